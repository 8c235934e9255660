#!/usr/bin/env python
"""Benchmark of the NVFP4 inference hot path (BASELINE.json metric: NVFP4 GEMM TFLOPS; MoE / TP layer tokens/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

The headline step is one pass of the W4A4 prompt projection (`Nvfp4.project(x, W4A4)`: device activation
quantizer + tcgen05 block-scaled GEMM) over one batch of synthetic activations at M = 8192 for the three
projection shapes of the sweep, (K, N) in {(4096, 4096), (4096, 14336), (14336, 4096)}. Inputs are seeded N(0, 1)
activations and N(0, 0.02) weights quantised once to NVFP4; they stand in for real checkpoints (none exist
offline) and are larger than L2 (126 MB) per step.

`value` is TFLOP/s with inputs resident in HBM; `e2e` runs the same step from pinned host activations to pinned
host outputs through the public API. `roofline` is the GEMM kernel alone (CUDA events around each launch);
`cpu_baseline` is the CPU oracle's restatement of the reference's CPU lane timed on a bounded sample.

With N > 1 (torchrun) every rank runs an independent replica of the GEMM step (the sweep does not shard, so
`value` scales weakly), and the one path that DOES shard, the tensor-parallel decoder layer of config 4, is
measured in the same process group: the JSON line carries a `tp_layer` object (decode and 8192-token prefill
tokens/s at this N, their reduce path, roofline and parity against the 1-rank layer on rank 0). At N = 1 the
line also carries `moe`, `attn_decode` and `attn_prefill` (configs 2 and 3), each with a CPU baseline.

Every row of the hot path also has a workload of its own (same JSON contract, its own metric):

    --workload moe           config 2: 4096 tokens, hidden 2048, 128 experts, top-8 (tokens/s)
    --workload attn_decode   config 3: batch 32 x 1 query over 32768 keys (GB/s of K/V read;
                             --kv nvfp4 reads the same keys as NVFP4 cache rows)
    --workload attn_prefill  config 3: batch 4 x 8192 causal (TFLOP/s)
    --workload tp_decode     config 4: decoder layer, batch 64 over a 4096-token cache (tokens/s),
    --workload tp_prefill    config 4: decoder layer, 8192-token prefill (tokens/s); both shard over
                             --gpus N ranks (strong scaling, two all-reduces per layer)
    --workload gemm_sweep    config 1 in full: M in {1, 16, 128, 1024, 8192} x the three (K, N) x the lanes
                             (W4A4, W4A4 per-row scale, W4A16, BF16 x BF16), weights rotated over >= 1 GiB of
                             distinct copies where the product is weight-streaming bound (one JSON line per point)
"""
import argparse
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(4096, 4096), (4096, 14336), (14336, 4096)]   # (K, N)
M = 8192
WORKLOAD = "nvfp4_w4a4_linear_prefill_M8192_KN{4096x4096,4096x14336,14336x4096}"
NOMINAL_FP4_TFLOPS = 9000.0


def step_flops(m=M):
    return sum(2.0 * m * n * k for (k, n) in SHAPES)


def main_config(world):
    return {"workload": WORKLOAD, "M": M, "KN": SHAPES, "lane": "W4A4 input_scale=1",
            "parallelism": f"replicas x{world}", "l2": "inputs+outputs per step exceed L2 (126 MB)"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def recorded_traffic(kernel_source, key):
    """dram bytes per launch of a kernel from the committed ncu summary profiles/<key>.json, valid only for the
    kernel source it was captured from (the file records that source's SHA-1); None when absent or stale."""
    path = os.path.join(ROOT, "profiles", key + ".json")
    if not os.path.exists(path):
        return None, "no capture on record"
    with open(path) as f:
        rec = json.load(f)
    with open(os.path.join(ROOT, kernel_source), "rb") as f:
        sha = hashlib.sha1(f.read()).hexdigest()
    if rec.get("source_sha1") != sha:
        return None, "the capture on record is of an older kernel source"
    return rec.get("traffic_bytes_per_launch"), rec.get("traffic_unit", "bytes/launch (ncu)")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        self.lines = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, args=(self.proc,), daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self, proc):
        for line in proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        self.proc = None
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's CPU lanes on bounded samples of the same workloads.
# Only these functions (and the smoke / tests) touch oracle/.
# --------------------------------------------------------------------------------------
def _oracle(threads=None):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import oracle
    orc = oracle()
    orc.set_threads(threads or host_threads())      # never inherit a launcher's OMP_NUM_THREADS=1
    return orc


def cpu_lane(sample_rows, threads=None, repeats=1):
    """Config 0/1: decode to dense f32, f32 matmul, bf16 result (src/leaf.rs:184-191, src/nvfp4.rs:170-182)."""
    orc = _oracle(threads)
    from oracle_lib import f32_to_bf16_bits
    cores = orc.threads()
    rng = np.random.default_rng(0)
    planes = []
    for (k, n) in SHAPES:
        w = (rng.standard_normal(n * k, dtype=np.float32) * np.float32(0.02))
        codes, scales, s2 = orc.pack_nearest(w, k)
        t0 = time.perf_counter()
        dense = orc.dequantize(codes, scales, s2)
        planes.append((k, n, dense, time.perf_counter() - t0))
    xs = {k: f32_to_bf16_bits(rng.standard_normal(sample_rows * k, dtype=np.float32)) for k in (4096, 14336)}
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        for (k, n, dense, _) in planes:
            orc.linear_cpu_lane(xs[k], dense, sample_rows, n, k)
        times.append(time.perf_counter() - t0)
    flops = step_flops(sample_rows)
    decode_s = sum(p[3] for p in planes)
    return {"seconds": times, "flops": flops, "cores": cores, "decode_s": decode_s,
            "sample": f"first {sample_rows} of {M} activation rows over the three (K,N) shapes; dense f32 decode of "
                      f"the weights ({decode_s:.2f} s, once, untimed) then f32 matmul with bf16 result"}


def _random_planes(rng, rows, k):
    """NVFP4 planes with random code bytes and block scales in a plausible range: the CPU lanes' time does not
    depend on the values, and packing hundreds of millions of weights on the host would dominate the sample."""
    codes = rng.integers(0, 256, rows * k // 2, dtype=np.uint8)
    scales = rng.integers(0x28, 0x48, rows * k // 16, dtype=np.uint8)
    return codes, scales


def cpu_moe(sample_tokens=32):
    """Config 2 on a token sample: the oracle's expert block (gather, quantize, grouped products, SwiGLU, ordered
    weighted sum) after its softmax top-8 router."""
    orc = _oracle()
    from oracle_lib import f32_to_bf16_bits
    h, inter, E, K = 2048, 768, 128, 8
    rng = np.random.default_rng(1)
    x = f32_to_bf16_bits(rng.standard_normal(sample_tokens * h, dtype=np.float32))
    gate = f32_to_bf16_bits(rng.standard_normal(E * h, dtype=np.float32) * np.float32(0.02))
    banks = [_random_planes(rng, E * n, k) + (np.full(E, 1e-3, np.float32),) for (n, k) in ((2 * inter, h), (h, inter))]
    t0 = time.perf_counter()
    logits = orc.router_logits(x, gate, sample_tokens, h, E)
    idx, w = orc.router_select(orc.router_scores_softmax(logits), K)
    orc.moe_experts(x, idx, w, banks[0], banks[1], h, inter, E)
    dt = time.perf_counter() - t0
    return {"value": sample_tokens / dt, "unit": "tokens/s", "cores": orc.threads(), "kind": "port",
            "sample": f"{sample_tokens} of 4096 tokens through the router and the expert block (all 128 experts' planes resident)"}


def cpu_attention(decode, sample):
    """Config 3 on a sample: the oracle's f64 two-pass attention (src/models/inkling/flash.rs:1937-1987)."""
    orc = _oracle()
    H, KVH, D = 32, 8, 128
    rng = np.random.default_rng(2)
    if decode:
        L, nq = 32768, 1
        k = rng.standard_normal(L * KVH * D, dtype=np.float32)
        v = rng.standard_normal(L * KVH * D, dtype=np.float32)
        t0 = time.perf_counter()
        for _ in range(sample):
            orc.attention(rng.standard_normal(nq * H * D, dtype=np.float32), k, v, H, KVH, D, L - 1, 1.0 / np.sqrt(D))
        dt = time.perf_counter() - t0
        byts = sample * 2 * L * KVH * D * 2
        return {"value": byts / dt / 1e9, "unit": "GB/s", "cores": orc.threads(), "kind": "port",
                "sample": f"{sample} of 32 sequences, one query over 32768 keys each (bf16-sized K/V bytes counted)"}
    S = sample
    q = rng.standard_normal(S * H * D, dtype=np.float32)
    k = rng.standard_normal(S * KVH * D, dtype=np.float32)
    v = rng.standard_normal(S * KVH * D, dtype=np.float32)
    t0 = time.perf_counter()
    orc.attention(q, k, v, H, KVH, D, 0, 1.0 / np.sqrt(D))
    dt = time.perf_counter() - t0
    return {"value": 4.0 * H * S * S * D / 2 / dt / 1e12, "unit": "TFLOP/s", "cores": orc.threads(), "kind": "port",
            "sample": f"one sequence of {S} tokens (of 4 x 8192), causal, 32 heads"}


_CPU_LAYER = {}


def cpu_layer(rows, past):
    """Config 4 on a row sample: one decoder layer from oracle pieces (norm, W4A4 projections, attention, SwiGLU,
    residual adds) with the reference's rounding points, every projection at full size; each sampled row is one
    query over `past` + 1 cached keys (the rotation of q and k is left out: it is a millionth of the work)."""
    orc = _oracle()
    from oracle_lib import f32_to_bf16_bits, bf16_bits_to_f32
    hidden, heads, kvh, D, inter = 4096, 32, 8, 128, 14336
    rng = np.random.default_rng(3)
    shapes = {"q": (heads * D, hidden), "k": (kvh * D, hidden), "v": (kvh * D, hidden), "o": (hidden, heads * D),
              "gate": (inter, hidden), "up": (inter, hidden), "down": (hidden, inter)}
    if not _CPU_LAYER:
        _CPU_LAYER.update({name: _random_planes(rng, n, k) for name, (n, k) in shapes.items()})
    w = _CPU_LAYER
    gain = f32_to_bf16_bits(np.ones(hidden, np.float32))
    x = f32_to_bf16_bits(rng.standard_normal(rows * hidden, dtype=np.float32))
    kc = rng.standard_normal((past + 1) * kvh * D, dtype=np.float32)
    vc = rng.standard_normal((past + 1) * kvh * D, dtype=np.float32)

    def lin(xb, name):
        n, k = shapes[name]
        c, s = w[name]
        ac, asc = orc.quantize_act_scaled(bf16_bits_to_f32(xb), rows, k, 1.0)
        return f32_to_bf16_bits(orc.linear_w4a4(ac, asc, c, s, np.float32(1e-3), rows, n, k))

    t0 = time.perf_counter()
    nrm = orc.rmsnorm_breeze(x, gain, rows, hidden, 1e-6)
    q, _, _ = lin(nrm, "q"), lin(nrm, "k"), lin(nrm, "v")
    att = np.concatenate([orc.attention(bf16_bits_to_f32(q.reshape(rows, -1)[r]), kc, vc, heads, kvh, D, past, 1.0 / np.sqrt(D))
                          for r in range(rows)]).astype(np.float32)
    resid = orc.add_bf16(x, lin(f32_to_bf16_bits(att), "o"))
    nrm = orc.rmsnorm_breeze(resid, gain, rows, hidden, 1e-6)
    orc.add_bf16(resid, lin(orc.swiglu_bf16(lin(nrm, "gate"), lin(nrm, "up")), "down"))
    dt = time.perf_counter() - t0
    return {"value": rows / dt, "unit": "tokens/s", "cores": orc.threads(), "kind": "port",
            "sample": f"{rows} token rows, each one query over {past + 1} cached keys, all seven projections at full size"}


def run_reference(args, rank, world):
    if rank != 0:
        return          # one CPU arm per job: the other ranks of a multi-process launch do no work
    sample_rows = 64
    res = cpu_lane(sample_rows, repeats=max(1, args.steps))
    secs = res["seconds"]
    total = sum(secs)
    tflops = res["flops"] * len(secs) / total / 1e12
    line = {
        "impl": "reference", "metric": "nvfp4_gemm_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": len(secs), "warmup": args.warmup, "ms_per_step": 1e3 * total / len(secs), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 (dequantised e2m1 x e4m3 weights, bf16 activations)",
        "data": "synthetic", "config": main_config(args.gpus),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": res["cores"], "kind": "port",
                         "sample": res["sample"]},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# GPU workloads. Each builder returns a dict: step (callable), e2e (callable or None), units per step, metric,
# unit, roof(ms) -> roofline dict, config, launches per step, h2d / d2h bytes per e2e step, cpu (callable -> dict).
# --------------------------------------------------------------------------------------
class Env:
    def __init__(self, rank, world, local_rank):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank, self.world, self.local_rank = rank, world, local_rank
        torch.cuda.set_device(local_rank)
        self.dev = torch.device("cuda", local_rank)
        import maryml_b200  # noqa: F401  (fails loudly if the CUDA library is missing)
        from maryml_b200 import _lib
        self.ctx = _lib.context(local_rank)
        if world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.stream = torch.cuda.current_stream()
        self.peaks = measured_peaks()
        self.sampler = ClockSampler(local_rank) if rank == 0 else None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.world == 1:
            return list(values)
        t = self.torch.tensor(list(values), device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def check_flags(self):
        rc, flags = self.ctx.check_flags(None)
        if rc != 0:
            raise SystemExit(f"bench.py: device status words set: {flags}")

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def time_steps(env, step, steps, warmup, sample_clocks=True):
    """W untimed steps, then exactly `steps` steps between two CUDA events on the launching stream, a barrier and a
    device synchronize on both sides; the caller takes the max over ranks."""
    torch = env.torch
    for _ in range(max(warmup, 3)):
        step()
    env.barrier()
    if env.sampler and sample_clocks:
        env.sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(env.stream)
    for _ in range(steps):
        step()
    t1.record(env.stream)
    env.barrier()
    clocks = env.sampler.stop() if (env.sampler and sample_clocks) else None
    return t0.elapsed_time(t1), clocks


def build_moe(env, args):
    torch = env.torch
    from maryml_b200 import _lib, moe
    dev = env.dev
    g = torch.Generator(device=dev)
    g.manual_seed(99)
    T, h, inter, E, K = 4096, 2048, 768, 128, 8
    x = torch.randn(T, h, device=dev, generator=g).to(torch.bfloat16)
    gate = (torch.randn(E, h, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    b13 = moe.ExpertBank.quantize((torch.randn(E, 2 * inter, h, device=dev, generator=g) * 0.02).to(torch.bfloat16))
    b2 = moe.ExpertBank.quantize((torch.randn(E, h, inter, device=dev, generator=g) * 0.02).to(torch.bfloat16))
    flop = T * K * 2 * (h * 2 * inter + inter * h) + 2 * T * h * E
    byts = (E * (2 * inter * h + h * inter)) * 0.5625 + T * h * 2 + T * h * 4 + E * h * 2
    hx = x.cpu().pin_memory()
    hy = torch.empty(T, h, dtype=torch.float32).pin_memory()
    dx = torch.empty_like(x)

    def e2e():
        dx.copy_(hx, non_blocking=True)
        out, _ = moe.moe_layer(dx, gate, K, b13, b2)
        hy.copy_(out, non_blocking=True)

    peaks = env.peaks
    return {
        "step": lambda: moe.moe_layer(x, gate, K, b13, b2), "e2e": e2e, "units": T, "metric": "moe_layer_tokens_per_s",
        "unit": "tokens/s", # quantizer, router projection, selection, plan, gather, two products, un-permute (the ncu launch list of a layer);
        # the plan is one kernel up to 4096 tokens and k <= 8 (its chunks as one cluster), else three
        "launches": 7 + (1 if T <= 4096 and K <= 8 and os.environ.get("MB_MOE_PLAN_CLUSTER", "1") != "0" else 3)
        + splitk_sum_launches(_lib.context(dev.index), 1, T, E, h),
        "h2d": T * h * 2, "d2h": T * h * 4,
        "roof": lambda ms: {"bound": "hbm", "kernel": "whole layer", "achieved": byts / (ms * 1e-3) / 1e9,
                            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": byts / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                            "peak_source": peaks["source"], "traffic": None, "flop_per_step": flop,
                            "note": "min bytes = expert planes + x + out; the layer is weight-streaming bound at 4096 tokens"},
        "config": {"workload": "moe_layer_T4096_h2048_E128_top8_inter768",
                   "lane": "SwiGLU and the second projection's quantizer fused into the first grouped product"},
        "cpu": lambda: cpu_moe(32),
    }


def build_attention(env, args, decode):
    torch = env.torch
    from maryml_b200 import attention as att, _lib
    dev = env.dev
    g = torch.Generator(device=dev)
    g.manual_seed(98)
    H, KVH, D = 32, 8, 128
    B, nq, L = (32, 1, 32768) if decode else (4, 8192, 8192)
    if args.batch:
        B = args.batch
    q = torch.randn(B, nq, H, D, device=dev, generator=g).to(torch.bfloat16)
    k = torch.randn(B, L, KVH, D, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(B, L, KVH, D, device=dev, generator=g).to(torch.bfloat16)
    ws = torch.empty(max(int(_lib.lib.mb_attention_workspace(B, nq, L, H, KVH, D)), 16), dtype=torch.uint8, device=dev)
    packed = decode and args.kv == "nvfp4"
    if packed:
        kc, ks = att.quantize_kv_rows(k)
        vc, vs = att.quantize_kv_rows(v)
        del k, v
        attend = lambda qq: att.flash_attention_fp4kv(qq, kc, ks, vc, vs, KVH, q0=L - nq, workspace=ws)
    else:
        attend = lambda qq: att.flash_attention(qq, k, v, q0=L - nq, workspace=ws)
    hq = q.cpu().pin_memory()
    ho = torch.empty_like(hq).pin_memory()
    dq = torch.empty_like(q)

    def e2e():
        dq.copy_(hq, non_blocking=True)
        ho.copy_(attend(dq), non_blocking=True)

    peaks = env.peaks
    cfg = {"workload": f"attn_{'decode' if decode else 'prefill'}_B{B}_nq{nq}_keys{L}_heads32_kv8_d128",
           "rope": "pre-applied (inputs drawn N(0,1))"}
    w = {"step": lambda: attend(q), "e2e": e2e, "h2d": q.numel() * 2, "d2h": q.numel() * 2, "config": cfg}
    if decode:
        byts = 2 * B * L * KVH * D * (0.5625 if packed else 2)
        w.update(units=byts / 1e9, metric="decode_attention_kv_gbytes_per_s", unit="GB/s", launches=2,
                 roof=lambda ms: {"bound": "hbm", "kernel": "attn_decode_kernel<nvfp4 rows>" if packed else "attn_decode_kernel",
                                  "achieved": byts / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                  "frac": byts / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "peak_source": peaks["source"],
                                  "frac_of_nominal_8tbs": byts / (ms * 1e-3) / 1e9 / 8000.0, "traffic": None},
                 cpu=lambda: cpu_attention(True, 2))
        if packed:
            cfg["workload"] += "_nvfp4rows"
            cfg["kv"] = "NVFP4 cache rows: 0.5625 B per value counted; the bf16 cache of the same keys is 3.56x the bytes"
    else:
        flop = 4.0 * B * H * nq * L * D / 2
        w.update(units=flop / 1e12, metric="prefill_attention_tflops", unit="TFLOP/s", launches=1,
                 roof=lambda ms: {"bound": "tensor", "kernel": "attn_prefill_tc5_kernel (tcgen05, TMEM-resident O)",
                                  "achieved": flop / (ms * 1e-3) / 1e12, "peak": peaks["bf16"], "unit": "TFLOP/s",
                                  "frac": flop / (ms * 1e-3) / 1e12 / peaks["bf16"], "peak_source": peaks["source"],
                                  "traffic": None},
                 cpu=lambda: cpu_attention(False, 1024))
    return w


class TpLayerSetup:
    """Config 4: the NVFP4 decoder layer cut over the job's ranks (the same stored tensors on every rank, cut after
    quantisation), one NCCL group and, for decode-sized messages, one fused peer-memory exchange."""

    def __init__(self, env, want_fused):
        torch, dist = env.torch, env.dist
        from maryml_b200 import nvfp4 as mb, layer
        self.env, self.layer = env, layer
        self.cfg = cfgL = layer.LayerConfig()
        rank, world, dev = env.rank, env.world, env.dev
        self.tp = layer.Tp(rank, world)

        def exchange(raw):
            obj = [raw]
            dist.broadcast_object_list(obj, src=0)
            return obj[0]
        self.group = layer.Group(self.tp, env.local_rank, exchange) if world > 1 else None
        D = cfgL.head_dim
        self.shapes = {"q": (cfgL.heads * D, cfgL.hidden), "k": (cfgL.kv_heads * D, cfgL.hidden),
                       "v": (cfgL.kv_heads * D, cfgL.hidden), "o": (cfgL.hidden, cfgL.heads * D),
                       "gate": (cfgL.inter, cfgL.hidden), "up": (cfgL.inter, cfgL.hidden), "down": (cfgL.hidden, cfgL.inter)}
        gw = torch.Generator(device=dev)
        gw.manual_seed(7)
        self.full = {}
        for name, (n, kk) in self.shapes.items():
            qz = mb.Nvfp4.quantize((torch.randn(n, kk, device=dev, generator=gw) * 0.02).to(torch.bfloat16))
            self.full[name] = (qz.codes, qz.scales, qz.scale2)
        self.gain = torch.ones(cfgL.hidden, dtype=torch.bfloat16, device=dev)
        self.fx = self.bulk = None

        def exchange_all(raw):
            got = [None] * world
            dist.all_gather_object(got, raw)
            return got
        if want_fused and world > 1:
            # decode-sized messages: the GEMM epilogue scatters its partial tiles into the peers (32-byte segments)
            self.fx = layer.FusedExchange(self.tp, env.local_rank, 64, cfgL.hidden, exchange_all)
        if world > 1 and os.environ.get("MB_TP_BULK", "1") != "0":
            # prompt-sized messages: reduce-scatter and all-gather kernels over a peer-mapped region
            # (MB_TP_BULK=0 in the environment keeps NCCL for them, for comparison runs)
            # every rank has to end up with the same answer: one that cannot map its peers sends all back to NCCL
            try:
                self.bulk = layer.BulkExchange(self.tp, env.local_rank, 8192, cfgL.hidden, exchange_all)
                mine = 1.0
            except Exception as exc:
                sys.stderr.write(f"bench.py: rank {rank}: no peer-memory region for the prompt exchanges ({exc}); NCCL instead\n")
                mine = 0.0
            (worst,) = env.max_over_ranks([1.0 - mine])
            if worst > 0.0 and self.bulk is not None:
                self.bulk.close()
                self.bulk = None
        self.params = sum(n * kk for (n, kk) in self.shapes.values())

    def make_layer(self, fused):
        return self.layer.DecoderLayer(self.cfg, self.full, self.gain, self.gain, tp=self.tp, group=self.group,
                                       device=self.env.dev, fused=self.fx if fused else None, bulk=self.bulk)

    def reference_layer(self):
        """The unsharded layer over the same stored planes (rank 0 only: the parity arm)."""
        return self.layer.DecoderLayer(self.cfg, self.full, self.gain, self.gain, device=self.env.dev)

    def inputs(self, decode):
        torch = self.env.torch
        cfgL, dev = self.cfg, self.env.dev
        batch, t, past = (64, 1, 4096) if decode else (1, 8192, 0)
        g = torch.Generator(device=dev)
        g.manual_seed(11 if decode else 12)          # the same bytes on every rank
        x = torch.randn(batch * t, cfgL.hidden, device=dev, generator=g).to(torch.bfloat16)
        kc = torch.randn(batch, past + t, cfgL.kv_heads, cfgL.head_dim, device=dev, generator=g).to(torch.bfloat16)
        vc = torch.randn(batch, past + t, cfgL.kv_heads, cfgL.head_dim, device=dev, generator=g).to(torch.bfloat16)
        return batch, t, past, x, kc, vc

    def close(self):
        if self.bulk is not None:
            self.bulk.close()
        if self.fx is not None:
            self.fx.close()
        if self.group is not None:
            self.group.close()


def splitk_sum_launches(ctx, operands, rows, n, k):
    """1 when a split-K product (operands 0: NVFP4, 1: bf16) needs its second kernel, the sum of f32 planes; 0 when
    it is not split or its K slices meet inside the product's own kernel (one cluster per output tile)."""
    import ctypes as C
    from maryml_b200 import _lib
    cs, ps = C.c_int(), C.c_int()
    ctx.check(_lib.lib.mb_gemm_splitk_plan(ctx.handle, operands, rows, n, k, C.byref(cs), C.byref(ps)))
    return 1 if ps.value > 1 and cs.value == 0 else 0


def tp_launches(setup, L_, rows, decode, fused):
    """Kernels of ours per layer step: norm+quantize, q|k|v product, rotation+append, attention, quantize, o product,
    add+norm+quantize, gate/up+SwiGLU+quantize product, down product, add = 10; the decode kernel adds its combine
    pass; a product with <= 128 rows and few tiles adds a split-K sum; the fused exchange swaps (sum, add) for its
    reduce+residual kernel and runs the second norm+quantize on its own."""
    from maryml_b200 import _lib
    cfgL = setup.cfg
    splitk = lambda n, k: splitk_sum_launches(_lib.context(setup.env.dev.index), 0, rows, n, k)
    n_qkv = (L_.local_heads + 2 * L_.local_kv_heads) * cfgL.head_dim
    launches = 10 + (1 if decode else 0) + splitk(n_qkv, cfgL.hidden)
    if fused:
        launches += 1
    else:
        launches += splitk(cfgL.hidden, L_.local_heads * cfgL.head_dim) + splitk(cfgL.hidden, L_.local_inter)
    return launches


def build_tp(env, args, decode, setup=None, fused=None):
    torch = env.torch
    own_setup = setup is None
    fused = args.fused if fused is None else fused
    if setup is None:
        setup = TpLayerSetup(env, fused)
    cfgL, world = setup.cfg, env.world
    batch, t, past, x, kc_full, vc_full = setup.inputs(decode)
    use_fused = bool(fused and setup.fx is not None and batch * t <= setup.fx.t_max)
    L_ = setup.make_layer(use_fused)
    kv = setup.tp.kv_heads(cfgL.kv_heads)
    kc = kc_full[:, :, kv.start:kv.stop].contiguous()
    vc = vc_full[:, :, kv.start:kv.stop].contiguous()
    hx = x.cpu().pin_memory()
    hy = torch.empty_like(hx).pin_memory()
    dx = torch.empty_like(x)

    def e2e():
        dx.copy_(hx, non_blocking=True)
        hy.copy_(L_.forward(dx, batch, past, kc, vc), non_blocking=True)

    peaks = env.peaks
    D = cfgL.head_dim
    if decode:
        byts = (setup.params * 0.5625 + 2 * batch * (past + t) * cfgL.kv_heads * D * 2) / world
        roof = lambda ms: {"bound": "hbm", "kernel": "whole layer per rank", "achieved": byts / (ms * 1e-3) / 1e9,
                           "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": byts / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                           "peak_source": peaks["source"], "traffic": None,
                           "note": "weights + KV per rank; the two exchanges of [64, 4096] are latency terms"}
    else:
        flop = (2.0 * t * setup.params + 4.0 * cfgL.heads * t * t * D / 2) / world
        roof = lambda ms: {"bound": "tensor", "kernel": "whole layer per rank", "achieved": flop / (ms * 1e-3) / 1e12,
                           "peak": 4 * peaks["bf16"], "unit": "TFLOP/s", "frac": flop / (ms * 1e-3) / 1e12 / (4 * peaks["bf16"]),
                           "peak_source": "4 x " + peaks["source"] + " bf16 burst", "traffic": None,
                           "note": "projections at the FP4 rate dominate; attention runs at the bf16 rate"}
    if use_fused:
        reduce = "fused: GEMM epilogue scatters to peers, one reduce+residual+gather kernel"
    elif world > 1 and L_._rows_shard(batch * t):
        how = ("peer-memory kernels (peer stores, flags)" if (L_.bulk is not None and L_.bulk.takes(batch * t, cfgL.hidden))
               else "nccl")
        reduce = (f"{how}, rows sharded between the exchanges: reduce-scatter f32 by rows, norm + quantizer on the rank's "
                  "rows, all-gather of NVFP4 planes; reduce-scatter f32 + add, all-gather of bf16 rows")
    else:
        reduce = "nccl all-reduce f32 + add" if world > 1 else "none (world 1)"
    w = {
        "step": lambda: L_.forward(x, batch, past, kc, vc), "e2e": e2e, "units": batch * t,
        "metric": f"tp_layer_{'decode' if decode else 'prefill'}_tokens_per_s", "unit": "tokens/s",
        "launches": tp_launches(setup, L_, batch * t, decode, use_fused) +
                    (4 if (not use_fused and world > 1 and L_._rows_shard(batch * t) and L_.bulk is not None
                           and L_.bulk.takes(batch * t, cfgL.hidden)) else 0),      # two reduce-scatters, two all-gathers
        "h2d": x.numel() * 2, "d2h": x.numel() * 2,
        "roof": roof, "reduce": reduce,
        "config": {"workload": f"tp_{'decode' if decode else 'prefill'}_hidden4096_heads32_kv8_ffn14336_batch{batch}_t{t}_past{past}",
                   "parallelism": f"tp{world}", "reduce": reduce},
        # a prompt token sees 4096 keys on average
        "cpu": (lambda: cpu_layer(4, 4096)) if decode else (lambda: cpu_layer(4, 4095)),
        "parity_inputs": (batch, t, past, x, kc_full, vc_full), "layer": L_, "kc": kc, "vc": vc,
        "cleanup": setup.close if own_setup else (lambda: None),
    }
    return w


def tp_parity(env, setup, w):
    """Parity of the sharded layer against the unsharded layer on rank 0 (same stored planes, same inputs), exchange
    by exchange. The cut changes one thing, the association of the K sums of the two row-parallel products, so each
    all-reduced partial is compared with the unsharded product of the SAME input bytes: `max_rel` is the larger of
    the two relative errors (|err| / max|ref|). The layer's output through the production path (fused exchange or
    row-sharded prompt path) against the unsharded layer end to end is reported beside it: W4A4 re-quantizes bf16
    intermediates three times per layer, so noise in the last bf16 bit of the attention output (another key-split
    count is enough) flips E2M1 codes downstream, and two correct evaluations of this layer sit a few percent of
    the output's rms apart (the CPU oracle included; the design notes carry the numbers). Returned on rank 0."""
    torch, dist = env.torch, env.dist
    L = w["layer"]
    batch, t, past, x, kc_full, vc_full = w["parity_inputs"]
    y_prod = L.forward(x, batch, past, w["kc"], w["vc"]).clone()
    a = L._attention(x, batch, past, w["kc"], w["vc"])
    o_sum = L._all_reduce(L._linear(a, L.wo, out_dtype=torch.float32))
    residual, down = L.half_mlp(x, o_sum)
    down_sum = L._all_reduce(down)
    y = L.finish(residual, down_sum)
    if env.world > 1:
        parts = [torch.empty_like(a) for _ in range(env.world)]
        dist.all_gather(parts, a.contiguous())
        a_full = torch.cat(parts, 1)          # heads in rank order
    else:
        a_full = a
    env.barrier()
    if env.rank != 0:
        return None
    L1 = setup.reference_layer()
    o1 = L1._linear(a_full, L1.wo, out_dtype=torch.float32)
    res1, down1 = L1.half_mlp(x, o_sum)
    y1 = L1.finish(res1, down1)
    e_o = float((o_sum - o1).abs().max() / o1.abs().max())
    e_d = float((down_sum - down1).abs().max() / down1.abs().max())
    same_resid = bool(torch.equal(res1.view(torch.int16), residual.view(torch.int16)))
    moved = float((y.view(torch.int16) != y1.view(torch.int16)).float().mean())
    y_ref = L1.forward(x, batch, past, kc_full.clone(), vc_full.clone()).float()
    torch.cuda.synchronize()

    def dist_of(got, ref):
        err = (got.float() - ref).abs()
        rms = ref.pow(2).mean().sqrt()
        cos = torch.nn.functional.cosine_similarity(got.float().ravel().double(), ref.ravel().double(), dim=0)
        return {"max_err_over_rms": float(err.max() / rms), "mean_err_over_rms": float(err.mean() / rms), "cosine": float(cos)}
    out = {"max_rel": max(e_o, e_d), "o_sum_rel": e_o, "down_sum_rel": e_d, "residual_bit_equal": same_resid,
           "output_bf16_moved": moved,
           "vs": "1-rank layer on rank 0 fed the same bytes at each exchange; rel = max|err| / max|ref| of the all-reduced f32 partial",
           "end_to_end": dict(dist_of(y_prod, y_ref), path=w["reduce"],
                              note="every stage on its own previous output: re-quantized bf16 intermediates amplify last-bit "
                                   "noise of the attention output, see the design notes"),
           "production_vs_allreduce_bf16_moved": float((y_prod.view(torch.int16) != y.view(torch.int16)).float().mean())}
    del L1
    return out


def measure_extra(env, w, steps, warmup, cpu=True, graph=False):
    """Times one workload as a leg of the default run; returns its record (rank 0) or None."""
    torch = env.torch
    ms, clocks = time_steps(env, w["step"], steps, warmup)
    (ms,) = env.max_over_ranks([ms])
    per = ms / steps
    rec = None
    graph_ms = None
    if graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(env.stream)
            with torch.cuda.stream(side):
                for _ in range(3):
                    w["step"]()
            env.stream.wait_stream(side)
            env.barrier()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                w["step"]()
            if env.world > 1:
                # two trial replays before the timed ones: a replay whose peer waits run out costs a second each, and
                # every rank has to agree on whether the timed replays run
                gr.replay()
                gr.replay()
                torch.cuda.synchronize()
                rc, flags = env.ctx.check_flags(None)
                (bad,) = env.max_over_ranks([1.0 if (rc != 0 or any(flags)) else 0.0])
                if bad:
                    raise RuntimeError(f"trial replay raised device status words {flags}")
            gms, _ = time_steps(env, gr.replay, steps, warmup, sample_clocks=False)
            (gms,) = env.max_over_ranks([gms])
            graph_ms = gms / steps
            del gr
        except Exception as exc:                          # a capture that fails costs the leg, not the line
            graph_ms = f"capture failed: {type(exc).__name__}: {exc}"[:200]
    env.check_flags()
    if env.rank == 0:
        mult = 1 if w["metric"].startswith("tp_") else env.world
        rec = {"metric": w["metric"], "value": mult * w["units"] / (per * 1e-3), "unit": w["unit"], "ms": per, "steps": steps,
               "gpu_launches_per_step": w["launches"], "roofline": w["roof"](per), "config": w["config"], "clocks": clocks}
        if "reduce" in w:
            rec["reduce"] = "fused" if w["reduce"].startswith("fused") else ("nccl" if env.world > 1 else "none")
        rec["launch"] = "host (Python, one C call per kernel)"
        if isinstance(graph_ms, float):
            rec["cuda_graph_replay"] = {"ms": graph_ms, "value": mult * w["units"] / (graph_ms * 1e-3)}
            if graph_ms < per:
                # the same kernels replayed as a CUDA graph: what the GPU needs for the step when the host layer
                # (about 40 us per call on an idle host, several times that on a busy one) is off the clock
                rec["host_launched"] = {"ms": per, "value": rec["value"]}
                rec.update(value=mult * w["units"] / (graph_ms * 1e-3), ms=graph_ms, roofline=w["roof"](graph_ms),
                           launch="cuda graph replay")
        elif graph_ms is not None:
            rec["cuda_graph_replay"] = graph_ms
        if cpu:
            try:
                rec["cpu_baseline"] = w["cpu"]()
            except Exception as exc:
                rec["cpu_baseline"] = {"error": f"{type(exc).__name__}: {exc}"}
    return rec


def run_ours(args, rank, world, local_rank):
    env = Env(rank, world, local_rank)
    torch, dev, ctx, stream = env.torch, env.dev, env.ctx, env.stream
    from maryml_b200 import nvfp4 as mb, _lib

    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    weights, acts, outs = [], {}, []
    for (k, n) in SHAPES:
        w = (torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        q = mb.Nvfp4.quantize(w)
        q.sf_tiled()
        weights.append(q)
        del w
        outs.append(torch.empty(M, n, dtype=torch.bfloat16, device=dev))
    for k in (4096, 14336):
        acts[k] = torch.randn(M, k, device=dev, generator=g).to(torch.bfloat16)
    # preallocated activation planes: the step allocates nothing
    a_codes = {k: torch.empty(M, k // 2, dtype=torch.uint8, device=dev) for k in acts}
    a_sf = {k: torch.empty(mb.sf_bytes(M, k), dtype=torch.uint8, device=dev) for k in acts}
    sp = lambda t: t.data_ptr()
    lib = _lib.lib
    gemm_events = []

    def step(record=False):
        for q, out in zip(weights, outs):
            k, n = q.k(), q.n()
            x = acts[k]
            ctx.check(lib.mb_nvfp4_quantize_act(ctx.handle, stream.cuda_stream, sp(x), _lib.DT_BF16, M, k,
                                                _lib.QUANT_SCALED, 1.0, None, 0, sp(a_codes[k]), sp(a_sf[k]),
                                                _lib.SF_TILED, None))
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            ctx.check(lib.mb_nvfp4_gemm_w4a4(ctx.handle, stream.cuda_stream, sp(a_codes[k]), sp(a_sf[k]), sp(q.codes),
                                             sp(q.sf_tiled()), None, q.scale2, M, n, k, sp(out), _lib.DT_BF16,
                                             _lib.EPI_PLAIN))
            if record:
                e1.record(stream)
                gemm_events.append((e0, e1, 2.0 * M * n * k))

    launches_per_step = 2 * len(SHAPES)        # 3 x (quantize + gemm); the scale plane's memset is the driver's
    for _ in range(max(args.warmup, 3)):
        step()
    env.barrier()
    if env.sampler:
        env.sampler.start()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(args.steps):
        step(record=True)
    t1.record(stream)
    env.barrier()
    clocks = env.sampler.stop() if env.sampler else None
    (ms,) = env.max_over_ranks([t0.elapsed_time(t1)])
    env.check_flags()

    # kernel-only roofline of the GEMM launches (CUDA events on the launching stream)
    gemm_ms = sum(e0.elapsed_time(e1) for (e0, e1, _) in gemm_events)
    gemm_fl = sum(f for (_, _, f) in gemm_events)
    achieved = gemm_fl / (gemm_ms * 1e-3) / 1e12
    peaks = env.peaks
    fp4_peak = 4.0 * peaks["bf16"]

    # A sustained leg beside the driver's short one: the same step for about a second, with the clocks it ran at.
    sustained = None
    if not args.no_extras:
        n_sus = max(200, int(1000.0 / max(ms / args.steps, 1e-3)))
        sms, sclk = time_steps(env, step, n_sus, 3)
        (sms,) = env.max_over_ranks([sms])
        sustained = {"steps": n_sus, "ms_per_step": sms / n_sus, "value": world * step_flops() * n_sus / (sms * 1e-3) / 1e12,
                     "unit": "TFLOP/s", "clocks": sclk,
                     "note": "the power cap, not the kernel, sets the clock of a second-long run"}

    # end to end: pinned host activations in, pinned host outputs back, every step
    h_x = {k: torch.empty(M, k, dtype=torch.bfloat16).pin_memory() for k in acts}
    for k in acts:
        h_x[k].copy_(acts[k])
    h_y = [torch.empty(M, q.n(), dtype=torch.bfloat16).pin_memory() for q in weights]
    # Three streams, as a serving host would run it: activations of the next projection travel up while
    # the current one computes and the previous result travels down (PCIe is full duplex). Device input
    # buffers are double-buffered per projection; every copy and every projection of every step is inside
    # the timed region, and the region ends only when the last result has landed in host memory.
    n_proj = len(weights)
    d_x2 = [[torch.empty(M, q.k(), dtype=torch.bfloat16, device=dev) for q in weights] for _ in range(2)]
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [[torch.cuda.Event() for _ in range(n_proj)] for _ in range(2)]
    ev_cmp = [[torch.cuda.Event() for _ in range(n_proj)] for _ in range(2)]
    e2e_count = [0]

    def e2e_step():
        slot = e2e_count[0] & 1
        first = e2e_count[0] < 2
        e2e_count[0] += 1
        for i, (q, hy) in enumerate(zip(weights, h_y)):
            with torch.cuda.stream(s_in):
                if not first:
                    s_in.wait_event(ev_cmp[slot][i])          # the projection that last read this buffer is done
                d_x2[slot][i].copy_(h_x[q.k()], non_blocking=True)
                ev_in[slot][i].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(ev_in[slot][i])
                y = q.project(d_x2[slot][i], mb.PromptLane.W4A4)
                ev_cmp[slot][i].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[slot][i])
                hy.copy_(y.view(M, q.n()), non_blocking=True)
                y.record_stream(s_out)

    def e2e_join():
        for st in (s_in, s_cmp, s_out):
            stream.wait_stream(st)

    e2e_steps = max(4, min(args.steps, 8))
    e2e_step()
    e2e_step()
    e2e_join()
    env.barrier()
    s0 = torch.cuda.Event(enable_timing=True)
    s1 = torch.cuda.Event(enable_timing=True)
    s0.record(stream)
    for st in (s_in, s_cmp, s_out):
        st.wait_stream(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()
    s1.record(stream)
    env.barrier()
    (e2e_ms,) = env.max_over_ranks([s0.elapsed_time(s1)])
    h2d = sum(M * q.k() * 2 for q in weights)
    d2h = sum(M * q.n() * 2 for q in weights)
    # the headline's buffers are not needed by the legs below
    del d_x2, h_x, h_y

    # ---- the other rows of the hot path, measured in the same process (group) ---------------------------------
    extras = {}
    if not args.no_extras:
        layer_steps = max(200, args.steps)
        try:
            setup = TpLayerSetup(env, want_fused=True)
            tp = {}
            for decode in (True, False):
                name = "decode" if decode else "prefill"
                wl = build_tp(env, args, decode, setup=setup, fused=decode)
                rec = measure_extra(env, wl, layer_steps if decode else max(50, min(layer_steps, 200)), 5, cpu=(world == 1),
                                    graph=(decode and (world == 1 or setup.fx is not None)))
                parity = tp_parity(env, setup, wl)
                if decode and world > 1 and setup.fx is not None:
                    alt = measure_extra(env, build_tp(env, args, True, setup=setup, fused=False), layer_steps, 5, cpu=False)
                    if rec is not None and alt is not None:
                        rec["alt"] = {"reduce": "nccl", "ms": alt["ms"], "value": alt["value"]}
                if rec is not None:
                    rec["tokens_per_s"] = rec["value"]
                    rec["parity"] = parity
                    tp[name] = rec
                del wl
                torch.cuda.empty_cache()
            setup.close()
            del setup
            torch.cuda.empty_cache()
            if rank == 0:
                extras["tp_layer"] = dict(tp, world=world,
                                          config="hidden 4096, 32 heads / 8 KV heads, FFN 14336, all projections NVFP4 W4A4; "
                                                 "decode: batch 64 over a 4096-token cache; prefill: 1 x 8192 tokens")
        except Exception as exc:
            if world > 1:
                raise                      # a rank that left a collective cannot be waited for: fail the job
            extras["tp_layer"] = {"error": f"{type(exc).__name__}: {exc}"}
        if world == 1:
            for name, build in (("moe", lambda: build_moe(env, args)),
                                ("attn_decode", lambda: build_attention(env, args, True)),
                                ("attn_prefill", lambda: build_attention(env, args, False))):
                try:
                    wl = build()
                    n_steps = {"moe": 200, "attn_decode": 100, "attn_prefill": 20}[name]
                    extras[name] = measure_extra(env, wl, n_steps, 3, graph=(name == "moe"))
                    del wl
                except Exception as exc:
                    extras[name] = {"error": f"{type(exc).__name__}: {exc}"}
                torch.cuda.empty_cache()

    if rank == 0:
        cpu = cpu_lane(256, repeats=1)
        cpu_tflops = cpu["flops"] / cpu["seconds"][0] / 1e12
        value = world * step_flops() * args.steps / (ms * 1e-3) / 1e12
        traffic, traffic_note = recorded_traffic("maryml_b200/csrc/gemm_tc5.cu", "gemm_tc5_pair_nvf4_prefill_M8192")
        line = {
            "metric": "nvfp4_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "e2m1 x e2m1 (ue4m3 block scales), f32 accumulate, bf16 out",
            "data": "synthetic", "config": main_config(world),
            "clocks": clocks,
            "e2e": {"value": world * step_flops() * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "tensor", "kernel": "gemm_tc5_pair_kernel (cta_group::2, 256x256 tiles)", "achieved": achieved,
                         "peak": fp4_peak, "unit": "TFLOP/s", "frac": achieved / fp4_peak,
                         "peak_source": f"4 x {peaks['source']} bf16 burst ({peaks['bf16']} TFLOP/s): no FP4 figure "
                                        f"in MEASURED_PEAKS.json",
                         "frac_of_nominal_9pf": achieved / NOMINAL_FP4_TFLOPS,
                         "regime": f"{args.steps} steps = {ms:.1f} ms timed: a burst figure unless the run is seconds long "
                                   f"(see `sustained`)",
                         "traffic": traffic, "traffic_unit": traffic_note},
            "cpu_baseline": {"value": cpu_tflops, "unit": "TFLOP/s", "cores": cpu["cores"], "kind": "port",
                             "sample": cpu["sample"]},
        }
        if sustained is not None:
            line["sustained"] = sustained
        line.update(extras)
        print(json.dumps(line), flush=True)
    env.close()


# --------------------------------------------------------------------------------------
# One workload per invocation
# --------------------------------------------------------------------------------------
def run_other(args, rank, world, local_rank):
    env = Env(rank, world, local_rank)
    torch = env.torch
    wl = args.workload
    if wl == "moe":
        w = build_moe(env, args)
    elif wl in ("attn_decode", "attn_prefill"):
        w = build_attention(env, args, wl == "attn_decode")
    else:
        w = build_tp(env, args, wl == "tp_decode")
    step = w["step"]
    cfg = w["config"]
    if args.graph:
        # Serving mode: the step is captured once into a CUDA graph (kernels, memsets and the NCCL
        # all-reduces alike) and replayed, which takes the host's ~30 launches per layer off the clock.
        side = torch.cuda.Stream()
        side.wait_stream(env.stream)
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        env.stream.wait_stream(side)
        env.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        step = graph.replay
        cfg["launch"] = "cuda graph replay"
    ms, clocks = time_steps(env, step, args.steps, args.warmup)
    e2e = w["e2e"]
    e2e()
    env.barrier()
    n_e2e = max(2, min(args.steps, 5))
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record(env.stream)
    for _ in range(n_e2e):
        e2e()
    s1.record(env.stream)
    env.barrier()
    ms, e2e_ms = env.max_over_ranks([ms, s0.elapsed_time(s1)])
    env.check_flags()
    tp_like = wl.startswith("tp_")
    mult = 1 if tp_like else world          # the TP layer is one job over all ranks; the others are replicas
    if rank == 0:
        per_step = ms / args.steps
        try:
            cpu = w["cpu"]()
        except Exception as exc:
            cpu = {"error": f"{type(exc).__name__}: {exc}"}
        line = {"metric": w["metric"], "value": mult * w["units"] / (per_step * 1e-3), "unit": w["unit"], "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": per_step, "higher_is_better": True,
                "scaling": "strong" if tp_like else "weak", "vs_baseline": None, "dtype": "nvfp4/bf16, f32 accumulate",
                "data": "synthetic", "config": cfg, "clocks": clocks,
                "e2e": {"value": mult * w["units"] / (e2e_ms / n_e2e * 1e-3), "unit": w["unit"],
                        "h2d_bytes_per_step": w["h2d"], "d2h_bytes_per_step": w["d2h"]},
                "gpu_launches": w["launches"] * args.steps, "roofline": w["roof"](per_step), "cpu_baseline": cpu}
        print(json.dumps(line), flush=True)
    if "cleanup" in w:
        w["cleanup"]()
    env.close()


def run_sweep(args, rank, world, local_rank):
    """Config 1 in full. One JSON line per (lane, M, K, N). Weight-streaming points (M <= 128) rotate over enough
    distinct weight copies to exceed 1 GiB, so every launch streams its weights from HBM (the reference's own rule,
    src/models/breeze/nvfp4.rs:28-33); `resident` repeats the point on ONE copy (served from L2) for comparison."""
    env = Env(rank, world, local_rank)
    torch, dev = env.torch, env.dev
    from maryml_b200 import nvfp4 as mb
    peaks = env.peaks
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    lanes = args.lanes.split(",")
    ms_list = [int(v) for v in args.ms.split(",")]
    for (k, n) in SHAPES:
        wbytes = n * k * 0.5625
        copies = max(1, int(np.ceil((1 << 30) / wbytes)))
        base = mb.Nvfp4.quantize((torch.randn(n, k, device=dev, generator=g) * 0.02).to(torch.bfloat16))
        qs = [base]
        for _ in range(copies - 1):
            qs.append(mb.Nvfp4.from_parts(base.codes.clone(), base.scales.clone(), base.scale2, n, k, torch.bfloat16, dev))
        for q in qs:
            q.sf_tiled()
        wb16 = None
        for m in ms_list:
            x = torch.randn(1, m, k, device=dev, generator=g).to(torch.bfloat16)
            for lane in lanes:
                rotating = m <= 128 and lane != "bf16"
                if lane == "w4a4":
                    fn = lambda q: q.project(x, mb.PromptLane.W4A4)
                elif lane == "w4a4_rows":
                    fn = lambda q: q.project_w4a4_rows(x)
                elif lane == "w4a16":
                    fn = (lambda q: q.gemv(x, m)) if m <= 8 else (lambda q: q.project(x, mb.PromptLane.W4A16))
                else:
                    if wb16 is None:
                        wb16 = mb.dequantize(base.codes, base.scales, base.scale2, n, k, dtype=torch.bfloat16)
                    fn = lambda q: mb.bf16_gemm(x.view(m, k), wb16, out_dtype=torch.bfloat16)
                res = {}
                for mode, pool in (("rotating", qs if rotating else qs[:1]), ("resident", qs[:1])):
                    if mode == "resident" and not rotating:
                        continue
                    # One CUDA graph of a pass over the pool (at least eight calls), replayed: the host layer's
                    # per-call cost (a few tens of microseconds of Python) would otherwise hide every kernel that
                    # is shorter than that, which is all of them below a thousand rows.
                    calls = max(8, len(pool))
                    for q_ in pool:
                        fn(q_)
                    torch.cuda.synchronize()
                    side = torch.cuda.Stream()
                    side.wait_stream(env.stream)
                    with torch.cuda.stream(side):
                        fn(pool[0])
                    env.stream.wait_stream(side)
                    torch.cuda.synchronize()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph):
                        for c in range(calls):
                            fn(pool[c % len(pool)])
                    replays = max(3, min(args.steps, 200) // calls + 1)
                    t, _ = time_steps(env, graph.replay, replays, 3, sample_clocks=False)
                    res[mode] = t / (replays * calls)
                    del graph
                ms_ = res["rotating"]
                flop = 2.0 * m * n * k
                byts = (wbytes if lane != "bf16" else n * k * 2) + 2 * m * k + 2 * m * n
                hbm_bound = m <= 128
                ach = byts / (ms_ * 1e-3) / 1e9 if hbm_bound else flop / (ms_ * 1e-3) / 1e12
                tensor_peak = 4 * peaks["bf16"] if lane.startswith("w4a4") else peaks["bf16"]
                peak = peaks["hbm_gbs"] if hbm_bound else tensor_peak
                line = {"metric": "nvfp4_gemm_sweep_point", "lane": lane, "M": m, "K": k, "N": n, "ms": ms_,
                        "tflops": flop / (ms_ * 1e-3) / 1e12, "gbytes_per_s": byts / (ms_ * 1e-3) / 1e9,
                        "weights": f"rotating over {len(qs)} copies ({len(qs) * wbytes / 2**30:.2f} GiB)" if rotating else "one copy",
                        "resident_ms": res.get("resident"),
                        "roofline": {"bound": "hbm" if hbm_bound else "tensor", "achieved": ach, "peak": peak,
                                     "unit": "GB/s" if hbm_bound else "TFLOP/s", "frac": ach / peak,
                                     "peak_source": peaks["source"] + ("" if hbm_bound or not lane.startswith("w4a4") else " bf16 burst x 4")},
                        "kernel": "gemv_w4a16_kernel" if (lane == "w4a16" and m <= 8) else lane}
                if rank == 0:
                    print(json.dumps(line), flush=True)
        del qs, base, wb16
        torch.cuda.empty_cache()
    env.check_flags()
    env.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="gemm",
                    choices=["gemm", "moe", "attn_decode", "attn_prefill", "tp_decode", "tp_prefill", "gemm_sweep"])
    ap.add_argument("--kv", default="bf16", choices=["bf16", "nvfp4"],
                    help="attn_decode: read the cache as bf16 rows (the BASELINE config) or as NVFP4 rows")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--fused", action="store_true",
                    help="tp workloads: reduce over peer memory from the GEMM epilogue instead of NCCL")
    ap.add_argument("--graph", action="store_true", help="capture the step into a CUDA graph and time replays")
    ap.add_argument("--batch", type=int, default=0, help="override the batch of the attention workloads (profiling)")
    ap.add_argument("--no-extras", action="store_true",
                    help="default workload: the headline step only (no sustained leg, no tp_layer / moe / attention legs)")
    ap.add_argument("--lanes", default="w4a4,w4a4_rows,w4a16,bf16", help="gemm_sweep: lanes to run")
    ap.add_argument("--ms", default="1,16,128,1024,8192", help="gemm_sweep: activation row counts")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.workload == "gemm":
        run_ours(args, rank, world, local_rank)
    elif args.workload == "gemm_sweep":
        run_sweep(args, rank, world, local_rank)
    else:
        run_other(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
