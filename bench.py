#!/usr/bin/env python
"""Benchmark of the NVFP4 linear hot path (BASELINE.json metric: NVFP4 GEMM TFLOPS).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the W4A4 prompt projection (`Nvfp4.project(x, W4A4)`: device
activation quantizer + tcgen05 block-scaled GEMM) over one batch of synthetic
activations at M = 8192 for the three projection shapes of the sweep,
(K, N) in {(4096, 4096), (4096, 14336), (14336, 4096)}. Inputs are seeded N(0, 1)
activations and N(0, 0.02) weights quantised once to NVFP4; they stand in for real
checkpoints (none exist offline) and are larger than L2 (126 MB) per step.

`value` is TFLOP/s with inputs resident in HBM; `e2e` runs the same step from pinned
host activations to pinned host outputs through the public API. `roofline` is the
GEMM kernel alone (CUDA events around each launch); `cpu_baseline` is the CPU oracle's
restatement of the reference's CPU lane timed on a bounded sample.

With N > 1 (torchrun) every rank runs an independent replica of the step: the GEMM
sweep does not shard (no collective on this path), so scaling is weak.

Other rows of the hot path have their own workloads (same JSON contract, their own metric):

    --workload moe           config 2: 4096 tokens, hidden 2048, 128 experts, top-8 (tokens/s)
    --workload attn_decode   config 3: batch 32 x 1 query over 32768 keys (GB/s of K/V read;
                             --kv nvfp4 reads the same keys as NVFP4 cache rows)
    --workload attn_prefill  config 3: batch 4 x 8192 causal (TFLOP/s)
    --workload tp_decode     config 4: decoder layer, batch 64 over a 4096-token cache (tokens/s),
    --workload tp_prefill    config 4: decoder layer, 8192-token prefill (tokens/s); both shard over
                             --gpus N ranks (strong scaling, two NCCL all-reduces per layer)
"""
import argparse
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


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


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
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
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
# CPU arm: the oracle's restatement of the reference's CPU lane (decode to dense f32,
# f32 matmul, bf16 result) on a bounded sample of the same workload.
# --------------------------------------------------------------------------------------
def cpu_lane(sample_rows, threads=None, repeats=1):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from oracle_lib import oracle, f32_to_bf16_bits
    orc = oracle()
    if threads:
        orc.set_threads(threads)
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


def run_reference(args, rank, world):
    if rank != 0:
        return
    sample_rows = 64
    for _ in range(args.warmup):
        pass  # the CPU lane has no cold caches worth warming beyond its first repeat below
    res = cpu_lane(sample_rows, repeats=max(1, args.steps))
    secs = res["seconds"]
    total = sum(secs)
    tflops = res["flops"] * len(secs) / total / 1e12
    line = {
        "impl": "reference", "metric": "nvfp4_gemm_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": len(secs), "warmup": args.warmup, "ms_per_step": 1e3 * total / len(secs), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 (dequantised e2m1 x e4m3 weights, bf16 activations)",
        "data": "synthetic", "config": {"workload": WORKLOAD, "sample_rows": sample_rows},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": res["cores"], "kind": "port",
                         "sample": res["sample"]},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------
def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the library has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import maryml_b200  # noqa: F401  (fails loudly if the CUDA library is missing)
    from maryml_b200 import nvfp4 as mb, _lib
    ctx = _lib.context(local_rank)

    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

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
    stream = torch.cuda.current_stream()
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

    # launches per step: 3 x (memset of the scale plane is a driver memset, not ours) quantize + gemm
    launches_per_step = 2 * len(SHAPES)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(args.steps):
        step(record=True)
    t1.record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = t0.elapsed_time(t1)
    if world > 1:
        tms = torch.tensor([ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    rc, flags = ctx.check_flags(None)
    if rc != 0:
        raise SystemExit(f"bench.py: device status words set: {flags}")

    # kernel-only roofline of the GEMM launches (CUDA events on the launching stream)
    gemm_ms = sum(e0.elapsed_time(e1) for (e0, e1, _) in gemm_events)
    gemm_fl = sum(f for (_, _, f) in gemm_events)
    achieved = gemm_fl / (gemm_ms * 1e-3) / 1e12
    peaks = measured_peaks()
    fp4_peak = 4.0 * peaks["bf16"]

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
    ev_out = [torch.cuda.Event() for _ in range(n_proj)]
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
                ev_out[i].record(s_out)

    def e2e_join():
        for st in (s_in, s_cmp, s_out):
            stream.wait_stream(st)

    e2e_steps = max(4, min(args.steps, 8))
    e2e_step()
    e2e_step()
    e2e_join()
    barrier()
    s0 = torch.cuda.Event(enable_timing=True)
    s1 = torch.cuda.Event(enable_timing=True)
    s0.record(stream)
    for st in (s_in, s_cmp, s_out):
        st.wait_stream(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e2e_join()
    s1.record(stream)
    barrier()
    e2e_ms = s0.elapsed_time(s1)
    if world > 1:
        tms = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        e2e_ms = float(tms.item())
    h2d = sum(M * q.k() * 2 for q in weights)
    d2h = sum(M * q.n() * 2 for q in weights)

    if rank == 0:
        cpu = cpu_lane(256, repeats=1)
        cpu_tflops = cpu["flops"] / cpu["seconds"][0] / 1e12
        value = world * step_flops() * args.steps / (ms * 1e-3) / 1e12
        line = {
            "metric": "nvfp4_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "e2m1 x e2m1 (ue4m3 block scales), f32 accumulate, bf16 out",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "M": M, "KN": SHAPES, "lane": "W4A4 input_scale=1",
                       "parallelism": f"replicas x{world}", "l2": "inputs+outputs per step exceed L2 (126 MB)"},
            "clocks": clocks,
            "e2e": {"value": world * step_flops() * e2e_steps / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "tensor", "kernel": "gemm_tc5_pair_kernel (cta_group::2, 256x256 tiles)", "achieved": achieved,
                         "peak": fp4_peak, "unit": "TFLOP/s", "frac": achieved / fp4_peak,
                         "peak_source": f"4 x {peaks['source']} bf16 burst ({peaks['bf16']} TFLOP/s): no FP4 figure "
                                        f"in MEASURED_PEAKS.json",
                         "frac_of_nominal_9pf": achieved / NOMINAL_FP4_TFLOPS,
                         # dram read+write per launch from one ncu capture, averaged over the three shapes
                         "traffic": 238.9e6, "traffic_unit": "bytes/launch (ncu, mean of 3 shapes)"},
            "cpu_baseline": {"value": cpu_tflops, "unit": "TFLOP/s", "cores": cpu["cores"], "kind": "port",
                             "sample": cpu["sample"]},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------
# Other workloads of the hot path
# --------------------------------------------------------------------------------------
def _time_steps(step, steps, warmup, stream, barrier, sampler):
    import torch
    for _ in range(max(warmup, 3)):
        step()
    barrier()
    if sampler:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(steps):
        step()
    t1.record(stream)
    barrier()
    clocks = sampler.stop() if sampler else None
    return t0.elapsed_time(t1), clocks


def run_other(args, rank, world, local_rank):
    import math
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from maryml_b200 import nvfp4 as mb, moe, attention as att, layer, _lib
    ctx = _lib.context(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream()
    g = torch.Generator(device=dev)
    g.manual_seed(99)
    peaks = measured_peaks()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    wl = args.workload
    extra = {}
    if wl == "moe":
        T, h, inter, E, K = 4096, 2048, 768, 128, 8
        x = torch.randn(T, h, device=dev, generator=g).to(torch.bfloat16)
        gate = (torch.randn(E, h, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        b13 = moe.ExpertBank.quantize((torch.randn(E, 2 * inter, h, device=dev, generator=g) * 0.02).to(torch.bfloat16))
        b2 = moe.ExpertBank.quantize((torch.randn(E, h, inter, device=dev, generator=g) * 0.02).to(torch.bfloat16))
        step = lambda: moe.moe_layer(x, gate, K, b13, b2)
        units, metric, unit = T, "moe_layer_tokens_per_s", "tokens/s"
        flop = T * K * 2 * (h * 2 * inter + inter * h) + 2 * T * h * E
        byts = (E * (2 * inter * h + h * inter)) * 0.5625 + T * h * 2 + T * h * 4 + E * h * 2
        h2d, d2h = T * h * 2, T * h * 4
        hx = x.cpu().pin_memory()
        hy = torch.empty(T, h, dtype=torch.float32).pin_memory()
        dx = torch.empty_like(x)

        def e2e():
            dx.copy_(hx, non_blocking=True)
            out, _ = moe.moe_layer(dx, gate, K, b13, b2)
            hy.copy_(out, non_blocking=True)
        roof = lambda ms: {"bound": "hbm", "kernel": "whole layer", "achieved": byts / (ms * 1e-3) / 1e9,
                           "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": byts / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                           "peak_source": peaks["source"], "traffic": None, "flop_per_step": flop,
                           "note": "min bytes = expert planes + x + out; the layer is weight-streaming bound at 4096 tokens"}
        cfg = {"workload": "moe_layer_T4096_h2048_E128_top8_inter768",
               "lane": "SwiGLU and the second projection's quantizer fused into the first grouped product"}
        launches = 14
    elif wl in ("attn_decode", "attn_prefill"):
        H, KVH, D = 32, 8, 128
        if wl == "attn_decode":
            B, nq, L = 32, 1, 32768
        else:
            B, nq, L = 4, 8192, 8192
        if args.batch:
            B = args.batch
        q = torch.randn(B, nq, H, D, device=dev, generator=g).to(torch.bfloat16)
        k = torch.randn(B, L, KVH, D, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(B, L, KVH, D, device=dev, generator=g).to(torch.bfloat16)
        ws = torch.empty(max(int(_lib.lib.mb_attention_workspace(B, nq, L, H, KVH, D)), 16), dtype=torch.uint8, device=dev)
        packed = wl == "attn_decode" and args.kv == "nvfp4"
        if packed:
            # NVFP4 cache rows (blocks of 16 along the features of a row, no global scale)
            kc, ks = att.quantize_kv_rows(k)
            vc, vs = att.quantize_kv_rows(v)
            del k, v
            attend = lambda qq: att.flash_attention_fp4kv(qq, kc, ks, vc, vs, KVH, q0=L - nq, workspace=ws)
        else:
            attend = lambda qq: att.flash_attention(qq, k, v, q0=L - nq, workspace=ws)
        step = lambda: attend(q)
        hq = q.cpu().pin_memory()
        ho = torch.empty_like(hq).pin_memory()
        dq = torch.empty_like(q)

        def e2e():
            dq.copy_(hq, non_blocking=True)
            ho.copy_(attend(dq), non_blocking=True)
        h2d = d2h = q.numel() * 2
        if wl == "attn_decode":
            byts = 2 * B * L * KVH * D * (0.5625 if packed else 2)
            units, metric, unit = byts / 1e9, "decode_attention_kv_gbytes_per_s", "GB/s"
            roof = lambda ms: {"bound": "hbm", "kernel": "attn_decode_kernel<nvfp4 rows>" if packed else "attn_decode_kernel",
                               "achieved": byts / (ms * 1e-3) / 1e9,
                               "peak": peaks["hbm_gbs"], "unit": "GB/s",
                               "frac": byts / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "peak_source": peaks["source"],
                               "frac_of_nominal_8tbs": byts / (ms * 1e-3) / 1e9 / 8000.0, "traffic": None}
            launches = 2
        else:
            flop = 4.0 * B * H * nq * L * D / 2
            units, metric, unit = flop / 1e12, "prefill_attention_tflops", "TFLOP/s"
            roof = lambda ms: {"bound": "tensor", "kernel": "attn_prefill_tc5_kernel (tcgen05, TMEM-resident O)", "achieved": flop / (ms * 1e-3) / 1e12,
                               "peak": peaks["bf16"], "unit": "TFLOP/s", "frac": flop / (ms * 1e-3) / 1e12 / peaks["bf16"],
                               "peak_source": peaks["source"], "traffic": None}
            launches = 1
        cfg = {"workload": f"{wl}_B{B}_nq{nq}_keys{L}_heads32_kv8_d128", "rope": "pre-applied (inputs drawn N(0,1))"}
        if packed:
            cfg["workload"] += "_nvfp4rows"
            cfg["kv"] = "NVFP4 cache rows: 0.5625 B per value counted; the bf16 cache of the same keys is 3.56x the bytes"
    else:
        cfgL = layer.LayerConfig()
        decode = wl == "tp_decode"
        batch, t, past = (64, 1, 4096) if decode else (1, 8192, 0)
        tp = layer.Tp(rank, world)

        def exchange(raw):
            obj = [raw]
            dist.broadcast_object_list(obj, src=0)
            return obj[0]
        group = layer.Group(tp, local_rank, exchange) if world > 1 else None
        D = cfgL.head_dim
        shapes = {"q": (cfgL.heads * D, cfgL.hidden), "k": (cfgL.kv_heads * D, cfgL.hidden),
                  "v": (cfgL.kv_heads * D, cfgL.hidden), "o": (cfgL.hidden, cfgL.heads * D),
                  "gate": (cfgL.inter, cfgL.hidden), "up": (cfgL.inter, cfgL.hidden), "down": (cfgL.hidden, cfgL.inter)}
        gw = torch.Generator(device=dev)
        gw.manual_seed(7)          # the same stored tensors on every rank, cut after quantisation
        full = {}
        for name, (n, kk) in shapes.items():
            qz = mb.Nvfp4.quantize((torch.randn(n, kk, device=dev, generator=gw) * 0.02).to(torch.bfloat16))
            full[name] = (qz.codes, qz.scales, qz.scale2)
        gain = torch.ones(cfgL.hidden, dtype=torch.bfloat16, device=dev)
        fx = None
        if args.fused and world > 1:
            def exchange_all(raw):
                got = [None] * world
                dist.all_gather_object(got, raw)
                return got
            # peer stores of 32-byte segments suit decode-sized messages; an 8192-token prompt's 134 MB
            # partial moves faster through NCCL's bulk all-reduce, so the exchange is sized for <= 1024 rows
            fx = layer.FusedExchange(tp, local_rank, min(batch * t, 1024), cfgL.hidden, exchange_all)
        L_ = layer.DecoderLayer(cfgL, full, gain, gain, tp=tp, group=group, device=dev, fused=fx)
        del full
        cap = past + t
        x = torch.randn(batch * t, cfgL.hidden, device=dev, generator=gw).to(torch.bfloat16)
        kc = torch.randn(batch, cap, L_.local_kv_heads, D, device=dev, generator=g).to(torch.bfloat16)
        vc = torch.randn(batch, cap, L_.local_kv_heads, D, device=dev, generator=g).to(torch.bfloat16)
        step = lambda: L_.forward(x, batch, past, kc, vc)
        hx = x.cpu().pin_memory()
        hy = torch.empty_like(hx).pin_memory()
        dx = torch.empty_like(x)

        def e2e():
            dx.copy_(hx, non_blocking=True)
            hy.copy_(L_.forward(dx, batch, past, kc, vc), non_blocking=True)
        h2d = d2h = x.numel() * 2
        units, metric, unit = batch * t, f"tp_layer_{'decode' if decode else 'prefill'}_tokens_per_s", "tokens/s"
        params = sum(n * kk for (n, kk) in shapes.values())
        if decode:
            byts = (params * 0.5625 + 2 * batch * cap * cfgL.kv_heads * D * 2) / world
            roof = lambda ms: {"bound": "hbm", "kernel": "whole layer per rank", "achieved": byts / (ms * 1e-3) / 1e9,
                               "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": byts / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                               "peak_source": peaks["source"], "traffic": None,
                               "note": "weights + KV per rank; 2 all-reduces of [64,4096] f32 are latency terms"}
        else:
            flop = (2.0 * t * params + 4.0 * cfgL.heads * t * t * D / 2) / world
            roof = lambda ms: {"bound": "tensor", "kernel": "whole layer per rank", "achieved": flop / (ms * 1e-3) / 1e12,
                               "peak": 4 * peaks["bf16"], "unit": "TFLOP/s", "frac": flop / (ms * 1e-3) / 1e12 / (4 * peaks["bf16"]),
                               "peak_source": "4 x " + peaks["source"] + " bf16 burst", "traffic": None,
                               "note": "projections at the FP4 rate dominate; attention runs at the bf16 rate"}
        cfg = {"workload": f"{wl}_hidden4096_heads32_kv8_ffn14336_batch{batch}_t{t}_past{past}", "parallelism": f"tp{world}",
               "reduce": "fused: GEMM epilogue scatters to peers, one reduce+residual+gather kernel" if (fx and batch * t <= 1024) else
                         ("nccl all-reduce f32 + add" if world > 1 else "none (world 1)")}
        # kernels of ours per step: norm+quantize, q|k|v product, rotation+append, attention, quantize, o product,
        # add+norm+quantize, gate/up+SwiGLU+quantize product, down product, add = 10; the decode kernel adds its
        # combine pass; a product with <= 128 rows and few tiles adds a split-K sum; the fused exchange swaps
        # (sum, add) for its reduce+residual kernel and runs the second norm+quantize on its own
        rows = batch * t
        from maryml_b200 import _lib as _l
        splitk = lambda n, k: 1 if _l.lib.mb_nvfp4_gemm_splitk_workspace(rows, n, k) else 0
        hd = cfgL.hidden
        n_qkv = (L_.local_heads + 2 * L_.local_kv_heads) * D
        launches = 10 + (1 if decode else 0) + splitk(n_qkv, hd)
        if fx and rows <= 1024:
            launches += 1
        else:
            launches += splitk(hd, L_.local_heads * D) + splitk(hd, L_.local_inter)

    if args.graph:
        # Serving mode: the step is captured once into a CUDA graph (kernels, memsets and the NCCL
        # all-reduces alike) and replayed, which takes the host's ~30 launches per layer off the clock.
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            for _ in range(3):
                step()
        stream.wait_stream(side)
        barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        captured = step
        step = graph.replay
        cfg["launch"] = "cuda graph replay"
    ms, clocks = _time_steps(step, args.steps, args.warmup, stream, barrier, sampler)
    e2e()
    barrier()
    n_e2e = max(2, min(args.steps, 5))
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record(stream)
    for _ in range(n_e2e):
        e2e()
    s1.record(stream)
    barrier()
    e2e_ms = s0.elapsed_time(s1)
    if world > 1:
        tms = torch.tensor([ms, e2e_ms], device=dev)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(tms[0].item()), float(tms[1].item())
    rc, flags = ctx.check_flags(None)
    if rc != 0:
        raise SystemExit(f"bench.py: device status words set: {flags}")
    tp_like = wl.startswith("tp_")
    mult = 1 if tp_like else world          # the TP layer is one job over all ranks; the others are replicas
    if rank == 0:
        per_step = ms / args.steps
        line = {"metric": metric, "value": mult * units / (per_step * 1e-3), "unit": unit, "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": per_step, "higher_is_better": True,
                "scaling": "strong" if tp_like else "weak", "vs_baseline": None, "dtype": "nvfp4/bf16, f32 accumulate",
                "data": "synthetic", "config": cfg, "clocks": clocks,
                "e2e": {"value": mult * units / (e2e_ms / n_e2e * 1e-3), "unit": unit, "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": d2h},
                "gpu_launches": launches * args.steps, "roofline": roof(per_step),
                "cpu_baseline": None}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="gemm",
                    choices=["gemm", "moe", "attn_decode", "attn_prefill", "tp_decode", "tp_prefill"])
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
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.workload == "gemm":
        run_ours(args, rank, world, local_rank)
    else:
        run_other(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
