"""The tensor-parallel decoder layer: the shard arithmetic of worlds 2, 4 and 8 at the benchmark's layer shapes
run rank after rank on ONE GPU (partials summed in rank order) against the unsharded layer and the CPU oracle,
and the layer on 2, 4 or 8 GPUs (one process each, NCCL or the fused peer-memory exchange) against the same layer
on 1 GPU; the multi-GPU cases are skipped when fewer devices are visible. Same stored planes everywhere, cut
after quantisation."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _fixture(cfg):
    sys.path.insert(0, HERE)
    from oracle_lib import oracle, f32_to_bf16_bits
    orc = oracle()
    D = cfg.head_dim
    shapes = {"q": (cfg.heads * D, cfg.hidden), "k": (cfg.kv_heads * D, cfg.hidden), "v": (cfg.kv_heads * D, cfg.hidden),
              "o": (cfg.hidden, cfg.heads * D), "gate": (cfg.inter, cfg.hidden), "up": (cfg.inter, cfg.hidden),
              "down": (cfg.hidden, cfg.inter)}
    full = {}
    for i, (name, (n, k)) in enumerate(shapes.items()):
        bits = f32_to_bf16_bits(orc.normal_f32(200 + i, n * k, 0.02))
        c, s, s2 = orc.quantize_weight_bf16(bits, n, k)
        full[name] = (torch.from_numpy(c).view(n, k // 2), torch.from_numpy(s).view(n, k // 16), float(s2))
    g1 = torch.from_numpy(f32_to_bf16_bits(1.0 + 0.05 * orc.normal_f32(220, cfg.hidden, 1.0)).view(np.int16)).view(torch.bfloat16)
    g2 = torch.from_numpy(f32_to_bf16_bits(1.0 + 0.05 * orc.normal_f32(221, cfg.hidden, 1.0)).view(np.int16)).view(torch.bfloat16)
    return orc, full, g1, g2


def _inputs(orc, cfg, batch, t, cap):
    from oracle_lib import f32_to_bf16_bits
    to_t = lambda b: torch.from_numpy(b.view(np.int16)).view(torch.bfloat16)
    x = to_t(f32_to_bf16_bits(orc.normal_f32(7, batch * t * cfg.hidden, 1.0))).view(batch * t, cfg.hidden)
    kc = to_t(f32_to_bf16_bits(orc.normal_f32(8, batch * cap * cfg.kv_heads * 128, 1.0))).view(batch, cap, cfg.kv_heads, 128)
    vc = to_t(f32_to_bf16_bits(orc.normal_f32(9, batch * cap * cfg.kv_heads * 128, 1.0))).view(batch, cap, cfg.kv_heads, 128)
    return x, kc, vc


def _worker(rank, world, port, out_path, fused=False):
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    sys.path.insert(0, os.path.dirname(HERE))
    sys.path.insert(0, HERE)
    torch.cuda.set_device(rank)
    from torch.distributed import TCPStore
    store = TCPStore("127.0.0.1", port, world, rank == 0)
    from maryml_b200 import layer

    def exchange(raw):
        if rank == 0:
            store.set("nccl_id", raw)
        return store.get("nccl_id")

    cfg = layer.LayerConfig(hidden=1024, heads=8, kv_heads=8, head_dim=128, inter=2048)   # divides by 2, 4 and 8
    orc, full, g1, g2 = _fixture(cfg)
    tp = layer.Tp(rank, world)
    group = layer.Group(tp, rank, exchange)
    fx = None
    if fused:
        def exchange_all(raw):
            store.set(f"ipc{rank}", raw)
            return [store.get(f"ipc{r}") for r in range(world)]
        fx = layer.FusedExchange(tp, rank, 64, cfg.hidden, exchange_all)
    L = layer.DecoderLayer(cfg, full, g1, g2, tp=tp, group=group, device=torch.device("cuda", rank), fused=fx)
    batch, t, past = 3, 1, 21
    x, kc, vc = _inputs(orc, cfg, batch, t, past + t)
    kv = tp.kv_heads(cfg.kv_heads)
    kd, vd = kc[:, :, kv.start:kv.stop].contiguous().cuda(), vc[:, :, kv.start:kv.stop].contiguous().cuda()
    y = L.forward(x.cuda(), batch, past, kd, vd)
    if fused:
        # a second and third step through the same exchange memory (both step parities, reused slots)
        for _ in range(2):
            y2 = L.forward(x.cuda(), batch, past, kd, vd)
        torch.cuda.synchronize()
        assert torch.equal(y2, y)
        from maryml_b200 import _lib
        rc, flags = _lib.context(rank).check_flags(None)
        assert rc == 0, flags
    y = y.clone()
    torch.cuda.synchronize()
    if not fused:
        # a prompt as a pipeline of chunks on two streams (all-reduces of the same communicator issued
        # from both) against one pass over the whole prompt, on every rank
        pt, ppast = 512, 0
        px, pk, pv = _inputs(orc, cfg, 1, pt, ppast + pt)
        pk, pv = pk[:, :, kv.start:kv.stop].contiguous().cuda(), pv[:, :, kv.start:kv.stop].contiguous().cuda()
        pk2, pv2 = pk.clone(), pv.clone()
        whole = L._forward_fused(px.cuda(), 1, ppast, pk, pv)
        parts = L.forward_chunked(px.cuda(), ppast, pk2, pv2, chunk=256)
        torch.cuda.synchronize()
        a, b = whole.float(), parts.float()
        rms = a.pow(2).mean().sqrt()
        assert (a - b).abs().max() <= 2e-2 * rms, float((a - b).abs().max() / rms)
        assert torch.equal(pk.view(torch.int16), pk2.view(torch.int16))
        _bulk_exchange_checks(rank, world, store, layer, cfg, full, g1, g2, tp, group, orc, kv, whole if world == 2 else None)
    if rank == 0:
        np.save(out_path, y.float().cpu().numpy())
    store.set(f"done{rank}", b"1")
    for r in range(world):
        store.get(f"done{r}")
    if fx is not None:
        fx.close()
    group.close()


def _bulk_exchange_checks(rank, world, store, layer, cfg, full, g1, g2, tp, group, orc, kv, whole_512):
    """The prompt path's exchanges as peer-memory kernels (mb_tp_bulk_*): the reduce-scatter against the sum of every
    rank's partial in rank order (bit for bit: each rank rebuilds all partials from their seeds), the all-gather
    against the slices every rank is known to have written, three rounds through both buffers of each kind; then the
    layer through them against the same layer through NCCL."""
    dev = torch.device("cuda", rank)

    def exchange_all(raw):
        key = f"bulk{len(raw)}_{exchange_all.n}"
        exchange_all.n += 1
        store.set(f"{key}_{rank}", raw)
        return [store.get(f"{key}_{r}") for r in range(world)]
    exchange_all.n = 0
    rows_max = 256 * world
    bulk = layer.BulkExchange(tp, rank, rows_max, cfg.hidden, exchange_all)
    for rnd in range(3):
        rows = rows_max if rnd != 1 else 128 * world
        parts = [torch.randn(rows, cfg.hidden, generator=torch.Generator().manual_seed(1000 * rnd + r)) for r in range(world)]
        got = bulk.reduce_scatter_f32(parts[rank].to(dev))
        local = rows // world
        want = parts[0][rank * local:(rank + 1) * local].clone()
        for r in range(1, world):
            want += parts[r][rank * local:(rank + 1) * local]
        assert torch.equal(got.cpu(), want), rnd
        codes, sf = bulk.planes(rows)
        sf_part = sf.numel() // world
        codes[rank * local:(rank + 1) * local] = (rank + 1 + rnd) & 0xFF
        sf[rank * sf_part:(rank + 1) * sf_part] = (0x40 + rank + rnd) & 0xFF
        bulk.all_gather_planes(rows)
        yb = bulk.rows_buffer(rows)
        yb[rank * local:(rank + 1) * local] = float(rank + 2 + rnd)
        bulk.all_gather_rows(rows)
        torch.cuda.synchronize()
        for r in range(world):
            assert bool((codes[r * local:(r + 1) * local] == ((r + 1 + rnd) & 0xFF)).all()), (rnd, r)
            assert bool((sf[r * sf_part:(r + 1) * sf_part] == ((0x40 + r + rnd) & 0xFF)).all()), (rnd, r)
            assert bool((yb[r * local:(r + 1) * local] == float(r + 2 + rnd)).all()), (rnd, r)
    # the layer's prompt path through these exchanges and through NCCL
    Lb = layer.DecoderLayer(cfg, full, g1, g2, tp=tp, group=group, device=dev, bulk=bulk)
    Ln = layer.DecoderLayer(cfg, full, g1, g2, tp=tp, group=group, device=dev)
    pt = rows_max
    assert Lb._rows_shard(pt)
    px, pk, pv = _inputs(orc, cfg, 1, pt, pt)
    pk, pv = pk[:, :, kv.start:kv.stop].contiguous().cuda(), pv[:, :, kv.start:kv.stop].contiguous().cuda()
    a = Lb._forward_fused(px.cuda(), 1, 0, pk.clone(), pv.clone()).clone()
    b = Ln._forward_fused(px.cuda(), 1, 0, pk.clone(), pv.clone())
    torch.cuda.synchronize()
    if world == 2:
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))       # two partials add in one order only
    else:
        rms = b.float().pow(2).mean().sqrt()
        assert (a.float() - b.float()).abs().max() <= 2e-2 * rms
    from maryml_b200 import _lib
    rc, flags = _lib.context(rank).check_flags(None)
    assert rc == 0, flags
    bulk.close()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("fused", [False, True])
def test_multi_gpu_layer_matches_one_gpu(tmp_path, fused, world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = str(tmp_path / "tp2.npy")
    mp.spawn(_worker, args=(world, port, out, fused), nprocs=world, join=True)
    from maryml_b200 import layer
    cfg = layer.LayerConfig(hidden=1024, heads=8, kv_heads=8, head_dim=128, inter=2048)
    orc, full, g1, g2 = _fixture(cfg)
    L = layer.DecoderLayer(cfg, full, g1, g2)
    batch, t, past = 3, 1, 21
    x, kc, vc = _inputs(orc, cfg, batch, t, past + t)
    y1 = L.forward(x.cuda(), batch, past, kc.cuda(), vc.cuda()).float().cpu().numpy()
    y2 = np.load(out)
    rms = np.sqrt(np.mean(y1.astype(np.float64) ** 2))
    # only the K sum of the row-parallel projections is re-associated across ranks
    assert np.abs(y1 - y2).max() <= 5e-2 * rms and np.abs(y1 - y2).mean() <= 5e-3 * rms


# ------------------------------------------------------------------- the shard arithmetic on one GPU
_CACHE = {}


def _config4():
    """Config 4 of the benchmark: hidden 4096, 32 heads / 8 KV heads, FFN 14336; batch 64 decode over a
    4096-token cache. Weights, inputs and the unsharded layer's stages, made once."""
    if "c4" in _CACHE:
        return _CACHE["c4"]
    sys.path.insert(0, HERE)
    from maryml_b200 import layer
    cfg = layer.LayerConfig()
    orc, full, g1, g2 = _fixture(cfg)
    batch, t, past = 64, 1, 4096
    cap = past + t
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(batch * t, cfg.hidden, device="cuda", generator=g).to(torch.bfloat16)
    kc = torch.randn(batch, cap, cfg.kv_heads, 128, device="cuda", generator=g).to(torch.bfloat16)
    vc = torch.randn(batch, cap, cfg.kv_heads, 128, device="cuda", generator=g).to(torch.bfloat16)
    L1 = layer.DecoderLayer(cfg, full, g1, g2)
    k1, v1 = kc.clone(), vc.clone()
    st = {}
    st["a"] = L1._attention(x, batch, past, k1, v1)                       # [64, 4096] bf16, all heads
    st["o"] = L1._linear(st["a"], L1.wo, out_dtype=torch.float32)          # the whole o projection
    st["residual"], st["down"] = L1.half_mlp(x, st["o"])
    st["y"] = layer.DecoderLayer.finish(st["residual"], st["down"])
    _CACHE["c4"] = (cfg, orc, full, g1, g2, x, kc, vc, L1, k1, v1, st, batch, t, past)
    return _CACHE["c4"]


def _bounds(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    rms = float(np.sqrt(np.mean(want ** 2)))
    err = np.abs(got - want)
    cos = float(np.dot(got.ravel(), want.ravel()) / (np.linalg.norm(got) * np.linalg.norm(want) + 1e-30))
    return err.max() / rms, err.mean() / rms, cos


def test_layer_products_at_benchmark_shapes_against_the_oracle(figures):
    """Every product of the layer at its real shape (64 rows; q|k|v stacked 6144 x 4096, o 4096 x 4096, gate/up
    stacked 28672 x 4096 with the SwiGLU + quantizer epilogue, down 4096 x 14336 through split-K) against f64 sums
    of the SAME quantized operands: each stage is fed the GPU's own previous bytes, as the reference's gates do
    (src/bin/k3_router_gate.rs:60-95), so a disagreement is that stage's and nothing is amplified downstream."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle_lib import bf16_bits_to_f32, f32_to_bf16_bits
    from maryml_b200 import nvfp4 as nv, _lib
    cfg, orc, full, g1, g2, x, kc, vc, L1, k1, v1, st, batch, t, past = _config4()
    rows = batch * t
    bits = lambda a: a.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)

    def planes(codes, sf, k):
        return codes.cpu().numpy().ravel(), nv.untile_scales(sf, rows, k).cpu().numpy().ravel()

    def oracle_product(a_c, a_s, name):
        c, s, s2 = full[name]
        n, k = c.shape[0], c.shape[1] * 2
        return orc.linear_w4a4(a_c, a_s, c.numpy().ravel(), s.numpy().ravel(), np.float32(s2), rows, n, k)

    # input norm + quantizer: the bytes of the oracle's norm + quantizer on the same rows (the f32 sum of squares is
    # ordered differently on the two sides, so a few values sit on the other side of a rounding)
    _, (xc, xsf, _) = L1._norm_quantize(x, None, L1.input_gain)
    y_or = orc.rmsnorm_breeze(bits(x).ravel(), bits(g1).ravel(), rows, cfg.hidden, cfg.eps)
    c_or, _ = orc.quantize_act_scaled(bf16_bits_to_f32(y_or), rows, cfg.hidden, 1.0)
    a_c, a_s = planes(xc, xsf, cfg.hidden)
    assert (a_c == c_or).mean() >= 0.999
    # q | k | v as one product, f32 out, against the three separate oracle products of the GPU's activation planes
    qkv = nv.gemm_w4a4_stacked(xc, xsf, L1.wqkv, rows, out_dtype=torch.float32).cpu().numpy()
    ref = np.concatenate([oracle_product(a_c, a_s, n_) for n_ in ("q", "k", "v")], 1)
    e_qkv = np.abs(qkv - ref).max() / np.abs(ref).max()
    # o projection of the GPU's own attention output
    oc, osf, _ = nv.quantize_act(st["a"], _lib.QUANT_SCALED, 1.0, tiled=True)
    o_c, o_s = planes(oc, osf, cfg.hidden)
    assert np.array_equal(o_c, orc.quantize_act_scaled(bf16_bits_to_f32(bits(st["a"])), rows, cfg.hidden, 1.0)[0])
    e_o = np.abs(st["o"].cpu().numpy() - oracle_product(o_c, o_s, "o")).max() / np.abs(st["o"].cpu().numpy()).max()
    # gate/up + SwiGLU (+ quantizer) epilogue on the GPU's own post-attention planes
    resid, (nc, nsf, _) = L1._norm_quantize(x, st["o"], L1.post_gain)
    n_c, n_s = planes(nc, nsf, cfg.hidden)
    act = nv.gemm_w4a4_stacked(nc, nsf, L1.wgu, rows, epilogue=_lib.EPI_SWIGLU_ROUNDED)
    gate = f32_to_bf16_bits(oracle_product(n_c, n_s, "gate"))
    up = f32_to_bf16_bits(oracle_product(n_c, n_s, "up"))
    act_ref = orc.swiglu_bf16(gate, up).reshape(rows, cfg.inter)
    act_bits = bits(act).reshape(rows, cfg.inter)
    moved = float((act_bits != act_ref).mean())          # f32 sums rounded to the other bf16 neighbour, then the expf ulp
    step = np.abs(bf16_bits_to_f32(act_bits) - bf16_bits_to_f32(act_ref))
    assert moved <= 2e-2 and (step <= 2.0 ** -6 * np.abs(bf16_bits_to_f32(act_ref)) + 1e-6).all(), moved
    qc, qsf = nv.gemm_w4a4_stacked(nc, nsf, L1.wgu, rows, epilogue=_lib.EPI_SWIGLU_ROUNDED | _lib.EPI_QUANT_SCALED)
    d_c, d_s = planes(qc, qsf, cfg.inter)
    c_ref, s_ref = orc.quantize_act_scaled(bf16_bits_to_f32(act_bits), rows, cfg.inter, 1.0)
    assert np.array_equal(d_c, c_ref) and np.array_equal(d_s, s_ref)      # the epilogue quantizes its own bf16 result
    # down projection (K = 14336: split-K planes summed in slice order) of the GPU's own activation planes
    e_d = np.abs(st["down"].cpu().numpy() - oracle_product(d_c, d_s, "down")).max() / np.abs(st["down"].cpu().numpy()).max()
    figures("layer_products_config4", qkv_rel=e_qkv, o_rel=e_o, swiglu_moved=moved, down_rel=e_d)
    # the reference's same-operand gate (src/bin/inkling_fp4_expert_gate.rs:16-28)
    assert e_qkv <= 1e-4 and e_o <= 1e-4 and e_d <= 1e-4, (e_qkv, e_o, e_d)
    # residual add after the exchange: bf16(x + bf16(o))
    want = orc.add_bf16(bits(x).ravel(), f32_to_bf16_bits(st["o"].cpu().numpy().ravel()))
    assert np.array_equal(bits(resid).ravel(), want)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_shard_arithmetic_of_worlds_2_4_8_on_one_gpu(world, figures):
    """Tp::shard / cut_rows / cut_cols at the benchmark's layer shapes (src/models/inkling/tp.rs:540-555,
    tpshard.rs:102-180; placement session.rs:2713-2717, 2843-2846): every rank's half-layers run on this one
    device and the f32 partials of the two row-parallel projections are summed in rank order, which is what the
    SUM all-reduce does.

    Checked exchange by exchange, each rank fed the same bytes the unsharded layer saw at that point: the cut
    re-associates the K sums of o and down and changes nothing else, so the summed partials agree with the
    unsharded products to f32 rounding and the replicated tensors agree to the bit. The layer run end to end
    (each stage on its own previous output) is then compared as well, and only recorded: W4A4 re-quantizes
    bf16 intermediates three times per layer, so the 2^-9 noise that a different key-split count puts on the
    attention output flips E2M1 codes downstream, and two correct evaluations of this layer (the CPU oracle
    included) sit a few percent of the output's rms apart."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    sys.path.insert(0, HERE)
    from test_gpu_nvfp4 import attn_check
    from maryml_b200 import layer
    cfg, orc, full, g1, g2, x, kc, vc, L1, k1, v1, st, batch, t, past = _config4()
    D = cfg.head_dim
    ranks = [layer.DecoderLayer(cfg, full, g1, g2, tp=layer.Tp(r, world)) for r in range(world)]
    # the cuts tile the axes: heads, KV heads and the intermediate width are covered once, in rank order
    assert sum(L.local_heads for L in ranks) == cfg.heads and sum(L.local_kv_heads for L in ranks) == cfg.kv_heads
    assert sum(L.local_inter for L in ranks) == cfg.inter
    o_sum = o_chain = None
    a_worst = 0.0
    for L in ranks:
        kv, qh = L.tp.kv_heads(cfg.kv_heads), L.tp.q_heads(cfg.heads)
        kr, vr = kc[:, :, kv.start:kv.stop].contiguous(), vc[:, :, kv.start:kv.stop].contiguous()
        a_r = L._attention(x, batch, past, kr, vr)
        # this rank's heads against the same heads of the unsharded layer: the attention bound (the key splits differ)
        a_ref = st["a"][:, qh.start * D:qh.stop * D]
        rel, cos = attn_check(a_r.float().cpu().numpy(), a_ref.float().cpu().numpy())
        a_worst = max(a_worst, rel)
        assert rel <= 1e-2 and cos >= 0.9999, (rel, cos)
        # every rank appended its own KV heads' new rows: together they are the unsharded layer's cache
        assert torch.equal(kr.view(torch.int16), k1[:, :, kv.start:kv.stop].contiguous().view(torch.int16))
        assert torch.equal(vr.view(torch.int16), v1[:, :, kv.start:kv.stop].contiguous().view(torch.int16))
        # first exchange, fed the unsharded layer's attention bytes for this rank's heads
        part = L._linear(a_ref.contiguous(), L.wo, out_dtype=torch.float32)
        o_sum = part if o_sum is None else o_sum + part
        chain = L._linear(a_r, L.wo, out_dtype=torch.float32)
        o_chain = chain if o_chain is None else o_chain + chain
    e_o = float((o_sum - st["o"]).abs().max() / st["o"].abs().max())
    # second exchange, fed the unsharded layer's summed o partial
    down_sum = None
    for L in ranks:
        res, part = L.half_mlp(x, st["o"])
        assert torch.equal(res.view(torch.int16), st["residual"].view(torch.int16))     # replicated, not sharded
        down_sum = part if down_sum is None else down_sum + part
    e_d = float((down_sum - st["down"]).abs().max() / st["down"].abs().max())
    y = layer.DecoderLayer.finish(st["residual"], down_sum)
    diff = (y.view(torch.int16) != st["y"].view(torch.int16)).float().mean().item()
    # where the two differ, by one bf16 step of the operands of the last add (residual + bf16(down sum)); the result
    # itself can be much smaller than its operands, so its own bit patterns may sit several steps apart
    step = 2.0 ** -7 * torch.maximum(st["residual"].float().abs(), st["down"].abs())
    steps = float(((y.float() - st["y"].float()).abs() / step.clamp_min(1e-30)).max())
    assert e_o <= 2e-5 and e_d <= 2e-5, (e_o, e_d)            # f32 re-association of 4096- and 14336-term sums
    assert diff <= 1e-3 and steps <= 3.0, (diff, steps)        # one step of bf16(down) plus the rounding of the sum
    # the layer as it runs, every stage on its own previous output
    down_chain = None
    for L in ranks:
        res_c, part = L.half_mlp(x, o_chain)
        down_chain = part if down_chain is None else down_chain + part
    y_chain = layer.DecoderLayer.finish(res_c, down_chain).float().cpu().numpy()
    mx, mean, cos = _bounds(y_chain, st["y"].float().cpu().numpy())
    figures("tp_layer_config4_shards_on_one_gpu", world=world, attention_max_rel=a_worst, o_sum_rel=e_o, down_sum_rel=e_d,
            output_bf16_moved=diff, chained_max_over_rms=mx, chained_mean_over_rms=mean, chained_cos=cos)
    assert cos >= 0.99 and mean <= 0.1, (mx, mean, cos)


def test_unsharded_layer_end_to_end_against_the_oracle_is_recorded(figures):
    """The whole layer against the all-CPU chain at the benchmark's shapes. Recorded with a loose bound: see the
    note on re-quantized intermediates above; the per-product test carries the parity claim."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    sys.path.insert(0, HERE)
    from oracle_lib import bf16_bits_to_f32
    from test_gpu_attention_layer import _oracle_layer
    cfg, orc, full, g1, g2, x, kc, vc, L1, k1, v1, st, batch, t, past = _config4()
    bits = lambda a: a.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    cap = past + t
    ref = _oracle_layer(orc, cfg, full, bits(g1), bits(g2), bits(x).ravel(), batch, t, past,
                        bits(kc).reshape(batch, cap, -1).copy(), bits(vc).reshape(batch, cap, -1).copy())
    mx, mean, cos = _bounds(st["y"].float().cpu().numpy(), bf16_bits_to_f32(ref).reshape(batch * t, cfg.hidden))
    figures("tp_layer_config4_world1_vs_oracle", max_over_rms=mx, mean_over_rms=mean, cosine=cos)
    assert cos >= 0.99 and mean <= 0.1, (mx, mean, cos)
