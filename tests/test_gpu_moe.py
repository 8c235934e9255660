"""GPU parity tests of the MoE lane: router indices and permutation maps bit-exact against the
oracle, expert outputs within tolerance. All calls go through the C ABI."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle_lib import bf16_bits_to_f32, f32_to_bf16_bits  # noqa: E402
from test_gpu_nvfp4 import dev_bf16, host_bits, rel_check  # noqa: E402


@pytest.fixture(scope="module")
def moe():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from maryml_b200 import moe as m
    return m


@pytest.mark.parametrize("tokens,n_experts,k", [(1, 32, 1), (37, 128, 8), (4096, 128, 8), (300, 256, 6), (70, 512, 8),
                                               (33, 96, 32)])
def test_router_indices_bit_exact(moe, orc, tokens, n_experts, k):
    logits = (orc.normal_f32(77 + tokens, tokens * n_experts, 2.0)).reshape(tokens, n_experts)
    if tokens > 2:
        logits[1, :] = 0.25          # an all-tie row: the lowest indices win
        logits[2, 5] = logits[2, 9]  # one exact tie
    idx, w = moe.router_topk_softmax(torch.from_numpy(logits).cuda(), k)
    scores = orc.router_scores_softmax(logits)
    idx_ref, w_ref = orc.router_select(scores, k)
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), idx_ref)
    # weights: f32 arithmetic of identical scores; the reference's own stage gate allows 1e-6
    # (src/bin/k3_router_gate.rs:60-95)
    assert np.abs(w.cpu().numpy() - w_ref).max() <= 1e-6
    # without the renormalising divide the weights are the gathered scores themselves: the oracle's bits
    idx_u, w_u = moe.router_topk_softmax(torch.from_numpy(logits).cuda(), k, renormalize=False)
    _, w_u_ref = orc.router_select(scores, k, renormalize=False)
    assert np.array_equal(idx_u.cpu().numpy().astype(np.uint32), idx_ref)
    assert np.array_equal(w_u.cpu().numpy().view(np.uint32), w_u_ref.view(np.uint32))


@pytest.mark.parametrize("activation", ["sigmoid", "softmax"])
@pytest.mark.parametrize("tokens,n_experts,k,scaling", [(1, 32, 2, 1.0), (37, 128, 8, 2.5), (1000, 384, 8, 2.827),
                                                        (300, 256, 6, 1.0)])
def test_router_activation_and_selection_bias(moe, orc, activation, tokens, n_experts, k, scaling):
    logits = (orc.normal_f32(177 + tokens, tokens * n_experts, 2.0)).reshape(tokens, n_experts)
    bias = (orc.normal_f32(9 + n_experts, n_experts, 0.2)).astype(np.float32)
    if tokens > 2:
        logits[1, :] = 0.25
        logits[2, 5] = logits[2, 9]
        bias[5] = bias[9]
    scores = orc.router_scores_sigmoid(logits) if activation == "sigmoid" else orc.router_scores_softmax(logits)
    for b in (None, bias):
        idx, w = moe.router_topk(torch.from_numpy(logits).cuda(), k, activation,
                                 None if b is None else torch.from_numpy(b).cuda(), True, scaling)
        idx_ref, w_ref = orc.router_select(scores, k, bias=b, scaling=scaling)
        assert np.array_equal(idx.cpu().numpy().astype(np.uint32), idx_ref)
        assert np.abs(w.cpu().numpy() - w_ref).max() <= 1e-6 * max(1.0, scaling)
    # without renormalisation the weights are the unbiased scores themselves: bit-exact
    idx, w = moe.router_topk(torch.from_numpy(logits).cuda(), k, activation, torch.from_numpy(bias).cuda(), False, 1.0)
    idx_ref, w_ref = orc.router_select(scores, k, bias=bias, renormalize=False)
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), idx_ref)
    assert np.array_equal(w.cpu().numpy().view(np.uint32), w_ref.view(np.uint32))
    assert np.array_equal(w.cpu().numpy(), np.take_along_axis(scores, idx_ref.astype(np.int64), 1))


def test_router_known_answer_bias_moves_selection(moe):
    # src/models/k3/router.rs:518-547 widened to 32 experts (the kernel's minimum): experts 4.. sit far below
    logits = np.full((1, 32), -30.0, np.float32)
    logits[0, :4] = [2.0, 1.0, 0.5, 0.0]
    bias = np.zeros(32, np.float32)
    idx, w = moe.router_topk(torch.from_numpy(logits).cuda(), 2, "sigmoid")
    assert idx.cpu().numpy().tolist() == [[0, 1]] and abs(float(w.sum()) - 1.0) < 1e-6
    bias[3] = 1.0
    idx, w = moe.router_topk(torch.from_numpy(logits).cuda(), 2, "sigmoid", torch.from_numpy(bias).cuda(), False)
    assert idx.cpu().numpy().tolist() == [[3, 0]]
    assert w.cpu().numpy().tolist() == [[0.5, float(np.float32(1.0 / (1.0 + np.exp(-2.0))))]]


@pytest.mark.parametrize("tokens,k,rows", [(300, 2048, 1000), (64, 192, 128), (5, 64, 37)])
def test_gather_of_quantized_planes_equals_quantizer_with_gather(moe, tokens, k, rows):
    from maryml_b200 import _lib, nvfp4 as nv
    g = torch.Generator(device="cuda").manual_seed(tokens + k)
    x = (torch.randn(tokens, k, device="cuda", generator=g) * 3).to(torch.bfloat16)
    rng = np.random.default_rng(rows)
    gather = rng.integers(-1, tokens, rows).astype(np.int32)
    gather[0] = -1
    gd = torch.from_numpy(gather).cuda()
    want_c, want_s, _ = nv.quantize_act(x, _lib.QUANT_RECIP, tiled=True, gather=gd)
    t_c, t_s, _ = nv.quantize_act(x, _lib.QUANT_RECIP, tiled=True)
    got_c, got_s = nv.gather_rows(t_c, t_s, tokens, k, gd)
    assert torch.equal(got_c, want_c)
    # pad rows of the last 128-row tile are unspecified in neither plane: both are zero-filled first
    assert torch.equal(nv.untile_scales(got_s, rows, k), nv.untile_scales(want_s, rows, k))
    ctx = _lib.context(0)
    assert ctx.check_flags(None)[0] == 0
    gd[1] = tokens                                   # a source row that does not exist
    c2, _ = nv.gather_rows(t_c, t_s, tokens, k, gd)
    rc, flags = ctx.check_flags(None)
    assert rc == _lib.ERR_DEVICE_FLAG and flags[2] == 2 and not c2[1].any()
    assert ctx.check_flags(None)[0] == 0


@pytest.mark.parametrize("tokens,n_routed,n_shared,k", [(1, 32, 0, 1), (37, 256, 2, 6), (512, 256, 1, 6), (300, 384, 4, 8),
                                                         (64, 64, 32, 32)])
def test_sink_router_against_the_cpu_rule(moe, orc, tokens, n_routed, n_shared, k):
    rows = n_routed + n_shared
    logits = (orc.normal_f32(277 + tokens, tokens * rows, 2.0)).reshape(tokens, rows)
    bias = (orc.normal_f32(5 + n_routed, n_routed, 0.1)).astype(np.float32)
    if tokens > 2:
        logits[1, :] = 0.25          # an all-tie row
        bias[: n_routed // 2] = bias[0]
        logits[2, 5] = logits[2, 9]
        bias[9] = bias[5]
    idx, w, gam = moe.router_topk_sinks(torch.from_numpy(logits).cuda(), torch.from_numpy(bias).cuda(), n_routed, k,
                                        global_scale=0.75, route_scale=2.5)
    idx_ref, w_ref, gam_ref = orc.router_sinks(logits, bias, n_routed, k, global_scale=0.75, route_scale=2.5)
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), idx_ref)
    # f32 chains of exp / log: the device takes each as the rounded f64 function, the host its libm
    assert np.allclose(w.cpu().numpy(), w_ref, rtol=2e-6, atol=1e-9)
    assert np.allclose(gam.cpu().numpy(), gam_ref, rtol=2e-6, atol=1e-9)
    total = w.sum(1) + gam.sum(1)
    assert float((total - 0.75 * 2.5).abs().max()) <= 1e-5


def test_sink_router_flags_non_finite_shared_logit(moe):
    # src/models/inkling/block.rs:273-279: a NaN in a sink column is loud too
    from maryml_b200 import _lib
    ctx = _lib.context(0)
    ctx.check_flags(None)
    logits = torch.zeros(4, 34, device="cuda")
    logits[2, 33] = float("nan")
    moe.router_topk_sinks(logits, torch.zeros(32, device="cuda"), 32, 2)
    rc, flags = ctx.check_flags(None)
    assert rc == _lib.ERR_DEVICE_FLAG and flags[1] == 3
    assert ctx.check_flags(None)[0] == 0


def test_router_flags_non_finite_logits(moe, orc):
    from maryml_b200 import _lib
    ctx = _lib.context(0)
    ctx.check_flags(None)
    logits = torch.zeros(8, 64, device="cuda")
    logits[3, 7] = float("nan")
    moe.router_topk_softmax(logits, 4)
    rc, flags = ctx.check_flags(None)
    assert rc == _lib.ERR_DEVICE_FLAG and flags[1] == 4   # token index + 1
    rc, flags = ctx.check_flags(None)
    assert rc == 0


@pytest.mark.parametrize("form", ["one kernel", "three passes"])
@pytest.mark.parametrize("tokens,n_experts,k", [(2, 3, 2), (130, 4, 3), (4096, 128, 8), (5, 128, 8), (300, 64, 12),
                                               (1000, 32, 1), (2000, 256, 6), (3000, 1024, 8), (4097, 64, 4)])
def test_row_plan_bit_exact(moe, orc, tokens, n_experts, k, form, monkeypatch):
    """Plans of up to 4096 tokens and k <= 8 are built by one kernel whose CTAs (one per 256 tokens) form a cluster
    and read one another's histograms; larger ones, and MB_MOE_PLAN_CLUSTER=0, by three passes through global memory."""
    monkeypatch.setenv("MB_MOE_PLAN_CLUSTER", "1" if form == "one kernel" else "0")
    rng = np.random.default_rng(tokens * 7 + k)
    idx = np.stack([rng.permutation(n_experts)[:k] for _ in range(tokens)]).astype(np.int32)
    wgt = rng.random((tokens, k), dtype=np.float32)
    plan = moe.RowPlan(torch.from_numpy(idx).cuda(), torch.from_numpy(wgt).cuda(), n_experts)
    ref = orc.row_plan(idx.astype(np.uint32), wgt, n_experts, 128)
    m = ref["m_total"]
    assert int(plan.n_tiles.item()) * 128 == m
    assert np.array_equal(plan.row_tok.cpu().numpy()[:m], ref["row_tok"])
    assert (plan.row_tok.cpu().numpy()[m:] == -1).all()
    assert np.array_equal(plan.row_wgt.cpu().numpy()[:m].view(np.uint32), ref["row_wgt"].view(np.uint32))
    assert np.array_equal(plan.tok_rows.cpu().numpy().astype(np.uint32), ref["tok_rows"])
    counts = np.bincount(idx.ravel(), minlength=n_experts)
    assert np.array_equal(plan.expert_rows.cpu().numpy(), counts)
    active = np.nonzero(counts)[0]
    assert np.array_equal(plan.expert_row0.cpu().numpy()[active], ref["slot_row0"])
    te = plan.tile_expert.cpu().numpy()[: m // 128]
    want = np.concatenate([np.full((c + 127) // 128, e) for e, c in enumerate(counts) if c]) if m else np.array([])
    assert np.array_equal(te, want)
    # the padding-free map: every (token, pick) owns exactly one row and sees its own weight
    rt, rw, tr = plan.row_tok.cpu().numpy(), plan.row_wgt.cpu().numpy(), plan.tok_rows.cpu().numpy()
    for t in range(min(tokens, 50)):
        assert (rt[tr[t]] == t).all() and np.all(np.diff(tr[t]) > 0)
        assert sorted(rw[tr[t]].tolist()) == sorted(wgt[t].tolist())


@pytest.mark.parametrize("form", ["one kernel", "three passes"])
def test_plan_fault_flag_on_duplicate_or_out_of_range(moe, orc, form, monkeypatch):
    from maryml_b200 import _lib
    monkeypatch.setenv("MB_MOE_PLAN_CLUSTER", "1" if form == "one kernel" else "0")
    ctx = _lib.context(0)
    ctx.check_flags(None)
    idx = torch.tensor([[0, 1], [2, 2]], dtype=torch.int32, device="cuda")
    moe.RowPlan(idx, torch.ones(2, 2, device="cuda"), 4)
    rc, flags = ctx.check_flags(None)
    assert rc == _lib.ERR_DEVICE_FLAG and flags[2] == 2
    idx = torch.tensor([[0, 9]], dtype=torch.int32, device="cuda")
    moe.RowPlan(idx, torch.ones(1, 2, device="cuda"), 4)
    rc, flags = ctx.check_flags(None)
    assert rc == _lib.ERR_DEVICE_FLAG and flags[2] == 1


def test_scatter_weighted_bit_exact(moe, orc):
    tokens, k, n_experts, h = 200, 4, 16, 256
    rng = np.random.default_rng(5)
    idx = np.stack([rng.permutation(n_experts)[:k] for _ in range(tokens)]).astype(np.int32)
    wgt = rng.random((tokens, k), dtype=np.float32)
    plan = moe.RowPlan(torch.from_numpy(idx).cuda(), torch.from_numpy(wgt).cuda(), n_experts)
    ybits = f32_to_bf16_bits(orc.normal_f32(3, plan.m_cap * h, 1.0))
    y = dev_bf16(ybits).view(plan.m_cap, h)
    out = moe.scatter_weighted(y, plan, h).cpu().numpy()
    ref = orc.scatter_weighted(bf16_bits_to_f32(ybits).reshape(plan.m_cap, h), plan.row_wgt.cpu().numpy(),
                               plan.tok_rows.cpu().numpy().astype(np.uint32), np.full(tokens, k, np.uint32), h)
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))
    out32 = moe.scatter_weighted(y.float(), plan, h).cpu().numpy()
    assert np.array_equal(out32.view(np.uint32), ref.view(np.uint32))


def _bank(orc, seed, experts, n, k):
    w = orc.normal_f32(seed, experts * n * k, 0.02)
    return f32_to_bf16_bits(w).reshape(experts, n, k)


@pytest.mark.parametrize("tokens,h,inter,n_experts,k", [(64, 256, 128, 8, 2), (300, 512, 256, 16, 4)])
def test_moe_experts_against_oracle(moe, orc, tokens, h, inter, n_experts, k):
    xbits = f32_to_bf16_bits(orc.normal_f32(1, tokens * h, 1.0)).reshape(tokens, h)
    gbits = f32_to_bf16_bits(orc.normal_f32(4, n_experts * h, 0.02)).reshape(n_experts, h) if n_experts >= 32 else None
    w13 = _bank(orc, 2, n_experts, 2 * inter, h)
    w2 = _bank(orc, 3, n_experts, h, inter)
    rng = np.random.default_rng(tokens)
    idx = np.stack([rng.permutation(n_experts)[:k] for _ in range(tokens)]).astype(np.int32)
    wgt = rng.random((tokens, k), dtype=np.float32)
    wgt /= wgt.sum(1, keepdims=True)
    b13 = moe.ExpertBank.quantize(dev_bf16(w13).view(n_experts, 2 * inter, h))
    b2 = moe.ExpertBank.quantize(dev_bf16(w2).view(n_experts, h, inter))
    x = dev_bf16(xbits).view(tokens, h)
    out, plan = moe.moe_experts(x, torch.from_numpy(idx).cuda(), torch.from_numpy(wgt).cuda(), b13, b2)
    out_unfused, _ = moe.moe_experts(x, torch.from_numpy(idx).cuda(), torch.from_numpy(wgt).cuda(), b13, b2,
                                     fuse_swiglu=False)
    ref = orc.moe_experts(xbits, idx.astype(np.uint32), wgt,
                          (b13.codes.cpu().numpy().ravel(), b13.scales.cpu().numpy().ravel(), b13.scale2.cpu().numpy()),
                          (b2.codes.cpu().numpy().ravel(), b2.scales.cpu().numpy().ravel(), b2.scale2.cpu().numpy()),
                          h, inter, n_experts)
    got = out.cpu().numpy()
    rel, cos = rel_check(got, ref, max_rel=1e-2)
    # re-quantisation of bf16-rounded intermediates can flip a code where the GPU and CPU sums
    # round to different bf16 neighbours; the bound on the whole block is the north-star one
    assert cos >= 0.9999 and rel <= 5e-2, (rel, cos)
    rel2, cos2 = rel_check(out_unfused.cpu().numpy(), got)
    assert cos2 >= 0.99999, (rel2, cos2)
    # the second projection's quantizer inside the first product's epilogue: the same bytes as
    # storing the bf16 activations and quantizing them in a pass of their own
    out_stored, _ = moe.moe_experts(x, torch.from_numpy(idx).cuda(), torch.from_numpy(wgt).cuda(), b13, b2,
                                    fuse_quant=False)
    assert torch.equal(out_stored, out)


@pytest.mark.parametrize("tokens,h,inter,n_experts,k", [(300, 512, 256, 16, 4), (256, 2048, 768, 128, 8)])
def test_moe_experts_stage_by_stage(moe, orc, figures, tokens, h, inter, n_experts, k):
    """The expert lane checked the way the reference's own gates do it (src/bin/k3_router_gate.rs:60-95 stage by
    stage, src/bin/fp4quant_gate.rs:12-24 counting near-ties): every stage is fed the GPU's OWN previous output, so
    identical inputs must give identical bytes where the arithmetic is integer (quantizers, scatter order) and
    agree within the same-operand gate where it is a sum (products). The end-to-end comparison then COUNTS the
    rows whose second-stage codes flipped against the all-CPU chain; tokens without a flipped row must meet the
    1e-2 bound, the others are bounded by what a flipped E2M1 code can move."""
    from maryml_b200 import _lib, nvfp4 as nv
    xbits = f32_to_bf16_bits(orc.normal_f32(1, tokens * h, 1.0)).reshape(tokens, h)
    rng = np.random.default_rng(tokens)
    idx = np.stack([rng.permutation(n_experts)[:k] for _ in range(tokens)]).astype(np.int32)
    wgt = rng.random((tokens, k), dtype=np.float32)
    wgt /= wgt.sum(1, keepdims=True)
    b13 = moe.ExpertBank.quantize(dev_bf16(_bank(orc, 2, n_experts, 2 * inter, h)).view(n_experts, 2 * inter, h))
    b2 = moe.ExpertBank.quantize(dev_bf16(_bank(orc, 3, n_experts, h, inter)).view(n_experts, h, inter))
    c13, s13, g13 = b13.codes.cpu().numpy(), b13.scales.cpu().numpy(), b13.scale2.cpu().numpy()
    c2w, s2w, g2 = b2.codes.cpu().numpy(), b2.scales.cpu().numpy(), b2.scale2.cpu().numpy()
    x = dev_bf16(xbits).view(tokens, h)
    plan = moe.RowPlan(torch.from_numpy(idx).cuda(), torch.from_numpy(wgt).cuda(), n_experts)
    row_tok = plan.row_tok.cpu().numpy()
    m_cap = plan.m_cap
    live = row_tok >= 0
    e_rows, e_row0 = plan.expert_rows.cpu().numpy(), plan.expert_row0.cpu().numpy()

    # stage 1: token planes, bit-exact; gathered into plan order
    t_codes, t_sf, _ = nv.quantize_act(x, _lib.QUANT_RECIP, tiled=True)
    tc_ref, ts_ref = orc.quantize_act_recip(bf16_bits_to_f32(xbits), tokens, h)
    assert np.array_equal(t_codes.cpu().numpy().ravel(), tc_ref)
    assert np.array_equal(nv.untile_scales(t_sf, tokens, h).cpu().numpy().ravel(), ts_ref)
    a_codes, a_sf = nv.gather_rows(t_codes, t_sf, tokens, h, plan.row_tok)
    a_c = a_codes.cpu().numpy()
    a_s = nv.untile_scales(a_sf, m_cap, h).cpu().numpy()
    assert np.array_equal(a_c[live], tc_ref.reshape(tokens, h // 2)[row_tok[live]])

    def per_expert(codes_rows, scales_rows, wc, ws, wg, n, kk):
        out = np.zeros((m_cap, n), np.float32)
        for e in range(n_experts):
            r0, cnt = int(e_row0[e]), int(e_rows[e])
            if cnt:
                out[r0:r0 + cnt] = orc.linear_w4a4(codes_rows[r0:r0 + cnt].ravel(), scales_rows[r0:r0 + cnt].ravel(),
                                                   wc[e].ravel(), ws[e].ravel(), np.float32(wg[e]), cnt, n, kk)
        return out

    # stage 2: first grouped product, f32 out, against f64 sums of the SAME operands (reference gate: 1e-4)
    both32 = moe.grouped_gemm(a_codes, a_sf, b13, plan, out_dtype=torch.float32).cpu().numpy()
    both_ref = per_expert(a_c, a_s, c13, s13, g13, 2 * inter, h)
    e2 = np.abs(both32[live] - both_ref[live]).max() / np.abs(both_ref[live]).max()
    assert e2 <= 1e-4, e2

    # stage 3: SwiGLU on the GPU's own product. The fused epilogue rounds gate and up to bf16, then silu * up in
    # f32 with the fast exponential, then bf16: against the CPU form on the same bf16 gate/up a few results land
    # on the neighbouring bf16 value; they are counted.
    act = moe.grouped_gemm(a_codes, a_sf, b13, plan, epilogue=_lib.EPI_SWIGLU_INTERLEAVED)
    act_bits = host_bits(act).reshape(m_cap, inter)
    act_ref = f32_to_bf16_bits(orc.gate_up_silu(bf16_bits_to_f32(f32_to_bf16_bits(both32)), m_cap, inter, round_bf16=True))
    act_ref = act_ref.reshape(m_cap, inter)
    moved = (act_bits[live] != act_ref[live])
    step = np.abs(bf16_bits_to_f32(act_bits[live]) - bf16_bits_to_f32(act_ref[live]))
    assert moved.mean() <= 5e-3 and (step <= 2.0 ** -7 * np.abs(bf16_bits_to_f32(act_ref[live])) + 1e-30).all()

    # stage 3b: the second projection's quantizer on the GPU's own activations: identical input, identical bytes
    q_c, q_sf, _ = nv.quantize_act(act, _lib.QUANT_RECIP, tiled=True)
    qc_ref, qs_ref = orc.quantize_act_recip(bf16_bits_to_f32(act_bits), m_cap, inter)
    q_cn, q_sn = q_c.cpu().numpy(), nv.untile_scales(q_sf, m_cap, inter).cpu().numpy()
    assert np.array_equal(q_cn[live], qc_ref.reshape(m_cap, -1)[live])
    assert np.array_equal(q_sn[live], qs_ref.reshape(m_cap, -1)[live])
    # and the epilogue that quantizes where it produces writes those bytes
    f_c, f_sf = moe.grouped_gemm(a_codes, a_sf, b13, plan, epilogue=_lib.EPI_SWIGLU_INTERLEAVED | _lib.EPI_QUANT_RECIP)
    assert np.array_equal(f_c.cpu().numpy()[live], q_cn[live])
    assert np.array_equal(nv.untile_scales(f_sf, m_cap, inter).cpu().numpy()[live], q_sn[live])

    # stage 4: second grouped product from the GPU's codes
    y32 = moe.grouped_gemm(q_c, q_sf, b2, plan, out_dtype=torch.float32).cpu().numpy()
    y_ref = per_expert(q_cn, q_sn, c2w, s2w, g2, h, inter)
    e4 = np.abs(y32[live] - y_ref[live]).max() / np.abs(y_ref[live]).max()
    assert e4 <= 1e-4, e4

    # stage 5: ordered weighted sum of the GPU's own bf16 rows: the fma chain in ascending row order, bit for bit
    y16 = moe.grouped_gemm(q_c, q_sf, b2, plan, skip_pad_rows=True)
    out = moe.scatter_weighted(y16, plan, h).cpu().numpy()
    yf = bf16_bits_to_f32(host_bits(y16)).reshape(m_cap, h)
    yf[~live] = 0.0
    tok_rows = plan.tok_rows.cpu().numpy().astype(np.uint32)
    out_ref = orc.scatter_weighted(yf, plan.row_wgt.cpu().numpy(), tok_rows, np.full(tokens, k, np.uint32), h)
    assert np.array_equal(out.view(np.uint32), out_ref.view(np.uint32))

    # end to end against the all-CPU chain, with the flipped rows counted
    both_cpu = bf16_bits_to_f32(f32_to_bf16_bits(both_ref))
    act_cpu = orc.gate_up_silu(both_cpu, m_cap, inter, round_bf16=True)
    qc_cpu, qs_cpu = orc.quantize_act_recip(act_cpu, m_cap, inter)
    flipped_rows = live & ((q_cn != qc_cpu.reshape(m_cap, -1)).any(1) | (q_sn != qs_cpu.reshape(m_cap, -1)).any(1))
    flipped_codes = int((((q_cn ^ qc_cpu.reshape(m_cap, -1)) & 0x0F) != 0)[live].sum() +
                        (((q_cn ^ qc_cpu.reshape(m_cap, -1)) & 0xF0) != 0)[live].sum())
    touched = np.zeros(tokens, bool)
    touched[row_tok[flipped_rows]] = True
    final, _ = moe.moe_experts(x, torch.from_numpy(idx).cuda(), torch.from_numpy(wgt).cuda(), b13, b2)
    ref = orc.moe_experts(xbits, idx.astype(np.uint32), wgt, (c13.ravel(), s13.ravel(), g13), (c2w.ravel(), s2w.ravel(), g2),
                          h, inter, n_experts)
    got = final.cpu().numpy()
    # relative to the larger of the element and the output's rms: the second product's rows are stored as bf16, and
    # where the GPU's and the CPU's f32 sums straddle a bf16 rounding boundary a row value moves by 2^-8 of itself,
    # an absolute error no element far below the rms can absorb
    rms = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    rel = np.abs(got - ref) / np.maximum(np.abs(ref), rms)
    clean = rel[~touched].max() if (~touched).any() else 0.0
    dirty = (np.abs(got - ref)[touched].max() / rms) if touched.any() else 0.0
    figures("moe_stagewise", tokens=tokens, experts=n_experts, gemm1_rel=e2, gemm2_rel=e4, swiglu_moved=moved.mean(),
            flipped_codes=flipped_codes, codes=int(live.sum()) * inter, tokens_touched=int(touched.sum()),
            clean_max_rel=clean, touched_max_over_rms=dirty)
    print(f"moe stage-wise: {flipped_codes} of {int(live.sum()) * inter} second-stage codes flipped in {int(flipped_rows.sum())} rows "
          f"({int(touched.sum())} of {tokens} tokens); clean tokens max rel {clean:.2e}, touched tokens max |err|/rms {dirty:.2e}")
    assert flipped_codes <= 2e-3 * int(live.sum()) * inter
    assert clean <= 1e-2, clean
    assert dirty <= 5e-2, dirty
    assert rel_check(got, ref)[1] >= 0.9999


def test_grouped_product_leaves_pad_rows_unwritten(moe, orc):
    from maryml_b200 import _lib, nvfp4 as nv
    tokens, h, n, n_experts, k = 150, 256, 384, 8, 2
    rng = np.random.default_rng(11)
    idx = np.stack([rng.permutation(n_experts)[:k] for _ in range(tokens)]).astype(np.int32)
    wgt = rng.random((tokens, k), dtype=np.float32)
    plan = moe.RowPlan(torch.from_numpy(idx).cuda(), torch.from_numpy(wgt).cuda(), n_experts)
    bank = moe.ExpertBank.quantize(dev_bf16(_bank(orc, 8, n_experts, n, h)).view(n_experts, n, h))
    x = dev_bf16(f32_to_bf16_bits(orc.normal_f32(6, tokens * h, 1.0))).view(tokens, h)
    t_c, t_s, _ = nv.quantize_act(x, _lib.QUANT_RECIP, tiled=True)
    a_c, a_s = nv.gather_rows(t_c, t_s, tokens, h, plan.row_tok)
    live = plan.row_tok >= 0
    assert int(live.sum()) == tokens * k and not bool(live.all())
    for dt in (torch.bfloat16, torch.float32):
        whole = moe.grouped_gemm(a_c, a_s, bank, plan, out_dtype=dt)
        ctx = _lib.context(0)
        out = torch.full((plan.m_cap, n), 7.0, dtype=dt, device="cuda")
        ctx.check(_lib.lib.mb_nvfp4_gemm_w4a4_grouped(
            ctx.handle, nv._stream(), nv._p(a_c), nv._p(a_s), nv._p(bank.codes), nv._p(bank.sf_tiled),
            nv._p(bank.scale2), nv._p(plan.tile_expert), nv._p(plan.n_tiles), plan.m_cap, n_experts, n, h, nv._p(out),
            _lib.DT_BF16 if dt == torch.bfloat16 else _lib.DT_F32, _lib.EPI_PLAIN, None, nv._p(plan.row_tok)))
        assert torch.equal(out[live], whole[live])
        assert bool((out[~live] == 7.0).all())
        # the rows of an expert are contiguous from its first row: products of zero rows are zero
        used = int(plan.n_tiles.item()) * 128
        assert bool((whole[:used][~live[:used]] == 0).all())


def test_moe_layer_config2_shapes_smoke(moe, orc):
    """Config 2 at reduced token count: 128 experts, top-8, hidden 2048, intermediate 768."""
    tokens, h, inter, n_experts, k = 256, 2048, 768, 128, 8
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(tokens, h, device="cuda", generator=g).to(torch.bfloat16)
    gate = (torch.randn(n_experts, h, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    b13 = moe.ExpertBank.quantize((torch.randn(n_experts, 2 * inter, h, device="cuda", generator=g) * 0.02).to(torch.bfloat16))
    b2 = moe.ExpertBank.quantize((torch.randn(n_experts, h, inter, device="cuda", generator=g) * 0.02).to(torch.bfloat16))
    out, (logits, idx, weight, plan) = moe.moe_layer(x, gate, k, b13, b2)
    # router parity from the GPU's own logits (indices bit-exact given identical logits)
    lg = logits.cpu().numpy()
    idx_ref, w_ref = orc.router_select(orc.router_scores_softmax(lg), k)
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), idx_ref)
    # logits against f64 accumulation of the same bf16 operands
    lg_ref = orc.router_logits(host_bits(x), host_bits(gate), tokens, h, n_experts)
    assert np.abs(lg - lg_ref).max() <= 1e-4
    ref = orc.moe_experts(host_bits(x), idx_ref, w_ref,
                          (b13.codes.cpu().numpy().ravel(), b13.scales.cpu().numpy().ravel(), b13.scale2.cpu().numpy()),
                          (b2.codes.cpu().numpy().ravel(), b2.scales.cpu().numpy().ravel(), b2.scale2.cpu().numpy()),
                          h, inter, n_experts)
    rel, cos = rel_check(out.cpu().numpy(), ref)
    assert cos >= 0.9999 and rel <= 5e-2, (rel, cos)
