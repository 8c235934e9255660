"""GPU parity tests of the entry points that complete the reference's boundary: attention over key runs
(flash_attention_launch's own argument list), the decode-time grouped experts, the W4A16 prompt product that
keeps the weight four bits in HBM, the Inkling op surface (linear_fp4 / linear_w4a16 / linear_w, rms_norm,
gate_up_silu) and a bounded wait on an absent peer. Oracle = the CPU restatement on the same seeded bytes."""
import ctypes as C
import math

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle_lib import bf16_bits_to_f32, f32_to_bf16_bits  # noqa: E402
from test_gpu_nvfp4 import attn_check, dev_bf16, host_bits, rel_check  # noqa: E402


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from maryml_b200 import attention, inkling, nvfp4, _lib
    return attention, inkling, nvfp4, _lib


def _rows(orc, seed, batch, rows, width, sigma=1.0):
    return f32_to_bf16_bits(orc.normal_f32(seed, batch * rows * width, sigma)).reshape(batch, rows, width)


# ------------------------------------------------------------------- attention over key runs
def test_one_run_longer_than_its_live_keys_equals_the_sliced_cache(mods, orc):
    """A cache allocated longer than `keys` is read in place: same bytes out as the call on a contiguous copy of
    the live rows, and what sits in the dead rows (NaN here) never reaches the output."""
    att, _, _, _ = mods
    batch, heads, kvh, D = 3, 8, 2, 128
    for nq, keys, cap in [(1, 700, 1024), (2, 3000, 4100), (300, 300, 512)]:
        q = dev_bf16(_rows(orc, 7 + keys, batch, nq, heads * D)).view(batch, nq, heads, D)
        k = dev_bf16(_rows(orc, 8 + keys, batch, cap, kvh * D)).view(batch, cap, kvh, D).clone()
        v = dev_bf16(_rows(orc, 9 + keys, batch, cap, kvh * D)).view(batch, cap, kvh, D).clone()
        k[:, keys:] = float("nan")
        v[:, keys:] = float("nan")
        got = att.flash_attention(q, k, v, q0=keys - nq, keys=keys)
        want = att.flash_attention(q, k[:, :keys].contiguous(), v[:, :keys].contiguous(), q0=keys - nq)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def _paged(orc, seed, batch, kvh, pages, D=128):
    """pages: (rows, lo, hi) per run. Returns the bf16 bit arrays per page and the live rows stitched in order."""
    ks, vs, live_k, live_v = [], [], [], []
    for i, (rows, lo, hi) in enumerate(pages):
        kb = _rows(orc, seed + 2 * i, batch, rows, kvh * D)
        vb = _rows(orc, seed + 2 * i + 1, batch, rows, kvh * D)
        ks.append(kb)
        vs.append(vb)
        live_k.append(kb[:, lo:hi])
        live_v.append(vb[:, lo:hi])
    return ks, vs, np.concatenate(live_k, 1), np.concatenate(live_v, 1)


@pytest.mark.parametrize("nq,pages,window", [
    (1, [(512, 0, 512), (512, 0, 512), (256, 0, 77)], 0),          # full pages and a partly filled tail page
    (1, [(300, 45, 300), (1024, 0, 1024), (128, 0, 128)], 0),      # a dropped prefix on the first page
    (2, [(640, 10, 640), (640, 0, 333)], 0),                       # two queries at the end
    (1, [(1024, 0, 1024), (1024, 0, 1024), (512, 0, 400)], 700),   # a window that starts inside the second page
])
@pytest.mark.parametrize("q_f32", [False, True])
def test_key_runs_of_a_paged_cache_do_not_move_the_answer(mods, orc, nq, pages, window, q_f32):
    """src/models/inkling/flash.rs:1575-2332: one run per page, a dropped prefix and tail padding excluded by
    lo..hi, against the CPU rule over the stitched live rows; f32 queries and output as the reference passes them."""
    att, _, _, _ = mods
    batch, heads, kvh, D = 2, 8, 2, 128
    ks, vs, lk, lv = _paged(orc, 31 + nq + window, batch, kvh, pages)
    keys = lk.shape[1]
    qb = _rows(orc, 5, batch, nq, heads * D)
    runs, base = [], 0
    for (rows, lo, hi), kb, vb in zip(pages, ks, vs):
        kd = dev_bf16(kb).view(batch, rows, kvh, D).clone()
        vd = dev_bf16(vb).view(batch, rows, kvh, D).clone()
        kd[:, :lo] = float("nan"); kd[:, hi:] = float("nan")
        vd[:, :lo] = float("nan"); vd[:, hi:] = float("nan")
        # `base` is the position of stored row 0, so the first live row stands at base + lo
        runs.append(att.KeyRunView(kd, vd, base=base - lo + 1000, lo=lo, hi=hi))
        base += hi - lo
    q0 = 1000 + keys - nq
    qd = dev_bf16(qb).view(batch, nq, heads, D)
    if q_f32:
        out = att.flash_attention_runs(qd.float(), runs, q0=q0, window=window)
        assert out.dtype == torch.float32
        got = out.cpu().numpy().reshape(batch, nq, heads * D)
    else:
        got = bf16_bits_to_f32(host_bits(att.flash_attention_runs(qd, runs, q0=q0, window=window))).reshape(batch, nq, -1)
    for b in range(batch):
        ref = orc.attention(bf16_bits_to_f32(qb[b]), bf16_bits_to_f32(lk[b]), bf16_bits_to_f32(lv[b]), heads, kvh, D,
                            keys - nq, 1.0 / math.sqrt(D), window=window)
        rel, cos = attn_check(got[b], ref)
        assert rel <= 1e-2 and cos >= 0.9999, (b, rel, cos)


def test_key_runs_of_nvfp4_rows_and_of_f32_rows(mods, orc):
    """KvElem::{Nvfp4, F32} (src/models/inkling/flash.rs:972-981): packed pages are read packed, f32 pages through a
    bf16 copy of their live rows; both against the CPU rule over the values the cache holds."""
    att, _, nv, _ = mods
    batch, heads, kvh, D = 2, 8, 2, 128
    pages = [(512, 0, 512), (384, 20, 384), (256, 0, 100)]
    ks, vs, lk, lv = _paged(orc, 77, batch, kvh, pages)
    keys = lk.shape[1]
    qb = _rows(orc, 3, batch, 1, heads * D)
    qd = dev_bf16(qb).view(batch, 1, heads, D)
    runs4, runs32, deq_k, deq_v, base = [], [], [], [], 0
    for (rows, lo, hi), kb, vb in zip(pages, ks, vs):
        kd = dev_bf16(kb).view(batch, rows, kvh, D)
        vd = dev_bf16(vb).view(batch, rows, kvh, D)
        kc, ksc = att.quantize_kv_rows(kd)
        vc, vsc = att.quantize_kv_rows(vd)
        runs4.append(att.KeyRunView(kc, vc, ksc, vsc, base=base - lo, lo=lo, hi=hi))
        runs32.append(att.KeyRunView(kd.float(), vd.float(), base=base - lo, lo=lo, hi=hi))
        dk = nv.dequantize(kc.view(batch * rows, -1), ksc.view(batch * rows, -1), 1.0, batch * rows, kvh * D).view(batch, rows, -1)
        dv = nv.dequantize(vc.view(batch * rows, -1), vsc.view(batch * rows, -1), 1.0, batch * rows, kvh * D).view(batch, rows, -1)
        deq_k.append(dk[:, lo:hi].cpu().numpy())
        deq_v.append(dv[:, lo:hi].cpu().numpy())
        base += hi - lo
    dk, dv = np.concatenate(deq_k, 1), np.concatenate(deq_v, 1)
    got4 = bf16_bits_to_f32(host_bits(att.flash_attention_runs(qd, runs4, q0=keys - 1))).reshape(batch, 1, -1)
    got32 = att.flash_attention_runs(qd.float(), runs32, q0=keys - 1).cpu().numpy().reshape(batch, 1, -1)
    for b in range(batch):
        ref4 = orc.attention(bf16_bits_to_f32(qb[b]), dk[b], dv[b], heads, kvh, D, keys - 1, 1.0 / math.sqrt(D))
        ref32 = orc.attention(bf16_bits_to_f32(qb[b]), bf16_bits_to_f32(lk[b]), bf16_bits_to_f32(lv[b]), heads, kvh, D,
                              keys - 1, 1.0 / math.sqrt(D))
        for got, ref in ((got4[b], ref4), (got32[b], ref32)):
            rel, cos = attn_check(got, ref)
            assert rel <= 1e-2 and cos >= 0.9999, (rel, cos)


def test_key_runs_with_relative_bias_and_gaps(mods, orc):
    """Gaps are indexed by the logical row (row0 + stored row) and shift every later key's position
    (src/models/inkling/flash.rs:751-785, 1017-1035), across two runs."""
    att, _, _, _ = mods
    batch, heads, kvh, D, eff = 1, 8, 2, 128, 40
    pages = [(512, 0, 512), (512, 0, 300)]
    ks, vs, lk, lv = _paged(orc, 91, batch, kvh, pages)
    keys = lk.shape[1]
    gaps = [(100, 7), (600, 30)]                       # logical rows, cumulative skips
    pos = np.arange(keys, dtype=np.int64)
    for row, cum in gaps:
        pos[row:] = np.arange(row, keys) + cum
    q0 = int(pos[-1])
    qb = _rows(orc, 4, batch, 1, heads * D)
    rel = orc.normal_f32(6, batch * heads * eff, 1.0).reshape(batch, 1, heads, eff).astype(np.float32)
    runs, base = [], 0
    for (rows, lo, hi), kb, vb in zip(pages, ks, vs):
        runs.append(att.KeyRunView(dev_bf16(kb).view(batch, rows, kvh, D), dev_bf16(vb).view(batch, rows, kvh, D),
                                   base=base, lo=lo, hi=hi, row0=base))
        base += hi - lo
    gd = (torch.tensor([g[0] for g in gaps], dtype=torch.int32, device="cuda"),
          torch.tensor([g[1] for g in gaps], dtype=torch.int32, device="cuda"))
    out = att.flash_attention_runs(dev_bf16(qb).view(batch, 1, heads, D), runs, q0=q0, rel=torch.from_numpy(rel).cuda(),
                                   gaps=gd, window=500)
    got = bf16_bits_to_f32(host_bits(out)).reshape(1, -1)
    ref = orc.attention(bf16_bits_to_f32(qb[0]), bf16_bits_to_f32(lk[0]), bf16_bits_to_f32(lv[0]), heads, kvh, D, q0,
                        1.0 / math.sqrt(D), key_pos=pos, window=500, rel=rel[0])
    r, cos = attn_check(got, ref)
    assert r <= 1e-2 and cos >= 0.9999, (r, cos)


def test_prompt_shapes_take_one_run_in_place_with_f32_in_and_out(mods, orc):
    att, _, _, _lib = mods
    batch, nq, past, cap, heads, kvh, D = 1, 200, 56, 384, 4, 2, 128
    keys = past + nq
    qb = _rows(orc, 12, batch, nq, heads * D)
    kb = _rows(orc, 13, batch, cap, kvh * D)
    vb = _rows(orc, 14, batch, cap, kvh * D)
    kd = dev_bf16(kb).view(batch, cap, kvh, D).clone()
    vd = dev_bf16(vb).view(batch, cap, kvh, D).clone()
    kd[:, keys:] = float("nan")
    vd[:, keys:] = float("nan")
    run = att.KeyRunView(kd, vd, hi=keys)
    out = att.flash_attention_runs(dev_bf16(qb).view(batch, nq, heads, D).float(), [run], q0=past)
    assert out.dtype == torch.float32
    ref = orc.attention(bf16_bits_to_f32(qb[0]), bf16_bits_to_f32(kb[0, :keys]), bf16_bits_to_f32(vb[0, :keys]), heads, kvh,
                        D, past, 1.0 / math.sqrt(D))
    r, cos = attn_check(out.cpu().numpy().reshape(nq, -1), ref)
    assert r <= 1.5e-2 and cos >= 0.9999, (r, cos)          # the prompt-shape bound of the attention tests
    with pytest.raises(_lib.MaryError):          # two live runs under a prompt-shaped block
        att.flash_attention_runs(dev_bf16(qb).view(batch, nq, heads, D), [run, run], q0=past)
    with pytest.raises(_lib.MaryError):          # a live range outside the buffer
        att.flash_attention_runs(dev_bf16(qb).view(batch, nq, heads, D), [att.KeyRunView(kd, vd, lo=10, hi=cap + 1)], q0=past)


def test_prompt_shaped_block_over_a_packed_page(mods, orc):
    """A prompt-shaped query block over NVFP4 rows goes through the dequantizing reader
    (src/models/inkling/flash.rs:520-540): the live rows are expanded to bf16 (exactly) and read by the prompt kernel.
    Against the CPU rule over the values the page holds; rows past the live ones are garbage on purpose."""
    att, _, nv, _lib = mods
    batch, nq, past, cap, heads, kvh, D = 2, 160, 96, 320, 8, 2, 128
    keys = past + nq
    qb = _rows(orc, 31, batch, nq, heads * D)
    kb = _rows(orc, 32, batch, cap, kvh * D)
    vb = _rows(orc, 33, batch, cap, kvh * D)
    kd = dev_bf16(kb).view(batch, cap, kvh, D)
    vd = dev_bf16(vb).view(batch, cap, kvh, D)
    kc, ksc = att.quantize_kv_rows(kd)
    vc, vsc = att.quantize_kv_rows(vd)
    dk = nv.dequantize(kc.view(batch * cap, -1), ksc.view(batch * cap, -1), 1.0, batch * cap, kvh * D).view(batch, cap, -1)
    dv = nv.dequantize(vc.view(batch * cap, -1), vsc.view(batch * cap, -1), 1.0, batch * cap, kvh * D).view(batch, cap, -1)
    ksc = ksc.clone()
    ksc.view(batch, cap, -1)[:, keys:] = 0x7F          # NaN scales beyond the live rows: they must never be read
    run = att.KeyRunView(kc, vc, ksc, vsc, hi=keys)
    out = att.flash_attention_runs(dev_bf16(qb).view(batch, nq, heads, D), [run], q0=past)
    got = bf16_bits_to_f32(host_bits(out)).reshape(batch, nq, -1)
    for b in range(batch):
        ref = orc.attention(bf16_bits_to_f32(qb[b]), dk[b, :keys].float().cpu().numpy(), dv[b, :keys].float().cpu().numpy(),
                            heads, kvh, D, past, 1.0 / math.sqrt(D))
        r, cos = attn_check(got[b], ref)
        assert r <= 1.5e-2 and cos >= 0.9999, (b, r, cos)


# ------------------------------------------------------------------- decode-time grouped experts
@pytest.mark.parametrize("groups,experts,n,k,per_group", [(8, 16, 1536, 2048, False), (4, 6, 264, 768, True),
                                                          (1, 3, 2048, 64, True)])
def test_grouped_decode_is_project_w4a4_scaled_on_one_row_per_group(mods, orc, groups, experts, n, k, per_group):
    """w4a4_grouped_bf16 (src/nn/nvfp4_gemm.rs:462-523): per group exactly project_w4a4_scaled on one row."""
    _, ink, nv, _lib = mods
    wb = f32_to_bf16_bits(orc.normal_f32(21, experts * n * k, 0.02)).reshape(experts, n, k)
    planes = [orc.quantize_weight_bf16(wb[e], n, k) for e in range(experts)]
    codes = np.stack([p[0] for p in planes]).reshape(experts, n, k // 2)
    scales = np.stack([p[1] for p in planes]).reshape(experts, n, k // 16)
    scale2 = np.array([p[2] for p in planes], np.float32)
    input_scale = (0.5 + np.arange(experts, dtype=np.float32) / 8).astype(np.float32)
    ids = np.sort(np.random.default_rng(3).choice(experts, groups, replace=False)).astype(np.int32)
    xb = f32_to_bf16_bits(orc.normal_f32(22, (groups if per_group else 1) * k, 1.0))
    bank = ink.GroupedBank(torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda(), torch.from_numpy(scale2),
                           torch.from_numpy(input_scale).cuda(), experts, n, k)
    out, (a_codes, a_scales) = ink.w4a4_grouped_bf16(dev_bf16(xb).view(-1, k), per_group, torch.from_numpy(ids).cuda(), bank)
    alpha = (scale2 * input_scale).astype(np.float32)
    ref, c_ref, s_ref = orc.w4a4_grouped(xb, per_group, ids.astype(np.uint32), input_scale, alpha, codes, scales, n, k)
    assert np.array_equal(a_codes.cpu().numpy(), c_ref) and np.array_equal(a_scales.cpu().numpy(), s_ref)
    got = bf16_bits_to_f32(host_bits(out)).reshape(groups, n)
    # products of the decoded operands are exact in f32, the sums are f32: the reference's same-operand gate
    # (src/bin/inkling_fp4_expert_gate.rs:16-28) plus the bf16 rounding of the stored result
    err = np.abs(got - ref).max(1) / (np.abs(ref).max(1) + 1e-30)
    assert err.max() <= 2 ** -8 + 1e-4, err
    # and the one-row projection itself
    for g in range(groups):
        w = nv.Nvfp4.from_parts(bank.codes[ids[g]], bank.scales[ids[g]], scale2[ids[g]], n, k, torch.bfloat16,
                                torch.device("cuda", 0))
        x_row = dev_bf16(xb).view(-1, k)[g if per_group else 0].view(1, 1, k)
        one = w.project_w4a4_scaled(x_row, float(input_scale[ids[g]])).view(-1).float()
        assert (one - out[g].float()).abs().max().item() <= 2 ** -7 * one.abs().max().item()
    bad = torch.from_numpy(ids.copy()).cuda()
    bad[0] = experts + 3                               # an id outside the bank raises the plan flag, the row is zeros
    out_bad, _ = ink.w4a4_grouped_bf16(dev_bf16(xb).view(-1, k), per_group, bad, bank)
    rc, flags = _lib.context(0).check_flags(None)
    assert rc == _lib.ERR_DEVICE_FLAG and flags[2] == 1 and not out_bad[0].any()


# ------------------------------------------------------------------- W4A16 without a 16-bit copy of the weight
@pytest.mark.parametrize("m,n,k", [(1, 256, 64), (16, 384, 512), (130, 4096, 4096), (300, 264, 1024), (1024, 512, 2048)])
def test_w4a16_prompt_product_decodes_the_weight_on_the_way_to_the_tensor_core(mods, orc, m, n, k):
    _, _, nv, _ = mods
    wb = f32_to_bf16_bits(orc.normal_f32(41, n * k, 0.02))
    xb = f32_to_bf16_bits(orc.normal_f32(42, m * k, 1.0))
    c, s, s2 = orc.quantize_weight_bf16(wb, n, k)
    q = nv.Nvfp4.from_parts(torch.from_numpy(c).cuda().view(n, k // 2), torch.from_numpy(s).cuda().view(n, k // 16), s2, n, k,
                            torch.bfloat16, torch.device("cuda", 0))
    got32 = nv.w4a16_gemm(dev_bf16(xb).view(m, k), q.codes, q.scales, q.scale2, n, k, out_dtype=torch.float32)
    ref = orc.linear_w4a16(xb, c, s, s2, m, n, k)
    # every product is exact in f32; only the f32 summation order separates the two (reference bound:
    # 64 eps of the absolute sum, src/nn/nvfp4_gemv.rs:690-724)
    xf, wf = np.abs(bf16_bits_to_f32(xb)).reshape(m, k), np.abs(orc.dequantize(c, s, s2)).reshape(n, k)
    bound = 64 * 2.0 ** -24 * (xf.astype(np.float64) @ wf.astype(np.float64).T)
    assert (np.abs(got32.cpu().numpy() - ref) <= bound + 1e-30).all()
    got16 = q.project(dev_bf16(xb).view(1, m, k), nv.PromptLane.W4A16)
    rel, cos = rel_check(bf16_bits_to_f32(host_bits(got16)).reshape(m, n), ref)
    assert rel <= 1e-2 and cos >= 0.9999
    # the lane that decodes to a scratch plane first multiplies the same bf16 operands
    w = nv.dequantize(q.codes, q.scales, 1.0, n, k, dtype=torch.bfloat16)
    via_scratch = nv.bf16_gemm(dev_bf16(xb).view(m, k), w, out_dtype=torch.float32, alpha=q.scale2)
    assert (via_scratch - got32).abs().max().item() <= 1e-4 * got32.abs().max().item()


# ------------------------------------------------------------------- Inkling op surface
@pytest.mark.parametrize("rows,width", [(5, 4096), (37, 2048), (3, 200), (2, 24), (1, 8192)])
def test_inkling_rms_norm_bit_exact(mods, orc, rows, width):
    """rms_norm_kernel (src/models/inkling/resid.rs:272-322): same summation order as the reference kernel, so the
    bytes are the oracle's."""
    _, ink, _, _ = mods
    xb = f32_to_bf16_bits(orc.normal_f32(51, rows * width, 1.5))
    gain = (1.0 + 0.1 * orc.normal_f32(52, width, 1.0)).astype(np.float32)
    g = torch.from_numpy(gain).cuda()
    y = ink.rms_norm(dev_bf16(xb).view(rows, width), g, 1e-6)
    assert np.array_equal(host_bits(y).reshape(rows, width), orc.rmsnorm_inkling(xb, gain, rows, width, 1e-6))
    x32 = orc.normal_f32(53, rows * width, 1.5)
    y32 = ink.rms_norm(torch.from_numpy(x32).cuda().view(rows, width), g, 1e-5)
    ref32 = orc.rmsnorm_inkling(x32, gain, rows, width, 1e-5, out_bf16=False)
    assert np.array_equal(y32.cpu().numpy().view(np.uint32), ref32.view(np.uint32))
    # and the host twin's formula (src/models/inkling/block.rs:31-46) within a few ulp
    scale = 1.0 / np.sqrt((x32.reshape(rows, width).astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-5)
    assert np.abs(y32.cpu().numpy() - gain * (x32.reshape(rows, width) * scale)).max() <= 1e-5 * np.abs(ref32).max()


@pytest.mark.parametrize("halved", [False, True])
def test_gate_up_silu_both_readings(mods, orc, halved):
    _, ink, _, _ = mods
    rows, inter = 9, 768
    both = orc.normal_f32(61, rows * 2 * inter, 2.0).reshape(rows, 2 * inter)
    act = ink.gate_up_silu(torch.from_numpy(both).cuda(), inter, halved=halved)
    ref = orc.gate_up_silu(both, rows, inter, halved=halved)
    assert np.abs(act.cpu().numpy() - ref).max() <= 4e-7 * np.abs(ref).max() + 1e-9     # expf differs by an ulp from the host's
    narrow = ink.gate_up_silu(torch.from_numpy(both).cuda().to(torch.bfloat16), inter, halved=halved)
    both16 = bf16_bits_to_f32(f32_to_bf16_bits(both))
    ref16 = bf16_bits_to_f32(f32_to_bf16_bits(orc.gate_up_silu(both16, rows, inter, halved=halved)))
    got16 = bf16_bits_to_f32(host_bits(narrow)).reshape(rows, inter)
    assert (got16 != ref16).mean() < 5e-3 and np.abs(got16 - ref16).max() <= 2 ** -7 * np.abs(ref16).max()
    # a halved w13 re-ordered row by row is the interleaved one
    codes = torch.arange(2 * inter, dtype=torch.int32).view(1, 2 * inter, 1)
    c2, _ = ink.interleave_halved(codes, codes)
    assert c2.view(-1).tolist()[:4] == [0, inter, 1, inter + 1]


def test_linear_w_lanes_against_the_oracle(mods, orc):
    """linear_fp4 / linear_w4a16 / linear_bf16 behind linear_w (src/models/inkling/burn.rs:203-311)."""
    _, ink, nv, _ = mods
    m, n, k = 21, 512, 1024
    wb = f32_to_bf16_bits(orc.normal_f32(71, n * k, 0.02))
    x32 = orc.normal_f32(72, m * k, 1.0)
    xb = f32_to_bf16_bits(x32)
    c, s, s2 = orc.quantize_weight_bf16(wb, n, k)
    w = ink.PackedW(torch.from_numpy(c).cuda().view(n, k // 2), torch.from_numpy(s).cuda().view(n, k // 16), s2, n, k)
    for x_t, x_host in ((dev_bf16(xb).view(m, k), bf16_bits_to_f32(xb)), (torch.from_numpy(x32).cuda().view(m, k), x32)):
        got = ink.linear_w(x_t, ink.ProjW("fp4", w))
        ac, asc = orc.quantize_act_recip(x_host, m, k)
        ref = orc.linear_w4a4(ac, asc, c, s, np.float32(s2), m, n, k)
        assert got.dtype == torch.float32
        # the reference's same-operand gate: <= 1e-4 relative (src/bin/inkling_fp4_expert_gate.rs:16-28)
        assert np.abs(got.cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()
    got = ink.linear_w(torch.from_numpy(x32).cuda().view(m, k), ink.ProjW("w4a16", w))
    ref = orc.linear_w4a16(xb, c, s, s2, m, n, k)
    assert np.abs(got.cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()
    got = ink.linear_w(dev_bf16(xb).view(m, k), ink.ProjW("bf16", dev_bf16(wb).view(n, k)))
    assert np.abs(got.cpu().numpy() - orc.linear_bf16(xb, wb, m, n, k)).max() <= 1e-4 * np.abs(ref).max()


def test_calibrated_planes_upload_and_project(mods, orc):
    """A linear packed by the calibrated packer (src/calibrate.rs:351-434) reaches the device as any stored NVFP4
    leaf does (payload -> Nvfp4::upload); the consumer applies 1 / s to the activation's columns."""
    _, _, nv, _ = mods
    from maryml_b200 import calibrate as cal
    n, k, m = 64, 128, 24
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    xs = rng.standard_normal((96, k)).astype(np.float32)
    xs[:, 3 * k // 4:] *= 8.0
    c = cal.pack_linear(w, k, xs, np.abs(xs).mean(0).astype(np.float32))
    assert c.error_ratio <= 1.0
    q = nv.Nvfp4.upload(c.packed.payload(), [n, k], torch.bfloat16, torch.device("cuda", 0))
    xb = f32_to_bf16_bits((xs[:m] * c.input_scale[None, :]).astype(np.float32))
    ref = bf16_bits_to_f32(xb).reshape(m, k).astype(np.float64) @ c.packed.decode().astype(np.float64).T
    for lane in (nv.PromptLane.W4A16,):
        y = q.project(dev_bf16(xb).view(1, m, k), lane)
        rel, cos = rel_check(bf16_bits_to_f32(host_bits(y)).reshape(m, n), ref)
        assert rel <= 1e-2 and cos >= 0.9999, (rel, cos)
    # and it tracks the unquantized layer better than plain rounding does on the same rows
    plain = cal.pack_nearest(w, k)
    assert cal.output_error(w, c.decode(), k, xs) <= cal.output_error(w, plain.decode(), k, xs)


def test_swiglu_epilogue_refuses_a_width_it_would_truncate(mods, orc):
    _, _, nv, _lib = mods
    m, n, k = 16, 24, 64
    z = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.MaryError):
        nv.gemm_w4a4(z, z, z, z, 1.0, m, n, k, epilogue=_lib.EPI_SWIGLU_INTERLEAVED)


# ------------------------------------------------------------------- a bounded wait on a peer that never answers
def test_wait_on_an_absent_peer_runs_out_and_the_context_stays_usable(mods, orc):
    """The fused exchange waits on flags its peers write. Here rank 0 of a world of two is attached to a second
    LOCAL buffer standing in for a peer that never runs: the wait gives up after the context's wait limit, the
    kernel ends, the status words say which wait, how long and for whom, and the next step works once the
    stand-in's flags are written by hand. Nothing faults, nothing spins beyond the limit."""
    _, _, nv, _lib = mods
    lib, ctx = _lib.lib, _lib.context(0)
    t, n, k = 64, 4096, 512
    assert lib.mb_tp_symm_destroy(ctx.handle) == 0
    handle = (C.c_uint8 * 64)()
    ctx.check(lib.mb_tp_symm_create(ctx.handle, t, n, handle))
    try:
        local = C.c_void_p()
        ctx.check(lib.mb_tp_symm_local(ctx.handle, C.byref(local)))
        nbytes = int(lib.mb_tp_symm_bytes(t, n))
        standin = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        peers = (C.c_void_p * 2)(local, standin.data_ptr())
        ctx.check(lib.mb_tp_symm_attach_ptrs(ctx.handle, peers, 0, 2))
        ctx.check(lib.mb_ctx_set_wait_limit_us(ctx.handle, 2000))
        wq = nv.Nvfp4.quantize(dev_bf16(f32_to_bf16_bits(orc.normal_f32(81, n * k, 0.02))).view(n, k))
        x = dev_bf16(f32_to_bf16_bits(orc.normal_f32(82, t * k, 1.0))).view(t, k)
        resid = dev_bf16(f32_to_bf16_bits(orc.normal_f32(83, t * n, 1.0))).view(t, n)
        codes, sf, _ = nv.quantize_act(x, _lib.QUANT_SCALED, 1.0, tiled=True)
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

        def step(s):
            ctx.check(lib.mb_nvfp4_gemm_w4a4_scatter(ctx.handle, stream, codes.data_ptr(), sf.data_ptr(), wq.codes.data_ptr(),
                                                     wq.sf_tiled().data_ptr(), wq.scale2, t, n, k, s))
            out = C.c_void_p()
            ctx.check(lib.mb_tp_reduce_residual(ctx.handle, stream, resid.data_ptr(), t, n, s, C.byref(out)))
            return out.value

        step(1)
        rc, flags = ctx.check_flags(None)
        assert rc == _lib.ERR_DEVICE_FLAG and flags[0] == 51, flags      # the wait for a peer's partials
        assert 1500 <= flags[3] <= 200000 and flags[4] == 1, flags       # microseconds waited, rank waited for
        # the peer "answers": its two flags of step 2 written by hand; its receive slot holds zeros
        from maryml_b200.layer import _wrap_bf16
        words = _wrap_bf16(local.value, 1, 256, torch.device("cuda", 0)).view(torch.int32).view(-1)   # the 128 flag words
        words[1] = 2
        words[65] = 2
        torch.cuda.synchronize()
        ptr = step(2)
        rc, flags = ctx.check_flags(None)
        assert rc == 0, flags
        got = _wrap_bf16(ptr, t, n, torch.device("cuda", 0))[:, : n // 2].float()
        partial = nv.gemm_w4a4(codes, sf, wq.codes, wq.sf_tiled(), wq.scale2, t, n, k, out_dtype=torch.float32)
        want = (resid.float() + partial.to(torch.bfloat16).float()).to(torch.bfloat16).float()[:, : n // 2]
        assert torch.equal(got, want)
    finally:
        lib.mb_ctx_set_wait_limit_us(ctx.handle, 1000000)
        lib.mb_tp_symm_destroy(ctx.handle)


def test_prompt_exchanges_give_up_on_an_absent_peer_and_work_once_it_answers(mods):
    """The prompt path's reduce-scatter and all-gather kernels (mb_tp_bulk_*) wait on flags their peers write. Rank 0
    of a world of two is attached to a second LOCAL buffer standing in for a peer that never runs: each kernel gives
    up after the context's wait limit with its own status code and ends; once the stand-in's flags are written by
    hand (its partial holds a known pattern) the same calls complete and the sums are exact."""
    _, _, _, _lib = mods
    from maryml_b200.layer import _DevBuf
    lib, ctx = _lib.lib, _lib.context(0)
    dev = torch.device("cuda", 0)
    rows, n = 256, 1024
    user = 2 * rows * n * 4
    hdr = int(lib.mb_tp_bulk_header_bytes())
    assert lib.mb_tp_bulk_destroy(ctx.handle) == 0
    handle = (C.c_uint8 * 64)()
    ctx.check(lib.mb_tp_bulk_create(ctx.handle, user, handle))
    try:
        region, mine = C.c_void_p(), C.c_void_p()
        ctx.check(lib.mb_tp_bulk_local(ctx.handle, C.byref(region), C.byref(mine)))
        standin = torch.zeros(hdr + user, dtype=torch.uint8, device=dev)
        peers = (C.c_void_p * 2)(region, standin.data_ptr())
        ctx.check(lib.mb_tp_bulk_attach_ptrs(ctx.handle, peers, 0, 2))
        ctx.check(lib.mb_ctx_set_wait_limit_us(ctx.handle, 2000))
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        my_partial = torch.as_tensor(_DevBuf(mine.value, (rows, n), "<f4"), device=dev)
        my_partial.copy_(torch.arange(rows * n, dtype=torch.float32, device=dev).view(rows, n) % 1024)
        peer_partial = standin[hdr:hdr + rows * n * 4].view(torch.float32).view(rows, n)
        peer_partial.fill_(0.25)
        out = torch.full((rows // 2, n), -1.0, device=dev)
        ctx.check(lib.mb_tp_bulk_reduce_scatter_f32(ctx.handle, stream, 0, rows, n, out.data_ptr(), 1))
        rc, flags = ctx.check_flags(None)
        assert rc == _lib.ERR_DEVICE_FLAG and flags[0] == 54 and flags[4] == 1, flags
        assert bool((out == -1.0).all())                                   # nothing was summed
        ctx.check(lib.mb_tp_bulk_all_gather(ctx.handle, stream, rows * n * 4, 4096, 0, 0, 1))
        rc, flags = ctx.check_flags(None)
        assert rc == _lib.ERR_DEVICE_FLAG and flags[0] == 55 and flags[4] == 1, flags
        # the peer "answers": its flag words of step 2 (reduce-scatter word 1, all-gather word 33) written by hand
        words = torch.as_tensor(_DevBuf(region.value, (hdr // 4,), "<i4"), device=dev)
        words[1] = 2
        words[33] = 2
        torch.cuda.synchronize()
        ctx.check(lib.mb_tp_bulk_reduce_scatter_f32(ctx.handle, stream, 0, rows, n, out.data_ptr(), 2))
        ctx.check(lib.mb_tp_bulk_all_gather(ctx.handle, stream, rows * n * 4, 4096, 0, 0, 2))
        rc, flags = ctx.check_flags(None)
        assert rc == 0, flags
        assert torch.equal(out, my_partial[: rows // 2] + 0.25)            # rank 0's rows: its own partial plus the peer's
        # the all-gather pushed this rank's slice into the stand-in's copy of the buffer
        src = torch.as_tensor(_DevBuf(mine.value + rows * n * 4, (4096,), "|u1"), device=dev)
        assert torch.equal(standin[hdr + rows * n * 4: hdr + rows * n * 4 + 4096], src)
    finally:
        lib.mb_ctx_set_wait_limit_us(ctx.handle, 1000000)
        lib.mb_tp_bulk_destroy(ctx.handle)
