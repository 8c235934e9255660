"""GPU parity tests of the NVFP4 codec, GEMV and tensor-core GEMMs against the CPU oracle.

Bit-exact for codes, scale bytes, scale2 and dequantised values; floating outputs
within the stated tolerances. Every call goes through the C ABI (ctypes).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle_lib import bf16_bits_to_f32, f32_to_bf16_bits  # noqa: E402


@pytest.fixture(scope="module")
def mb():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import maryml_b200
    from maryml_b200 import nvfp4
    return nvfp4


def dev_bf16(bits):
    return torch.from_numpy(np.ascontiguousarray(bits, np.uint16).view(np.int16)).cuda().view(torch.bfloat16)


def host_bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def adversarial(orc, n, k):
    """The fixture of src/nn/nvfp4_gemv.rs:726-738 on bf16."""
    w = orc.normal_f32(0xF160FF4, n * k, 0.5)
    w[0] = 2688.0
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], np.float32)
    small = orc.normal_f32(0x0F169E77, 2 * k, 1.0)
    for i in range(k):
        w[k + i] = (-1.0 if i % 3 == 0 else 1.0) * ties[i % 8]
        w[2 * k + i] = small[i] * 1e-3
        w[3 * k + i] = small[k + i] * 1e-6
        w[4 * k + i] = -0.0 if i % 2 == 0 else 0.0
    return f32_to_bf16_bits(w)


def rel_check(got, ref, max_rel=1e-2, cos_min=0.9999):
    """north_star tolerance: max relative error <= 1e-2 (relative to max(|ref|, 1/64 of the
    reference rms, so that cancelled sums do not divide by ~0), cosine >= 0.9999."""
    got = np.asarray(got, np.float64).ravel()
    ref = np.asarray(ref, np.float64).ravel()
    rms = np.sqrt(np.mean(ref ** 2)) + 1e-30
    rel = np.abs(got - ref) / np.maximum(np.abs(ref), rms / 64 + 1e-30)
    # bf16 outputs carry a 2^-9 rounding of their own
    cos = float(np.dot(got, ref) / (np.linalg.norm(got) * np.linalg.norm(ref) + 1e-30))
    return float(rel.max()), cos


def attn_check(got, ref, d=128):
    """The attention bound, per output vector (one query row of one head, `d` values): every element within 1e-2
    of max(|ref|, rms of its own vector), cosine >= 0.9999 overall. The probabilities enter the second product as
    bf16 (f16 over NVFP4 rows), which puts an absolute error of about 2^-9 of the VECTOR's magnitude on each of
    its elements, so an element far below its vector's rms cannot meet a bound relative to itself; and vectors of
    one call differ widely in magnitude (a causal row that sees three keys against one that sees thousands), so
    the rms is taken per vector, not per call."""
    got = np.asarray(got, np.float64).reshape(-1, d)
    ref = np.asarray(ref, np.float64).reshape(-1, d)
    rms = np.sqrt(np.mean(ref ** 2, axis=1, keepdims=True)) + 1e-30
    rel = np.abs(got - ref) / np.maximum(np.abs(ref), rms)
    cos = float(np.dot(got.ravel(), ref.ravel()) / (np.linalg.norm(got) * np.linalg.norm(ref) + 1e-30))
    return float(rel.max()), cos


# --------------------------------------------------------------------------- codec
@pytest.mark.parametrize("n,k", [(8, 128), (64, 4096), (33, 96)])
def test_weight_quantizer_bit_exact(mb, orc, n, k):
    bits = adversarial(orc, n, k) if n >= 8 and k >= 96 else f32_to_bf16_bits(orc.normal_f32(3, n * k, 0.02))
    w = dev_bf16(bits).view(n, k)
    q = mb.Nvfp4.quantize(w)
    codes, scales = q.read_planes()
    c_ref, s_ref, g_ref = orc.quantize_weight_bf16(bits, n, k)
    assert np.float32(q.scale2).tobytes() == g_ref.tobytes()
    assert np.array_equal(scales, s_ref)
    assert np.array_equal(codes, c_ref)
    # pack_matching (src/nn/nvfp4_gemv.rs:468-501): the host packing equals the device planes
    c_host, s_host, g_host = orc.pack_nearest(bf16_bits_to_f32(bits), k)
    assert np.array_equal(codes, c_host) and np.array_equal(scales, s_host) and g_host.tobytes() == g_ref.tobytes()
    # dequantised values bit-exact
    dq = mb.dequantize(q.codes, q.scales, q.scale2, n, k).cpu().numpy().ravel()
    assert np.array_equal(dq.view(np.uint32), orc.dequantize(c_ref, s_ref, g_ref).view(np.uint32))


def test_weight_quantizer_refuses_non_finite_and_zero_tensor(mb, orc):
    from maryml_b200 import MaryError
    w = torch.ones(4, 64, dtype=torch.bfloat16, device="cuda")
    w[1, 3] = float("nan")
    with pytest.raises(MaryError):
        mb.Nvfp4.quantize(w)
    w[1, 3] = float("inf")
    with pytest.raises(MaryError):
        mb.Nvfp4.quantize(w)
    z = mb.Nvfp4.quantize(torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda"))
    assert z.scale2 == 1.0
    codes, scales = z.read_planes()
    assert not codes.any() and not scales.any()


def test_upload_round_trip_and_refusals(mb, orc):
    from maryml_b200 import MaryError
    n, k = 16, 64
    w = orc.normal_f32(5, n * k, 0.02)
    codes, scales, s2 = orc.pack_nearest(w, k)
    payload = orc.payload(codes, scales, s2)
    q = mb.Nvfp4.upload(payload, [n, k], torch.bfloat16, torch.device("cuda", 0))
    assert np.array_equal(q.payload(), payload)
    with pytest.raises(MaryError):
        mb.Nvfp4.upload(payload[:-1], [n, k], torch.bfloat16, torch.device("cuda", 0))
    with pytest.raises(MaryError):
        mb.Nvfp4.upload(payload, [n, k + 16], torch.bfloat16, torch.device("cuda", 0))
    bad = payload.copy()
    bad[-4:] = np.frombuffer(np.float32(-1.0).tobytes(), np.uint8)
    with pytest.raises(MaryError):
        mb.Nvfp4.upload(bad, [n, k], torch.bfloat16, torch.device("cuda", 0))


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("rows,k", [(1, 64), (37, 256), (130, 2048), (5, 48), (7, 96), (300, 14336)])
def test_activation_quantizers_bit_exact(mb, orc, dtype, rows, k):
    from maryml_b200 import _lib
    x32 = orc.normal_f32(100 + rows, rows * k, 1.0)
    x32[: min(k, 16)] = 0.0  # a zero block
    x32[16 + 5::29] = -0.0   # negative zeros inside live blocks: their codes keep the sign (src/nvfp4.rs:117-126)
    x32[16 + 9::31] = 0.0
    if rows > 2:
        x32[k:2 * k] *= 1e-4  # a row deep in the subnormal scale range
    if dtype == "bf16":
        bits = f32_to_bf16_bits(x32)
        x = dev_bf16(bits).view(rows, k)
        wide = bf16_bits_to_f32(bits)
    else:
        x = torch.from_numpy(x32).cuda().view(rows, k)
        wide = x32
    for recipe, ref in [
        (_lib.QUANT_SCALED, lambda: orc.quantize_act_scaled(wide, rows, k, 1.0)),
        (_lib.QUANT_RECIP, lambda: orc.quantize_act_recip(wide, rows, k)),
    ]:
        c_ref, s_ref = ref()
        for tiled in (False, True):
            codes, scales, _ = mb.quantize_act(x, recipe, 1.0, tiled=tiled)
            if tiled:
                scales = mb.untile_scales(scales, rows, k)
            assert np.array_equal(codes.cpu().numpy().ravel(), c_ref), (recipe, tiled)
            assert np.array_equal(scales.cpu().numpy().ravel(), s_ref), (recipe, tiled)
    # calibrated input scale
    c_ref, s_ref = orc.quantize_act_scaled(wide, rows, k, 0.0123)
    codes, scales, _ = mb.quantize_act(x, _lib.QUANT_SCALED, 0.0123, tiled=False)
    assert np.array_equal(codes.cpu().numpy().ravel(), c_ref) and np.array_equal(scales.cpu().numpy().ravel(), s_ref)
    # per-row scale
    c_ref, s_ref, rs_ref = orc.quantize_act_rows(wide, rows, k)
    codes, scales, rs = mb.quantize_act(x, _lib.QUANT_ROWS, 1.0, tiled=False)
    assert np.array_equal(rs.cpu().numpy().view(np.uint32), rs_ref.view(np.uint32))
    assert np.array_equal(codes.cpu().numpy().ravel(), c_ref) and np.array_equal(scales.cpu().numpy().ravel(), s_ref)


def test_quantize_gather_and_nan_row(mb, orc):
    from maryml_b200 import _lib
    rows, k = 12, 128
    x32 = orc.normal_f32(9, rows * k, 1.0).reshape(rows, k)
    x32[5, 17] = np.nan
    x = torch.from_numpy(x32).cuda()
    gather = torch.tensor([3, -1, 0, 11, 5], dtype=torch.int32, device="cuda")
    codes, scales, rs = mb.quantize_act(x, _lib.QUANT_ROWS, 1.0, tiled=False, gather=gather)
    src = np.stack([x32[3], np.zeros(k, np.float32), x32[0], x32[11], x32[5]])
    c_ref, s_ref, rs_ref = orc.quantize_act_rows(src, 5, k)
    assert np.isnan(rs.cpu().numpy()[4]) and rs.cpu().numpy()[1] == 1.0
    assert np.array_equal(rs.cpu().numpy()[:4].view(np.uint32), rs_ref[:4].view(np.uint32))
    assert np.array_equal(codes.cpu().numpy().ravel(), c_ref) and np.array_equal(scales.cpu().numpy().ravel(), s_ref)


def test_scale_tiling_is_a_bijection(mb, orc):
    rows, k = 200, 576
    s = torch.randint(0, 127, (rows, k // 16), dtype=torch.uint8, device="cuda")
    t = mb.tile_scales(s, rows, k)
    assert t.numel() == 2 * 3 * 4 * 512
    assert torch.equal(mb.untile_scales(t, rows, k), s)
    # atom-internal offset (row%32)*16 + (row/32%4)*4 + kb%4, atoms [row/128][kb/4]
    th = t.cpu().numpy()
    sh = s.cpu().numpy()
    for (r, kb) in [(0, 0), (31, 3), (32, 0), (127, 35), (128, 4), (199, 35)]:
        off = ((r // 128) * 12 + kb // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + kb % 4
        assert th[off] == sh[r, kb]


# --------------------------------------------------------------------------- GEMV
@pytest.mark.parametrize("form", ["one kernel", "two pass"])
@pytest.mark.parametrize("n,k", [(512, 4096), (200, 96), (33, 4128), (1024, 14336)])
@pytest.mark.parametrize("rows", [1, 3, 8])
def test_gemv_w4a16_against_f64(mb, orc, rows, n, k, form, monkeypatch):
    """(200, 96) and (33, 4128): output rows that do not fill a 16-row block, K that does not fill a 128-value slice;
    (1024, 14336): K ranges (a cluster per 16-row block in the one-kernel form, workspace sums in the two-pass form)."""
    monkeypatch.setenv("MB_GEMV_TWO_PASS", "1" if form == "two pass" else "0")
    wbits = f32_to_bf16_bits(orc.normal_f32(0x0F16CAFE, n * k, 0.02))
    xbits = f32_to_bf16_bits(orc.normal_f32(21 + rows, rows * k, 1.0))
    q = mb.Nvfp4.quantize(dev_bf16(wbits).view(n, k))
    x = dev_bf16(xbits).view(1, rows, k)
    assert q.takes(x) == rows
    y = q.gemv(x, rows)
    codes, scales = q.read_planes()
    ref = orc.linear_w4a16(xbits, codes, scales, q.scale2, rows, n, k)
    got = bf16_bits_to_f32(host_bits(y)).reshape(rows, n).astype(np.float64)
    # the reference's own bound (src/nn/nvfp4_gemv.rs:890-905): f32 accumulation error below
    # 64 eps * sum|x w|, and the output within half a bf16 ulp of that
    dq = orc.dequantize(codes, scales, q.scale2).reshape(n, k).astype(np.float64)
    xa = np.abs(bf16_bits_to_f32(xbits).reshape(rows, k).astype(np.float64))
    bound = 64 * 2.0 ** -24 * (xa @ np.abs(dq).T) + np.abs(ref) * 2.0 ** -8 + 1e-30
    assert np.all(np.abs(got - ref) <= bound)


def test_gemv_takes_the_bf16_form_when_a_value_does_not_fit_f16(mb, orc, monkeypatch):
    """The two-pass GEMV multiplies an f16 copy of the activation rows when that copy is exact; one value outside f16's normal
    range (70000, 1e30, 1e-30 and a bf16 subnormal; 1e30 times a decoded weight still fits the f32 accumulator, which
    the reference scales by scale2 only at the end) sends the whole call through the bf16 product.
    Both forms stay inside the reference's bound, and with the plain entry point (no workspace) they agree to f32
    summation order."""
    import ctypes as C
    from maryml_b200 import _lib
    monkeypatch.setenv("MB_GEMV_TWO_PASS", "1")
    n, k, rows = 272, 4096, 4
    wbits = f32_to_bf16_bits(orc.normal_f32(0x0F16CAFE, n * k, 0.02))
    q = mb.Nvfp4.quantize(dev_bf16(wbits).view(n, k))
    codes, scales = q.read_planes()
    dq = np.abs(orc.dequantize(codes, scales, q.scale2).reshape(n, k).astype(np.float64))
    for poke in (None, 70000.0, 1.0e30, 1.0e-30, 9.2e-41, float("inf")):
        x32 = orc.normal_f32(77, rows * k, 1.0)
        if poke is not None:
            x32[k + 5] = poke
        xbits = f32_to_bf16_bits(x32)
        x = dev_bf16(xbits).view(1, rows, k)
        y = q.gemv(x, rows)
        ref = orc.linear_w4a16(xbits, codes, scales, q.scale2, rows, n, k)
        got = bf16_bits_to_f32(host_bits(y)).reshape(rows, n).astype(np.float64)
        xa = np.abs(bf16_bits_to_f32(xbits).reshape(rows, k).astype(np.float64))
        with np.errstate(all="ignore"):
            bound = 64 * 2.0 ** -24 * (xa @ dq.T) + np.abs(ref) * 2.0 ** -8 + 1e-30
        fin = np.isfinite(ref)
        assert np.all(np.abs(got - ref)[fin] <= bound[fin]), poke
        assert np.array_equal(np.isfinite(got), fin)
        # the entry point without a workspace is the one-kernel form on the bf16 rows
        ctx = _lib.context(0)
        plain = torch.empty_like(y)
        ctx.check(_lib.lib.mb_nvfp4_gemv_w4a16(ctx.handle, None, C.c_void_p(x.data_ptr()), rows, C.c_void_p(q.codes.data_ptr()),
                                               C.c_void_p(q.scales.data_ptr()), q.scale2, n, k, C.c_void_p(plain.data_ptr()),
                                               _lib.DT_BF16))
        torch.cuda.synchronize()
        a, b = y.float(), plain.float()
        ok = torch.isfinite(b)
        assert bool(((a - b).abs()[ok] <= 2.0 ** -7 * b.abs()[ok] + 1e-6).all()), poke


def test_takes_refuses_what_the_reference_refuses(mb, orc):
    q = mb.Nvfp4.quantize(torch.randn(64, 128, device="cuda").to(torch.bfloat16))
    assert q.takes(torch.zeros(1, 9, 128, dtype=torch.bfloat16, device="cuda")) is None
    assert q.takes(torch.zeros(1, 2, 64, dtype=torch.bfloat16, device="cuda")) is None
    assert q.takes(torch.zeros(1, 2, 128, dtype=torch.float32, device="cuda")) is None
    assert q.takes(torch.zeros(2, 2, 128, dtype=torch.bfloat16, device="cuda")) is None
    assert q.takes(torch.zeros(1, 2, 256, dtype=torch.bfloat16, device="cuda")[:, :, ::2]) is None


# --------------------------------------------------------------------------- tensor-core GEMM
def _pow2_planes(orc, rng, rows, k):
    """Random codes with power-of-two block scales: every partial sum is exact in f32."""
    codes = rng.integers(0, 256, size=rows * k // 2, dtype=np.uint8)
    scales = rng.choice(np.array([0x30, 0x38, 0x40], np.uint8), size=rows * k // 16)
    return codes, scales


@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (128, 256, 256), (128, 128, 1024), (256, 512, 1024),
                                   (100, 136, 320), (300, 768, 448), (640, 1024, 1024)])
def test_gemm_w4a4_exact_on_power_of_two_scales(mb, orc, m, n, k):
    """One-hot/pow2 probe in the spirit of src/bin/nvfp4_mma_probe.rs:32-58: with exactly
    representable partial sums the tensor-core result must equal the oracle to the bit, which
    pins the operand, scale-factor and accumulator layouts."""
    rng = np.random.default_rng(m * 131 + n * 17 + k)
    a_codes, a_scales = _pow2_planes(orc, rng, m, k)
    b_codes, b_scales = _pow2_planes(orc, rng, n, k)
    ref = orc.linear_w4a4(a_codes, a_scales, b_codes, b_scales, 1.0, m, n, k)
    ac = torch.from_numpy(a_codes).cuda()
    bc = torch.from_numpy(b_codes).cuda()
    asf = mb.tile_scales(torch.from_numpy(a_scales).cuda(), m, k)
    bsf = mb.tile_scales(torch.from_numpy(b_scales).cuda(), n, k)
    out = mb.gemm_w4a4(ac, asf, bc, bsf, 1.0, m, n, k, out_dtype=torch.float32)
    got = out.cpu().numpy()
    assert np.array_equal(got, ref), f"max abs err {np.abs(got - ref).max()}"


@pytest.mark.parametrize("m,n,k", [(16, 4096, 4096), (64, 512, 7168), (100, 1280, 2048), (1, 256, 2816),
                                   (128, 384, 2816)])
def test_gemm_w4a4_split_k_exact_and_ordered(mb, orc, m, n, k):
    """Decode-sized products are cut along K into f32 planes and summed in slice order. With
    power-of-two scales every partial sum is exact, so the split result equals the oracle to the
    bit (f32 output) and the unsplit entry point to the bit (bf16 output with a row scale)."""
    from maryml_b200 import _lib
    need = int(_lib.lib.mb_nvfp4_gemm_splitk_workspace(m, n, k))
    assert need > 0 and need % (m * n * 4) == 0
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a_codes, a_scales = _pow2_planes(orc, rng, m, k)
    b_codes, b_scales = _pow2_planes(orc, rng, n, k)
    ref = orc.linear_w4a4(a_codes, a_scales, b_codes, b_scales, 1.0, m, n, k)
    ac = torch.from_numpy(a_codes).cuda()
    bc = torch.from_numpy(b_codes).cuda()
    asf = mb.tile_scales(torch.from_numpy(a_scales).cuda(), m, k)
    bsf = mb.tile_scales(torch.from_numpy(b_scales).cuda(), n, k)
    got = mb.gemm_w4a4(ac, asf, bc, bsf, 1.0, m, n, k, out_dtype=torch.float32).cpu().numpy()
    assert np.array_equal(got, ref), f"max abs err {np.abs(got - ref).max()}"
    # bf16 + row scale, twice (the workspace is reused), against the single-pass kernel
    rowscale = torch.from_numpy(rng.choice(np.array([0.5, 1.0, 2.0], np.float32), size=m)).cuda()
    ctx = _lib.context(0)
    plain = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ctx.check(_lib.lib.mb_nvfp4_gemm_w4a4(ctx.handle, None, ac.data_ptr(), asf.data_ptr(), bc.data_ptr(), bsf.data_ptr(),
                                          rowscale.data_ptr(), 0.25, m, n, k, plain.data_ptr(), _lib.DT_BF16,
                                          _lib.EPI_PLAIN))
    for _ in range(2):
        split = mb.gemm_w4a4(ac, asf, bc, bsf, 0.25, m, n, k, rowscale=rowscale)
        assert torch.equal(split.view(torch.int16), plain.view(torch.int16))
    # a short workspace falls back to the single pass instead of overrunning it
    short = torch.empty(16, dtype=torch.uint8, device="cuda")
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ctx.check(_lib.lib.mb_nvfp4_gemm_w4a4_splitk(ctx.handle, None, ac.data_ptr(), asf.data_ptr(), bc.data_ptr(),
                                                 bsf.data_ptr(), rowscale.data_ptr(), 0.25, m, n, k, out.data_ptr(),
                                                 _lib.DT_BF16, short.data_ptr(), 16))
    assert torch.equal(out.view(torch.int16), plain.view(torch.int16))


@pytest.mark.parametrize("m,n,k", [(16, 4096, 4096), (128, 256, 4096), (1000, 1280, 2048)])
def test_project_w4a4_against_same_operand_f64(mb, orc, m, n, k):
    wbits = f32_to_bf16_bits(orc.normal_f32(2, n * k, 0.02))
    xbits = f32_to_bf16_bits(orc.normal_f32(1, m * k, 1.0))
    q = mb.Nvfp4.quantize(dev_bf16(wbits).view(n, k))
    x = dev_bf16(xbits).view(1, m, k)
    y = q.project(x, mb.PromptLane.W4A4)
    assert tuple(y.shape) == (1, m, n)
    # oracle: the same quantised operands, f64 accumulation, one rounding
    a_codes, a_scales = orc.quantize_act_scaled(bf16_bits_to_f32(xbits), m, k, 1.0)
    codes, scales = q.read_planes()
    ref = orc.linear_w4a4(a_codes, a_scales, codes, scales, np.float32(q.scale2), m, n, k)
    got = bf16_bits_to_f32(host_bits(y)).reshape(m, n)
    rel, cos = rel_check(got, ref)
    assert rel <= 1e-2 and cos >= 0.9999, (rel, cos)
    # f32 output: the reference's own gate is 1e-4 relative vs f64 of the same operands
    # (src/bin/inkling_fp4_expert_gate.rs:16-28)
    a_c, a_sf, _ = mb.quantize_act(x.view(m, k), tiled=True)
    out32 = mb.gemm_w4a4(a_c, a_sf, q.codes, q.sf_tiled(), q.scale2, m, n, k, out_dtype=torch.float32).cpu().numpy()
    scale = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    assert np.abs(out32 - ref).max() <= 1e-4 * scale * 8


def test_project_w4a4_rows_and_scaled(mb, orc):
    m, n, k = 150, 512, 1024
    wbits = f32_to_bf16_bits(orc.normal_f32(12, n * k, 0.02))
    x32 = orc.normal_f32(13, m * k, 1.0).reshape(m, k)
    x32[7] *= 1e-3
    x32[9] = 0.0
    xbits = f32_to_bf16_bits(x32)
    q = mb.Nvfp4.quantize(dev_bf16(wbits).view(n, k))
    x = dev_bf16(xbits).view(1, m, k)
    codes, scales = q.read_planes()
    wide = bf16_bits_to_f32(xbits)
    # rows lane
    y = q.project_w4a4_rows(x)
    a_codes, a_scales, rs = orc.quantize_act_rows(wide, m, k)
    ref = orc.linear_w4a4(a_codes, a_scales, codes, scales, np.float32(q.scale2), m, n, k, rowscale=rs)
    got = bf16_bits_to_f32(host_bits(y)).reshape(m, n)
    rel, cos = rel_check(got, ref)
    assert rel <= 1e-2 and cos >= 0.9999, (rel, cos)
    assert not got[9].any()
    # calibrated global
    y = q.project_w4a4_scaled(x, 0.05)
    a_codes, a_scales = orc.quantize_act_scaled(wide, m, k, 0.05)
    alpha = np.float32(np.float32(q.scale2) * np.float32(0.05))
    ref = orc.linear_w4a4(a_codes, a_scales, codes, scales, alpha, m, n, k)
    rel, cos = rel_check(bf16_bits_to_f32(host_bits(y)).reshape(m, n), ref)
    assert rel <= 1e-2 and cos >= 0.9999, (rel, cos)
    from maryml_b200 import MaryError
    with pytest.raises(MaryError):
        q.project_w4a4_scaled(x, float("nan"))
    with pytest.raises(MaryError):
        q.project_w4a4_scaled(x, 0.0)


def test_w4a4_rows_nan_row_poisons_only_itself(mb, orc):
    # src/nn/nvfp4_gemm.rs:1123-1166
    m, n, k = 40, 256, 256
    w = torch.randn(n, k, device="cuda").to(torch.bfloat16) * 0.02
    q = mb.Nvfp4.quantize(w)
    x = torch.randn(1, m, k, device="cuda").to(torch.bfloat16)
    clean = q.project_w4a4_rows(x).clone()
    x2 = x.clone()
    x2[0, 17, 5] = float("nan")
    dirty = q.project_w4a4_rows(x2)
    assert torch.isnan(dirty[0, 17]).all()
    keep = [i for i in range(m) if i != 17]
    assert torch.equal(dirty[0, keep].view(torch.int16), clean[0, keep].view(torch.int16))


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (200, 264, 1032), (512, 1024, 2048), (512, 128, 2048), (100, 128, 1096),
                                   (300, 512, 192), (1024, 768, 4096), (2304, 256, 64), (2900, 2048, 128), (5000, 1024, 320)])
def test_bf16_gemm_against_f64(mb, orc, m, n, k):
    """(512, 128, 2048) and (100, 128, 1096) have few output tiles and a long K: they run as K slices (split-K).
    Shapes with n % 256 == 0, k % 64 == 0 and at least 74 tiles of 256 x 256 run on CTA pairs: (2900, 2048, 128)
    leaves the last row pair 84 rows (its second CTA none), (5000, 1024, 320) leaves the last pair's second CTA eight
    rows and has five K steps; (300, 512, 192), (1024, 768, 4096) and (2304, 256, 64) stay on the single-CTA kernel."""
    abits = f32_to_bf16_bits(orc.normal_f32(31, m * k, 1.0))
    bbits = f32_to_bf16_bits(orc.normal_f32(32, n * k, 0.02))
    ref = orc.linear_bf16(abits, bbits, m, n, k)
    out = mb.bf16_gemm(dev_bf16(abits).view(m, k), dev_bf16(bbits).view(n, k), out_dtype=torch.float32).cpu().numpy()
    scale = np.sqrt(np.mean(ref.astype(np.float64) ** 2))
    assert np.abs(out - ref).max() <= 2e-5 * scale * np.sqrt(k / 64)
    rel, cos = rel_check(out, ref)
    assert rel <= 1e-2 and cos >= 0.9999
    # the bf16 output is the f32 one rounded once
    out16 = mb.bf16_gemm(dev_bf16(abits).view(m, k), dev_bf16(bbits).view(n, k), out_dtype=torch.bfloat16)
    assert torch.equal(out16.cpu().view(torch.int16), torch.from_numpy(out).to(torch.bfloat16).view(torch.int16))


def test_project_w4a16_and_linear_dispatch(mb, orc):
    m, n, k = 41, 512, 1024
    wbits = f32_to_bf16_bits(orc.normal_f32(41, n * k, 0.02))
    xbits = f32_to_bf16_bits(orc.normal_f32(42, m * k, 1.0))
    q = mb.Nvfp4.quantize(dev_bf16(wbits).view(n, k))
    x = dev_bf16(xbits).view(1, m, k)
    y = mb.linear(x, q)  # 41 rows -> prompt lane, default W4A16
    codes, scales = q.read_planes()
    ref = orc.linear_w4a16(xbits, codes, scales, q.scale2, m, n, k)
    got = bf16_bits_to_f32(host_bits(y)).reshape(m, n)
    # the reference's bound for this lane: relative rms below 4e-3 (src/models/breeze/nvfp4.rs:339-380)
    assert np.sqrt(np.mean((got - ref) ** 2)) / np.sqrt(np.mean(ref ** 2)) < 4e-3
    y8 = mb.linear(x[:, :8].contiguous(), q)  # 8 rows -> the GEMV
    assert np.sqrt(np.mean((bf16_bits_to_f32(host_bits(y8)).reshape(8, n) - ref[:8]) ** 2)) / np.sqrt(np.mean(ref[:8] ** 2)) < 4e-3


def test_full_size_linearity_property(mb, orc):
    """At the benchmark's full shape the oracle is too slow; the size-independent property is
    linearity in the weight's global scale and agreement of the W4A4 lane with the dequantised
    bf16 tensor-core product of the same quantised operands."""
    m, n, k = 1024, 4096, 4096
    w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    q = mb.Nvfp4.quantize(w)
    a_c, a_sf, _ = mb.quantize_act(x, tiled=True)
    y1 = mb.gemm_w4a4(a_c, a_sf, q.codes, q.sf_tiled(), q.scale2, m, n, k, out_dtype=torch.float32)
    y2 = mb.gemm_w4a4(a_c, a_sf, q.codes, q.sf_tiled(), 2.0 * q.scale2, m, n, k, out_dtype=torch.float32)
    assert torch.equal(y2, 2.0 * y1)
    a_sf_rm = mb.untile_scales(a_sf, m, k)
    xa = mb.dequantize(a_c, a_sf_rm, 1.0, m, k, dtype=torch.bfloat16)
    wb = mb.dequantize(q.codes, q.scales, 1.0, n, k, dtype=torch.bfloat16)
    y3 = mb.bf16_gemm(xa, wb, out_dtype=torch.float32, alpha=q.scale2)
    err = (y1 - y3).abs().max().item()
    assert err <= 1e-4 * y3.abs().max().item() + 1e-6


@pytest.mark.parametrize("k,n", [(4096, 4096), (4096, 14336), (14336, 4096)])
def test_config1_full_shapes_against_the_oracle_at_128_rows(mb, orc, figures, k, n):
    """The three projection shapes of the sweep at their full (K, N), 128 activation rows: quantizer bytes and
    the three lanes (W4A4, W4A4 per-row scale, W4A16) compared directly with the CPU restatement."""
    m = 128
    wb = f32_to_bf16_bits(orc.normal_f32(2, n * k, 0.02))
    xb = f32_to_bf16_bits(orc.normal_f32(1, m * k, 1.0))
    q = mb.Nvfp4.quantize(dev_bf16(wb).view(n, k))
    codes, scales = q.read_planes()
    c_ref, s_ref, g_ref = orc.quantize_weight_bf16(wb, n, k)
    assert np.array_equal(codes, c_ref) and np.array_equal(scales, s_ref) and np.float32(q.scale2) == g_ref
    x = dev_bf16(xb).view(1, m, k)
    xf = bf16_bits_to_f32(xb)
    # W4A4, unit input scale: against f64 sums of the SAME quantized operands (reference gate 1e-4 on f32 output)
    a_c, a_s = orc.quantize_act_scaled(xf, m, k, 1.0)
    ref = orc.linear_w4a4(a_c, a_s, c_ref, s_ref, g_ref, m, n, k)
    d_c, d_sf, _ = mb.quantize_act(x.view(m, k), tiled=True)
    assert np.array_equal(d_c.cpu().numpy().ravel(), a_c)
    y32 = mb.gemm_w4a4(d_c, d_sf, q.codes, q.sf_tiled(), q.scale2, m, n, k, out_dtype=torch.float32).cpu().numpy()
    e_w4a4 = np.abs(y32 - ref).max() / np.abs(ref).max()
    assert e_w4a4 <= 1e-4, e_w4a4
    y = bf16_bits_to_f32(host_bits(q.project(x, mb.PromptLane.W4A4))).reshape(m, n)
    rel, cos = rel_check(y, ref)
    assert rel <= 1e-2 and cos >= 0.9999, (rel, cos)
    # per-row activation scale
    r_c, r_s, r_rs = orc.quantize_act_rows(xf, m, k)
    ref_rows = orc.linear_w4a4(r_c, r_s, c_ref, s_ref, g_ref, m, n, k, rowscale=r_rs)
    rel_r, cos_r = rel_check(bf16_bits_to_f32(host_bits(q.project_w4a4_rows(x))).reshape(m, n), ref_rows)
    assert rel_r <= 1e-2 and cos_r >= 0.9999, (rel_r, cos_r)
    # W4A16: exact weights, bf16 activations
    ref16 = orc.linear_w4a16(xb, c_ref, s_ref, g_ref, m, n, k)
    rel_16, cos_16 = rel_check(bf16_bits_to_f32(host_bits(q.project(x, mb.PromptLane.W4A16))).reshape(m, n), ref16)
    assert rel_16 <= 1e-2 and cos_16 >= 0.9999, (rel_16, cos_16)
    figures("config1_m128", k=k, n=n, w4a4_f32_rel=e_w4a4, w4a4_bf16_rel=rel, rows_rel=rel_r, w4a16_rel=rel_16)


def test_mxfp4_relabelled_as_nvfp4_decodes_to_the_same_bits(mb, orc):
    """transcode_to_nvfp4 (src/nn/mxfp4.rs:319-375) on the device: scale bytes equal the CPU relabelling, and the
    NVFP4 decode of (same codes, new scales, 2^g) equals the MXFP4 decode bit for bit."""
    nv = mb
    from maryml_b200 import _lib
    rows, cols = 96, 256
    rng = np.random.default_rng(4)
    packed = rng.integers(0, 256, rows * cols // 2, dtype=np.uint8)
    exps = rng.integers(-15, -4, rows * cols // 32)              # an 11-octave span like the reference's checkpoint
    exps[:18] = np.arange(-20, -2)                                # and the full 18-octave window somewhere
    scale = (exps + 127).astype(np.uint8)
    pd, sd = torch.from_numpy(packed).cuda(), torch.from_numpy(scale).cuda()
    codes, bs, gscale, gexp = nv.mxfp4_to_nvfp4(pd, sd, rows, cols)
    bs_ref, g_ref, _ = orc.mxfp4_transcode(scale)
    assert codes.data_ptr() == pd.data_ptr()                      # the codes are borrowed, not rebuilt
    assert gexp == g_ref == int(exps.max()) - 8 and gscale == 2.0 ** g_ref
    assert np.array_equal(bs.cpu().numpy().ravel(), bs_ref)
    back = nv.dequantize(codes.view(rows, cols // 2), bs, gscale, rows, cols).cpu().numpy().ravel()
    want = orc.mxfp4_decode(packed, scale, rows, cols)
    assert np.array_equal(back.view(np.uint32), want.view(np.uint32))
    # refusals: a 19-octave span, a NaN scale (the first index is named)
    wide = scale.copy()
    wide[5] = np.uint8(127 - 21)                                   # exponents now run -21 .. -3
    with pytest.raises(_lib.MaryError, match="span 19 octaves"):
        nv.mxfp4_to_nvfp4(pd, torch.from_numpy(wide).cuda(), rows, cols)
    bad = scale.copy()
    bad[[7, 300]] = 0xFF
    with pytest.raises(_lib.MaryError, match=r"scale\[7\] is NaN"):
        nv.mxfp4_to_nvfp4(pd, torch.from_numpy(bad).cuda(), rows, cols)


def _splitk_plan(operands, m, n, k):
    import ctypes as C
    from maryml_b200 import _lib
    cs, ps = C.c_int(), C.c_int()
    ctx = _lib.context(0)
    ctx.check(_lib.lib.mb_gemm_splitk_plan(ctx.handle, operands, m, n, k, C.byref(cs), C.byref(ps)))
    return cs.value, ps.value


@pytest.mark.parametrize("m,n,k", [(64, 6144, 4096), (64, 4096, 14336), (16, 14336, 4096), (128, 4096, 4096), (1, 1024, 2048),
                                   (37, 1280, 2048), (64, 1000, 4096), (5, 2056, 3072)])
def test_split_k_in_a_cluster_gives_the_bits_of_the_summed_planes(mb, m, n, k, monkeypatch):
    """The K slices of a decode-sized product meet either in distributed shared memory (one cluster per output tile)
    or as f32 planes summed by a second kernel; both add the slices in slice order, so the results are the same
    bits for ordinary (inexact) operands, for f32 and bf16 outputs, with a row scale and with per-column scales."""
    from maryml_b200 import _lib
    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    q = mb.Nvfp4.quantize(w)
    ac, asf, _ = mb.quantize_act(x, tiled=True)
    rowscale = (torch.rand(m, device="cuda", generator=g) + 0.5).float()
    stacked = mb.Stacked([q, q]) if n <= 6144 and n % 128 == 0 else None

    def run():
        outs = [mb.gemm_w4a4(ac, asf, q.codes, q.sf_tiled(), q.scale2, m, n, k, out_dtype=torch.float32),
                mb.gemm_w4a4(ac, asf, q.codes, q.sf_tiled(), 0.37, m, n, k, rowscale=rowscale)]
        if stacked is not None:
            outs.append(mb.gemm_w4a4_stacked(ac, asf, stacked, m))
        torch.cuda.synchronize()
        return outs

    assert int(_lib.lib.mb_nvfp4_gemm_splitk_workspace(m, n, k)) > 0
    monkeypatch.setenv("MB_SPLITK_CLUSTER", "0")
    planes = run()
    monkeypatch.setenv("MB_SPLITK_CLUSTER", "1")
    cs, ps = _splitk_plan(0, m, n, k)
    assert ps > 1 and (cs == 0 or 2 <= cs <= 8)
    cluster = run()
    again = run()
    for a, b, c in zip(planes, cluster, again):
        if cs == ps or cs == 0:      # the same slices in the same order: the same bits
            assert torch.equal(a.view(torch.int32 if a.dtype == torch.float32 else torch.int16),
                               b.view(torch.int32 if b.dtype == torch.float32 else torch.int16))
        else:                        # fewer, longer slices: f32 sums associated differently
            d = (a.float() - b.float()).abs().max().item()
            assert d <= 2e-2 * a.float().abs().max().item() * (2.0 ** -7 if a.dtype == torch.bfloat16 else 2.0 ** -12), d
        assert torch.equal(b, c)
    assert _lib.context(0).check_flags(None)[0] == 0


@pytest.mark.parametrize("m,n,k", [(4096, 128, 2048), (32, 256, 4096), (300, 128, 1024)])
def test_bf16_split_k_in_a_cluster_gives_the_bits_of_the_summed_planes(mb, m, n, k, monkeypatch):
    from maryml_b200 import _lib
    g = torch.Generator(device="cuda").manual_seed(m * 3 + n + k)
    a = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    assert int(_lib.lib.mb_bf16_gemm_splitk_workspace(m, n, k)) > 0
    monkeypatch.setenv("MB_SPLITK_CLUSTER", "0")
    planes = [mb.bf16_gemm(a, b, out_dtype=torch.float32), mb.bf16_gemm(a, b, out_dtype=torch.bfloat16, alpha=0.5)]
    monkeypatch.setenv("MB_SPLITK_CLUSTER", "1")
    cs, ps = _splitk_plan(1, m, n, k)
    cluster = [mb.bf16_gemm(a, b, out_dtype=torch.float32), mb.bf16_gemm(a, b, out_dtype=torch.bfloat16, alpha=0.5)]
    torch.cuda.synchronize()
    if cs == ps or cs == 0:
        assert torch.equal(planes[0], cluster[0]) and torch.equal(planes[1], cluster[1])
    ref = a.float() @ b.float().T
    assert (planes[0] - ref).abs().max() <= 2e-3 * ref.abs().max()
    assert (cluster[0] - ref).abs().max() <= 2e-3 * ref.abs().max()
    assert _lib.context(0).check_flags(None)[0] == 0


@pytest.mark.parametrize("m,n,k", [(16, 4096, 4096), (128, 4096, 14336), (100, 2048, 8192), (64, 1000, 4096)])
def test_w4a16_split_k_in_a_cluster_gives_the_bits_of_the_summed_planes(mb, m, n, k, monkeypatch):
    """The W4A16 prompt kernel cuts K the same way; its slices are the same in both forms, so the bits are too."""
    from maryml_b200 import _lib
    g = torch.Generator(device="cuda").manual_seed(m + 2 * n + k)
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    q = mb.Nvfp4.quantize(w)
    assert int(_lib.lib.mb_nvfp4_gemm_w4a16_workspace(m, n, k)) > 0
    outs = {}
    for form in ("0", "1"):
        monkeypatch.setenv("MB_SPLITK_CLUSTER", form)
        outs[form] = [mb.w4a16_gemm(x, q.codes, q.scales, q.scale2, n, k),
                      mb.w4a16_gemm(x, q.codes, q.scales, q.scale2, n, k, out_dtype=torch.float32)]
    torch.cuda.synchronize()
    assert torch.equal(outs["0"][0], outs["1"][0]) and torch.equal(outs["0"][1], outs["1"][1])
    ref = x.float() @ mb.dequantize(q.codes, q.scales, q.scale2, n, k).float().T
    assert (outs["1"][1] - ref).abs().max() <= 2e-3 * ref.abs().max()
    assert _lib.context(0).check_flags(None)[0] == 0
