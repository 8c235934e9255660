"""The oracle's codec against the reference's own known-answer tests.

Each test restates one in-source test of the reference (cited by file:line, paths
relative to the reference root) on the oracle's functions. These pin the oracle;
the CUDA kernels are then checked against the oracle.
"""
import numpy as np
import pytest

E4M3_MAX_BYTE = 0x7E


def e4m3_search(orc, v):
    """Nearest pattern, ties to the even one: the search of src/nvfp4.rs:313-330."""
    v = np.float32(v)
    if not (v > 0):
        return 0
    if v >= 448.0:
        return E4M3_MAX_BYTE
    best, best_err = 0, float("inf")
    for b in range(E4M3_MAX_BYTE + 1):
        err = abs(float(orc.e4m3_to_f32(b)) - float(v))
        if err < best_err or (err == best_err and b & 1 == 0):
            best, best_err = b, err
    return best


def test_arithmetic_e4m3_is_the_nearest_pattern_everywhere(orc):
    # src/nvfp4.rs:333-353
    probes = [0.0, 1e-30, 2.0 ** -10, 2.0 ** -9, 447.9, 448.0, 1e9]
    for b in range(E4M3_MAX_BYTE + 1):
        lo = np.float32(orc.e4m3_to_f32(b))
        probes.append(lo)
        if b < E4M3_MAX_BYTE:
            mid = np.float32((float(lo) + float(orc.e4m3_to_f32(b + 1))) / 2.0)
            bits = mid.view(np.uint32)
            probes += [mid, np.uint32(bits - 1).view(np.float32), np.uint32(bits + 1).view(np.float32)]
    v = np.float32(2.0 ** -12)
    while v < 460.0:
        probes.append(v)
        v = np.float32(v * np.float32(1.0007))
    for v in probes:
        assert orc.e4m3_from_f32(v) == e4m3_search(orc, v), f"{float(v):e}"


def test_every_finite_e4m3_pattern_round_trips(orc):
    # src/nvfp4.rs:356-362
    for b in range(1, E4M3_MAX_BYTE + 1):
        assert orc.e4m3_from_f32(orc.e4m3_to_f32(b)) == b
    assert orc.e4m3_from_f32(0.0) == 0
    assert orc.e4m3_to_f32(E4M3_MAX_BYTE) == 448.0
    assert np.isnan(orc.e4m3_to_f32(0x7F))


def test_e4m3_saturates_and_ties_to_even(orc):
    # src/nvfp4.rs:365-371
    assert orc.e4m3_from_f32(1000.0) == E4M3_MAX_BYTE
    assert orc.e4m3_from_f32(1.0625) == 0x38
    assert orc.e4m3_from_f32(1.1875) == 0x3A
    assert orc.e4m3_from_f32(1.1) == 0x39


def test_e2m1_ties_go_to_the_even_code_and_saturate(orc):
    # src/nvfp4.rs:374-383
    assert orc.e2m1_code(0.25) == 0
    assert orc.e2m1_code(1.25) == 2
    assert orc.e2m1_code(2.5) == 4
    assert orc.e2m1_code(5.0) == 6
    assert orc.e2m1_code(0.75) == 2
    assert orc.e2m1_code(9.0) == 7
    assert orc.code_of(-3.1, 1.0) == 8 | 5
    assert orc.code_of(-0.0, 1.0) == 8


def test_sixteen_codes_and_values(orc):
    # src/models/inkling/fp4quant.rs:552-569: the 16 codes <-> values incl. -0.0
    mags = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for c in range(16):
        v = orc.decode_code(c)
        assert abs(v) == mags[c & 7]
        assert np.signbit(np.float32(v)) == bool(c & 8)
        assert orc.lib.orc_cvt_e2m1(v) == c


def test_pack_then_decode_is_the_reference_arithmetic(orc):
    # src/nvfp4.rs:396-414
    rows, cols = 5, 48
    w = orc.sample(rows, cols)
    codes, scales, scale2 = orc.pack_nearest(w, cols)
    dec = orc.decode_payload(orc.payload(codes, scales, scale2), rows * cols)
    assert scale2 == orc.global_scale(w)
    for blk in range(rows * cols // 16):
        block = w[blk * 16:(blk + 1) * 16]
        byte, unit = orc.block_unit(block, scale2)
        assert scales[blk] == byte
        for i, v in enumerate(block):
            want = np.float32(np.float32(orc.decode_code(orc.code_of(v, unit))) * unit)
            assert dec[blk * 16 + i] == want
            assert abs(dec[blk * 16 + i] - v) <= unit + 1e-6 or abs(v) > 6.0 * unit


def test_payload_round_trips_and_the_flat_decoder_agrees(orc):
    # src/nvfp4.rs:417-426
    rows, cols = 3, 64
    w = orc.sample(rows, cols)
    codes, scales, scale2 = orc.pack_nearest(w, cols)
    payload = orc.payload(codes, scales, scale2)
    assert payload.size == orc.lib.orc_payload_len(rows * cols) == rows * cols // 2 + rows * cols // 16 + 4
    assert np.array_equal(payload[:codes.size], codes)
    assert np.array_equal(payload[codes.size:codes.size + scales.size], scales)
    assert payload[-4:].tobytes() == np.float32(scale2).tobytes()
    assert np.array_equal(orc.decode_payload(payload, rows * cols), orc.dequantize(codes, scales, scale2))
    with pytest.raises(ValueError):
        orc.decode_payload(payload[:-1], rows * cols)


def test_the_lower_index_is_the_low_nibble(orc):
    # src/nvfp4.rs:446-455
    block = np.zeros(16, np.float32)
    block[0], block[1] = 6.0, -1.0
    codes, scales, scale2 = orc.pack_nearest(block, 16)
    assert codes[0] == 0x07 | (0x0A << 4)
    dec = orc.dequantize(codes, scales, scale2)
    assert dec[0] == 6.0 and dec[1] == -1.0


def test_a_zero_block_and_a_zero_tensor_decode_to_zero(orc):
    # src/nvfp4.rs:458-462
    codes, scales, scale2 = orc.pack_nearest(np.zeros(32, np.float32), 32)
    assert scale2 == 1.0
    assert np.all(orc.dequantize(codes, scales, scale2) == 0.0)
    assert np.all(codes == 0) and np.all(scales == 0)


def test_recipe_inverts_on_representable_blocks(orc):
    # src/nn/nvfp4_gemv.rs:753-767: 2688 -> scale2 1.0, E4M3 1.0 = 0x38, all 8 magnitudes invert
    from oracle_lib import f32_to_bf16_bits
    w = np.zeros(32, np.float32)
    w[0] = 2688.0
    w[16:24] = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    codes, scales, s2 = orc.quantize_weight_bf16(f32_to_bf16_bits(w), 1, 32)
    assert s2 == 1.0
    assert scales[0] == 0x7E and scales[1] == 0x38
    dec = orc.dequantize(codes, scales, s2)
    assert np.array_equal(dec[16:24], w[16:24])
    assert dec[0] == 2688.0


def test_device_recipe_equals_host_packing(orc):
    # src/nn/nvfp4_gemv.rs:468-501 (`pack_matching`): quantize_block == pack_nearest, bit for bit,
    # including on the adversarial fixture of :726-738 (ties, tiny blocks, signed zeros).
    from oracle_lib import f32_to_bf16_bits, bf16_bits_to_f32
    n, k = 8, 128
    w = orc.normal_f32(0xF160FF4, n * k, 0.5)
    w[0] = 2688.0
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], np.float32)
    small = orc.normal_f32(0x0F169E77, 2 * k, 1.0)
    for i in range(k):
        sign = -1.0 if i % 3 == 0 else 1.0
        w[k + i] = sign * ties[i % 8]
        w[2 * k + i] = small[i] * 1e-3
        w[3 * k + i] = small[k + i] * 1e-6
        w[4 * k + i] = -0.0 if i % 2 == 0 else 0.0
    bits = f32_to_bf16_bits(w)
    wide = bf16_bits_to_f32(bits)
    c1, s1, g1 = orc.quantize_weight_bf16(bits, n, k)
    c2, s2, g2 = orc.pack_nearest(wide, k)
    assert g1.tobytes() == g2.tobytes()
    assert np.array_equal(c1, c2) and np.array_equal(s1, s2)
    # -0.0 keeps its sign as code 8 under a live unit; the zero row's blocks flush to +0 codes
    assert np.all(c1[4 * k // 2:5 * k // 2] == 0)


def test_non_finite_weight_is_refused(orc):
    # src/nn/nvfp4_gemv.rs:101-117, :593-600
    from oracle_lib import f32_to_bf16_bits
    w = np.ones(32, np.float32)
    w[5] = np.nan
    with pytest.raises(ValueError):
        orc.quantize_weight_bf16(f32_to_bf16_bits(w), 1, 32)
    w[5] = np.inf
    with pytest.raises(ValueError):
        orc.quantize_weight_bf16(f32_to_bf16_bits(w), 1, 32)


def test_activation_recipes_differ_only_where_stated(orc):
    # K2 with input_scale 1 divides; fp4quant multiplies by a rounded reciprocal
    # (src/models/inkling/fp4quant.rs:199-238). Scales agree; codes agree except near ties.
    x = orc.normal_f32(7, 64 * 256, 1.0)
    c_div, s_div = orc.quantize_act_scaled(x, 64, 256, 1.0)
    c_rec, s_rec = orc.quantize_act_recip(x, 64, 256)
    assert np.array_equal(s_div, s_rec)
    assert np.mean(c_div != c_rec) < 1e-3


def test_row_scale_recipe(orc):
    # src/nn/nvfp4_gemm.rs:757-796: amax/2688, 1.0 for a zero row, NaN for a NaN row
    x = orc.normal_f32(11, 4 * 64, 1.0).reshape(4, 64)
    x[1] = 0.0
    x[2, 7] = np.nan
    codes, scales, rs = orc.quantize_act_rows(x, 4, 64)
    assert rs[0] == np.float32(np.abs(x[0]).max() / np.float32(2688.0))
    assert rs[1] == 1.0
    assert np.isnan(rs[2])
    # the largest block of a live row lands on E4M3's top code
    assert scales.reshape(4, 4)[0].max() == 0x7E
