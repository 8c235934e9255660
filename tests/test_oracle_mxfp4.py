"""The oracle's MXFP4 -> NVFP4 relabelling against the reference's own known-answer tests
(src/nn/mxfp4.rs:405-563). CPU only."""
import numpy as np
import pytest

MX_BLOCK = 32


def _synthetic(exps):
    # mxfp4.rs:473-481: code bytes i % 256, one scale byte per 32 values
    packed = (np.arange(len(exps) * MX_BLOCK // 2) % 256).astype(np.uint8)
    scale = (np.asarray(exps) + 127).astype(np.uint8)
    return packed, scale


def test_e4m3_pow2_window_and_known_bytes(orc):
    # e4m3_pow2_window_is_18_octaves, e4m3_from_pow2_emits_known_bytes, e4m3_known_encodings
    f = orc.lib.orc_e4m3_from_pow2
    exact = [e for e in range(-30, 31) if f(e) >= 0 and orc.e4m3_to_f32(f(e)) == 2.0 ** e]
    assert exact[0] == -9 and exact[-1] == 8 and len(exact) == 18
    assert f(0) == 0x38 and f(8) == 0x78 and f(-9) == 0x01 and f(-6) == 0x08 and f(9) < 0 and f(-10) < 0
    assert all(f(e) & 0x80 == 0 for e in range(-9, 9))
    assert orc.e4m3_to_f32(0x38) == 1.0 and orc.e4m3_to_f32(0x78) == 256.0 and orc.e4m3_to_f32(0x7E) == 448.0
    assert orc.e4m3_to_f32(0x01) == 1.0 / 512.0 and np.isnan(orc.e4m3_to_f32(0x7F)) and np.isnan(orc.e4m3_to_f32(0xFF))


def test_e8m0_is_the_f32_exponent_field(orc):
    one = np.zeros(16, np.uint8)      # code 0 everywhere except element 0 = 1.0 (code 2)
    one[0] = 0x02
    val = lambda b: float(orc.mxfp4_decode(one, np.array([b], np.uint8), 1, 32)[0])
    tiny = float(np.finfo(np.float32).tiny)
    assert val(127) == 1.0 and val(122) == 0.03125 and val(112) == 3.0517578125e-05
    assert val(1) == tiny and val(0) * 2.0 == tiny and val(254) == 2.0 ** 127
    assert np.isnan(val(0xFF))


def test_transcode_is_bit_exact_across_the_whole_window(orc):
    exps = list(range(-9, 9))         # 18 octaves, the maximum
    packed, scale = _synthetic(exps)
    rows, cols = len(exps), MX_BLOCK
    mx = orc.mxfp4_decode(packed, scale, rows, cols)
    block_scale, g, sub = orc.mxfp4_transcode(scale)
    assert g == 0 and sub
    back = orc.dequantize(packed, block_scale, 2.0 ** g)
    assert np.array_equal(mx.view(np.uint32), back.view(np.uint32))
    assert np.array_equal(block_scale[0::2], block_scale[1::2])


def test_transcode_refuses_a_19_octave_span_and_nan(orc):
    _, scale = _synthetic(list(range(-9, 10)))
    with pytest.raises(ValueError, match="ExponentSpan e_min -9 e_max 9 octaves 19"):
        orc.mxfp4_transcode(scale)
    with pytest.raises(ValueError, match="ScaleNan index 2"):
        orc.mxfp4_transcode(np.array([127, 120, 0xFF, 0xFF], np.uint8))


def test_a_kimi_shaped_span_stays_in_e4m3_normals(orc):
    _, scale = _synthetic(list(range(-15, -4)))
    _, g, sub = orc.mxfp4_transcode(scale)
    assert g == -13 and not sub


def test_negative_zero_survives_the_decode(orc):
    out = orc.mxfp4_decode(np.full(16, 0x80, np.uint8), np.array([122], np.uint8), 1, 32)
    assert out[0].view(np.uint32) == 0 and out[1].view(np.uint32) == 0x80000000
