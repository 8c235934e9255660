"""The calibrated packers (AWQ channel scales, GPTQ error feedback) against the reference's own tests
(src/calibrate.rs:436-522, restated with its deterministic generators) and the host codec they are built on
against the oracle's restatement of src/nvfp4.rs, bit for bit."""
import numpy as np
import pytest

from maryml_b200 import calibrate as cal


def matrix(rows, cols):
    """src/calibrate.rs:440-449: column j carries a magnitude that grows with j."""
    i = np.arange(rows * cols)
    x = ((i * 7919) % 1000).astype(np.float32) / np.float32(1000.0) - np.float32(0.5)
    return (x * (np.float32(1.0) + (i % cols).astype(np.float32) / np.float32(cols))).astype(np.float32)


def inputs(n, cols):
    """src/calibrate.rs:451-463: the last quarter of the channels is busy."""
    r, j = np.meshgrid(np.arange(n), np.arange(cols), indexing="ij")
    x = ((r * 131 + j * 17) % 997).astype(np.float32) / np.float32(997.0) - np.float32(0.5)
    return np.where(j >= 3 * cols // 4, x * np.float32(8.0), x).astype(np.float32)


def mean_abs(rows):
    return (np.abs(rows).sum(0, dtype=np.float32) / np.float32(rows.shape[0])).astype(np.float32)


def test_host_codec_is_the_oracles_codec(orc):
    # every E4M3 pattern, every midpoint between neighbours and one ulp either side, a dense sweep (src/nvfp4.rs:333-353)
    vals = [orc.e4m3_to_f32(b) for b in range(0x7F)]
    probes = list(vals)
    for a, b in zip(vals[:-1], vals[1:]):
        mid = np.float32((np.float64(a) + np.float64(b)) / 2)
        probes += [mid, np.nextafter(mid, np.float32(0)), np.nextafter(mid, np.float32(1e9))]
    probes += list(np.exp(np.linspace(np.log(2.0 ** -12), np.log(460.0), 4000)).astype(np.float32))
    probes = np.array(probes, np.float32)
    got = cal.e4m3_from_f32(probes)
    assert np.array_equal(got, np.array([orc.e4m3_from_f32(v) for v in probes], np.uint8))
    assert np.array_equal(cal.e4m3_to_f32(np.arange(0x7F, dtype=np.uint8)).view(np.uint32), np.array(vals, np.float32).view(np.uint32))
    # E2M1 ties and signs (src/nvfp4.rs:374-383)
    for m, c in [(0.25, 0), (1.25, 2), (2.5, 4), (5.0, 6), (0.75, 2), (9.0, 7)]:
        assert int(cal.e2m1_code(np.float32(m))) == c == orc.e2m1_code(m)
    assert int(cal.code_of(np.float32(-3.1), np.float32(1.0))) == (8 | 5) == orc.code_of(-3.1, 1.0)
    assert int(cal.code_of(np.float32(-0.0), np.float32(1.0))) == 8 and int(cal.code_of(np.float32(2.0), np.float32(0.0))) == 0
    # whole tensors: the reference's sample generator, the adversarial magnitudes, an all-zero tensor
    for rows, cols in [(7, 64), (33, 256)]:
        w = orc.sample(rows, cols)
        w[3] = -0.0
        p = cal.pack_nearest(w, cols)
        c, s, g = orc.pack_nearest(w, cols)
        assert np.array_equal(p.codes.ravel(), c) and np.array_equal(p.scales.ravel(), s) and p.scale2.tobytes() == g.tobytes()
        assert np.array_equal(p.decode().ravel().view(np.uint32), orc.dequantize(c, s, g).view(np.uint32))
        assert np.array_equal(p.payload(), orc.payload(c, s, g))
    z = cal.pack_nearest(np.zeros(64, np.float32), 16)
    assert z.scale2 == 1.0 and not z.codes.any() and not z.scales.any()
    with pytest.raises(ValueError):
        cal.pack_nearest(np.zeros(60, np.float32), 24)


def test_calibration_never_loses_to_plain_rounding():
    rows, cols = 8, 64
    w, x = matrix(rows, cols), inputs(64, cols)
    c = cal.pack_linear(w, cols, x, mean_abs(x))
    assert c.error_ratio <= 1.0, c.error_ratio
    assert c.input_scale.size == cols and c.decode().size == rows * cols
    # alpha zero alone and no feedback is plain rounding
    p = cal.pack_linear(w, cols, x, mean_abs(x), alphas=(0.0,), feedback=False)
    assert p.error_ratio == 1.0 and p.alpha == 0.0 and not p.feedback_used and np.all(p.input_scale == 1.0)


def test_feedback_alone_beats_nearest_on_correlated_inputs():
    rows, cols = 4, 32
    w, x = matrix(rows, cols), inputs(48, cols)
    plain = cal.pack_nearest(w, cols)
    fed = cal.pack_gptq(w, cols, x)
    e_plain = cal.output_error(w, plain.decode(), cols, x)
    e_fed = cal.output_error(w, fed.decode(), cols, x)
    assert e_fed <= e_plain, (e_fed, e_plain)
    assert fed.scale2 == plain.scale2          # the global scale is the tensor's, not the feedback's
    with pytest.raises(ValueError):
        cal.pack_gptq(w, cols, np.zeros((0, cols), np.float32))


def test_decode_folds_the_input_scale_into_the_columns():
    cols = 16
    packed = cal.pack_nearest(np.ones(cols, np.float32), cols)
    c = cal.Calibrated(packed, np.arange(cols, dtype=np.float32), alpha=0.5)
    assert np.array_equal(c.decode().ravel(), np.arange(cols, dtype=np.float32))


def test_channel_scales_have_geometric_mean_one():
    m = np.abs(np.random.default_rng(0).standard_normal(256)).astype(np.float32) + np.float32(0.01)
    assert np.all(cal.channel_scales(m, 0.0) == 1.0)
    s = cal.channel_scales(m, 0.5)
    assert abs(float(np.exp(np.mean(np.log(s.astype(np.float64))))) - 1.0) < 1e-5
    assert np.argmax(s) == np.argmax(m)
