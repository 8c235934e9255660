"""Activation-aware NVFP4 packing of one linear layer: AWQ channel scales and GPTQ error feedback.

Host-side weight preprocessing, done once per model, as in the reference (src/calibrate.rs:1-34 says why it is
host code by design): `output_error` (:106-135), `pack_gptq` (:212-321), `channel_scales` / `scale_columns`
(:324-345), `pack_linear` (:351-434) and `Calibrated` (:67-101). The codes, block scales and global scale follow
the scalar codec rules of src/nvfp4.rs:52-150, restated here on numpy arrays in f32 (one rounding per operation,
as the reference's f32 arithmetic has); the decoded planes upload unchanged through `Nvfp4.from_parts`.

The channel scale cannot live inside the codes (it is per input column, the codes are per element under a
per-block scale), so a calibrated linear is the codes of W * diag(s) plus the vector 1 / s applied to the input.
"""
import numpy as np

BLOCK = 16
E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)
_MIDPOINTS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], np.float32)
AWQ_ALPHAS = (0.0, 0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9)
_f32 = np.float32


# ---- scalar codec on arrays (src/nvfp4.rs:52-150) ----------------------------------------------------
def e4m3_to_f32(b):
    b = np.asarray(b, np.uint8).astype(np.int32)
    exp, man = (b >> 3) & 0xF, b & 7
    sub = man.astype(np.float32) * _f32(2.0 ** -9)
    nor = np.ldexp((8 + man).astype(np.float32), exp - 10).astype(np.float32)
    mag = np.where(exp == 0, sub, nor).astype(np.float32)
    mag = np.where((exp == 15) & (man == 7), _f32(np.nan), mag)
    return np.where(b & 0x80, -mag, mag).astype(np.float32)


def e4m3_from_f32(v):
    """Nearest E4M3 pattern of a non-negative value, ties to the even significand, saturating at 448."""
    v = np.asarray(v, np.float32)
    pos = v > 0
    vv = np.where(pos, v, _f32(1.0))
    e = np.maximum(((vv.view(np.uint32) >> 23) & 0xFF).astype(np.int32) - 127, -6)
    steps = np.rint(np.ldexp(vv, 3 - e)).astype(np.int64)           # the scaling is exact; rint ties to even
    carry = steps == 16
    byte = np.where((e == -6) & (steps < 8), steps, ((np.where(carry, e + 1, e) + 7) << 3) | np.where(carry, 0, steps - 8))
    byte = np.minimum(byte, 0x7E)
    byte = np.where(v >= _f32(448.0), 0x7E, byte)
    return np.where(pos, byte, 0).astype(np.uint8)


def e2m1_code(m):
    """Nearest E2M1 code of a magnitude in E2M1 units, an exact midpoint to the even code, saturating at 6."""
    m = np.asarray(m, np.float32)
    code = np.zeros(m.shape, np.uint8)
    for i, mid in enumerate(_MIDPOINTS):
        take = (m > mid) | ((m == mid) & ((i + 1) % 2 == 0))
        code = np.where(take, np.uint8(i + 1), code)
    return np.where(np.isnan(m), np.uint8(7), code).astype(np.uint8)


def code_of(v, unit):
    """Signed code of v at `unit` per E2M1 step; a zero unit codes every value as +0; a zero keeps its sign."""
    v = np.asarray(v, np.float32)
    unit = np.broadcast_to(np.asarray(unit, np.float32), v.shape)
    sign = np.where(np.signbit(v), np.uint8(8), np.uint8(0))
    with np.errstate(all="ignore"):
        mag = e2m1_code((np.abs(v) / np.where(unit > 0, unit, _f32(1.0))).astype(np.float32))
    code = np.where((v == 0) | np.isnan(v), sign, mag | sign)
    return np.where(unit > 0, code, np.uint8(0)).astype(np.uint8)


def decode_code(code):
    code = np.asarray(code, np.uint8)
    m = E2M1[code & 7]
    return np.where(code & 8, -m, m).astype(np.float32)


def global_scale(w):
    absmax = _f32(np.max(np.abs(np.asarray(w, np.float32)))) if np.size(w) else _f32(0.0)
    if absmax > 0 and np.isfinite(absmax):
        return _f32(absmax / _f32(6.0 * 448.0))
    return _f32(1.0)


def block_unit(blocks, scale2):
    """blocks [..., 16] -> (scale bytes, value of one E2M1 step) per block."""
    bmax = np.max(np.abs(np.asarray(blocks, np.float32)), axis=-1)
    with np.errstate(all="ignore"):
        t = np.minimum(((bmax / _f32(6.0)).astype(np.float32) / _f32(scale2)).astype(np.float32), _f32(448.0))
    byte = e4m3_from_f32(t)
    return byte, (e4m3_to_f32(byte) * _f32(scale2)).astype(np.float32)


class Packed:
    """Packed (src/nvfp4.rs:186-230): codes [rows, cols/2] (lower index in the LOW nibble), scales [rows, cols/16],
    one f32 scale2."""

    def __init__(self, rows, cols, codes, scales, scale2):
        self.rows, self.cols, self.codes, self.scales, self.scale2 = rows, cols, codes, scales, _f32(scale2)

    def decode(self):
        unit = (e4m3_to_f32(self.scales) * self.scale2).astype(np.float32).reshape(self.rows, self.cols // BLOCK, 1)
        c = self.codes.reshape(self.rows, self.cols // 2)
        codes = np.stack([c & 0xF, c >> 4], -1).reshape(self.rows, self.cols // BLOCK, BLOCK)
        return (decode_code(codes) * unit).astype(np.float32).reshape(self.rows, self.cols)

    def payload(self):
        return np.concatenate([self.codes.ravel(), self.scales.ravel(), np.frombuffer(self.scale2.tobytes(), np.uint8)])


def _pack_codes(codes):
    """[rows, cols] nibbles -> [rows, cols/2] bytes, the lower index in the low nibble."""
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)


def pack_nearest(w, cols):
    """pack_nearest (src/nvfp4.rs:268-305): nearest rounding under the tensor's own global scale."""
    if cols <= 0 or cols % BLOCK != 0:
        raise ValueError(f"cols {cols} is not a positive multiple of {BLOCK}")
    w = np.ascontiguousarray(w, np.float32).reshape(-1)
    if w.size % cols != 0:
        raise ValueError(f"{w.size} values do not fill rows of {cols}")
    rows = w.size // cols
    scale2 = global_scale(w)
    blocks = w.reshape(rows, cols // BLOCK, BLOCK)
    byte, unit = block_unit(blocks, scale2)
    codes = code_of(blocks, unit[..., None]).reshape(rows, cols)
    return Packed(rows, cols, _pack_codes(codes), byte.reshape(rows, cols // BLOCK), scale2)


# ---- calibration (src/calibrate.rs) --------------------------------------------------------------------
def output_error(w, wq, cols, rows):
    """sum over input rows of |(W - Wq) x|^2, the quantity AWQ minimises (src/calibrate.rs:106-135): each dot
    product is carried in f32, squared and summed in f64."""
    diff = (np.asarray(w, np.float32).reshape(-1, cols) - np.asarray(wq, np.float32).reshape(-1, cols)).astype(np.float32)
    x = np.asarray(rows, np.float32).reshape(-1, cols)
    acc = (x @ diff.T).astype(np.float32)
    return float(np.sum(acc.astype(np.float64) ** 2))


def pack_gptq(w, cols, x):
    """Error-feedback (GPTQ) NVFP4 of w [rows, cols] against input rows x [R, cols], under one global scale from
    w's own maximum (src/calibrate.rs:212-321): H = X^T X / R damped by one percent of its mean diagonal,
    U = chol(H^-1)^T; the columns are rounded left to right and each column's rounding error is pushed onto the
    columns still to come through row j of U; a block's scale is fixed when its first column is reached, from
    the values the feedback has left there."""
    if cols <= 0 or cols % BLOCK != 0:
        raise ValueError(f"cols {cols} is not a positive multiple of {BLOCK}")
    w = np.ascontiguousarray(w, np.float32).reshape(-1)
    if w.size % cols != 0:
        raise ValueError(f"{w.size} values do not fill rows of {cols}")
    x = np.asarray(x, np.float32).reshape(-1, cols)
    if x.shape[0] == 0:
        raise ValueError("error feedback needs input rows")
    rows, n = w.size // cols, cols
    x64 = x.astype(np.float64)
    h = (x64.T @ x64) / x.shape[0]
    damp = 0.01 * max(float(np.mean(np.diag(h))), 1e-12)
    h[np.diag_indices(n)] += damp
    hinv = np.linalg.inv(h)
    hinv = (hinv + hinv.T) / 2
    u = np.linalg.cholesky(hinv).T                       # upper; the feedback uses its rows
    scale2 = global_scale(w)
    work = w.reshape(rows, cols).copy()
    codes = np.zeros((rows, cols), np.uint8)
    scales = np.zeros((rows, cols // BLOCK), np.uint8)
    units = np.zeros(rows, np.float32)
    for j in range(cols):
        if j % BLOCK == 0:
            byte, units = block_unit(work[:, j:j + BLOCK], scale2)
            scales[:, j // BLOCK] = byte
        v = work[:, j]
        code = code_of(v, units)
        codes[:, j] = code
        qv = (decode_code(code) * units).astype(np.float32)
        err = ((v - qv).astype(np.float64) / u[j, j]).astype(np.float32)
        if j + 1 < cols:
            work[:, j + 1:] -= (err[:, None] * u[j, j + 1:].astype(np.float32)[None, :]).astype(np.float32)
    return Packed(rows, cols, _pack_codes(codes), scales, scale2)


def channel_scales(mean_abs, alpha):
    """mean|x|^alpha with geometric mean one, or all ones at alpha zero (src/calibrate.rs:324-335)."""
    mean_abs = np.asarray(mean_abs, np.float32)
    if alpha == 0.0:
        return np.ones(mean_abs.size, np.float32)
    s = np.power(mean_abs + _f32(1e-8), _f32(alpha)).astype(np.float32)
    norm = _f32(np.exp(np.mean(np.log(s).astype(np.float64))))
    return (s / norm).astype(np.float32)


def scale_columns(w, cols, s):
    return (np.asarray(w, np.float32).reshape(-1, cols) * np.asarray(s, np.float32)[None, :]).astype(np.float32)


class Calibrated:
    """One packed linear and how it was made (src/calibrate.rs:67-101)."""

    def __init__(self, packed, input_scale, alpha=0.0, error_ratio=1.0, feedback_used=False):
        self.packed, self.input_scale = packed, np.asarray(input_scale, np.float32)
        self.alpha, self.error_ratio, self.feedback_used = float(alpha), float(error_ratio), bool(feedback_used)

    @staticmethod
    def plain(packed):
        return Calibrated(packed, np.ones(packed.cols, np.float32))

    def decode(self):
        """The dense f32 matrix a consumer of W should use: decoded codes with the input scale folded into the columns."""
        return (self.packed.decode() * self.input_scale[None, :]).astype(np.float32)


def pack_linear(w, cols, rows, mean_abs, alphas=AWQ_ALPHAS, feedback=True):
    """Calibrated NVFP4 of one linear w [n, cols] (src/calibrate.rs:351-434): the channel-scale exponent is chosen
    from `alphas` by least output error over the captured input rows; error feedback is kept only where it beats
    the best nearest rounding on the same rows."""
    w = np.ascontiguousarray(w, np.float32).reshape(-1)
    rows = np.asarray(rows, np.float32).reshape(-1, cols)
    mean_abs = np.asarray(mean_abs, np.float32)
    if rows.shape[0] == 0:
        raise ValueError("calibration needs input rows")
    if mean_abs.size != cols:
        raise ValueError(f"mean_abs has {mean_abs.size} entries for {cols} columns")
    plain = pack_nearest(w, cols)
    plain_err = output_error(w, plain.decode(), cols, rows)
    best, best_err = Calibrated.plain(plain), plain_err
    for alpha in alphas:
        if alpha == 0.0:
            continue
        s = channel_scales(mean_abs, alpha)
        cal = Calibrated(pack_nearest(scale_columns(w, cols, s), cols), (_f32(1.0) / s).astype(np.float32), alpha)
        err = output_error(w, cal.decode(), cols, rows)
        if err < best_err:
            best, best_err = cal, err
    if feedback:
        s = channel_scales(mean_abs, best.alpha)
        xs = (rows / s[None, :]).astype(np.float32)
        cal = Calibrated(pack_gptq(scale_columns(w, cols, s), cols, xs), (_f32(1.0) / s).astype(np.float32), best.alpha,
                         feedback_used=True)
        err = output_error(w, cal.decode(), cols, rows)
        if err < best_err:
            best, best_err = cal, err
    best.error_ratio = best_err / plain_err if plain_err > 0.0 else 1.0
    return best
