"""Host-side mirror of the Inkling op surface that Burn model code calls, over the C ABI.

Follows src/models/inkling/burn.rs:40-329 (`PackedW`, `ProjW`, `linear`, `linear_bf16`, `linear_fp4`,
`linear_w4a16`, `linear_w`, `rms_norm`, `silu`), src/models/inkling/resid.rs:272-365 (the narrow
`rms_norm`), src/models/inkling/fp4gemm.rs:472-623 (`gate_up_silu*`) and the decode-time grouped
experts of src/nn/nvfp4_gemm.rs:293-523 (`GroupedBank`, `w4a4_grouped_bf16`).

The reference pads the activation to 16 rows before its MMA kernels and slices the result back; the
kernels here take any row count, so nothing is padded and the result is the sliced one.
"""
import numpy as np
import torch

from . import _lib
from ._lib import lib, context, MaryError
from . import nvfp4 as nv

_p = nv._p
_stream = nv._stream


def _dt(t):
    return _lib.DT_BF16 if t == torch.bfloat16 else _lib.DT_F32


class PackedW:
    """PackedW (src/models/inkling/burn.rs:110-150): a resident NVFP4 weight [n, k] as row-major codes and
    scales plus its global scale."""

    def __init__(self, codes, scales, scale2, n, k):
        if k % 64 != 0 or n % 8 != 0:
            raise MaryError(_lib.ERR_INVALID, f"PackedW [{n}, {k}]: k must be a multiple of 64 and n of 8")
        self.codes, self.scales, self.scale2, self.n, self.k = codes, scales, float(np.float32(scale2)), n, k
        self.swizzled = False          # the fragment-order layout of the reference is internal to its kernels
        self._sf_tiled = None

    @staticmethod
    def quantize(w):
        q = nv.Nvfp4.quantize(w)
        return PackedW(q.codes, q.scales, q.scale2, q.n(), q.k())

    def sf_tiled(self):
        if self._sf_tiled is None:
            self._sf_tiled = nv.tile_scales(self.scales, self.n, self.k)
        return self._sf_tiled


class ProjW:
    """ProjW (src/models/inkling/burn.rs:160-200): a projection weight bound to one of three lanes."""

    def __init__(self, lane, w):
        assert lane in ("bf16", "fp4", "w4a16")
        self.lane, self.w = lane, w

    def k(self):
        return self.w.shape[1] if self.lane == "bf16" else self.w.k


def _check_2d(x, k, who):
    if x.dim() != 2 or x.shape[1] != k:
        raise MaryError(_lib.ERR_INVALID, f"{who}: x is {list(x.shape)} but the weight is [_, {k}]")
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise MaryError(_lib.ERR_INVALID, f"{who}: no lane for a {x.dtype} activation")
    return x if x.is_contiguous() else x.contiguous()


def linear_bf16(x, w):
    """linear_bf16 (src/models/inkling/burn.rs:56-108): x [m, k] bf16 or f32 (rounded to bf16) against a bf16
    weight [n, k]; f32 result."""
    x = _check_2d(x, w.shape[1], "linear_bf16")
    if x.dtype == torch.float32:
        x = x.to(torch.bfloat16)
    return nv.bf16_gemm(x, w, out_dtype=torch.float32)


def linear_fp4(x, w):
    """linear_fp4 (src/models/inkling/burn.rs:214-259): the activation (bf16 or f32) is quantised on the device
    by the reciprocal recipe without a second-level scale (quantize_nvfp4(_bf16)), then the dense W4A4
    product with epilogue scale2; f32 result [m, n]."""
    x = _check_2d(x, w.k, "linear_fp4")
    if w.swizzled:
        raise MaryError(_lib.ERR_INVALID, "linear_fp4 was handed a weight in fragment order")
    m = x.shape[0]
    codes, sf, _ = nv.quantize_act(x, _lib.QUANT_RECIP, tiled=True)
    return nv.gemm_w4a4(codes, sf, w.codes, w.sf_tiled(), w.scale2, m, w.n, w.k, out_dtype=torch.float32)


def linear_w4a16(x, w):
    """linear_w4a16 (src/models/inkling/burn.rs:261-311): the weight reaches the product as the same four bits,
    the activation stays bf16 (an f32 one is rounded to bf16 first); f32 result [m, n]."""
    x = _check_2d(x, w.k, "linear_w4a16")
    if x.dtype == torch.float32:
        x = x.to(torch.bfloat16)
    return nv.w4a16_gemm(x, w.codes, w.scales, w.scale2, w.n, w.k, out_dtype=torch.float32)


def linear_w(x, w):
    """linear_w (src/models/inkling/burn.rs:203-209): x @ w^T for a weight in whichever lane it is bound to."""
    if w.lane == "bf16":
        return linear_bf16(x, w.w)
    if w.lane == "fp4":
        return linear_fp4(x, w.w)
    return linear_w4a16(x, w.w)


def rms_norm(x, gain, eps):
    """rms_norm (src/models/inkling/resid.rs:365-380 over rms_norm_kernel :272-322): bf16 in gives bf16 out, f32 in
    f32 out; f32 gain; one rounding."""
    assert x.dim() == 2 and x.is_contiguous() and gain.dtype == torch.float32 and gain.numel() == x.shape[1]
    ctx = context(x.device.index)
    out = torch.empty_like(x)
    ctx.check(lib.mb_rmsnorm_inkling(ctx.handle, _stream(), _p(x), _dt(x.dtype), _p(gain), x.shape[0], x.shape[1],
                                     float(eps), _p(out), _dt(out.dtype)))
    return out


def gate_up_silu(both, inter, halved=False, out_dtype=None):
    """gate_up_silu_launch / _narrow / _bf16 (src/models/inkling/fp4gemm.rs:574-623): both [rows, 2 * inter]
    (f32 or bf16) -> silu(gate) * up [rows, inter]."""
    assert both.dim() == 2 and both.is_contiguous() and both.shape[1] == 2 * inter
    out_dtype = out_dtype or both.dtype
    ctx = context(both.device.index)
    act = torch.empty((both.shape[0], inter), dtype=out_dtype, device=both.device)
    ctx.check(lib.mb_gate_up_silu(ctx.handle, _stream(), _p(both), _dt(both.dtype), both.shape[0], inter, int(halved),
                                  _p(act), _dt(out_dtype)))
    return act


def interleave_halved(codes, scales):
    """A w13 stored HALVED (all gate rows, then all up rows) re-ordered row by row into the INTERLEAVED order
    (g0, u0, g1, u1, ...) the fused SwiGLU epilogues read; a permutation of stored rows, no byte changes
    (src/models/inkling/fp4gemm.rs:466-471 names the two readings)."""
    n2 = codes.shape[-2]
    half = n2 // 2
    order = torch.stack([torch.arange(half), torch.arange(half) + half], 1).reshape(-1).to(codes.device)
    return codes.index_select(-2, order).contiguous(), scales.index_select(-2, order).contiguous()


class GroupedBank:
    """GroupedBank (src/nn/nvfp4_gemm.rs:438-451): `experts` NVFP4 weights [n, k], planes contiguous
    [experts, n, ...] with row-major scales, every expert's activation input scale and its f32 epilogue
    product alpha = scale2 * input_scale, both indexed by expert id."""

    def __init__(self, codes, scales, scale2, input_scale, experts, n, k):
        if k % 64 != 0 or n % 8 != 0:
            raise MaryError(_lib.ERR_INVALID, f"grouped W4A4 geometry [{experts} x {n}, {k}]")
        self.codes, self.scales, self.experts, self.n, self.k = codes, scales, experts, n, k
        self.input_scale = input_scale.to(torch.float32).contiguous()
        s2 = scale2.to(torch.float32).to(self.input_scale.device)
        self.alpha = (s2 * self.input_scale).contiguous()        # f32 product, as the host forms it
        for name, v in (("input_scale", self.input_scale), ("alpha", self.alpha)):
            if not bool(torch.isfinite(v).all() and (v > 0).all()):
                raise MaryError(_lib.ERR_INVALID, f"W4A4 calibrated globals/product must be finite positive ({name})")


def w4a4_grouped_bf16(x, x_per_group, ids, bank):
    """w4a4_grouped_bf16 (src/nn/nvfp4_gemm.rs:462-523): one bf16 activation row per group (x [groups, k]) or one
    shared row (x [k] or [1, k]) times bank expert ids[g]; bf16 [groups, n]. ids: int32 CUDA tensor."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and ids.dtype == torch.int32 and ids.is_contiguous()
    groups = ids.numel()
    if x_per_group:
        assert x.numel() == groups * bank.k
    else:
        assert x.numel() == bank.k
    ctx = context(x.device.index)
    codes = torch.empty((groups, bank.k // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((groups, bank.k // 16), dtype=torch.uint8, device=x.device)
    ctx.check(lib.mb_nvfp4_quantize_grouped(ctx.handle, _stream(), _p(x), int(bool(x_per_group)), _p(ids), groups,
                                            _p(bank.input_scale), bank.experts, bank.k, _p(codes), _p(scales)))
    out = torch.empty((groups, bank.n), dtype=torch.bfloat16, device=x.device)
    ctx.check(lib.mb_nvfp4_gemv_w4a4_grouped(ctx.handle, _stream(), _p(codes), _p(scales), _p(bank.codes), _p(bank.scales),
                                             _p(bank.alpha), _p(ids), groups, bank.experts, bank.n, bank.k, _p(out),
                                             _lib.DT_BF16))
    return out, (codes, scales)
