"""Host-side mirror of the reference's NVFP4 operator surface over the C ABI.

`Nvfp4` follows `mary::nn::Nvfp4` (src/nn/nvfp4_gemv.rs:281-579,
src/nn/nvfp4_gemm.rs:558-1043 in the reference): the same constructors
(`quantize`, `upload`, `from_parts`), the same predicates (`takes`), the same
projections (`gemv`, `project`, `project_w4a4_scaled`, `project_w4a4_rows`) with
the same argument meaning and the same refusals. torch is used only for device
memory and streams; every computation is a call into libmary_b200.so.
"""
import ctypes as C
import enum

import os

import numpy as np
import torch

from . import _lib
from ._lib import lib, context, MaryError

GROUP = 16        # weights per E4M3 block scale (src/nn/nvfp4_gemv.rs:65)
CHUNK = 32        # weights one GEMV lane takes per step (:67)
W4A16_FUSED_ROWS = 512
MAX_ROWS = 8      # activation rows the GEMV takes (:73)
KTILE4 = 64       # K of the block-scaled instruction (src/nn/nvfp4_gemm.rs:43)
NTILE = 8


class PromptLane(enum.Enum):
    """src/nvfp4.rs:242-264."""
    W4A4 = "w4a4"
    W4A16 = "w4a16"

    @staticmethod
    def parse(value):
        for lane in PromptLane:
            if lane.value == value:
                return lane
        raise ValueError(f"NVFP4 prompt lane must be w4a4 or w4a16, not {value!r}")


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def sf_bytes(rows, k):
    return int(lib.mb_nvfp4_sf_bytes(rows, k))


def quantize_act(x, recipe=_lib.QUANT_SCALED, input_scale=1.0, tiled=True, gather=None, rows=None):
    """Activation quantizer (see MB_QUANT_* in the header). x: [rows, k] bf16/f32 CUDA tensor.
    Returns (codes [rows, k/2] u8, scales, rowscale or None)."""
    assert x.is_cuda and x.dim() == 2 and x.is_contiguous()
    ctx = context(x.device.index)
    src_rows, k = x.shape
    rows = int(rows if rows is not None else (gather.numel() if gather is not None else src_rows))
    dt = _lib.DT_BF16 if x.dtype == torch.bfloat16 else _lib.DT_F32
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise MaryError(_lib.ERR_INVALID, f"activations are bf16 or f32, not {x.dtype}")
    codes = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    if tiled:
        scales = torch.empty(sf_bytes(rows, k), dtype=torch.uint8, device=x.device)
    else:
        scales = torch.empty((rows, k // GROUP), dtype=torch.uint8, device=x.device)
    rowscale = torch.empty(rows, dtype=torch.float32, device=x.device) if recipe == _lib.QUANT_ROWS else None
    ctx.check(lib.mb_nvfp4_quantize_act(ctx.handle, _stream(), _p(x), dt, rows, k, recipe, float(input_scale),
                                        _p(gather), src_rows, _p(codes), _p(scales),
                                        _lib.SF_TILED if tiled else _lib.SF_ROWMAJOR, _p(rowscale)))
    return codes, scales, rowscale


def mxfp4_to_nvfp4(packed, e8m0, rows, cols):
    """transcode_to_nvfp4 (src/nn/mxfp4.rs:319-375): an MXFP4 tensor ([rows, cols/2] code bytes, [rows, cols/32]
    E8M0 scales) relabelled as NVFP4 without touching the codes. Returns (codes (the same tensor), row-major
    E4M3 block scales [rows, cols/16], global scale, global exponent)."""
    assert packed.dtype == torch.uint8 and e8m0.dtype == torch.uint8 and cols % 32 == 0
    assert packed.numel() == rows * cols // 2 and e8m0.numel() == rows * cols // 32
    ctx = context(packed.device.index)
    out = torch.empty((rows, cols // 16), dtype=torch.uint8, device=packed.device)
    gs, ge = C.c_float(), C.c_int()
    ctx.check(lib.mb_mxfp4_to_nvfp4_scales(ctx.handle, _stream(), _p(e8m0.contiguous()), e8m0.numel(), _p(out),
                                           C.byref(gs), C.byref(ge)))
    return packed, out, float(gs.value), int(ge.value)


def gather_rows(codes, sf_tiled, src_rows, k, gather):
    """Quantized activation planes copied into the row order of `gather` (negative = zero row)."""
    ctx = context(codes.device.index)
    rows = gather.numel()
    out = torch.empty((rows, k // 2), dtype=torch.uint8, device=codes.device)
    out_sf = torch.empty(sf_bytes(rows, k), dtype=torch.uint8, device=codes.device)
    ctx.check(lib.mb_nvfp4_gather_rows(ctx.handle, _stream(), _p(codes), _p(sf_tiled), src_rows, k, _p(gather), rows,
                                       _p(out), _p(out_sf)))
    return out, out_sf


def dequantize(codes, scales_rowmajor, scale2, rows, k, dtype=torch.float32):
    ctx = context(codes.device.index)
    out = torch.empty((rows, k), dtype=dtype, device=codes.device)
    ctx.check(lib.mb_nvfp4_dequantize(ctx.handle, _stream(), _p(codes), _p(scales_rowmajor), float(scale2), rows, k,
                                      _p(out), _lib.DT_F32 if dtype == torch.float32 else _lib.DT_BF16))
    return out


def tile_scales(scales_rowmajor, rows, k):
    ctx = context(scales_rowmajor.device.index)
    out = torch.empty(sf_bytes(rows, k), dtype=torch.uint8, device=scales_rowmajor.device)
    ctx.check(lib.mb_nvfp4_tile_scales(ctx.handle, _stream(), _p(scales_rowmajor), rows, k, _p(out)))
    return out


def untile_scales(scales_tiled, rows, k):
    ctx = context(scales_tiled.device.index)
    out = torch.empty((rows, k // GROUP), dtype=torch.uint8, device=scales_tiled.device)
    ctx.check(lib.mb_nvfp4_untile_scales(ctx.handle, _stream(), _p(scales_tiled), rows, k, _p(out)))
    return out


_SPLITK_WS = {}


def _splitk_workspace(device, nbytes):
    """One reusable split-K workspace per device and stream (grown on demand, never shrunk): calls on one stream
    are ordered and may share it, calls on different streams may overlap and may not."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _SPLITK_WS.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _SPLITK_WS[key] = ws
    return ws


_GEMV_WS = {}


def _gemv_workspace(device, nbytes):
    """The GEMV's f16 activation copy: one reusable buffer per device and stream (calls on one stream are ordered,
    so they may share it)."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _GEMV_WS.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _GEMV_WS[key] = ws
    return ws


def gemm_w4a4(a_codes, a_sf, b_codes, b_sf, alpha, m, n, k, rowscale=None, out_dtype=torch.bfloat16,
              epilogue=_lib.EPI_PLAIN, out=None):
    ctx = context(a_codes.device.index)
    cols = n // 2 if epilogue == _lib.EPI_SWIGLU_INTERLEAVED else n
    if out is None:
        out = torch.empty((m, cols), dtype=out_dtype, device=a_codes.device)
    if epilogue == _lib.EPI_PLAIN and m <= 128:
        need = int(lib.mb_nvfp4_gemm_splitk_workspace(m, n, k))
        if need:
            ws = _splitk_workspace(a_codes.device, need)
            ctx.check(lib.mb_nvfp4_gemm_w4a4_splitk(ctx.handle, _stream(), _p(a_codes), _p(a_sf), _p(b_codes), _p(b_sf),
                                                    _p(rowscale), float(alpha), m, n, k, _p(out),
                                                    _lib.DT_BF16 if out.dtype == torch.bfloat16 else _lib.DT_F32,
                                                    _p(ws), need))
            return out
    ctx.check(lib.mb_nvfp4_gemm_w4a4(ctx.handle, _stream(), _p(a_codes), _p(a_sf), _p(b_codes), _p(b_sf), _p(rowscale),
                                     float(alpha), m, n, k, _p(out),
                                     _lib.DT_BF16 if out.dtype == torch.bfloat16 else _lib.DT_F32, epilogue))
    return out


class Stacked:
    """Several stored NVFP4 tensors with the same k laid one after another along n, so that
    projections of one input run as one product; every tensor keeps its own global scale in
    `colscale` (one f32 per output column). `interleave` lays two tensors row by row (gate,
    up, gate, up ...), the order the SwiGLU epilogues read."""

    def __init__(self, parts, interleave=False):
        k = parts[0].k()
        assert all(w.k() == k for w in parts)
        dev = parts[0].codes.device
        if interleave:
            assert len(parts) == 2 and parts[0].n() == parts[1].n()
            n = parts[0].n()
            self.codes = torch.stack([parts[0].codes.view(n, k // 2), parts[1].codes.view(n, k // 2)], 1) \
                .reshape(2 * n, k // 2).contiguous()
            scales = torch.stack([parts[0].scales.view(n, k // GROUP), parts[1].scales.view(n, k // GROUP)], 1) \
                .reshape(2 * n, k // GROUP).contiguous()
            self.colscale = torch.tensor([parts[0].scale2, parts[1].scale2], dtype=torch.float32, device=dev).repeat(n)
        else:
            self.codes = torch.cat([w.codes.view(w.n(), k // 2) for w in parts]).contiguous()
            scales = torch.cat([w.scales.view(w.n(), k // GROUP) for w in parts]).contiguous()
            self.colscale = torch.cat([torch.full((w.n(),), w.scale2, dtype=torch.float32, device=dev) for w in parts])
        self.n, self.k = self.codes.shape[0], k
        self.sf_tiled = tile_scales(scales, self.n, k)


def gemm_w4a4_stacked(a_codes, a_sf, w, m, out_dtype=torch.bfloat16, epilogue=_lib.EPI_PLAIN):
    """One product against a `Stacked` weight. Plain epilogue: [m, n] in out_dtype. SwiGLU
    epilogues: [m, n/2] bf16, or with an EPI_QUANT_* flag the (codes, tiled scale plane) of it."""
    ctx = context(a_codes.device.index)
    dev = a_codes.device
    swiglu = (epilogue & 0xFF) in (_lib.EPI_SWIGLU_INTERLEAVED, _lib.EPI_SWIGLU_ROUNDED)
    quant = epilogue & (_lib.EPI_QUANT_RECIP | _lib.EPI_QUANT_SCALED)
    ws, need, out_sf = None, 0, None
    if quant:
        out = torch.empty((m, w.n // 4), dtype=torch.uint8, device=dev)
        out_sf = torch.empty(sf_bytes(m, w.n // 2), dtype=torch.uint8, device=dev)
        dt = _lib.DT_BF16
    else:
        out = torch.empty((m, w.n // 2 if swiglu else w.n), dtype=torch.bfloat16 if swiglu else out_dtype, device=dev)
        dt = _lib.DT_BF16 if out.dtype == torch.bfloat16 else _lib.DT_F32
        if not swiglu and m <= 128:
            need = int(lib.mb_nvfp4_gemm_splitk_workspace(m, w.n, w.k))
            ws = _splitk_workspace(dev, need) if need else None
    ctx.check(lib.mb_nvfp4_gemm_w4a4_stacked(ctx.handle, _stream(), _p(a_codes), _p(a_sf), _p(w.codes), _p(w.sf_tiled),
                                             _p(w.colscale), m, w.n, w.k, _p(out), dt, epilogue, _p(out_sf), _p(ws),
                                             need))
    return (out, out_sf) if quant else out


def bf16_gemm(a, b, out_dtype=torch.float32, out=None, alpha=1.0):
    """bf16_linear_launch (src/models/inkling/bf16gemm.rs:64-152): [m,k] x [n,k]^T -> [m,n]."""
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_contiguous() and b.is_contiguous()
    ctx = context(a.device.index)
    m, k = a.shape
    n = b.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    dt = _lib.DT_BF16 if out.dtype == torch.bfloat16 else _lib.DT_F32
    need = int(lib.mb_bf16_gemm_splitk_workspace(m, n, k))
    if need:        # few output tiles, long K (the router projection): K slices, summed in order
        ws = _splitk_workspace(a.device, need)
        ctx.check(lib.mb_bf16_gemm_splitk(ctx.handle, _stream(), _p(a), _p(b), float(alpha), m, n, k, _p(out), dt,
                                          _p(ws), need))
        return out
    ctx.check(lib.mb_bf16_gemm(ctx.handle, _stream(), _p(a), _p(b), float(alpha), m, n, k, _p(out), dt))
    return out


def w4a16_gemm(x, codes, scales, scale2, n, k, out_dtype=torch.bfloat16):
    """The W4A16 prompt product (src/nn/nvfp4_gemm.rs:93-197): x [m, k] bf16 against resident NVFP4 planes
    (row-major scales); the weight is decoded between shared memory and the tensor core, never into HBM."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.dim() == 2 and x.shape[1] == k
    ctx = context(x.device.index)
    m = x.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    need = int(lib.mb_nvfp4_gemm_w4a16_workspace(m, n, k))
    ws = _splitk_workspace(x.device, need) if need else None
    ctx.check(lib.mb_nvfp4_gemm_w4a16(ctx.handle, _stream(), _p(x), _p(codes), _p(scales), float(scale2), m, n, k, _p(out),
                                      _lib.DT_BF16 if out_dtype == torch.bfloat16 else _lib.DT_F32, _p(ws), need))
    return out


class Nvfp4:
    """A resident NVFP4 weight [n, k]: row-major code and scale planes (the
    canonical payload layout) plus the tiled scale plane the tensor-core GEMM reads."""

    def __init__(self, codes, scales, scale2, n, k, dtype, device):
        self.codes, self.scales, self.scale2 = codes, scales, float(np.float32(scale2))
        self._n, self._k, self._dtype, self._device = n, k, dtype, device
        self._sf_tiled = None

    # ---- constructors -------------------------------------------------------
    @staticmethod
    def quantize(w):
        """Nvfp4::quantize (src/nn/nvfp4_gemv.rs:284-351)."""
        if not (w.is_cuda and w.dim() == 2 and w.is_contiguous()):
            raise MaryError(_lib.ERR_INVALID, "NVFP4 quantizes contiguous rank-2 CUDA weights")
        if w.dtype != torch.bfloat16:
            raise MaryError(_lib.ERR_INVALID, "NVFP4 quantizes unquantized BF16 weights")
        n, k = w.shape
        ctx = context(w.device.index)
        codes = torch.empty((n, k // 2), dtype=torch.uint8, device=w.device)
        scales = torch.empty((n, max(k // GROUP, 1)), dtype=torch.uint8, device=w.device)
        s2 = C.c_float()
        ctx.check(lib.mb_nvfp4_quantize_weight(ctx.handle, _stream(), _p(w), n, k, _p(codes), _p(scales), C.byref(s2)))
        return Nvfp4(codes, scales, s2.value, n, k, w.dtype, w.device)

    @staticmethod
    def upload(payload, dims, dtype, device):
        """Nvfp4::upload (src/nn/nvfp4_gemv.rs:364-388): a stored leaf payload
        (codes || scales || scale2_le) copied to the device; nothing is converted."""
        n, k = int(dims[0]), int(dims[1])
        elements = n * k
        if not (0 < elements <= 0xFFFFFFFF):
            raise MaryError(_lib.ERR_INVALID, f"NVFP4 [{n}, {k}] is empty or exceeds u32 indexing")
        payload = np.ascontiguousarray(np.frombuffer(bytes(payload), np.uint8) if not isinstance(payload, np.ndarray)
                                       else payload, np.uint8)
        codes_len, scales_len = elements // 2, elements // GROUP
        if payload.size != codes_len + scales_len + 4:
            raise MaryError(_lib.ERR_INVALID,
                            f"NVFP4 payload has {payload.size} bytes; [{n}, {k}] requires {codes_len + scales_len + 4}")
        scale2 = np.frombuffer(payload[codes_len + scales_len:].tobytes(), np.float32)[0]
        codes = torch.from_numpy(payload[:codes_len].copy()).to(device).view(n, k // 2)
        scales = torch.from_numpy(payload[codes_len:codes_len + scales_len].copy()).to(device).view(n, k // GROUP)
        return Nvfp4.from_parts(codes, scales, scale2, n, k, dtype, device)

    @staticmethod
    def from_parts(codes, scales, scale2, n, k, dtype, device):
        """Nvfp4::from_parts (src/nn/nvfp4_gemv.rs:392-427)."""
        if not (n > 0 and k > 0 and k % CHUNK == 0):
            raise MaryError(_lib.ERR_INVALID, f"NVFP4 weight [{n}, {k}] needs k a multiple of {CHUNK}")
        if dtype != torch.bfloat16:
            raise MaryError(_lib.ERR_INVALID, f"NVFP4 weights multiply BF16 activations, not {dtype}")
        s2 = float(np.float32(scale2))
        if not (np.isfinite(s2) and s2 > 0.0):
            raise MaryError(_lib.ERR_INVALID, f"NVFP4 global scale {s2} is not a positive finite number")
        if codes.numel() < n * k // 2 or scales.numel() < n * k // GROUP:
            raise MaryError(_lib.ERR_INVALID, f"NVFP4 planes are shorter than [{n}, {k}]")
        return Nvfp4(codes, scales, s2, n, k, dtype, torch.device(device))

    # ---- accessors ----------------------------------------------------------
    def n(self):
        return self._n

    def k(self):
        return self._k

    def dtype(self):
        return self._dtype

    def device(self):
        return self._device

    def bytes(self):
        return self._n * self._k // 2 + self._n * self._k // GROUP

    def read_planes(self):
        """Nvfp4::read_planes: the canonical planes as host bytes."""
        return (self.codes.reshape(-1)[: self._n * self._k // 2].cpu().numpy(),
                self.scales.reshape(-1)[: self._n * self._k // GROUP].cpu().numpy())

    def payload(self):
        codes, scales = self.read_planes()
        return np.concatenate([codes, scales, np.frombuffer(np.float32(self.scale2).tobytes(), np.uint8)])

    def sf_tiled(self):
        if self._sf_tiled is None:
            self._sf_tiled = tile_scales(self.scales, self._n, self._k)
        return self._sf_tiled

    # ---- GEMV ---------------------------------------------------------------
    def takes(self, x):
        """Activation rows t if x is a [1, t, k] this GEMV takes, else None
        (src/nn/nvfp4_gemv.rs:510-525)."""
        s = tuple(x.shape)
        ok = (len(s) == 3 and s[0] == 1 and 1 <= s[1] <= MAX_ROWS and s[2] == self._k and x.stride(2) == 1
              and (s[1] == 1 or x.stride(1) == self._k) and x.dtype == self._dtype and x.device == self._device
              and x.data_ptr() % 16 == 0)
        return s[1] if ok else None

    def gemv(self, x, rows):
        """[1, rows, k] x [n, k]^T -> [1, rows, n] (src/nn/nvfp4_gemv.rs:529-578)."""
        assert 1 <= rows <= MAX_ROWS, f"NVFP4 GEMV takes 1..={MAX_ROWS} rows"
        ctx = context(self._device.index)
        out = torch.empty((1, rows, self._n), dtype=self._dtype, device=self._device)
        need = int(lib.mb_nvfp4_gemv_workspace(rows, self._n, self._k))
        ws = _gemv_workspace(self._device, need)
        ctx.check(lib.mb_nvfp4_gemv_w4a16_ws(ctx.handle, _stream(), _p(x), rows, _p(self.codes), _p(self.scales),
                                             self.scale2, self._n, self._k, _p(out), _lib.DT_BF16, _p(ws), need))
        return out

    # ---- prompt projections ---------------------------------------------------
    def _rows_of(self, x):
        """src/nn/nvfp4_gemm.rs:527-556."""
        s = tuple(x.shape)
        if len(s) == 3 and s[0] == 1:
            t, k = s[1], s[2]
        elif len(s) == 2:
            t, k = s
        else:
            raise MaryError(_lib.ERR_INVALID, f"NVFP4 prompt projection takes [1, t, k], got {list(s)}")
        if not (k == self._k and t > 0):
            raise MaryError(_lib.ERR_INVALID, f"NVFP4 prompt projection needs contiguous [t, {self._k}], got {list(s)}")
        if x.dtype != self._dtype or x.device != self._device:
            raise MaryError(_lib.ERR_INVALID,
                            f"NVFP4 prompt projection: activation is {x.dtype} on {x.device}, weight wants {self._dtype}")
        if t * k > 0xFFFFFFFF or self._n * k > 0xFFFFFFFF:
            raise MaryError(_lib.ERR_INVALID, "NVFP4 prompt projection exceeds u32 indexing")
        return t

    def project(self, x, lane=PromptLane.W4A16):
        return self._project_with_scale(x, lane, 1.0)

    def project_w4a4_scaled(self, x, input_scale):
        calibrated_scale(input_scale, self.scale2)
        return self._project_with_scale(x, PromptLane.W4A4, input_scale)

    def _project_with_scale(self, x, lane, input_scale):
        if not x.is_contiguous() or x.data_ptr() % 4 != 0:
            x = x.contiguous()
        t = self._rows_of(x)
        if self._n % NTILE != 0:
            raise MaryError(_lib.ERR_INVALID, f"NVFP4 prompt projection needs n a multiple of {NTILE}, got {self._n}")
        x2 = x.reshape(t, self._k)
        if lane == PromptLane.W4A16:
            out = self._w4a16(x2, t)
        else:
            if self._k % KTILE4 != 0:
                raise MaryError(_lib.ERR_INVALID, f"W4A4 needs k a multiple of {KTILE4}, got {self._k}")
            codes, sf, _ = quantize_act(x2, _lib.QUANT_SCALED, input_scale, tiled=True)
            alpha = float(np.float32(self.scale2) * np.float32(input_scale))
            out = gemm_w4a4(codes, sf, self.codes, self.sf_tiled(), alpha, t, self._n, self._k,
                            out_dtype=self._dtype)
        return out.view(1, t, self._n)

    def _w4a16(self, x2, t):
        # The weight stays four bits in HBM: code x block scale is expanded to bf16 (exact) between shared
        # memory and the tensor core, f32 accumulation, scale2 applied once to the accumulator, as in the
        # reference's W4A16 kernel. k % 64 != 0 (the reference's W4A16 takes k % 32) goes through a decoded
        # scratch plane and the bf16 product instead, and so do prompts beyond W4A16_FUSED_ROWS rows: there the
        # product is bound by the tensor core, the decode of a weight tile would be repeated for every row tile, and
        # decoding once (the same exact values) costs a few percent of the product. MB_W4A16_FUSED=0 / 1 forces
        # one way for comparison.
        fused = os.environ.get("MB_W4A16_FUSED")
        fused = (t <= W4A16_FUSED_ROWS) if fused is None else fused != "0"
        if fused and self._k % KTILE4 == 0 and x2.data_ptr() % 16 == 0:
            return w4a16_gemm(x2, self.codes, self.scales, self.scale2, self._n, self._k, out_dtype=self._dtype)
        w = dequantize(self.codes, self.scales, 1.0, self._n, self._k, dtype=torch.bfloat16)
        return bf16_gemm(x2, w, out_dtype=self._dtype, alpha=self.scale2)

    def project_w4a4_rows(self, x):
        """Per-row activation scale (src/nn/nvfp4_gemm.rs:947-1043)."""
        if not w4a4_rows_takes(self._n, self._k):
            raise MaryError(_lib.ERR_INVALID, f"W4A4 rows needs k % {KTILE4} == 0 and n % {NTILE} == 0")
        if not x.is_contiguous():
            x = x.contiguous()
        t = self._rows_of(x)
        x2 = x.reshape(t, self._k)
        codes, sf, rowscale = quantize_act(x2, _lib.QUANT_ROWS, 1.0, tiled=True)
        out = gemm_w4a4(codes, sf, self.codes, self.sf_tiled(), self.scale2, t, self._n, self._k, rowscale=rowscale,
                        out_dtype=self._dtype)
        return out.view(1, t, self._n)


def w4a4_rows_takes(n, k):
    """src/nn/nvfp4_gemm.rs:743-745."""
    return k % KTILE4 == 0 and n % NTILE == 0 and k % GROUP == 0


def calibrated_scale(input_scale, weight_scale):
    """src/nn/nvfp4_gemm.rs:700-706: reject underflow/overflow of the product."""
    i, w = np.float32(input_scale), np.float32(weight_scale)
    with np.errstate(all="ignore"):
        product = np.float32(i * w)
    if not (np.isfinite(i) and i > 0 and np.isfinite(w) and w > 0 and np.isfinite(product) and product > 0):
        raise MaryError(_lib.ERR_INVALID, "W4A4 calibrated globals/product must be finite positive")
    return float(product)


def linear(x, q, lane=PromptLane.W4A16):
    """breeze::backbone::linear (src/models/breeze/backbone.rs:20-34): the GEMV when
    it takes the activation, else the prompt projection."""
    rows = q.takes(x)
    if rows is not None:
        return q.gemv(x, rows)
    return q.project(x, lane)
