"""ctypes binding of the C ABI (include/mary_b200.h).

Importing this module loads maryml_b200/libmary_b200.so and fails loudly when it
is missing: there is no CPU or eager fallback anywhere in the package.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmary_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build the CUDA library first (python maryml_b200/build.py). "
        "maryml_b200 has no fallback path.")

lib = C.CDLL(LIB_PATH)

OK, ERR_INVALID, ERR_CUDA, ERR_NONFINITE, ERR_DEVICE_FLAG, ERR_UNAVAILABLE = 0, -1, -2, -3, -4, -5
DT_BF16, DT_F32 = 0, 1
SF_ROWMAJOR, SF_TILED = 0, 1
QUANT_SCALED, QUANT_RECIP, QUANT_ROWS = 0, 1, 2
EPI_PLAIN, EPI_SWIGLU_INTERLEAVED, EPI_SWIGLU_ROUNDED = 0, 1, 3
EPI_QUANT_RECIP, EPI_QUANT_SCALED = 0x100, 0x200
KV_F32, KV_BF16, KV_NVFP4 = 0, 1, 2


class KeyRun(C.Structure):
    """mb_key_run: one run of key/value rows (a page of a paged cache)."""
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("k_scales", C.c_void_p), ("v_scales", C.c_void_p),
                ("rows", C.c_size_t), ("base", C.c_size_t), ("lo", C.c_size_t), ("hi", C.c_size_t),
                ("row0", C.c_size_t)]

_vp, _sz, _f, _i = C.c_void_p, C.c_size_t, C.c_float, C.c_int

SIGNATURES = {
    "mb_ctx_create": (_i, [_i, C.POINTER(_vp)]),
    "mb_ctx_destroy": (None, [_vp]),
    "mb_ctx_set_sm_limit": (_i, [_vp, _i]),
    "mb_ctx_set_wait_limit_us": (_i, [_vp, C.c_uint32]),
    "mb_last_error": (C.c_char_p, [_vp]),
    "mb_version": (C.c_char_p, []),
    "mb_check_flags": (_i, [_vp, _vp, C.POINTER(C.c_int32)]),
    "mb_nvfp4_quantize_weight": (_i, [_vp, _vp, _vp, _sz, _sz, _vp, _vp, C.POINTER(_f)]),
    "mb_nvfp4_quantize_act": (_i, [_vp, _vp, _vp, _i, _sz, _sz, _i, _f, _vp, _sz, _vp, _vp, _i, _vp]),
    "mb_mxfp4_to_nvfp4_scales": (_i, [_vp, _vp, _vp, _sz, _vp, C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "mb_nvfp4_gather_rows": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _vp, _sz, _vp, _vp]),
    "mb_nvfp4_dequantize": (_i, [_vp, _vp, _vp, _vp, _f, _sz, _sz, _vp, _i]),
    "mb_nvfp4_sf_bytes": (_sz, [_sz, _sz]),
    "mb_nvfp4_tile_scales": (_i, [_vp, _vp, _vp, _sz, _sz, _vp]),
    "mb_nvfp4_untile_scales": (_i, [_vp, _vp, _vp, _sz, _sz, _vp]),
    "mb_nvfp4_gemv_w4a16": (_i, [_vp, _vp, _vp, _sz, _vp, _vp, _f, _sz, _sz, _vp, _i]),
    "mb_nvfp4_gemv_workspace": (_sz, [_sz, _sz, _sz]),
    "mb_nvfp4_gemv_w4a16_ws": (_i, [_vp, _vp, _vp, _sz, _vp, _vp, _f, _sz, _sz, _vp, _i, _vp, _sz]),
    "mb_nvfp4_gemm_w4a4": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _sz, _sz, _sz, _vp, _i, _i]),
    "mb_nvfp4_gemm_splitk_workspace": (_sz, [_sz, _sz, _sz]),
    "mb_nvfp4_gemm_w4a4_splitk": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _sz, _sz, _sz, _vp, _i, _vp, _sz]),
    "mb_nvfp4_gemm_w4a4_grouped": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp, _i, _i,
                                        _vp, _vp]),
    "mb_nvfp4_quantize_grouped": (_i, [_vp, _vp, _vp, _i, _vp, _sz, _vp, _sz, _sz, _vp, _vp]),
    "mb_nvfp4_gemv_w4a4_grouped": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp, _i]),
    "mb_nvfp4_gemm_w4a4_stacked": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _vp, _i, _i, _vp, _vp, _sz]),
    "mb_bf16_gemm": (_i, [_vp, _vp, _vp, _vp, _f, _sz, _sz, _sz, _vp, _i]),
    "mb_nvfp4_gemm_w4a16_workspace": (_sz, [_sz, _sz, _sz]),
    "mb_nvfp4_gemm_w4a16": (_i, [_vp, _vp, _vp, _vp, _vp, _f, _sz, _sz, _sz, _vp, _i, _vp, _sz]),
    "mb_bf16_gemm_splitk_workspace": (_sz, [_sz, _sz, _sz]),
    "mb_gemm_splitk_plan": (C.c_int, [_vp, C.c_int, _sz, _sz, _sz, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "mb_bf16_gemm_splitk": (_i, [_vp, _vp, _vp, _vp, _f, _sz, _sz, _sz, _vp, _i, _vp, _sz]),
    "mb_router_topk_softmax": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _i, _f, _vp, _vp]),
    "mb_router_topk_sinks": (_i, [_vp, _vp, _vp, _vp, _f, _f, _sz, _sz, _sz, _sz, _vp, _vp, _vp]),
    "mb_router_topk": (_i, [_vp, _vp, _vp, _vp, _i, _sz, _sz, _sz, _i, _f, _vp, _vp]),
    "mb_moe_plan_rows": (_sz, [_sz, _sz, _sz]),
    "mb_moe_plan_workspace": (_sz, [_sz, _sz, _sz]),
    "mb_moe_plan": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz]),
    "mb_moe_scatter_weighted": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _sz, _sz, _sz, _vp]),
    "mb_attention_workspace": (_sz, [_sz, _sz, _sz, _sz, _sz, _sz]),
    "mb_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _f, _i, _vp, _vp, _sz]),
    "mb_attention_window": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _f, _sz, _vp, _vp, _sz]),
    "mb_attention_decode_ext": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _f, _sz, _vp, _sz, _vp, _vp,
                                     _sz, _vp, _vp, _sz]),
    "mb_attention_fp4kv": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _f, _i, _sz,
                                _vp, _vp, _sz]),
    "mb_attention_runs_workspace": (_sz, [_vp, _sz, _i, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _i, _i]),
    "mb_attention_runs": (_i, [_vp, _vp, _vp, _i, _vp, _sz, _i, _vp, _sz, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz,
                               _sz, _f, _vp, _i, _vp, _sz]),
    "mb_attention_decode_static_warm": (_i, [_vp]),
    "mb_attention_decode_static": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _sz, _f, _i, _vp]),
    "mb_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _sz, _sz, _f, _vp]),
    "mb_rmsnorm_inkling": (_i, [_vp, _vp, _vp, _i, _vp, _sz, _sz, _f, _vp, _i]),
    "mb_gate_up_silu": (_i, [_vp, _vp, _vp, _i, _sz, _sz, _i, _vp, _i]),
    "mb_add": (_i, [_vp, _vp, _vp, _vp, _sz, _vp]),
    "mb_add_f32": (_i, [_vp, _vp, _vp, _vp, _sz, _vp]),
    "mb_swiglu": (_i, [_vp, _vp, _vp, _vp, _sz, _vp]),
    "mb_rope": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _vp, _vp]),
    "mb_residual_norm_quantize": (_i, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _f, _vp, _vp, _vp]),
    "mb_rope_append": (_i, [_vp, _vp, _vp, _sz, _sz, _sz, _sz, _sz, _sz, _vp, _vp, _vp, _vp, _sz]),
    "mb_tp_shard": (_i, [_sz, _sz, _sz, C.POINTER(_sz), C.POINTER(_sz)]),
    "mb_tp_unique_id": (_i, [_vp, C.POINTER(C.c_uint8)]),
    "mb_tp_form": (_i, [_vp, C.POINTER(C.c_uint8), _i, _i]),
    "mb_tp_warm": (_i, [_vp, _vp]),
    "mb_tp_all_reduce": (_i, [_vp, _vp, _vp, _sz, _i]),
    "mb_tp_reduce_scatter_f32": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "mb_tp_all_gather": (_i, [_vp, _vp, _vp, _vp, _sz]),
    "mb_tp_close": (_i, [_vp]),
    "mb_tp_symm_bytes": (_sz, [_sz, _sz]),
    "mb_tp_symm_create": (_i, [_vp, _sz, _sz, C.POINTER(C.c_uint8)]),
    "mb_tp_symm_attach": (_i, [_vp, C.POINTER(C.c_uint8), _i, _i]),
    "mb_tp_symm_local": (_i, [_vp, C.POINTER(_vp)]),
    "mb_tp_symm_attach_ptrs": (_i, [_vp, C.POINTER(_vp), _i, _i]),
    "mb_nvfp4_gemm_w4a4_scatter": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _f, _sz, _sz, _sz, _i]),
    "mb_tp_reduce_residual": (_i, [_vp, _vp, _vp, _sz, _sz, _i, C.POINTER(_vp)]),
    "mb_tp_symm_destroy": (_i, [_vp]),
    "mb_tp_bulk_header_bytes": (_sz, []),
    "mb_tp_bulk_create": (_i, [_vp, _sz, C.POINTER(C.c_uint8)]),
    "mb_tp_bulk_attach": (_i, [_vp, C.POINTER(C.c_uint8), _i, _i]),
    "mb_tp_bulk_attach_ptrs": (_i, [_vp, C.POINTER(_vp), _i, _i]),
    "mb_tp_bulk_local": (_i, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "mb_tp_bulk_reduce_scatter_f32": (_i, [_vp, _vp, _sz, _sz, _sz, _vp, _i]),
    "mb_tp_bulk_all_gather": (_i, [_vp, _vp, _sz, _sz, _sz, _sz, _i]),
    "mb_tp_bulk_destroy": (_i, [_vp]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)   # AttributeError here means header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args


class MaryError(RuntimeError):
    """A refusal or failure reported by the C ABI (code + mb_last_error text)."""

    def __init__(self, code, text):
        super().__init__(f"[{code}] {text}")
        self.code = code


class Context:
    """One mb_ctx: a device plus its status words. Mirrors the compute client the
    reference's launch functions take."""

    def __init__(self, device=0):
        h = _vp()
        rc = lib.mb_ctx_create(int(device), C.byref(h))
        if rc != OK:
            raise MaryError(rc, f"mb_ctx_create({device}) failed: no sm_100 CUDA device, and no fallback exists")
        self.handle = h
        self.device = int(device)

    def close(self):
        if self.handle:
            lib.mb_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, rc):
        if rc != OK:
            raise MaryError(rc, lib.mb_last_error(self.handle).decode())

    def check_flags(self, stream=None):
        out = (C.c_int32 * 8)()
        rc = lib.mb_check_flags(self.handle, stream, out)
        return rc, list(out)


_CONTEXTS = {}


def context(device=None):
    """The process-wide context of a device (created on first use)."""
    import torch
    if device is None:
        device = torch.cuda.current_device()
    device = int(device)
    if device not in _CONTEXTS:
        _CONTEXTS[device] = Context(device)
    return _CONTEXTS[device]
