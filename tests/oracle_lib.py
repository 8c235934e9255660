"""ctypes binding of the CPU oracle (oracle/liboracle.so) for the tests.

The oracle is the checker: only tests, the smoke entry and the CPU-baseline leg of
the benchmark load it. The product package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(_ROOT, "oracle", "liboracle.so")


def build():
    src = os.path.join(_ROOT, "oracle", "oracle.cpp")
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", os.path.join(_ROOT, "oracle")],
                              stdout=subprocess.DEVNULL)
    return _SO


def _ptr(a, t):
    return a.ctypes.data_as(C.POINTER(t))


class Oracle:
    def __init__(self):
        self.lib = L = C.CDLL(build())
        u8, u16, u32, f32, f64 = C.c_uint8, C.c_uint16, C.c_uint32, C.c_float, C.c_double
        sz, i32, i64 = C.c_size_t, C.c_int32, C.c_int64
        P = C.POINTER
        sig = {
            "orc_e4m3_to_f32": (f32, [u8]),
            "orc_e4m3_from_f32": (u8, [f32]),
            "orc_e2m1_code": (u8, [f32]),
            "orc_code_of": (u8, [f32, f32]),
            "orc_decode_code": (f32, [u8]),
            "orc_cvt_e2m1": (u8, [f32]),
            "orc_f32_to_bf16": (u16, [f32]),
            "orc_bf16_to_f32": (f32, [u16]),
            "orc_global_scale": (f32, [P(f32), sz]),
            "orc_scale2_of_tensor": (C.c_int, [P(f32), sz, P(f32)]),
            "orc_block_unit": (None, [P(f32), f32, P(u8), P(f32)]),
            "orc_pack_nearest": (C.c_int, [P(f32), sz, sz, P(u8), P(u8), P(f32)]),
            "orc_payload_len": (sz, [sz]),
            "orc_decode_payload": (C.c_int, [P(u8), sz, sz, P(f32)]),
            "orc_dequantize": (None, [P(u8), P(u8), f32, sz, P(f32)]),
            "orc_quantize_weight_bf16": (C.c_int, [P(u16), sz, sz, P(u8), P(u8), P(f32)]),
            "orc_quantize_act_scaled": (None, [P(f32), sz, sz, f32, P(u8), P(u8)]),
            "orc_quantize_act_rows": (None, [P(f32), sz, sz, P(f32), P(u8), P(u8)]),
            "orc_quantize_act_recip": (None, [P(f32), sz, sz, P(u8), P(u8)]),
            "orc_linear_w4a16": (None, [P(u16), P(u8), P(u8), f32, sz, sz, sz, P(f64)]),
            "orc_linear_cpu_lane": (None, [P(u16), P(f32), sz, sz, sz, P(u16)]),
            "orc_linear_w4a4": (None, [P(u8), P(u8), P(u8), P(u8), P(f32), f32, sz, sz, sz, P(f32)]),
            "orc_w4a4_grouped": (None, [P(u16), C.c_int, P(u32), sz, P(f32), P(f32), P(u8), P(u8), sz, sz, P(u8), P(u8),
                                        P(f32)]),
            "orc_rmsnorm_inkling": (None, [P(u16), P(f32), P(f32), sz, sz, f32, P(u16), P(f32)]),
            "orc_linear_bf16": (None, [P(u16), P(u16), sz, sz, sz, P(f32)]),
            "orc_e4m3_from_pow2": (C.c_int, [C.c_int]),
            "orc_mxfp4_transcode": (C.c_int, [P(u8), sz, P(u8), P(C.c_longlong)]),
            "orc_mxfp4_decode": (None, [P(u8), P(u8), sz, sz, P(f32)]),
            "orc_router_scores_softmax": (None, [P(f32), sz, sz, P(f32)]),
            "orc_router_scores_sigmoid": (None, [P(f32), sz, sz, P(f32)]),
            "orc_router_select": (C.c_int, [P(f32), P(f32), sz, sz, sz, C.c_int, f32, P(u32), P(f32)]),
            "orc_router_sinks": (C.c_int, [P(f32), P(f32), f32, f32, sz, sz, sz, sz, P(u32), P(f32), P(f32), P(sz)]),
            "orc_router_logits": (None, [P(u16), P(u16), sz, sz, sz, P(f32)]),
            "orc_row_plan": (C.c_longlong, [P(u32), P(f32), sz, sz, sz, sz, sz, P(i32), P(f32), P(u32), P(u32),
                                            P(u32), P(u32), P(u32), P(u32), P(u32)]),
            "orc_gather_rows_bf16": (None, [P(u16), P(i32), sz, sz, P(u16)]),
            "orc_gate_up_silu": (None, [P(f32), sz, sz, C.c_int, C.c_int, P(f32)]),
            "orc_scatter_weighted": (None, [P(f32), P(f32), P(u32), P(u32), sz, sz, sz, P(f32)]),
            "orc_moe_experts": (C.c_int, [P(u16), sz, sz, sz, sz, P(u32), P(f32), sz, P(u8), P(u8), P(f32), P(u8),
                                          P(u8), P(f32), C.c_int, P(f32)]),
            "orc_attention": (C.c_int, [P(f32), P(f32), P(f32), sz, sz, sz, sz, sz, sz, P(i64), f32, C.c_longlong,
                                        P(f64)]),
            "orc_attention_rel": (C.c_int, [P(f32), P(f32), P(f32), sz, sz, sz, sz, sz, sz, P(i64), f32, C.c_longlong,
                                            P(f32), sz, P(f64)]),
            "orc_rmsnorm_breeze": (None, [P(u16), P(u16), sz, sz, f32, P(u16)]),
            "orc_add_bf16": (None, [P(u16), P(u16), sz, P(u16)]),
            "orc_swiglu_bf16": (None, [P(u16), P(u16), sz, P(u16)]),
            "orc_rope_bf16": (None, [P(u16), sz, sz, sz, sz, P(f32), P(u16)]),
            "orc_tp_shard": (C.c_int, [sz, sz, sz, P(sz), P(sz)]),
            "orc_rng_normal_f32": (None, [C.c_uint64, sz, f64, P(f32)]),
            "orc_rng_normal_bf16": (None, [C.c_uint64, sz, f64, P(u16)]),
            "orc_sample": (None, [sz, sz, P(f32)]),
            "orc_threads": (C.c_int, []),
            "orc_set_threads": (None, [C.c_int]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args

    # ---- scalar codec -----------------------------------------------------
    def e4m3_to_f32(self, b):
        return float(self.lib.orc_e4m3_to_f32(int(b)))

    def e4m3_from_f32(self, v):
        return int(self.lib.orc_e4m3_from_f32(float(np.float32(v))))

    def e2m1_code(self, m):
        return int(self.lib.orc_e2m1_code(float(np.float32(m))))

    def code_of(self, v, unit):
        return int(self.lib.orc_code_of(float(np.float32(v)), float(np.float32(unit))))

    def decode_code(self, c):
        return float(self.lib.orc_decode_code(int(c)))

    # ---- planes -----------------------------------------------------------
    def global_scale(self, w):
        w = np.ascontiguousarray(w, np.float32)
        return np.float32(self.lib.orc_global_scale(_ptr(w, C.c_float), w.size))

    def block_unit(self, block, scale2):
        block = np.ascontiguousarray(block, np.float32)
        b = C.c_uint8()
        u = C.c_float()
        self.lib.orc_block_unit(_ptr(block, C.c_float), float(np.float32(scale2)), C.byref(b), C.byref(u))
        return b.value, np.float32(u.value)

    def pack_nearest(self, w, cols):
        w = np.ascontiguousarray(w, np.float32).reshape(-1)
        rows = w.size // cols
        codes = np.empty(w.size // 2, np.uint8)
        scales = np.empty(w.size // 16, np.uint8)
        s2 = C.c_float()
        rc = self.lib.orc_pack_nearest(_ptr(w, C.c_float), rows, cols, _ptr(codes, C.c_uint8),
                                       _ptr(scales, C.c_uint8), C.byref(s2))
        if rc != 0:
            raise ValueError("cols is not a positive multiple of 16")
        return codes, scales, np.float32(s2.value)

    @staticmethod
    def payload(codes, scales, scale2):
        return np.concatenate([codes, scales, np.frombuffer(np.float32(scale2).tobytes(), np.uint8)])

    def decode_payload(self, payload, elems):
        payload = np.ascontiguousarray(payload, np.uint8)
        out = np.empty(elems, np.float32)
        rc = self.lib.orc_decode_payload(_ptr(payload, C.c_uint8), payload.size, elems, _ptr(out, C.c_float))
        if rc != 0:
            raise ValueError("payload length mismatch")
        return out

    def dequantize(self, codes, scales, scale2=1.0):
        codes = np.ascontiguousarray(codes, np.uint8).reshape(-1)
        scales = np.ascontiguousarray(scales, np.uint8).reshape(-1)
        out = np.empty(codes.size * 2, np.float32)
        self.lib.orc_dequantize(_ptr(codes, C.c_uint8), _ptr(scales, C.c_uint8), float(np.float32(scale2)),
                                out.size, _ptr(out, C.c_float))
        return out

    def quantize_weight_bf16(self, w_bits, n, k):
        w_bits = np.ascontiguousarray(w_bits, np.uint16).reshape(-1)
        codes = np.empty(n * k // 2, np.uint8)
        scales = np.empty(n * k // 16, np.uint8)
        s2 = C.c_float()
        rc = self.lib.orc_quantize_weight_bf16(_ptr(w_bits, C.c_uint16), n, k, _ptr(codes, C.c_uint8),
                                               _ptr(scales, C.c_uint8), C.byref(s2))
        if rc != 0:
            raise ValueError("NVFP4 source has a non-finite weight")
        return codes, scales, np.float32(s2.value)

    def quantize_act_scaled(self, x, rows, k, input_scale=1.0):
        x = np.ascontiguousarray(x, np.float32).reshape(-1)
        codes = np.empty(rows * k // 2, np.uint8)
        scales = np.empty(rows * k // 16, np.uint8)
        self.lib.orc_quantize_act_scaled(_ptr(x, C.c_float), rows, k, float(np.float32(input_scale)),
                                         _ptr(codes, C.c_uint8), _ptr(scales, C.c_uint8))
        return codes, scales

    def quantize_act_rows(self, x, rows, k):
        x = np.ascontiguousarray(x, np.float32).reshape(-1)
        codes = np.empty(rows * k // 2, np.uint8)
        scales = np.empty(rows * k // 16, np.uint8)
        rs = np.empty(rows, np.float32)
        self.lib.orc_quantize_act_rows(_ptr(x, C.c_float), rows, k, _ptr(rs, C.c_float), _ptr(codes, C.c_uint8),
                                       _ptr(scales, C.c_uint8))
        return codes, scales, rs

    def quantize_act_recip(self, x, rows, k):
        x = np.ascontiguousarray(x, np.float32).reshape(-1)
        codes = np.empty(rows * k // 2, np.uint8)
        scales = np.empty(rows * k // 16, np.uint8)
        self.lib.orc_quantize_act_recip(_ptr(x, C.c_float), rows, k, _ptr(codes, C.c_uint8), _ptr(scales, C.c_uint8))
        return codes, scales

    # ---- linears ----------------------------------------------------------
    def linear_w4a16(self, x_bits, codes, scales, scale2, M, N, K):
        x_bits = np.ascontiguousarray(x_bits, np.uint16).reshape(-1)
        out = np.empty(M * N, np.float64)
        self.lib.orc_linear_w4a16(_ptr(x_bits, C.c_uint16), _ptr(codes, C.c_uint8), _ptr(scales, C.c_uint8),
                                  float(np.float32(scale2)), M, N, K, _ptr(out, C.c_double))
        return out.reshape(M, N)

    def linear_cpu_lane(self, x_bits, w_dense, M, N, K):
        x_bits = np.ascontiguousarray(x_bits, np.uint16).reshape(-1)
        w_dense = np.ascontiguousarray(w_dense, np.float32).reshape(-1)
        out = np.empty(M * N, np.uint16)
        self.lib.orc_linear_cpu_lane(_ptr(x_bits, C.c_uint16), _ptr(w_dense, C.c_float), M, N, K,
                                     _ptr(out, C.c_uint16))
        return out.reshape(M, N)

    def linear_w4a4(self, a_codes, a_scales, b_codes, b_scales, alpha, M, N, K, rowscale=None):
        out = np.empty(M * N, np.float32)
        rs = None
        if rowscale is not None:
            rowscale = np.ascontiguousarray(rowscale, np.float32)
            rs = _ptr(rowscale, C.c_float)
        self.lib.orc_linear_w4a4(_ptr(a_codes, C.c_uint8), _ptr(a_scales, C.c_uint8), _ptr(b_codes, C.c_uint8),
                                 _ptr(b_scales, C.c_uint8), rs, float(np.float32(alpha)), M, N, K,
                                 _ptr(out, C.c_float))
        return out.reshape(M, N)

    def w4a4_grouped(self, x_bits, x_per_group, ids, input_scale, alpha, bank_codes, bank_scales, n, k):
        """w4a4_grouped_bf16 (src/nn/nvfp4_gemm.rs:462-523) -> (out f32 [groups, n], activation codes, scales)."""
        x_bits = np.ascontiguousarray(x_bits, np.uint16).reshape(-1)
        ids = np.ascontiguousarray(ids, np.uint32)
        input_scale = np.ascontiguousarray(input_scale, np.float32)
        alpha = np.ascontiguousarray(alpha, np.float32)
        bank_codes = np.ascontiguousarray(bank_codes, np.uint8).reshape(-1)
        bank_scales = np.ascontiguousarray(bank_scales, np.uint8).reshape(-1)
        groups = ids.size
        out = np.empty((groups, n), np.float32)
        a_codes = np.empty((groups, k // 2), np.uint8)
        a_scales = np.empty((groups, k // 16), np.uint8)
        self.lib.orc_w4a4_grouped(_ptr(x_bits, C.c_uint16), int(x_per_group), _ptr(ids, C.c_uint32), groups,
                                  _ptr(input_scale, C.c_float), _ptr(alpha, C.c_float), _ptr(bank_codes, C.c_uint8),
                                  _ptr(bank_scales, C.c_uint8), n, k, _ptr(a_codes, C.c_uint8),
                                  _ptr(a_scales, C.c_uint8), _ptr(out, C.c_float))
        return out, a_codes, a_scales

    def rmsnorm_inkling(self, x, gain, rows, width, eps, out_bf16=True):
        """rms_norm_kernel (src/models/inkling/resid.rs:272-322). x: uint16 array = bf16 bits, float32 array = f32."""
        gain = np.ascontiguousarray(gain, np.float32)
        x = np.ascontiguousarray(x)
        xb = _ptr(x, C.c_uint16) if x.dtype == np.uint16 else None
        xf = _ptr(x, C.c_float) if x.dtype == np.float32 else None
        assert (xb is None) != (xf is None)
        out = np.empty(rows * width, np.uint16 if out_bf16 else np.float32)
        self.lib.orc_rmsnorm_inkling(xb, xf, _ptr(gain, C.c_float), rows, width, float(np.float32(eps)),
                                     _ptr(out, C.c_uint16) if out_bf16 else None,
                                     None if out_bf16 else _ptr(out, C.c_float))
        return out.reshape(rows, width)

    def linear_bf16(self, x_bits, w_bits, M, N, K):
        x_bits = np.ascontiguousarray(x_bits, np.uint16).reshape(-1)
        w_bits = np.ascontiguousarray(w_bits, np.uint16).reshape(-1)
        out = np.empty(M * N, np.float32)
        self.lib.orc_linear_bf16(_ptr(x_bits, C.c_uint16), _ptr(w_bits, C.c_uint16), M, N, K, _ptr(out, C.c_float))
        return out.reshape(M, N)

    # ---- MXFP4 relabelling ------------------------------------------------
    def mxfp4_transcode(self, scale):
        """transcode_to_nvfp4's scale half (src/nn/mxfp4.rs:319-375) -> (block scales [2n], global exponent g,
        any subnormal block scale); raises ValueError with the reference's error kinds."""
        scale = np.ascontiguousarray(scale, np.uint8).reshape(-1)
        out = np.empty(2 * scale.size, np.uint8)
        info = (C.c_longlong * 3)()
        rc = self.lib.orc_mxfp4_transcode(_ptr(scale, C.c_uint8), scale.size, _ptr(out, C.c_uint8), info)
        if rc == 1:
            raise ValueError(f"ScaleNan index {info[0]}")
        if rc == 2:
            raise ValueError(f"ExponentSpan e_min {info[0]} e_max {info[1]} octaves {info[2]}")
        if rc == 3:
            raise ValueError(f"GlobalScaleRange g {info[0]}")
        return out, int(info[0]), bool(info[1])

    def mxfp4_decode(self, packed, scale, rows, cols):
        packed = np.ascontiguousarray(packed, np.uint8).reshape(-1)
        scale = np.ascontiguousarray(scale, np.uint8).reshape(-1)
        out = np.empty(rows * cols, np.float32)
        self.lib.orc_mxfp4_decode(_ptr(packed, C.c_uint8), _ptr(scale, C.c_uint8), rows, cols, _ptr(out, C.c_float))
        return out

    # ---- router / MoE -----------------------------------------------------
    def router_scores_softmax(self, logits):
        logits = np.ascontiguousarray(logits, np.float32)
        t, n = logits.shape
        v = np.empty((t, n), np.float32)
        self.lib.orc_router_scores_softmax(_ptr(logits, C.c_float), t, n, _ptr(v, C.c_float))
        return v

    def router_scores_sigmoid(self, logits):
        logits = np.ascontiguousarray(logits, np.float32)
        t, n = logits.shape
        v = np.empty((t, n), np.float32)
        self.lib.orc_router_scores_sigmoid(_ptr(logits, C.c_float), t, n, _ptr(v, C.c_float))
        return v

    def router_select(self, scores, k, bias=None, renormalize=True, scaling=1.0):
        scores = np.ascontiguousarray(scores, np.float32)
        t, n = scores.shape
        idx = np.empty((t, k), np.uint32)
        w = np.empty((t, k), np.float32)
        b = None
        if bias is not None:
            bias = np.ascontiguousarray(bias, np.float32)
            b = _ptr(bias, C.c_float)
        rc = self.lib.orc_router_select(_ptr(scores, C.c_float), b, t, n, k, int(renormalize),
                                        float(np.float32(scaling)), _ptr(idx, C.c_uint32), _ptr(w, C.c_float))
        if rc != 0:
            raise ValueError("router: non-finite score")
        return idx, w

    def router_sinks(self, logits, bias, n_routed, k, global_scale=1.0, route_scale=1.0):
        """route_from_logits (src/models/inkling/block.rs:176-258) -> (experts, weights, shared_gammas)."""
        logits = np.ascontiguousarray(logits, np.float32)
        tokens, rows = logits.shape
        n_shared = rows - n_routed
        bias = np.ascontiguousarray(bias, np.float32)
        assert bias.size == n_routed
        idx = np.empty((tokens, k), np.uint32)
        w = np.empty((tokens, k), np.float32)
        gam = np.empty((tokens, max(n_shared, 1)), np.float32)
        bad = (C.c_size_t * 2)()
        rc = self.lib.orc_router_sinks(_ptr(logits, C.c_float), _ptr(bias, C.c_float), float(np.float32(global_scale)),
                                       float(np.float32(route_scale)), tokens, n_routed, n_shared, k,
                                       _ptr(idx, C.c_uint32), _ptr(w, C.c_float), _ptr(gam, C.c_float), bad)
        if rc != 0:
            raise ValueError(f"router logit is non-finite at token {bad[0]}, row {bad[1]}")
        return idx, w, gam[:, :n_shared]

    def router_logits(self, h_bits, gate_bits, tokens, hid, n):
        h_bits = np.ascontiguousarray(h_bits, np.uint16).reshape(-1)
        gate_bits = np.ascontiguousarray(gate_bits, np.uint16).reshape(-1)
        out = np.empty((tokens, n), np.float32)
        self.lib.orc_router_logits(_ptr(h_bits, C.c_uint16), _ptr(gate_bits, C.c_uint16), tokens, hid, n,
                                   _ptr(out, C.c_float))
        return out

    def row_plan(self, idx, weight, n_experts, mtile):
        idx = np.ascontiguousarray(idx, np.uint32)
        weight = np.ascontiguousarray(weight, np.float32)
        tokens, k = idx.shape
        m_cap = tokens * k + n_experts * mtile
        row_tok = np.empty(m_cap, np.int32)
        row_wgt = np.empty(m_cap, np.float32)
        slot_e = np.empty(n_experts, np.uint32)
        slot_r0 = np.empty(n_experts, np.uint32)
        slot_n = np.empty(n_experts, np.uint32)
        tok_rows = np.zeros((tokens, k), np.uint32)
        tok_cnt = np.empty(tokens, np.uint32)
        ns = C.c_uint32()
        kmax = C.c_uint32()
        m = self.lib.orc_row_plan(_ptr(idx, C.c_uint32), _ptr(weight, C.c_float), tokens, k, n_experts, mtile, m_cap,
                                  _ptr(row_tok, C.c_int32), _ptr(row_wgt, C.c_float), _ptr(slot_e, C.c_uint32),
                                  _ptr(slot_r0, C.c_uint32), _ptr(slot_n, C.c_uint32), C.byref(ns),
                                  _ptr(tok_rows, C.c_uint32), _ptr(tok_cnt, C.c_uint32), C.byref(kmax))
        assert m >= 0
        s = ns.value
        return dict(m_total=int(m), row_tok=row_tok[:m], row_wgt=row_wgt[:m], slot_expert=slot_e[:s],
                    slot_row0=slot_r0[:s], slot_rows=slot_n[:s], tok_rows=tok_rows, tok_cnt=tok_cnt,
                    kmax=int(kmax.value))

    def gate_up_silu(self, both, rows, inter, halved=False, round_bf16=False):
        both = np.ascontiguousarray(both, np.float32).reshape(-1)
        act = np.empty(rows * inter, np.float32)
        self.lib.orc_gate_up_silu(_ptr(both, C.c_float), rows, inter, int(halved), int(round_bf16),
                                  _ptr(act, C.c_float))
        return act.reshape(rows, inter)

    def scatter_weighted(self, y, row_wgt, tok_rows, tok_cnt, h):
        y = np.ascontiguousarray(y, np.float32)
        row_wgt = np.ascontiguousarray(row_wgt, np.float32)
        tok_rows = np.ascontiguousarray(tok_rows, np.uint32)
        tok_cnt = np.ascontiguousarray(tok_cnt, np.uint32)
        tokens, ks = tok_rows.shape
        out = np.empty((tokens, h), np.float32)
        self.lib.orc_scatter_weighted(_ptr(y, C.c_float), _ptr(row_wgt, C.c_float), _ptr(tok_rows, C.c_uint32),
                                      _ptr(tok_cnt, C.c_uint32), tokens, ks, h, _ptr(out, C.c_float))
        return out

    def moe_experts(self, x_bits, idx, weight, w13, w2, h, inter, n_experts, halved=False):
        """w13/w2: (codes, scales, scale2[E]) with expert-major planes."""
        x_bits = np.ascontiguousarray(x_bits, np.uint16)
        tokens = x_bits.size // h
        idx = np.ascontiguousarray(idx, np.uint32)
        weight = np.ascontiguousarray(weight, np.float32)
        k = idx.shape[1]
        out = np.empty((tokens, h), np.float32)
        c13, s13, g13 = [np.ascontiguousarray(a) for a in w13]
        c2, s2, g2 = [np.ascontiguousarray(a) for a in w2]
        g13 = np.ascontiguousarray(g13, np.float32)
        g2 = np.ascontiguousarray(g2, np.float32)
        rc = self.lib.orc_moe_experts(_ptr(x_bits, C.c_uint16), tokens, h, inter, n_experts, _ptr(idx, C.c_uint32),
                                      _ptr(weight, C.c_float), k, _ptr(c13, C.c_uint8), _ptr(s13, C.c_uint8),
                                      _ptr(g13, C.c_float), _ptr(c2, C.c_uint8),
                                      _ptr(s2, C.c_uint8), _ptr(g2, C.c_float), int(halved),
                                      _ptr(out, C.c_float))
        assert rc == 0
        return out

    # ---- attention / layer glue --------------------------------------------
    def attention(self, q, k, v, heads, kv_heads, D, q0, scale, key_pos=None, window=0, rel=None):
        q = np.ascontiguousarray(q, np.float32)
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        nq = q.size // (heads * D)
        keys = k.size // (kv_heads * D)
        out = np.empty(q.size, np.float64)
        kp = None
        if key_pos is not None:
            key_pos = np.ascontiguousarray(key_pos, np.int64)
            kp = _ptr(key_pos, C.c_int64)
        rp, eff = None, 0
        if rel is not None:
            rel = np.ascontiguousarray(rel, np.float32)
            eff = rel.size // (nq * heads)
            rp = _ptr(rel, C.c_float)
        rc = self.lib.orc_attention_rel(_ptr(q, C.c_float), _ptr(k, C.c_float), _ptr(v, C.c_float), nq, keys, heads,
                                        kv_heads, D, q0, kp, float(np.float32(scale)), int(window), rp, eff,
                                        _ptr(out, C.c_double))
        if rc != 0:
            raise ValueError("a query has no visible key")
        return out.reshape(nq, heads * D)

    def rmsnorm_breeze(self, x_bits, w_bits, rows, width, eps):
        x_bits = np.ascontiguousarray(x_bits, np.uint16).reshape(-1)
        w_bits = np.ascontiguousarray(w_bits, np.uint16).reshape(-1)
        y = np.empty(rows * width, np.uint16)
        self.lib.orc_rmsnorm_breeze(_ptr(x_bits, C.c_uint16), _ptr(w_bits, C.c_uint16), rows, width,
                                    float(np.float32(eps)), _ptr(y, C.c_uint16))
        return y.reshape(rows, width)

    def add_bf16(self, a, b):
        a = np.ascontiguousarray(a, np.uint16).reshape(-1)
        b = np.ascontiguousarray(b, np.uint16).reshape(-1)
        out = np.empty(a.size, np.uint16)
        self.lib.orc_add_bf16(_ptr(a, C.c_uint16), _ptr(b, C.c_uint16), a.size, _ptr(out, C.c_uint16))
        return out

    def swiglu_bf16(self, g, u):
        g = np.ascontiguousarray(g, np.uint16).reshape(-1)
        u = np.ascontiguousarray(u, np.uint16).reshape(-1)
        out = np.empty(g.size, np.uint16)
        self.lib.orc_swiglu_bf16(_ptr(g, C.c_uint16), _ptr(u, C.c_uint16), g.size, _ptr(out, C.c_uint16))
        return out

    def rope_bf16(self, x_bits, tokens, heads, d, past, inv_freq):
        x_bits = np.ascontiguousarray(x_bits, np.uint16).reshape(-1)
        inv_freq = np.ascontiguousarray(inv_freq, np.float32)
        out = np.empty(x_bits.size, np.uint16)
        self.lib.orc_rope_bf16(_ptr(x_bits, C.c_uint16), tokens, heads, d, past, _ptr(inv_freq, C.c_float),
                               _ptr(out, C.c_uint16))
        return out

    def tp_shard(self, rank, world, extent):
        lo, hi = C.c_size_t(), C.c_size_t()
        rc = self.lib.orc_tp_shard(rank, world, extent, C.byref(lo), C.byref(hi))
        if rc != 0:
            raise ValueError(f"extent {extent} does not divide by world {world}")
        return lo.value, hi.value

    # ---- fixtures -----------------------------------------------------------
    def normal_f32(self, seed, n, sigma=1.0):
        out = np.empty(n, np.float32)
        self.lib.orc_rng_normal_f32(seed, n, float(sigma), _ptr(out, C.c_float))
        return out

    def normal_bf16(self, seed, n, sigma=1.0):
        out = np.empty(n, np.uint16)
        self.lib.orc_rng_normal_bf16(seed, n, float(sigma), _ptr(out, C.c_uint16))
        return out

    def sample(self, rows, cols):
        out = np.empty(rows * cols, np.float32)
        self.lib.orc_sample(rows, cols, _ptr(out, C.c_float))
        return out

    def threads(self):
        return int(self.lib.orc_threads())

    def set_threads(self, n):
        self.lib.orc_set_threads(int(n))


_ORACLE = None


def oracle():
    global _ORACLE
    if _ORACLE is None:
        _ORACLE = Oracle()
    return _ORACLE


def bf16_bits_to_f32(bits):
    bits = np.ascontiguousarray(bits, np.uint16)
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    """Round-to-nearest-even narrowing, NaN kept quiet."""
    x = np.ascontiguousarray(x, np.float32)
    u = x.view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r
