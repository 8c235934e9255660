"""Host-side mirror of the reference's MoE expert lane over the C ABI.

Follows the Inkling grouped lane (src/models/inkling/assembly.rs:3048-3075 for the
algorithm, :3429-3588 for the launch order; routing per src/models/k3/router.rs):

    router logits (bf16 GEMM, f32 out) -> softmax top-k -> row plan ->
    gather + NVFP4 quantize -> grouped GEMM w13 (+ fused SwiGLU) ->
    NVFP4 quantize -> grouped GEMM w2 -> ordered weighted un-permute.
"""
import ctypes as C
import os

import numpy as np
import torch

from . import _lib
from ._lib import lib, context
from . import nvfp4 as nv

_p = nv._p
_stream = nv._stream


def router_topk_softmax(logits, k, renormalize=True, scaling=1.0):
    """Router::route from logits (src/models/k3/router.rs:343-488, softmax branch)."""
    assert logits.dtype == torch.float32 and logits.is_contiguous() and logits.dim() == 2
    tokens, n_experts = logits.shape
    ctx = context(logits.device.index)
    idx = torch.empty((tokens, k), dtype=torch.int32, device=logits.device)
    weight = torch.empty((tokens, k), dtype=torch.float32, device=logits.device)
    ctx.check(lib.mb_router_topk_softmax(ctx.handle, _stream(), _p(logits), tokens, n_experts, k, int(renormalize),
                                         float(scaling), _p(idx), _p(weight)))
    return idx, weight


ROUTER_SOFTMAX, ROUTER_SIGMOID = 0, 1


def router_topk(logits, k, activation="softmax", bias=None, renormalize=True, scaling=1.0):
    """Router::route from logits with either activation and the selection-only correction bias
    (src/models/k3/router.rs:343-488): the bias moves which experts are picked, never their weights."""
    assert logits.dtype == torch.float32 and logits.is_contiguous() and logits.dim() == 2
    tokens, n_experts = logits.shape
    act = {"softmax": ROUTER_SOFTMAX, "sigmoid": ROUTER_SIGMOID}[activation]
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == n_experts
        assert bias.device == logits.device
    ctx = context(logits.device.index)
    idx = torch.empty((tokens, k), dtype=torch.int32, device=logits.device)
    weight = torch.empty((tokens, k), dtype=torch.float32, device=logits.device)
    ctx.check(lib.mb_router_topk(ctx.handle, _stream(), _p(logits), _p(bias) if bias is not None else None, act,
                                 tokens, n_experts, k, int(renormalize), float(scaling), _p(idx), _p(weight)))
    return idx, weight


def router_topk_sinks(logits, bias, n_routed, k, global_scale=1.0, route_scale=1.0):
    """route_from_logits (src/models/inkling/block.rs:176-258; device form routetopk.rs): the k routed experts
    picked by sigmoid + bias, weighted together with the shared-expert sinks in one softmax over log_sigmoid.
    Returns (experts [tokens, k] int32, weights [tokens, k], shared_gammas [tokens, n_shared])."""
    assert logits.dtype == torch.float32 and logits.is_contiguous() and logits.dim() == 2
    assert bias.dtype == torch.float32 and bias.is_contiguous() and bias.numel() == n_routed
    tokens, rows = logits.shape
    n_shared = rows - n_routed
    ctx = context(logits.device.index)
    idx = torch.empty((tokens, k), dtype=torch.int32, device=logits.device)
    weight = torch.empty((tokens, k), dtype=torch.float32, device=logits.device)
    gammas = torch.empty((tokens, n_shared), dtype=torch.float32, device=logits.device)
    ctx.check(lib.mb_router_topk_sinks(ctx.handle, _stream(), _p(logits), _p(bias), float(global_scale),
                                       float(route_scale), tokens, n_routed, n_shared, k, _p(idx), _p(weight),
                                       _p(gammas) if n_shared else None))
    return idx, weight, gammas


class RowPlan:
    """RowPlan::build on the device (src/models/inkling/moegroup.rs:1850-1909)."""

    def __init__(self, idx, weight, n_experts):
        tokens, k = idx.shape
        dev = idx.device
        ctx = context(dev.index)
        self.tokens, self.k, self.n_experts = tokens, k, n_experts
        self.m_cap = int(lib.mb_moe_plan_rows(tokens, k, n_experts))
        self.row_tok = torch.empty(self.m_cap, dtype=torch.int32, device=dev)
        self.row_wgt = torch.empty(self.m_cap, dtype=torch.float32, device=dev)
        self.tok_rows = torch.empty((tokens, k), dtype=torch.int32, device=dev)
        self.expert_rows = torch.empty(n_experts, dtype=torch.int32, device=dev)
        self.expert_row0 = torch.empty(n_experts, dtype=torch.int32, device=dev)
        self.tile_expert = torch.empty(self.m_cap // 128, dtype=torch.int32, device=dev)
        self.n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
        ws_bytes = int(lib.mb_moe_plan_workspace(tokens, k, n_experts))
        self._ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
        ctx.check(lib.mb_moe_plan(ctx.handle, _stream(), _p(idx), _p(weight), tokens, k, n_experts, _p(self.row_tok),
                                  _p(self.row_wgt), _p(self.tok_rows), _p(self.expert_rows), _p(self.expert_row0),
                                  _p(self.tile_expert), _p(self.n_tiles), _p(self._ws), ws_bytes))


def scatter_weighted(y, plan, h):
    """scatter_weighted(_bf16) (src/models/inkling/moegroup.rs:1690-1716)."""
    ctx = context(y.device.index)
    out = torch.empty((plan.tokens, h), dtype=torch.float32, device=y.device)
    dt = _lib.DT_BF16 if y.dtype == torch.bfloat16 else _lib.DT_F32
    ctx.check(lib.mb_moe_scatter_weighted(ctx.handle, _stream(), _p(y), dt, _p(plan.row_wgt), _p(plan.tok_rows),
                                          plan.tokens, plan.k, h, _p(out)))
    return out


class ExpertBank:
    """An expert bank [experts, n, k] of NVFP4 planes with one scale2 per expert
    (GroupedBank, src/nn/nvfp4_gemm.rs:293-330; the mapped expert buffer of
    src/models/inkling/moegroup.rs:612-751)."""

    def __init__(self, codes, scales_rowmajor, scale2, experts, n, k):
        assert n % 128 == 0 and k % 64 == 0
        self.codes, self.scales, self.experts, self.n, self.k = codes, scales_rowmajor, experts, n, k
        self.scale2 = scale2.to(torch.float32).contiguous()
        per = nv.sf_bytes(n, k)
        self.sf_tiled = torch.empty(experts * per, dtype=torch.uint8, device=codes.device)
        ctx = context(codes.device.index)
        sc = scales_rowmajor.view(experts, n * k // 16)
        for e in range(experts):
            ctx.check(lib.mb_nvfp4_tile_scales(ctx.handle, _stream(), _p(sc[e]), n, k,
                                               C.c_void_p(self.sf_tiled.data_ptr() + e * per)))

    @staticmethod
    def quantize(w):
        """w: [experts, n, k] bf16; every expert gets its own global scale."""
        experts, n, k = w.shape
        codes = torch.empty((experts, n, k // 2), dtype=torch.uint8, device=w.device)
        scales = torch.empty((experts, n, k // 16), dtype=torch.uint8, device=w.device)
        s2 = torch.empty(experts, dtype=torch.float32)
        for e in range(experts):
            q = nv.Nvfp4.quantize(w[e].contiguous())
            codes[e], scales[e], s2[e] = q.codes, q.scales, q.scale2
        return ExpertBank(codes, scales, s2.to(w.device), experts, n, k)


def grouped_gemm(a_codes, a_sf, bank, plan, out_dtype=torch.bfloat16, epilogue=_lib.EPI_PLAIN, skip_pad_rows=False):
    """fp4_linear_grouped(_bf16)_launch (src/models/inkling/moegroup.rs:612-751). With an
    EPI_QUANT_* flag on a SwiGLU epilogue the result comes back as (codes, tiled scale plane).
    skip_pad_rows leaves the plan's padding rows of a bf16/f32 result unwritten (nothing reads them)."""
    ctx = context(a_codes.device.index)
    dev = a_codes.device
    swiglu = (epilogue & 0xFF) in (_lib.EPI_SWIGLU_INTERLEAVED, _lib.EPI_SWIGLU_ROUNDED)
    quant = epilogue & (_lib.EPI_QUANT_RECIP | _lib.EPI_QUANT_SCALED)
    out_sf = None
    if quant:
        out = torch.empty((plan.m_cap, bank.n // 4), dtype=torch.uint8, device=dev)
        out_sf = torch.empty(nv.sf_bytes(plan.m_cap, bank.n // 2), dtype=torch.uint8, device=dev)
    else:
        out = torch.empty((plan.m_cap, bank.n // 2 if swiglu else bank.n), dtype=out_dtype, device=dev)
    ctx.check(lib.mb_nvfp4_gemm_w4a4_grouped(ctx.handle, _stream(), _p(a_codes), _p(a_sf), _p(bank.codes),
                                             _p(bank.sf_tiled), _p(bank.scale2), _p(plan.tile_expert),
                                             _p(plan.n_tiles), plan.m_cap, bank.experts, bank.n, bank.k, _p(out),
                                             _lib.DT_BF16 if out.dtype != torch.float32 else _lib.DT_F32, epilogue,
                                             _p(out_sf), _p(plan.row_tok) if skip_pad_rows else None))
    return (out, out_sf) if quant else out


def moe_experts(x, idx, weight, w13, w2, fuse_swiglu=True, fuse_quant=True, token_planes=None):
    """grouped_experts_core on the narrow (bf16) lane. x [tokens, h] bf16; w13 bank
    [E, 2*inter, h] with interleaved gate/up rows; w2 bank [E, h, inter]. Returns [tokens, h] f32.
    token_planes: the (codes, tiled scales) of quantize_act(x, QUANT_RECIP) when the caller already has them."""
    tokens, h = x.shape
    inter = w2.k
    plan = RowPlan(idx, weight, w13.experts)
    if h % 64 == 0:
        # a row's bytes do not depend on its place in the plan: quantize each token once, copy planes
        t_codes, t_sf = token_planes if token_planes is not None else nv.quantize_act(x, _lib.QUANT_RECIP, tiled=True)[:2]
        a_codes, a_sf = nv.gather_rows(t_codes, t_sf, tokens, h, plan.row_tok)
    else:
        a_codes, a_sf, _ = nv.quantize_act(x, _lib.QUANT_RECIP, tiled=True, gather=plan.row_tok)
    if fuse_swiglu and fuse_quant:
        # SwiGLU and the second projection's activation quantizer both in the first product's epilogue
        c2, sf2 = grouped_gemm(a_codes, a_sf, w13, plan, epilogue=_lib.EPI_SWIGLU_INTERLEAVED | _lib.EPI_QUANT_RECIP)
        return scatter_weighted(grouped_gemm(c2, sf2, w2, plan, skip_pad_rows=True), plan, h), plan
    if fuse_swiglu:
        act = grouped_gemm(a_codes, a_sf, w13, plan, epilogue=_lib.EPI_SWIGLU_INTERLEAVED)
    else:
        # the reference's own order: the fused gate/up product stored, then gate_up_silu as a pass of its own
        from .inkling import gate_up_silu
        act = gate_up_silu(grouped_gemm(a_codes, a_sf, w13, plan), inter)
    c2, sf2, _ = nv.quantize_act(act, _lib.QUANT_RECIP, tiled=True)
    y = grouped_gemm(c2, sf2, w2, plan, skip_pad_rows=True)
    return scatter_weighted(y, plan, h), plan


_side_streams = {}


def _side_stream(device):
    s = _side_streams.get(device.index)
    if s is None:
        s = _side_streams[device.index] = torch.cuda.Stream(device=device)
    return s


def moe_layer(x, gate_w, k, w13, w2, renormalize=True, scaling=1.0):
    """One MoE block of config 2: router projection (bf16 GEMM, f32 logits), softmax top-k, experts.
    The tokens' NVFP4 planes do not depend on the routing: their quantizer runs on a second stream beside the
    router projection, the selection and the row plan (short, latency-bound kernels), and joins before the planes
    are copied into plan order. MB_MOE_SIDE_STREAM=0 keeps everything on the caller's stream."""
    planes = None
    if x.shape[1] % 64 == 0 and os.environ.get("MB_MOE_SIDE_STREAM", "1") != "0":
        cur, side = torch.cuda.current_stream(x.device), _side_stream(x.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            planes = nv.quantize_act(x, _lib.QUANT_RECIP, tiled=True)[:2]
        for t in planes:
            t.record_stream(cur)
    logits = nv.bf16_gemm(x, gate_w, out_dtype=torch.float32)
    idx, weight = router_topk_softmax(logits, k, renormalize, scaling)
    if planes is not None:
        torch.cuda.current_stream(x.device).wait_stream(_side_stream(x.device))
    out, plan = moe_experts(x, idx, weight, w13, w2, token_planes=planes)
    return out, (logits, idx, weight, plan)
