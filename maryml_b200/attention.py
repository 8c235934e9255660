"""Host-side mirror of the reference's attention entry points over the C ABI.

`flash_attention` follows flash_attention_launch (src/models/inkling/flash.rs:1140-1316)
for the plain GQA case (no window, no relative bias, no eviction gaps) with a batch axis
of independent sequences; `attention_prefill` / `attention_step` are the op-surface names
of src/models/inkling/burn.rs:1732, 2741.
"""
import math

import torch

from . import _lib
from ._lib import lib, context
from .nvfp4 import _p, _stream


def flash_attention(q, k, v, q0=0, scale=None, causal=True, workspace=None, window=0):
    """q [batch, nq, heads, D], k/v [batch, keys, kv_heads, D] bf16 -> out like q.
    Query i sits at absolute position q0 + i, key j at j. window > 0: the query at position p sees the keys
    in (p - window, p] only (sliding-window attention; causal)."""
    assert q.dtype == k.dtype == v.dtype == torch.bfloat16
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    batch, nq, heads, d = q.shape
    _, keys, kv_heads, _ = k.shape
    ctx = context(q.device.index)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    out = torch.empty_like(q)
    need = int(lib.mb_attention_workspace(batch, nq, keys, heads, kv_heads, d))
    if need and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    if window:
        assert causal, "a sliding window is a causal window"
        ctx.check(lib.mb_attention_window(ctx.handle, _stream(), _p(q), _p(k), _p(v), batch, nq, keys, heads, kv_heads, d,
                                          q0, float(scale), int(window), _p(out), _p(workspace) if need else None, need))
        return out
    ctx.check(lib.mb_attention(ctx.handle, _stream(), _p(q), _p(k), _p(v), batch, nq, keys, heads, kv_heads, d, q0,
                               float(scale), int(causal), _p(out), _p(workspace) if need else None, need))
    return out


def decode_attention_ext(q, k, v, q0, scale=None, window=0, rel=None, gaps=None, workspace=None):
    """Causal decode attention with a relative bias table rel [batch, nq, heads, eff] and eviction gaps
    (src/models/inkling/flash.rs:751-785). gaps: (gap_rows, gap_cums) int32 CUDA tensors, rows ascending: the key in
    cache row r sits at position r + gap_cums[g] for the last g with gap_rows[g] <= r. q0 is a position."""
    assert q.dtype == k.dtype == v.dtype == torch.bfloat16
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    batch, nq, heads, d = q.shape
    _, keys, kv_heads, _ = k.shape
    ctx = context(q.device.index)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    eff = 0
    if rel is not None:
        assert rel.dtype == torch.float32 and rel.is_contiguous() and rel.shape[:3] == (batch, nq, heads)
        eff = rel.shape[3]
    rows = cums = None
    ngaps = 0
    if gaps is not None:
        rows, cums = gaps
        assert rows.dtype == cums.dtype == torch.int32 and rows.numel() == cums.numel()
        ngaps = rows.numel()
    out = torch.empty_like(q)
    need = int(lib.mb_attention_workspace(batch, nq, keys, heads, kv_heads, d))
    if need and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    ctx.check(lib.mb_attention_decode_ext(ctx.handle, _stream(), _p(q), _p(k), _p(v), batch, nq, keys, heads, kv_heads, d,
                                          q0, float(scale), int(window), _p(rel), eff, _p(rows), _p(cums), ngaps,
                                          _p(out), _p(workspace) if need else None, need))
    return out


def quantize_kv_rows(x):
    """[batch, keys, kv_heads, D] bf16 cache rows -> (codes [batch, keys, kv_heads*D/2], scales
    [batch, keys, kv_heads*D/16]) in the Fp4Rows layout (src/models/inkling/kvpages.rs:1378-1404):
    every row quantized on its own, blocks of 16 along the features, no global scale."""
    from . import nvfp4 as nv
    batch, keys, kv_heads, d = x.shape
    codes, scales, _ = nv.quantize_act(x.reshape(batch * keys, kv_heads * d), _lib.QUANT_RECIP, tiled=False)
    return codes.view(batch, keys, kv_heads * d // 2), scales.view(batch, keys, kv_heads * d // 16)


def flash_attention_fp4kv(q, k_codes, k_scales, v_codes, v_scales, kv_heads, q0=0, scale=None, causal=True,
                          workspace=None, window=0):
    """Decode attention reading NVFP4 cache rows (the packed reader of src/models/inkling/flash.rs:520-540)."""
    assert q.dtype == torch.bfloat16 and q.is_contiguous()
    for t in (k_codes, k_scales, v_codes, v_scales):
        assert t.dtype == torch.uint8 and t.is_contiguous()
    batch, nq, heads, d = q.shape
    keys = k_codes.shape[1]
    ctx = context(q.device.index)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    out = torch.empty_like(q)
    need = int(lib.mb_attention_workspace(batch, nq, keys, heads, kv_heads, d))
    if need and (workspace is None or workspace.numel() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    ctx.check(lib.mb_attention_fp4kv(ctx.handle, _stream(), _p(q), _p(k_codes), _p(k_scales), _p(v_codes), _p(v_scales),
                                     batch, nq, keys, heads, kv_heads, d, q0, float(scale), int(causal), int(window),
                                     _p(out), _p(workspace) if need else None, need))
    return out


def attention_prefill(q, k, v, scale=None):
    """Causal self-attention over a fresh sequence (q0 = 0)."""
    return flash_attention(q, k, v, 0, scale, True)


def attention_step(q, k_cache, v_cache, scale=None):
    """One decode step: the single query of each sequence sits after all cached keys."""
    keys = k_cache.shape[1]
    return flash_attention(q, k_cache, v_cache, keys - q.shape[1], scale, True)
