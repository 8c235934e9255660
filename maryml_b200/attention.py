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


def flash_attention(q, k, v, q0=0, scale=None, causal=True, workspace=None, window=0, keys=None):
    """q [batch, nq, heads, D], k/v [batch, capacity, kv_heads, D] bf16 -> out like q.
    Query i sits at absolute position q0 + i, key j at j. window > 0: the query at position p sees the keys
    in (p - window, p] only (sliding-window attention; causal). keys: live rows of a cache allocated longer
    than that (read in place as one key run); None = all rows."""
    assert q.dtype == k.dtype == v.dtype == torch.bfloat16
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    batch, nq, heads, d = q.shape
    _, cap, kv_heads, _ = k.shape
    if keys is not None and keys != cap:
        assert causal, "a cache read through its live rows is read causally"
        return flash_attention_runs(q, [KeyRunView(k, v, hi=keys)], q0=q0, scale=scale, window=window,
                                    workspace=workspace)
    keys = cap
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


class KeyRunView:
    """KeyRun (src/models/inkling/flash.rs:995-1015): one run of contiguous key/value rows, e.g. one page of a
    paged cache. k, v: [batch, rows, kv_heads, D] bf16 or f32 tensors, or uint8 code planes
    [batch, rows, kv_heads * D / 2] with k_scales, v_scales [batch, rows, kv_heads * D / 16] for NVFP4 rows.
    base: absolute position of row 0; rows [lo, hi) are live; row0: logical row of stored row 0."""

    def __init__(self, k, v, k_scales=None, v_scales=None, base=0, lo=0, hi=None, row0=0):
        self.k, self.v, self.k_scales, self.v_scales = k, v, k_scales, v_scales
        self.rows = k.shape[1]
        self.base, self.lo, self.hi, self.row0 = base, lo, self.rows if hi is None else hi, row0


def flash_attention_runs(q, runs, q0=0, scale=None, window=0, rel=None, gaps=None, workspace=None, out_dtype=None):
    """flash_attention_launch (src/models/inkling/flash.rs:1140-1316): the query block q [batch, nq, heads, D]
    (bf16 or f32) over the key runs `runs` (KeyRunView objects of one element type), causal on absolute
    positions. rel [batch, nq, heads, eff] f32 and gaps (rows, cums int32 tensors) as in decode_attention_ext.
    Returns [batch, nq, heads, D] in out_dtype (default: q's dtype)."""
    assert q.is_contiguous() and q.dtype in (torch.bfloat16, torch.float32)
    batch, nq, heads, d = q.shape
    first = runs[0]
    if first.k_scales is not None:
        kv_elem, kv_heads = _lib.KV_NVFP4, first.k.shape[2] * 2 // d
    else:
        kv_elem = _lib.KV_BF16 if first.k.dtype == torch.bfloat16 else _lib.KV_F32
        kv_heads = first.k.shape[2]
    arr = (_lib.KeyRun * len(runs))()
    for i, r in enumerate(runs):
        for t in (r.k, r.v, r.k_scales, r.v_scales):
            assert t is None or (t.is_contiguous() and t.device == q.device and t.shape[0] == batch)
        assert (r.k_scales is not None) == (kv_elem == _lib.KV_NVFP4)
        arr[i] = _lib.KeyRun(r.k.data_ptr(), r.v.data_ptr(), r.k_scales.data_ptr() if r.k_scales is not None else None,
                             r.v_scales.data_ptr() if r.v_scales is not None else None, r.rows, r.base, r.lo, r.hi,
                             r.row0)
    ctx = context(q.device.index)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    eff = 0
    if rel is not None:
        assert rel.dtype == torch.float32 and rel.is_contiguous() and rel.shape[:3] == (batch, nq, heads)
        eff = rel.shape[3]
    g_rows = g_cums = None
    ngaps = 0
    if gaps is not None:
        g_rows, g_cums = gaps
        assert g_rows.dtype == g_cums.dtype == torch.int32 and g_rows.numel() == g_cums.numel()
        ngaps = g_rows.numel()
    out_dtype = out_dtype or q.dtype
    out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
    dt = lambda t: _lib.DT_BF16 if t == torch.bfloat16 else _lib.DT_F32
    need = int(lib.mb_attention_runs_workspace(arr, len(runs), kv_elem, batch, nq, q0, heads, kv_heads, d, int(window),
                                               ngaps, dt(q.dtype), dt(out_dtype)))
    if need and (workspace is None or workspace.numel() < need or workspace.data_ptr() % 256):
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    ctx.check(lib.mb_attention_runs(ctx.handle, _stream(), _p(q), dt(q.dtype), arr, len(runs), kv_elem, _p(rel), eff,
                                    _p(g_rows), _p(g_cums), ngaps, batch, nq, q0, heads, kv_heads, d, int(window),
                                    float(scale), _p(out), dt(out_dtype), _p(workspace) if need else None, need))
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
