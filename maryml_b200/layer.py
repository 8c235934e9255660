"""The NVFP4 decoder layer and its tensor-parallel placement, over the C ABI.

The layer follows Breeze's `Decoder::forward` body (src/models/breeze/backbone.rs:287-333)
with its bf16 rounding points (src/models/breeze/cuda_ops.rs:88-117, 230-255, 286-320);
the placement follows the reference's TP path (src/models/inkling/tp.rs:283-325, 564-640;
src/models/inkling/session.rs:2713-2717, 2843-2846): QKV / gate / up column-parallel (row
ranges of the [out, in] planes), o / down row-parallel (column ranges, gathered at load),
one SUM all-reduce of the f32 partial after o and after down, before the residual add.
"""
import ctypes as C
import math
import os

import numpy as np
import torch

from . import _lib
from ._lib import lib, context, MaryError
from . import nvfp4 as nv
from .attention import flash_attention

_p = nv._p
_stream = nv._stream


# ---- elementwise glue ----------------------------------------------------------------
def rmsnorm(x, gain, eps):
    rows, width = x.shape
    ctx = context(x.device.index)
    out = torch.empty_like(x)
    ctx.check(lib.mb_rmsnorm(ctx.handle, _stream(), _p(x), _p(gain), rows, width, float(eps), _p(out)))
    return out


def add(a, b, out=None):
    ctx = context(a.device.index)
    if out is None:
        out = torch.empty_like(a)
    ctx.check(lib.mb_add(ctx.handle, _stream(), _p(a), _p(b), a.numel(), _p(out)))
    return out


def add_f32(a, b_f32, out=None):
    ctx = context(a.device.index)
    if out is None:
        out = torch.empty_like(a)
    ctx.check(lib.mb_add_f32(ctx.handle, _stream(), _p(a), _p(b_f32), a.numel(), _p(out)))
    return out


def swiglu(gate, up):
    ctx = context(gate.device.index)
    out = torch.empty_like(gate)
    ctx.check(lib.mb_swiglu(ctx.handle, _stream(), _p(gate), _p(up), gate.numel(), _p(out)))
    return out


def rope(x, tokens, heads, d, past, inv_freq):
    """x viewed as [tokens, heads, d]; position of token t is past + t."""
    ctx = context(x.device.index)
    out = torch.empty_like(x)
    ctx.check(lib.mb_rope(ctx.handle, _stream(), _p(x), tokens, heads, d, past, _p(inv_freq), _p(out)))
    return out


def inv_freq(d, theta):
    """theta^(-2f/d) as f32 (the frequency table the rope kernel takes)."""
    f = np.arange(d // 2, dtype=np.float64)
    return (1.0 / (np.float64(theta) ** (2.0 * f / d))).astype(np.float32)


# ---- tensor-parallel placement (host arithmetic; works on CPU tensors too) -----------
class Indivisible(ValueError):
    """A tensor axis that does not divide by the world size (src/models/inkling/tp.rs:461-470)."""

    def __init__(self, axis, extent, world):
        super().__init__(f"{axis} = {extent} does not divide by world {world}")
        self.axis, self.extent, self.world = axis, extent, world


class Tp:
    """Which rank this process is and how many there are (src/models/inkling/tp.rs:449-555).
    world == 1 is the identity: every cut returns the whole axis."""

    def __init__(self, rank=0, world=1):
        if world < 1 or not (0 <= rank < world):
            raise ValueError(f"rank {rank} of world {world}")
        self.rank, self.world = rank, world

    def is_split(self):
        return self.world > 1

    def shard(self, axis, extent):
        if extent % self.world != 0:
            raise Indivisible(axis, extent, self.world)
        per = extent // self.world
        return range(self.rank * per, (self.rank + 1) * per)

    def share(self, axis, extent):
        return len(self.shard(axis, extent))

    def q_heads(self, heads):
        return self.shard("num_attention_heads", heads)

    def kv_heads(self, kv_heads):
        return self.shard("num_key_value_heads", kv_heads)

    def dense_inter(self, inter):
        return self.shard("intermediate_size", inter)


def cut_rows(codes, scales, rows):
    """Column-parallel cut of stored planes [n, k/2], [n, k/16]: a contiguous row range
    (src/models/inkling/tpshard.rs:102-140). The global scale stays the whole tensor's."""
    return codes[rows.start:rows.stop].contiguous(), scales[rows.start:rows.stop].contiguous()


def cut_cols(codes, scales, cols):
    """Row-parallel cut along K: the range must land on a 16-element block and a byte
    (src/models/inkling/tpshard.rs:526-556 refuses a cut inside a byte)."""
    if cols.start % 16 != 0 or cols.stop % 16 != 0:
        raise ValueError(f"a K cut [{cols.start}, {cols.stop}) is not on 16-element block boundaries")
    return (codes[:, cols.start // 2:cols.stop // 2].contiguous(),
            scales[:, cols.start // 16:cols.stop // 16].contiguous())


class Group:
    """Group::form / warm / all_reduce_f32 (src/models/inkling/tpcomm.rs:217-429) over NCCL.
    The 128-byte id minted on rank 0 travels through `exchange` (a callable that broadcasts bytes)."""

    def __init__(self, tp, device, exchange=None):
        self.tp = tp
        self.ctx = context(device)
        if tp.world > 1:
            uid = (C.c_uint8 * 128)()
            if tp.rank == 0:
                self.ctx.check(lib.mb_tp_unique_id(self.ctx.handle, uid))
            raw = exchange(bytes(uid))
            uid = (C.c_uint8 * 128).from_buffer_copy(raw)
            self.ctx.check(lib.mb_tp_form(self.ctx.handle, uid, tp.rank, tp.world))
            self.warm()

    def warm(self):
        self.ctx.check(lib.mb_tp_warm(self.ctx.handle, _stream()))

    def all_reduce_f32(self, t):
        assert t.dtype == torch.float32 and t.is_contiguous()
        self.ctx.check(lib.mb_tp_all_reduce(self.ctx.handle, _stream(), _p(t), t.numel(), _lib.DT_F32))
        return t

    def reduce_scatter_f32(self, t):
        """SUM reduce-scatter by rows: t [rows, n] f32 on every rank -> this rank's [rows / world, n] of the sum."""
        assert t.dtype == torch.float32 and t.is_contiguous() and t.shape[0] % self.tp.world == 0
        out = torch.empty((t.shape[0] // self.tp.world, t.shape[1]), dtype=torch.float32, device=t.device)
        self.ctx.check(lib.mb_tp_reduce_scatter_f32(self.ctx.handle, _stream(), _p(t), _p(out), out.numel()))
        return out

    def all_gather_rows(self, whole):
        """In-place all-gather of a contiguous buffer cut evenly in rank order: this rank's slice is already in
        its place, the others' slices arrive."""
        assert whole.is_contiguous()
        nbytes = whole.numel() * whole.element_size()
        assert nbytes % self.tp.world == 0
        part = nbytes // self.tp.world
        base = whole.data_ptr()
        self.ctx.check(lib.mb_tp_all_gather(self.ctx.handle, _stream(), C.c_void_p(base + self.tp.rank * part),
                                            C.c_void_p(base), part))
        return whole

    def close(self):
        lib.mb_tp_close(self.ctx.handle)


class FusedExchange:
    """Peer-mapped exchange memory of the fused row-parallel path (see mb_tp_symm_* in the header):
    the GEMM epilogue scatters f32 partial tiles into the owning ranks, one kernel reduces, adds the
    residual and gathers. `exchange_all` all-gathers one bytes object per rank, in rank order."""

    def __init__(self, tp, device, t_max, n, exchange_all):
        self.tp, self.ctx, self.t_max, self.n, self.step = tp, context(device), t_max, n, 0
        h = (C.c_uint8 * 64)()
        self.ctx.check(lib.mb_tp_symm_create(self.ctx.handle, t_max, n, h))
        handles = b"".join(exchange_all(bytes(h)))
        buf = (C.c_uint8 * (64 * tp.world)).from_buffer_copy(handles)
        self.ctx.check(lib.mb_tp_symm_attach(self.ctx.handle, buf, tp.rank, tp.world))

    def gemm_reduce_residual(self, a_codes, a_sf, w, resid, t):
        """bf16(resid + bf16(sum over ranks of a . w^T * scale2)) as a [t, n] bf16 tensor living in the
        exchange memory (valid until the step after next)."""
        self.step += 1
        self.ctx.check(lib.mb_nvfp4_gemm_w4a4_scatter(self.ctx.handle, _stream(), _p(a_codes), _p(a_sf), _p(w.codes),
                                                      _p(w.sf_tiled()), w.scale2, t, w.n(), w.k(), self.step))
        out = C.c_void_p()
        self.ctx.check(lib.mb_tp_reduce_residual(self.ctx.handle, _stream(), _p(resid), t, self.n, self.step,
                                                 C.byref(out)))
        return _wrap_bf16(out.value, t, self.n, resid.device)

    def close(self):
        lib.mb_tp_symm_destroy(self.ctx.handle)


class _DevBuf:
    def __init__(self, ptr, shape, typestr="<i2"):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 3}


def _wrap_bf16(ptr, rows, cols, device):
    return torch.as_tensor(_DevBuf(ptr, (rows, cols)), device=device).view(torch.bfloat16)


def _wrap_bytes(ptr, nbytes, device):
    return torch.as_tensor(_DevBuf(ptr, (nbytes,), "|u1"), device=device)


def _align256(n):
    return (n + 255) // 256 * 256


class BulkExchange:
    """Peer-mapped region for the prompt path's exchanges (mb_tp_bulk_* in the header): reduce-scatter of the f32
    partial by rows and all-gather of the next product's NVFP4 planes or of the output rows, as peer stores from
    kernels of the library instead of NCCL rings. Sized for activations up to [rows_max, hidden]; two of every
    partial and gathered buffer, used in turn. All exchanges of one object are issued on one stream (their step
    numbers are their issue order). `exchange_all` all-gathers one bytes object per rank."""

    def __init__(self, tp, device, rows_max, hidden, exchange_all):
        self.tp, self.ctx, self.rows_max, self.hidden = tp, context(device), rows_max, hidden
        self.device = torch.device("cuda", device) if isinstance(device, int) else device
        recv = _align256(rows_max * hidden * 4)
        codes = _align256(rows_max * hidden // 2)
        sf = _align256(nv.sf_bytes(rows_max, hidden))
        out = _align256(rows_max * hidden * 2)
        self.off_recv = [0, recv]
        self.off_codes = [2 * recv, 2 * recv + codes]
        self.off_sf = [2 * recv + 2 * codes, 2 * recv + 2 * codes + sf]
        self.off_out = [2 * recv + 2 * codes + 2 * sf, 2 * recv + 2 * codes + 2 * sf + out]
        total = 2 * (recv + codes + sf + out)
        h = (C.c_uint8 * 64)()
        self.ctx.check(lib.mb_tp_bulk_create(self.ctx.handle, total, h))
        handles = b"".join(exchange_all(bytes(h)))
        buf = (C.c_uint8 * (64 * tp.world)).from_buffer_copy(handles)
        self.ctx.check(lib.mb_tp_bulk_attach(self.ctx.handle, buf, tp.rank, tp.world))
        user = C.c_void_p()
        self.ctx.check(lib.mb_tp_bulk_local(self.ctx.handle, None, C.byref(user)))
        self.user = user.value
        self.n_rs = self.n_ag = 0            # exchanges of each kind so far (the kernels' step numbers)
        self.n_planes = self.n_rows = 0      # gathers of each buffer kind so far (which of the two buffers is next)

    def takes(self, rows, hidden):
        return hidden == self.hidden and rows <= self.rows_max

    def partial_buffer(self, rows):
        """Where the next reduce-scatter's f32 partial [rows, hidden] goes: inside the region, so that the peers can
        read it (the row-parallel product writes it there directly)."""
        ptr = self.user + self.off_recv[(self.n_rs + 1) & 1]
        return torch.as_tensor(_DevBuf(ptr, (rows, self.hidden), "<f4"), device=self.device)

    def reduce_scatter_f32(self, t):
        """SUM reduce-scatter by rows of the partial in partial_buffer (t is that buffer, or is copied into it):
        this rank's [rows / world, hidden] of the sum."""
        assert t.dtype == torch.float32 and t.is_contiguous() and t.shape[0] % self.tp.world == 0
        buf = self.partial_buffer(t.shape[0])
        if t.data_ptr() != buf.data_ptr():
            buf.copy_(t)
        self.n_rs += 1
        out = torch.empty((t.shape[0] // self.tp.world, t.shape[1]), dtype=torch.float32, device=t.device)
        self.ctx.check(lib.mb_tp_bulk_reduce_scatter_f32(self.ctx.handle, _stream(), self.off_recv[self.n_rs & 1], t.shape[0],
                                                         t.shape[1], _p(out), self.n_rs))
        return out

    def planes(self, rows):
        """The next all-gather's activation planes as tensors inside the region: codes [rows, hidden / 2] and the
        tiled scale plane; the caller writes its own rows' part, all_gather_planes brings the others'."""
        par = (self.n_planes + 1) & 1
        codes = _wrap_bytes(self.user + self.off_codes[par], rows * self.hidden // 2, self.device).view(rows, self.hidden // 2)
        sf = _wrap_bytes(self.user + self.off_sf[par], nv.sf_bytes(rows, self.hidden), self.device)
        return codes, sf

    def all_gather_planes(self, rows):
        self.n_ag += 1
        self.n_planes += 1
        par = self.n_planes & 1
        w = self.tp.world
        self.ctx.check(lib.mb_tp_bulk_all_gather(self.ctx.handle, _stream(), self.off_codes[par], rows * self.hidden // 2 // w,
                                                 self.off_sf[par], nv.sf_bytes(rows, self.hidden) // w, self.n_ag))

    def rows_buffer(self, rows):
        """The next all-gather's bf16 rows [rows, hidden] inside the region."""
        par = (self.n_rows + 1) & 1
        return _wrap_bf16(self.user + self.off_out[par], rows, self.hidden, self.device)

    def all_gather_rows(self, rows):
        self.n_ag += 1
        self.n_rows += 1
        self.ctx.check(lib.mb_tp_bulk_all_gather(self.ctx.handle, _stream(), self.off_out[self.n_rows & 1],
                                                 rows * self.hidden * 2 // self.tp.world, 0, 0, self.n_ag))

    def close(self):
        lib.mb_tp_bulk_destroy(self.ctx.handle)


# ---- the layer -----------------------------------------------------------------------
class LayerConfig:
    def __init__(self, hidden=4096, heads=32, kv_heads=8, head_dim=128, inter=14336, eps=1e-6, theta=1e6):
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.inter, self.eps, self.theta = inter, eps, theta


class DecoderLayer:
    """One Llama-style NVFP4 decoder layer, this rank's shard of it.

    `full` maps names (q, k, v, o, gate, up, down) to whole-tensor planes
    (codes [n, k/2], scales [n, k/16], scale2) quantised BEFORE the cut, so every rank
    holds bytes of the same stored tensor (the reference cuts stored planes)."""

    def __init__(self, cfg, full, input_gain, post_gain, tp=None, group=None, device=None, fused=None, fuse=True,
                 bulk=None):
        self.cfg, self.tp, self.group, self.fused, self.fuse = cfg, tp or Tp(), group, fused, fuse
        self.bulk = bulk              # BulkExchange: the prompt path's exchanges over peer memory instead of NCCL
        self._chunked = False         # inside forward_chunked
        dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        D = cfg.head_dim
        qh, kvh = self.tp.q_heads(cfg.heads), self.tp.kv_heads(cfg.kv_heads)
        inter = self.tp.dense_inter(cfg.inter)
        self.local_heads, self.local_kv_heads, self.local_inter = len(qh), len(kvh), len(inter)

        def col_parallel(name, rows):
            c, s, s2 = full[name]
            cc, ss = cut_rows(c, s, rows)
            return nv.Nvfp4.from_parts(cc.to(dev), ss.to(dev), s2, len(rows), c.shape[1] * 2, torch.bfloat16, dev)

        def row_parallel(name, cols):
            c, s, s2 = full[name]
            cc, ss = cut_cols(c, s, cols)
            return nv.Nvfp4.from_parts(cc.to(dev), ss.to(dev), s2, c.shape[0], len(cols), torch.bfloat16, dev)

        self.wq = col_parallel("q", range(qh.start * D, qh.stop * D))
        self.wk = col_parallel("k", range(kvh.start * D, kvh.stop * D))
        self.wv = col_parallel("v", range(kvh.start * D, kvh.stop * D))
        self.wo = row_parallel("o", range(qh.start * D, qh.stop * D))
        self.wgate = col_parallel("gate", inter)
        self.wup = col_parallel("up", inter)
        self.wdown = row_parallel("down", inter)
        self.input_gain, self.post_gain = input_gain.to(dev), post_gain.to(dev)
        self.inv_freq = torch.from_numpy(inv_freq(D, cfg.theta)).to(dev)
        for w in (self.wo, self.wdown):
            w.sf_tiled()
        if fuse:
            # Projections of one input run as one product: q|k|v stacked, gate and up interleaved
            # row by row for the SwiGLU epilogue. The separate planes are not kept.
            self.wqkv = nv.Stacked([self.wq, self.wk, self.wv])
            self.wgu = nv.Stacked([self.wgate, self.wup], interleave=True)
            self.wq = self.wk = self.wv = self.wgate = self.wup = None
        else:
            for w in (self.wq, self.wk, self.wv, self.wgate, self.wup):
                w.sf_tiled()

    @staticmethod
    def _quantize(x):
        """The W4A4 lane's activation planes (per-16 scales, unit global; src/nn/nvfp4_gemm.rs:644-669).
        Projections that share an input share these planes: the bytes are the same as if each
        projection had quantised the input itself."""
        codes, sf, _ = nv.quantize_act(x, _lib.QUANT_SCALED, 1.0, tiled=True)
        return codes, sf, x.shape[0]

    @staticmethod
    def _project(xq, w, out_dtype=torch.bfloat16, out=None):
        codes, sf, t = xq
        return nv.gemm_w4a4(codes, sf, w.codes, w.sf_tiled(), w.scale2, t, w.n(), w.k(), out_dtype=out_dtype, out=out)

    def _linear(self, x, w, out_dtype=torch.bfloat16, out=None):
        """W4A4 projection (src/nn/nvfp4_gemm.rs:644-694)."""
        return self._project(self._quantize(x), w, out_dtype, out=out)

    def _reduced_residual(self, resid, x, w):
        """bf16(resid + bf16(all-reduced x . w^T)): NCCL all-reduce of the f32 partial then the add,
        or the fused peer-memory exchange when one is attached."""
        t = x.shape[0]
        if self.fused is not None and t <= self.fused.t_max:      # decode-sized messages; long prompts go through NCCL
            codes, sf, _ = nv.quantize_act(x, _lib.QUANT_SCALED, 1.0, tiled=True)
            return self.fused.gemm_reduce_residual(codes, sf, w, resid, t)
        partial = self._linear(x, w, out_dtype=torch.float32)
        if self.group is not None and self.tp.is_split():
            self.group.all_reduce_f32(partial)
        return add_f32(resid, partial)

    def _norm_quantize(self, resid, partial, gain):
        """(new residual, activation planes of rmsnorm(new residual)) in one pass; the new residual
        is resid itself without a partial sum."""
        rows, width = resid.shape
        dev = resid.device
        codes = torch.empty((rows, width // 2), dtype=torch.uint8, device=dev)
        sf = torch.empty(nv.sf_bytes(rows, width), dtype=torch.uint8, device=dev)
        out = torch.empty_like(resid) if partial is not None else resid
        ctx = context(dev.index)
        ctx.check(lib.mb_residual_norm_quantize(ctx.handle, _stream(), _p(resid), _p(partial), _p(gain), rows, width,
                                                float(self.cfg.eps), _p(out) if partial is not None else None,
                                                _p(codes), _p(sf)))
        return out, (codes, sf, rows)

    def _attention(self, x, batch, past, k_cache, v_cache, after_rope=None, before_rope=None):
        """Input norm + quantizer, q|k|v as one product, rotation + cache append, attention of this rank's
        heads: [batch * t, local_heads * D] bf16."""
        cfg = self.cfg
        D = cfg.head_dim
        t = x.shape[0] // batch
        dev = x.device
        ctx = context(dev.index)
        _, xq = self._norm_quantize(x, None, self.input_gain)
        qkv = nv.gemm_w4a4_stacked(xq[0], xq[1], self.wqkv, xq[2])
        q = torch.empty((batch, t, self.local_heads, D), dtype=torch.bfloat16, device=dev)
        assert k_cache.is_contiguous() and v_cache.is_contiguous()
        if before_rope is not None:
            before_rope()
        ctx.check(lib.mb_rope_append(ctx.handle, _stream(), _p(qkv), batch, t, self.local_heads, self.local_kv_heads, D,
                                     past, _p(self.inv_freq), _p(q), _p(k_cache), _p(v_cache), k_cache.shape[1]))
        if after_rope is not None:
            after_rope()
        # a cache allocated longer than its live keys is read in place (one key run of past + t live rows)
        return flash_attention(q, k_cache, v_cache, q0=past, scale=1.0 / math.sqrt(D), causal=True,
                               keys=past + t).view(batch * t, self.local_heads * D)

    def half_attention(self, x, batch, past, k_cache, v_cache, after_rope=None, before_rope=None, out=None):
        """The attention half up to the exchange step: this rank's f32 share of the o projection, [rows, hidden].
        The shares of all ranks sum to the whole projection (src/models/inkling/session.rs:2713-2717)."""
        a = self._attention(x, batch, past, k_cache, v_cache, after_rope, before_rope)
        return self._linear(a, self.wo, out_dtype=torch.float32, out=out)

    def half_mlp(self, x, o_sum, down_dtype=torch.float32):
        """The MLP half between the two exchange steps: given the layer input and the SUMMED o partial, the new
        residual bf16(x + bf16(o_sum)) and this rank's f32 share of the down projection
        (src/models/inkling/session.rs:2843-2846). down_dtype = bf16 is for a layer that is not split: the product
        then rounds its result itself, to the bytes the f32 share would round to in `finish`."""
        residual, nq_ = self._norm_quantize(x, o_sum, self.post_gain)
        act = nv.gemm_w4a4_stacked(nq_[0], nq_[1], self.wgu, nq_[2],
                                   epilogue=_lib.EPI_SWIGLU_ROUNDED | _lib.EPI_QUANT_SCALED)
        return residual, self._project((act[0], act[1], x.shape[0]), self.wdown, out_dtype=down_dtype)

    @staticmethod
    def finish(residual, down_sum, out=None):
        """bf16(residual + bf16(down_sum)): the layer's output from the SUMMED down partial."""
        return add_f32(residual, down_sum, out=out)

    def _all_reduce(self, partial):
        if self.group is not None and self.tp.is_split():
            self.group.all_reduce_f32(partial)
        return partial

    def _forward_fused(self, x, batch, past, k_cache, v_cache, out=None, after_rope=None, before_rope=None):
        """The same layer in fewer passes: norm + quantize in one kernel, q|k|v as one product,
        rotation + cache append in one kernel, gate/up + SwiGLU + quantize in one product, the
        residual add folded into the next norm. Every value is computed by the arithmetic of the
        separate kernels. `before_rope` / `after_rope` are hooks of the chunked prompt path."""
        rows = x.shape[0]
        if self.fused is not None and rows <= self.fused.t_max:
            # peer-memory exchange: the row-parallel products scatter their partial tiles, one kernel per
            # exchange reduces, adds the residual and gathers
            a = self._attention(x, batch, past, k_cache, v_cache, after_rope, before_rope)
            residual = self._reduced_residual(x, a, self.wo)
            _, nq_ = self._norm_quantize(residual, None, self.post_gain)
            act = nv.gemm_w4a4_stacked(nq_[0], nq_[1], self.wgu, nq_[2],
                                       epilogue=_lib.EPI_SWIGLU_ROUNDED | _lib.EPI_QUANT_SCALED)
            y = self.fused.gemm_reduce_residual(act[0], act[1], self.wdown, residual, rows)
            if out is not None:
                out.copy_(y)
                return out
            return y
        if self._rows_shard(rows):
            return self._forward_rows_sharded(x, batch, past, k_cache, v_cache, out, after_rope, before_rope)
        o_sum = self._all_reduce(self.half_attention(x, batch, past, k_cache, v_cache, after_rope, before_rope))
        if not (self.group is not None and self.tp.is_split()):
            # nothing to sum across ranks: the down product hands over bf16 (half the bytes written and read back),
            # bf16(residual + bf16(down)) either way
            residual, down = self.half_mlp(x, o_sum, down_dtype=torch.bfloat16)
            return add(residual, down, out=out)
        residual, down = self.half_mlp(x, o_sum)
        return self.finish(residual, self._all_reduce(down), out=out)

    # Prompts of at least this many rows per rank keep their rows sharded between the two exchanges
    # (MB_TP_ROW_SHARD=0 in the environment keeps the plain all-reduce, for comparison runs).
    ROW_SHARD_MIN = 256

    def _rows_shard(self, rows):
        w = self.tp.world
        return (self.group is not None and w > 1 and rows % (128 * w) == 0 and rows // w >= self.ROW_SHARD_MIN
                and self.cfg.hidden % 256 == 0 and os.environ.get("MB_TP_ROW_SHARD", "1") != "0")

    def _forward_rows_sharded(self, x, batch, past, k_cache, v_cache, out=None, after_rope=None, before_rope=None):
        """The split layer for prompt-sized activations. An f32 all-reduce of [rows, hidden] moves 8 bytes per
        element and rank over the links, and every rank then repeats the same residual add, norm and quantizer on
        all rows. Here each exchange is the all-reduce's first half only, a SUM reduce-scatter by rows (the same
        f32 sums); this rank adds the residual, normalises and quantizes its OWN rows, and what is gathered is what
        the next product reads: NVFP4 planes at 0.5625 bytes per element. The output rows are gathered as bf16 at
        the end. Per element the arithmetic is that of the all-reduce path."""
        cfg, w, r = self.cfg, self.tp.world, self.tp.rank
        rows, hidden = x.shape
        local = rows // w
        lo = r * local
        dev = x.device
        ctx = context(dev.index)
        # the peer-memory exchanges count their steps in issue order on ONE stream; the chunked path runs its chunks
        # on two streams and keeps NCCL
        bulk = self.bulk if (self.bulk is not None and self.bulk.takes(rows, hidden) and not self._chunked) else None
        ex = bulk or self.group                       # peer-memory kernels of this library, or NCCL
        # with the peer-memory exchange the row-parallel products write their partials where the peers read them
        part_out = (lambda: bulk.partial_buffer(rows)) if bulk is not None else (lambda: None)
        o_local = ex.reduce_scatter_f32(self.half_attention(x, batch, past, k_cache, v_cache, after_rope, before_rope,
                                                            out=part_out()))
        if bulk is not None:
            codes, sf = bulk.planes(rows)
        else:
            codes = torch.empty((rows, hidden // 2), dtype=torch.uint8, device=dev)
            sf = torch.empty(nv.sf_bytes(rows, hidden), dtype=torch.uint8, device=dev)
        sf_part = sf.numel() // w                      # whole 128-row tiles per rank: a contiguous range of the plane
        resid_local = torch.empty((local, hidden), dtype=torch.bfloat16, device=dev)
        ctx.check(lib.mb_residual_norm_quantize(ctx.handle, _stream(), _p(x[lo:lo + local]), _p(o_local), _p(self.post_gain),
                                                local, hidden, float(cfg.eps), _p(resid_local), _p(codes[lo:lo + local]),
                                                C.c_void_p(sf.data_ptr() + r * sf_part)))
        if bulk is not None:
            bulk.all_gather_planes(rows)
        else:
            self.group.all_gather_rows(codes)
            self.group.all_gather_rows(sf)
        act = nv.gemm_w4a4_stacked(codes, sf, self.wgu, rows, epilogue=_lib.EPI_SWIGLU_ROUNDED | _lib.EPI_QUANT_SCALED)
        d_local = ex.reduce_scatter_f32(self._project((act[0], act[1], rows), self.wdown, out_dtype=torch.float32,
                                                      out=part_out()))
        if bulk is not None:
            y = bulk.rows_buffer(rows)                 # lives in the region until the exchange after next
            add_f32(resid_local, d_local, out=y[lo:lo + local])
            bulk.all_gather_rows(rows)
            if out is not None:
                out.copy_(y)
                return out
            return y
        y = out if out is not None else torch.empty((rows, hidden), dtype=torch.bfloat16, device=dev)
        assert y.is_contiguous()
        add_f32(resid_local, d_local, out=y[lo:lo + local])
        return self.group.all_gather_rows(y)

    # rows per chunk of the pipelined prompt path, and the SMs left to the all-reduce that runs beside the products
    PROMPT_CHUNK = 2048
    COLLECTIVE_SMS = 20

    def forward_chunked(self, x, past, k_cache, v_cache, chunk=None):
        """One long prompt (batch 1) as a pipeline of token chunks on two streams: while chunk c's f32
        all-reduce crosses NVLink, chunk c + 1 runs its products and attention. Causal attention
        only needs the keys of earlier chunks, which their rope + append passes wrote (ordered by
        events). Per query row the arithmetic is that of the unchunked layer."""
        chunk = chunk or self.PROMPT_CHUNK
        rows = x.shape[0]
        assert rows % chunk == 0 and chunk % 256 == 0, "chunks are whole 256-row attention tiles"
        n = rows // chunk
        main = torch.cuda.current_stream()
        if getattr(self, "_side", None) is None:
            self._side = [torch.cuda.Stream(device=x.device), torch.cuda.Stream(device=x.device)]
        out = torch.empty_like(x)
        ev_rope = [torch.cuda.Event() for _ in range(n)]
        ctx = context(x.device.index)
        split = self.group is not None and self.tp.is_split()
        if split:
            sms = torch.cuda.get_device_properties(x.device).multi_processor_count
            ctx.check(lib.mb_ctx_set_sm_limit(ctx.handle, sms - self.COLLECTIVE_SMS))
        self._chunked = True
        try:
            for st in self._side:
                st.wait_stream(main)
            for c in range(n):
                st = self._side[c & 1]
                with torch.cuda.stream(st):
                    before = (lambda c=c, st=st: st.wait_event(ev_rope[c - 1])) if c > 0 else None
                    after = lambda c=c, st=st: ev_rope[c].record(st)
                    self._forward_fused(x[c * chunk:(c + 1) * chunk], 1, past + c * chunk, k_cache, v_cache,
                                        out=out[c * chunk:(c + 1) * chunk], after_rope=after, before_rope=before)
            for st in self._side:
                main.wait_stream(st)
        finally:
            self._chunked = False
            if split:
                ctx.check(lib.mb_ctx_set_sm_limit(ctx.handle, 0))
        return out

    def forward(self, x, batch, past, k_cache, v_cache):
        """x [batch * t, hidden] bf16 (t new tokens per sequence, sequence-major). Caches
        [batch, capacity, local_kv_heads, D]; the new keys/values land at [past, past + t)."""
        if self.fuse:
            # the pipelined prompt path is opt-in (MB_TP_PROMPT_CHUNK=rows): at two GPUs the all-reduce is too
            # short to pay for the extra launches (1.58 vs 1.50 ms on the 8192-token prompt)
            chunk = int(os.environ.get("MB_TP_PROMPT_CHUNK", 0))
            if (batch == 1 and chunk > 0 and x.shape[0] >= 2 * chunk and x.shape[0] % chunk == 0
                    and self.group is not None and self.tp.is_split()):
                return self.forward_chunked(x, past, k_cache, v_cache, chunk)
            return self._forward_fused(x, batch, past, k_cache, v_cache)
        cfg = self.cfg
        D = cfg.head_dim
        t = x.shape[0] // batch
        nq_ = self._quantize(rmsnorm(x, self.input_gain, cfg.eps))
        q = self._project(nq_, self.wq)
        k = self._project(nq_, self.wk)
        v = self._project(nq_, self.wv)
        # rope positions restart for every sequence: one call per sequence when t > 1, one call when t == 1
        if t == 1:
            q = rope(q, 1, batch * self.local_heads, D, past, self.inv_freq)
            k = rope(k, 1, batch * self.local_kv_heads, D, past, self.inv_freq)
        else:
            qs, ks = q.view(batch, t * self.local_heads * D), k.view(batch, t * self.local_kv_heads * D)
            q = torch.stack([rope(qs[b], t, self.local_heads, D, past, self.inv_freq) for b in range(batch)])
            k = torch.stack([rope(ks[b], t, self.local_kv_heads, D, past, self.inv_freq) for b in range(batch)])
        k_cache[:, past:past + t].copy_(k.view(batch, t, self.local_kv_heads, D))
        v_cache[:, past:past + t].copy_(v.view(batch, t, self.local_kv_heads, D))
        a = flash_attention(q.view(batch, t, self.local_heads, D), k_cache, v_cache, q0=past,
                            scale=1.0 / math.sqrt(D), causal=True, keys=past + t)
        residual = self._reduced_residual(x, a.view(batch * t, self.local_heads * D), self.wo)
        nq_ = self._quantize(rmsnorm(residual, self.post_gain, cfg.eps))
        gate = self._project(nq_, self.wgate)
        up = self._project(nq_, self.wup)
        return self._reduced_residual(residual, swiglu(gate, up), self.wdown)
