"""Tensor-parallel host logic on CPU: two gloo ranks cut the stored NVFP4 planes the way the
decoder layer does, compute their partials with the CPU oracle, all-reduce, and must agree with
the unsharded oracle. No GPU, no NCCL: this covers the shard arithmetic and the placement rules."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def _worker(rank, world, port, result_path):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle_lib import oracle, f32_to_bf16_bits, bf16_bits_to_f32
    from maryml_b200.layer import Tp, cut_rows, cut_cols, Indivisible
    orc = oracle()
    orc.set_threads(2)
    tp = Tp(rank, world)
    hidden, inter, rows = 256, 512, 5
    # one column-parallel (up) followed by one row-parallel (down) projection, planes cut AFTER
    # quantising the whole tensors (every rank holds bytes of the same stored tensor)
    w_up = f32_to_bf16_bits(orc.normal_f32(1, inter * hidden, 0.02))
    w_down = f32_to_bf16_bits(orc.normal_f32(2, hidden * inter, 0.02))
    cu, su, gu = orc.quantize_weight_bf16(w_up, inter, hidden)
    cd, sd, gd = orc.quantize_weight_bf16(w_down, hidden, inter)
    x = f32_to_bf16_bits(orc.normal_f32(3, rows * hidden, 1.0))

    def lin(xb, codes, scales, s2, n, k):
        ac, asc = orc.quantize_act_scaled(bf16_bits_to_f32(xb), rows, k, 1.0)
        return orc.linear_w4a4(ac, asc, codes, scales, np.float32(s2), rows, n, k)

    cut = tp.dense_inter(inter)
    cu_r, su_r = cut_rows(torch.from_numpy(cu).view(inter, hidden // 2), torch.from_numpy(su).view(inter, hidden // 16), cut)
    cd_r, sd_r = cut_cols(torch.from_numpy(cd).view(hidden, inter // 2), torch.from_numpy(sd).view(hidden, inter // 16), cut)
    up_local = f32_to_bf16_bits(lin(x, cu_r.numpy().ravel(), su_r.numpy().ravel(), gu, len(cut), hidden))
    partial = lin(up_local.ravel(), cd_r.numpy().ravel(), sd_r.numpy().ravel(), gd, hidden, len(cut))
    t = torch.from_numpy(partial.copy())
    dist.all_reduce(t)                      # the SUM all-reduce of the f32 partial activation
    # unsharded reference on every rank
    up_full = f32_to_bf16_bits(lin(x, cu, su, gu, inter, hidden))
    # the column-parallel shard is a slice of the full result, bit for bit
    assert np.array_equal(up_full.reshape(rows, inter)[:, cut.start:cut.stop], up_local.reshape(rows, len(cut)))
    full = lin(up_full.ravel(), cd, sd, gd, hidden, inter)
    err = np.abs(t.numpy() - full).max() / (np.abs(full).max() + 1e-30)
    ok = err < 1e-5                          # only the f32 re-association of the K sum differs
    # warm(): the sum of ones equals the world (src/models/inkling/tpcomm.rs:377-404)
    one = torch.ones(1)
    dist.all_reduce(one)
    ok = ok and one.item() == world
    try:
        Tp(0, 3).shard("intermediate_size", inter)
        ok = False
    except Indivisible:
        pass
    try:
        cut_cols(torch.zeros(4, 32, dtype=torch.uint8), torch.zeros(4, 4, dtype=torch.uint8), range(8, 40))
        ok = False
    except ValueError:
        pass
    flag = torch.tensor([1.0 if ok else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        with open(result_path, "w") as f:
            f.write(f"{flag.item()} {err}")
    dist.destroy_process_group()


def _rows_worker(rank, world, port, result_path):
    """The prompt path's exchange: SUM reduce-scatter of the f32 partial by rows, residual + norm + quantizer on the
    rank's own rows, all-gather of the NVFP4 planes, against the all-reduce form (every rank norms and quantizes all
    rows). Same sums, same per-row arithmetic: the gathered planes and the residual rows must be the same bytes."""
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle_lib import oracle, f32_to_bf16_bits, bf16_bits_to_f32
    orc = oracle()
    orc.set_threads(2)
    rows, hidden = 8 * world, 256
    local = rows // world
    x = f32_to_bf16_bits(orc.normal_f32(11, rows * hidden, 1.0)).reshape(rows, hidden)
    gain = f32_to_bf16_bits(1.0 + orc.normal_f32(12, hidden, 0.1))
    partial = orc.normal_f32(100 + rank, rows * hidden, 0.5).reshape(rows, hidden).astype(np.float32)   # this rank's share

    def finish(x_rows, summed, n):
        """bf16(x + bf16(sum)) -> norm -> W4A4 activation planes, row by row (the layer's second half opens so)."""
        res = orc.add_bf16(x_rows, f32_to_bf16_bits(summed)).reshape(n, hidden)
        normed = orc.rmsnorm_breeze(res, gain, n, hidden, 1e-5)
        codes, scales = orc.quantize_act_scaled(bf16_bits_to_f32(normed), n, hidden, 1.0)
        return res, np.asarray(codes).reshape(n, hidden // 2), np.asarray(scales).reshape(n, hidden // 16)

    # all-reduce form
    t = torch.from_numpy(partial.copy())
    dist.all_reduce(t)
    res_all, codes_all, scales_all = finish(x, t.numpy(), rows)
    # rows stay sharded: reduce-scatter, local finish, all-gather of the planes
    mine = torch.empty(local, hidden)
    dist.reduce_scatter_tensor(mine, torch.from_numpy(partial.copy()))
    res_l, codes_l, scales_l = finish(x[rank * local:(rank + 1) * local], mine.numpy(), local)
    codes_g = torch.empty(rows, hidden // 2, dtype=torch.uint8)
    scales_g = torch.empty(rows, hidden // 16, dtype=torch.uint8)
    dist.all_gather_into_tensor(codes_g, torch.from_numpy(codes_l.copy()))
    dist.all_gather_into_tensor(scales_g, torch.from_numpy(scales_l.copy()))
    ok = (np.array_equal(codes_g.numpy(), codes_all) and np.array_equal(scales_g.numpy(), scales_all)
          and np.array_equal(res_l, res_all[rank * local:(rank + 1) * local]))
    flag = torch.tensor([1.0 if ok else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        with open(result_path, "w") as f:
            f.write(f"{flag.item()}")
    dist.destroy_process_group()


def test_two_rank_rows_sharded_exchange_gathers_the_all_reduce_forms_planes(tmp_path):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    result = tmp_path / "rows_result.txt"
    mp.spawn(_rows_worker, args=(2, port, str(result)), nprocs=2, join=True)
    assert float(result.read_text()) == 1.0


def test_two_rank_row_and_column_parallel_projection(tmp_path):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    result = tmp_path / "tp_result.txt"
    mp.spawn(_worker, args=(2, port, str(result)), nprocs=2, join=True)
    ok, err = result.read_text().split()
    assert float(ok) == 1.0, f"sharded projection disagrees with the whole: rel err {err}"


def test_identity_world_and_gqa_cuts():
    from maryml_b200.layer import Tp
    t = Tp()
    assert not t.is_split() and t.q_heads(32) == range(0, 32)
    a, b = Tp(0, 2), Tp(1, 2)
    assert a.q_heads(32) == range(0, 16) and b.q_heads(32) == range(16, 32)
    assert a.kv_heads(8) == range(0, 4) and b.kv_heads(8) == range(4, 8)
    for world in (1, 2, 4, 8):
        seen = np.zeros(14336, np.uint8)
        for r in range(world):
            sh = Tp(r, world).dense_inter(14336)
            seen[sh.start:sh.stop] += 1
            assert sh.start % 64 == 0        # a K cut of `down` lands on whole scale atoms
        assert (seen == 1).all()
