"""The committed golden vectors (tests/golden/hot_path_golden.npz, written by tests/golden/make_golden.py).

CPU: the oracle still reproduces them. GPU: the CUDA path, through the C ABI, against the file alone."""
import importlib.util
import math
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden", "hot_path_golden.npz")

EXACT_FLOATS = {"w_scale2", "w_decoded", "act_x", "act_rows_rowscale", "router_logits", "router_bias", "router_sink_logits",
                "plan_row_wgt"}


@pytest.fixture(scope="module")
def golden():
    return dict(np.load(GOLDEN))


def test_oracle_reproduces_the_golden_file(orc, golden):
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fresh = mod.build(orc)
    assert sorted(fresh) == sorted(golden)
    for name, want in golden.items():
        got = np.asarray(fresh[name])
        assert got.shape == want.shape and got.dtype == want.dtype, name
        if want.dtype.kind in "iu" or name in EXACT_FLOATS:
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), name
        else:   # outputs that pass through the host's exp / log
            assert np.allclose(got, want, rtol=1e-6, atol=1e-12), name


# ---------------------------------------------------------------------------- GPU
def _dev_bf16(torch, bits):
    return torch.from_numpy(np.ascontiguousarray(bits, np.uint16).view(np.int16)).cuda().view(torch.bfloat16)


@pytest.mark.gpu
def test_cuda_quantizers_against_the_golden_file(golden):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from maryml_b200 import _lib, nvfp4 as nv
    q = nv.Nvfp4.quantize(_dev_bf16(torch, golden["w_bits"]).view(8, 128))
    codes, scales = q.read_planes()
    assert np.array_equal(codes.ravel(), golden["w_codes"]) and np.array_equal(scales.ravel(), golden["w_scales"])
    assert np.float32(q.scale2) == golden["w_scale2"][0]
    dq = nv.dequantize(q.codes, q.scales, q.scale2, 8, 128).cpu().numpy().ravel()
    assert np.array_equal(dq.view(np.uint32), golden["w_decoded"].view(np.uint32))
    x = torch.from_numpy(golden["act_x"]).cuda()
    for recipe, tag, arg in [(_lib.QUANT_SCALED, "scaled", 0.5), (_lib.QUANT_RECIP, "recip", 1.0), (_lib.QUANT_ROWS, "rows", 1.0)]:
        c, s, rs = nv.quantize_act(x, recipe, arg, tiled=False)
        assert np.array_equal(c.cpu().numpy().ravel(), golden[f"act_{tag}_codes"]), tag
        assert np.array_equal(s.cpu().numpy().ravel(), golden[f"act_{tag}_scales"]), tag
        if rs is not None:
            assert np.array_equal(rs.cpu().numpy().view(np.uint32), golden["act_rows_rowscale"].view(np.uint32))
    _, bs, gscale, gexp = nv.mxfp4_to_nvfp4(torch.zeros(18 * 16, dtype=torch.uint8, device="cuda"),
                                            torch.from_numpy(golden["mx_e8m0"]).cuda(), 18, 32)
    assert np.array_equal(bs.cpu().numpy().ravel(), golden["mx_block_scales"]) and gexp == int(golden["mx_global_exp"][0])
    assert gscale == 2.0 ** gexp


@pytest.mark.gpu
def test_cuda_routing_against_the_golden_file(golden):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from maryml_b200 import moe
    logits = torch.from_numpy(golden["router_logits"]).cuda()
    bias = torch.from_numpy(golden["router_bias"]).cuda()
    idx, w = moe.router_topk(logits, 4, "softmax")
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), golden["router_softmax_idx"])
    assert np.abs(w.cpu().numpy() - golden["router_softmax_w"]).max() <= 1e-6
    plan = moe.RowPlan(idx, w, 64)
    m = golden["plan_row_tok"].size
    assert int(plan.n_tiles.item()) * 128 == m
    assert np.array_equal(plan.row_tok.cpu().numpy()[:m], golden["plan_row_tok"])
    assert np.array_equal(plan.tok_rows.cpu().numpy().astype(np.uint32), golden["plan_tok_rows"])
    idx, w = moe.router_topk(logits, 4, "sigmoid", bias, False)
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), golden["router_sigmoid_idx"])
    assert np.array_equal(w.cpu().numpy().view(np.uint32), golden["router_sigmoid_w"].view(np.uint32))
    idx, w, gam = moe.router_topk_sinks(torch.from_numpy(golden["router_sink_logits"]).cuda(), bias, 64, 4,
                                        global_scale=0.5, route_scale=2.5)
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), golden["router_sinks_idx"])
    assert np.allclose(w.cpu().numpy(), golden["router_sinks_w"], rtol=2e-6, atol=1e-9)
    assert np.allclose(gam.cpu().numpy(), golden["router_sinks_gammas"], rtol=2e-6, atol=1e-9)


@pytest.mark.gpu
def test_cuda_decode_attention_against_the_golden_file(golden):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from maryml_b200 import attention as att
    heads, kvh, D, nq, keys = 4, 1, 128, 2, 70
    q = _dev_bf16(torch, golden["attn_q"]).view(1, nq, heads, D)
    k = _dev_bf16(torch, golden["attn_k"]).view(1, keys, kvh, D)
    v = _dev_bf16(torch, golden["attn_v"]).view(1, keys, kvh, D)
    for window, name in [(0, "attn_out"), (33, "attn_out_window33")]:
        out = att.flash_attention(q, k, v, q0=keys - nq, window=window).float().cpu().numpy().reshape(nq, heads * D)
        ref = golden[name]
        assert np.abs(out - ref).max() <= 2e-2 * np.abs(ref).max(), name
        cos = float((out * ref).sum() / (np.linalg.norm(out) * np.linalg.norm(ref)))
        assert cos >= 0.9999, (name, cos)
    assert math.isfinite(float(np.abs(golden["attn_out"]).max()))
