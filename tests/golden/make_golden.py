"""Writes tests/golden/hot_path_golden.npz: small input/output vectors of the hot path made by the
CPU oracle (oracle/oracle.cpp, pinned by the reference's known-answer tests).

The reference is a Rust project whose kernels are generated at run time for another GPU, so it
cannot be run to produce fixtures; these vectors freeze the pinned oracle instead. The CPU suite
checks that the oracle still reproduces them (a changed oracle shows up as a diff of this file),
the GPU suite checks the CUDA path against them without the oracle in the loop.

    python tests/golden/make_golden.py        # rewrites the .npz next to this script
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from oracle_lib import oracle, f32_to_bf16_bits, bf16_bits_to_f32  # noqa: E402


def adversarial(orc, n, k):
    """The weight fixture of src/nn/nvfp4_gemv.rs:726-738 on bf16: the saturating 2688, exact ties,
    tiny rows and signed zeros."""
    w = orc.normal_f32(0xF160FF4, n * k, 0.5)
    w[0] = 2688.0
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0], np.float32)
    small = orc.normal_f32(0x0F169E77, 2 * k, 1.0)
    for i in range(k):
        w[k + i] = (-1.0 if i % 3 == 0 else 1.0) * ties[i % 8]
        w[2 * k + i] = small[i] * 1e-3
        w[3 * k + i] = small[k + i] * 1e-6
        w[4 * k + i] = -0.0 if i % 2 == 0 else 0.0
    return f32_to_bf16_bits(w)


def build(orc):
    g = {}
    # weight quantizer (codes, scales, scale2) and decode on the adversarial fixture
    n, k = 8, 128
    wbits = adversarial(orc, n, k)
    codes, scales, s2 = orc.quantize_weight_bf16(wbits, n, k)
    g["w_bits"], g["w_codes"], g["w_scales"] = wbits, codes, scales
    g["w_scale2"] = np.array([s2], np.float32).reshape(1)
    g["w_decoded"] = orc.dequantize(codes, scales, s2)
    # the three activation recipes on one [5, 96] block of rows
    rows, ka = 5, 96
    x = bf16_bits_to_f32(f32_to_bf16_bits(orc.normal_f32(41, rows * ka, 1.5)))
    g["act_x"] = x.reshape(rows, ka)
    c, s = orc.quantize_act_scaled(x, rows, ka, 0.5)
    g["act_scaled_codes"], g["act_scaled_scales"] = c, s
    c, s = orc.quantize_act_recip(x, rows, ka)
    g["act_recip_codes"], g["act_recip_scales"] = c, s
    c, s, rs = orc.quantize_act_rows(x, rows, ka)
    g["act_rows_codes"], g["act_rows_scales"], g["act_rows_rowscale"] = c, s, rs
    # routers: softmax, sigmoid with a selection bias, and the sink form
    tokens, n_exp, topk = 6, 64, 4
    logits = orc.normal_f32(43, tokens * n_exp, 2.0).reshape(tokens, n_exp)
    logits[1, :] = 0.25
    bias = orc.normal_f32(44, n_exp, 0.2).astype(np.float32)
    g["router_logits"], g["router_bias"] = logits, bias
    idx, w = orc.router_select(orc.router_scores_softmax(logits), topk)
    g["router_softmax_idx"], g["router_softmax_w"] = idx, w
    idx, w = orc.router_select(orc.router_scores_sigmoid(logits), topk, bias=bias, renormalize=False)
    g["router_sigmoid_idx"], g["router_sigmoid_w"] = idx, w
    sink_logits = np.concatenate([logits, orc.normal_f32(48, tokens * 2, 2.0).reshape(tokens, 2)], axis=1)
    g["router_sink_logits"] = np.ascontiguousarray(sink_logits, np.float32)       # 64 routed + 2 shared columns
    idx, w, gam = orc.router_sinks(g["router_sink_logits"], bias, n_exp, topk, global_scale=0.5, route_scale=2.5)
    g["router_sinks_idx"], g["router_sinks_w"], g["router_sinks_gammas"] = idx, w, gam
    # row plan of the softmax routing over 64 experts, 128-row tiles
    plan = orc.row_plan(g["router_softmax_idx"], g["router_softmax_w"], n_exp, 128)
    g["plan_row_tok"], g["plan_row_wgt"], g["plan_tok_rows"] = plan["row_tok"], plan["row_wgt"], plan["tok_rows"]
    # MXFP4 relabelling across the whole 18-octave window
    e8 = (np.arange(-9, 9) + 127).astype(np.uint8)
    bs, gexp, _ = orc.mxfp4_transcode(e8)
    g["mx_e8m0"], g["mx_block_scales"], g["mx_global_exp"] = e8, bs, np.array([gexp], np.int32)
    # one decode-attention case: 2 queries, GQA 4:1, 70 keys, a window of 33
    heads, kvh, D, nq, keys = 4, 1, 128, 2, 70
    q = f32_to_bf16_bits(orc.normal_f32(45, nq * heads * D, 1.0))
    kk = f32_to_bf16_bits(orc.normal_f32(46, keys * kvh * D, 1.0))
    vv = f32_to_bf16_bits(orc.normal_f32(47, keys * kvh * D, 1.0))
    g["attn_q"], g["attn_k"], g["attn_v"] = q, kk, vv
    g["attn_out"] = orc.attention(bf16_bits_to_f32(q), bf16_bits_to_f32(kk), bf16_bits_to_f32(vv), heads, kvh, D,
                                  keys - nq, 1.0 / np.sqrt(D))
    g["attn_out_window33"] = orc.attention(bf16_bits_to_f32(q), bf16_bits_to_f32(kk), bf16_bits_to_f32(vv), heads, kvh,
                                           D, keys - nq, 1.0 / np.sqrt(D), window=33)
    return g


if __name__ == "__main__":
    out = os.path.join(HERE, "hot_path_golden.npz")
    np.savez_compressed(out, **build(oracle()))
    print(out, os.path.getsize(out), "bytes")
