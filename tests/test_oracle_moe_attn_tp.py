"""The oracle's router, row plan, attention and shard arithmetic against the reference's
in-source known-answer tests (cited by file:line, paths relative to the reference root)."""
import numpy as np
import pytest

from oracle_lib import bf16_bits_to_f32, f32_to_bf16_bits  # noqa: E402

MTILE = 16  # the reference's m16 MMA tile (src/models/inkling/moegroup.rs)


def test_rows_are_stacked_in_expert_order_with_padding(orc):
    # src/models/inkling/moegroup.rs:1947-1989: e0=[(1,.5)], e1=[(0,.25),(1,.125)], e2=[(0,.75)]
    idx = np.array([[1, 2], [0, 1]], np.uint32)
    wgt = np.array([[0.25, 0.75], [0.5, 0.125]], np.float32)
    plan = orc.row_plan(idx, wgt, 3, MTILE)
    assert plan["m_total"] == 3 * MTILE
    assert list(plan["slot_expert"]) == [0, 1, 2]
    assert list(plan["slot_row0"] // MTILE) == [0, 1, 2]          # blk_tile0, one tile each
    rt = plan["row_tok"]
    assert rt[0] == 1 and rt[1] == -1 and rt[MTILE] == 0 and rt[MTILE + 1] == 1 and rt[2 * MTILE] == 0
    assert plan["kmax"] == 2 and list(plan["tok_cnt"]) == [2, 2]
    assert list(plan["tok_rows"][0]) == [MTILE, 2 * MTILE]
    assert list(plan["tok_rows"][1]) == [0, MTILE + 1]
    rw = plan["row_wgt"]
    assert rw[0] == 0.5 and rw[1] == 0.0 and rw[MTILE] == 0.25 and rw[MTILE + 1] == 0.125 and rw[2 * MTILE] == 0.75


def test_every_tile_of_the_layer_is_served_once(orc):
    # src/models/inkling/moegroup.rs:1991-2007: 65, 3 and 130 tokens -> 5 + 1 + 9 tiles of 16 rows
    counts = [4 * MTILE + 1, 3, 8 * MTILE + 2]
    n = counts[2]
    idx = np.full((n, 3), 0, np.uint32)
    # token t picks expert 0 if t < 65, expert 1 if t < 3, expert 2 always; unused picks go to a 4th expert
    rows = []
    for t in range(n):
        picks = [e for e, c in enumerate(counts) if t < c]
        picks += [3] * (3 - len(picks))
        rows.append(picks)
    idx = np.array(rows, np.uint32)
    plan = orc.row_plan(idx, np.ones(idx.shape, np.float32), 4, MTILE)
    tiles = [(int(c) + MTILE - 1) // MTILE for c in plan["slot_rows"][:3]]
    assert tiles == [5, 1, 9]
    assert list(plan["slot_row0"][:3] // MTILE) == [0, 5, 6]
    # rows of one expert keep token order
    rt = plan["row_tok"][: counts[0]]
    assert list(rt) == list(range(counts[0]))


def test_bias_moves_selection_not_weights_and_renormalise(orc):
    # src/models/k3/router.rs:518-556 restated on the softmax branch the BASELINE config uses
    w = np.array([[2.0, 0], [1.0, 0], [0.5, 0], [0.0, 0]], np.float32)
    h = np.array([1.0, 0.0], np.float32)
    logits = (w @ h).reshape(1, 4).astype(np.float32)
    scores = orc.router_scores_softmax(logits)
    idx0, w0 = orc.router_select(scores, 2)
    assert list(idx0[0]) == [0, 1]
    assert abs(float(w0.sum()) - 1.0) < 1e-6
    idx1, w1 = orc.router_select(scores, 2, bias=[0, 0, 0, 1.0], renormalize=False)
    assert list(idx1[0]) == [3, 0]
    assert w1[0, 0] == scores[0, 3] and w1[0, 1] == scores[0, 0] and w1[0, 0] < 1.0
    # ties go to the lower index (router.rs:410-419)
    flat = np.zeros((1, 8), np.float32)
    idx, wt = orc.router_select(orc.router_scores_softmax(flat), 3)
    assert list(idx[0]) == [0, 1, 2]
    with pytest.raises(ValueError):
        orc.router_select(np.array([[np.nan, 1.0]], np.float32), 1)


def test_sigmoid_router_known_answers(orc):
    # src/models/k3/router.rs:518-556 as written there (RouterActivation::Sigmoid, hidden 2, 4 experts, top-2)
    w = np.array([[2.0, 0], [1.0, 0], [0.5, 0], [0.0, 0]], np.float32)
    logits = (w @ np.array([1.0, 0.0], np.float32)).reshape(1, 4).astype(np.float32)
    scores = orc.router_scores_sigmoid(logits)
    want = (1.0 / (1.0 + np.exp(-logits.astype(np.float64)))).astype(np.float32)
    assert np.array_equal(scores, want)
    idx0, w0 = orc.router_select(scores, 2)
    assert list(idx0[0]) == [0, 1]
    assert abs(float(w0.sum()) - 1.0) < 1e-6            # weights_renormalise_to_one
    idx1, w1 = orc.router_select(scores, 2, bias=[0, 0, 0, 1.0], renormalize=False)
    assert list(idx1[0]) == [3, 0]                      # bias_moves_selection_not_weights
    assert w1[0, 0] == scores[0, 3] and w1[0, 1] == scores[0, 0]
    assert w1[0, 0] < 1.0                               # the bias is not in the weight


def test_sink_router_known_answers(orc):
    # src/models/inkling/block.rs:273-300 as written there
    with pytest.raises(ValueError, match="token 0, row 3"):
        orc.router_sinks(np.array([[0.25, -0.5, 1.0, np.nan]], np.float32), [0.0, 0.0], 2, 1)
    logits = np.array([[0.25, -0.5, 1.0, -2.0], [0.75, 0.125, -0.25, 0.5]], np.float32)
    idx, w, gam = orc.router_sinks(logits, [0.0, 0.0], 2, 1)
    assert w.size + gam.size == 6 and np.isfinite(w).all() and np.isfinite(gam).all()
    assert idx.tolist() == [[0], [0]]
    # the chosen routed experts and the sinks share one softmax: the weights sum to route_scale * global_scale
    idx, w, gam = orc.router_sinks(logits, [0.0, 0.0], 2, 1, global_scale=0.5, route_scale=2.5)
    assert np.allclose(w.sum(1) + gam.sum(1), 1.25, rtol=1e-6)
    # restated: weights are softmax(log_sigmoid(logits)) over [chosen, sinks], i.e. sigmoid / sum of sigmoids
    sg = 1.0 / (1.0 + np.exp(-logits.astype(np.float64)))
    want = sg[0, [0, 2, 3]] / sg[0, [0, 2, 3]].sum() * 1.25
    assert np.allclose(np.concatenate([w[0], gam[0]]), want, rtol=1e-5)
    # the bias moves the selection and takes no part in the weights (block.rs:236-252)
    idx_b, w_b, gam_b = orc.router_sinks(logits, [0.0, 1.0], 2, 1)
    assert idx_b.tolist() == [[1], [1]]
    sg1 = sg[1, [1, 2, 3]] / sg[1, [1, 2, 3]].sum()
    assert np.allclose(np.concatenate([w_b[1], gam_b[1]]), sg1, rtol=1e-5)
    # ties go to the lower index
    idx_t, _, _ = orc.router_sinks(np.zeros((1, 6), np.float32), np.zeros(4, np.float32), 4, 3)
    assert idx_t.tolist() == [[0, 1, 2]]


def test_softmax_scores_follow_the_f64_recipe(orc):
    # router.rs:352-368: f64 exp, f32 store, f32(f64(v)/s)
    rng = np.random.default_rng(0)
    logits = rng.standard_normal((5, 128)).astype(np.float32) * 3
    got = orc.router_scores_softmax(logits)
    for t in range(5):
        m = logits[t].astype(np.float64).max()
        e = np.exp(logits[t].astype(np.float64) - m)
        v = e.astype(np.float32)
        s = 0.0
        for x in e:
            s += x
        want = (v.astype(np.float64) / s).astype(np.float32)
        assert np.array_equal(got[t], want)


def test_bf16_widening_is_a_shift(orc):
    # router.rs:567-572
    from oracle_lib import bf16_bits_to_f32
    assert list(bf16_bits_to_f32(np.array([0x3F80, 0xBF80], np.uint16))) == [1.0, -1.0]
    assert orc.lib.orc_bf16_to_f32(0x3F80) == 1.0


def test_cpu_attention_uses_absolute_positions_and_window_edges(orc):
    # src/models/inkling/flash.rs:1989-2016 (scale plays the role of 1/head_dim there: zero logits anyway)
    for window, expected in [(0, [5.5, 5.5, 37.0]), (3, [10.0, 10.0, 100.0])]:
        out = orc.attention(np.zeros(3), np.zeros(4), np.array([1.0, 10.0, 100.0, 1000.0]), heads=1, kv_heads=1, D=1,
                            q0=3, scale=1.0, key_pos=[0, 2, 5, 9], window=window)
        assert np.allclose(out.ravel(), expected, atol=1e-12)


def test_packed_kv_reader_index_rule(orc):
    # src/models/inkling/flash.rs:520-540 `nvfp4_at`: element idx of a [rows, kv_heads * head_dim] page lives in
    # word idx / 8 at nibble idx % 8, its scale is E4M3 byte idx / 16, value = E2M1[code] * scale (no global scale);
    # src/models/inkling/kvpages.rs:1378-1404: the page is the row-major quantization of those rows.
    rows, kvh, D = 5, 2, 128
    width = kvh * D
    x = orc.normal_f32(31, rows * width, 2.0)
    codes, scales = orc.quantize_act_recip(x, rows, width)
    words = codes.view(np.uint32)
    e2m1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0.0, -.5, -1, -1.5, -2, -3, -4, -6], np.float32)
    idx = np.arange(rows * width)
    code = (words[idx // 8] >> ((idx % 8) * 4).astype(np.uint32)) & 15
    sc = np.array([orc.e4m3_to_f32(int(b)) for b in scales], np.float32)[idx // 16]
    want = e2m1[code] * sc
    got = orc.dequantize(codes, scales, 1.0)
    assert np.array_equal(got.reshape(-1), want)
    # a row's bytes are its own: appending rows changes no earlier byte (kvpages.rs: "paged-safe")
    c2, s2 = orc.quantize_act_recip(x[: 3 * width], 3, width)
    assert np.array_equal(c2, codes[: 3 * width // 2]) and np.array_equal(s2, scales[: 3 * width // 16])
    # every value is exact in f16 and in bf16 (at most 7 significant bits, magnitude within [2^-10, 2688])
    assert np.array_equal(want.astype(np.float16).astype(np.float32), want)
    assert np.array_equal(bf16_bits_to_f32(f32_to_bf16_bits(want)), want)


def test_fp4_cache_rows_geometry_blocks_and_round_trip_bound(orc):
    # src/models/inkling/kvpages.rs:2996-3010: [rows, width/8] code words, [rows, width/64] scale words, 4.5 bits a value
    FW = 128
    x = orc.normal_f32(7, 3 * FW, 1.0)
    codes, scales = orc.quantize_act_recip(x, 3, FW)
    assert codes.size == 3 * (FW // 8) * 4 and scales.size == 3 * (FW // 64) * 4
    assert (FW // 8 + FW // 64) * 4 * 32 == FW * 2 * 9
    # kvpages.rs:3014-3030: alternating 16-blocks of 0.5 and 200 survive, so the blocks run along the features
    vals = np.array([0.5 if (j // 16) % 2 == 0 else 200.0 for j in range(FW)], np.float32)
    c, s = orc.quantize_act_recip(vals, 1, FW)
    got = orc.dequantize(c, s, 1.0)
    assert np.all(np.abs(got - vals) <= vals / 16.0)
    # kvpages.rs:3032-3100: a 1024-wide bf16 row loses less than 1/3 + 1/16 of its block amax
    KW, n = 1024, 40
    i = np.arange(n * KW, dtype=np.uint64)
    t = ((i * np.uint64(2654435761)) % np.uint64(2003)).astype(np.float32) / np.float32(1001.5) - np.float32(1.0)
    a = bf16_bits_to_f32(f32_to_bf16_bits((t * t * t * np.float32(8.0)).astype(np.float32)))
    c, s = orc.quantize_act_recip(a, n, KW)
    b = orc.dequantize(c, s, 1.0)
    amax = np.maximum(np.abs(a).reshape(-1, 16).max(1), 1e-6)
    worst = (np.abs(a - b).reshape(-1, 16) / amax[:, None]).max()
    assert worst < 1.0 / 3.0 + 1.0 / 16.0, worst


def _band_inputs(tokens, heads, kvh, D, window):
    fill = lambda n, ph: (np.sin(np.arange(n) * 0.37 + ph) * 0.5).astype(np.float32)
    eff = min(window, tokens)
    return (fill(tokens * heads * D, 0.1), fill(tokens * kvh * D, 0.3), fill(tokens * kvh * D, 0.5),
            fill(tokens * heads * eff, 0.7).reshape(tokens, heads, eff))


def test_window_reach_and_group_isolation(orc):
    # src/models/inkling/banded.rs:412-460: a key `window` back from the last query is outside its window (the
    # answer does not move at all), the query's own key is inside (it moves)
    for tokens, heads, kvh, D, window in [(40, 4, 2, 8, 8), (70, 8, 2, 16, 12), (11, 4, 2, 4, 5)]:
        q, k, v, rel = _band_inputs(tokens, heads, kvh, D, window)
        band = lambda kk, vv: orc.attention(q, kk, vv, heads, kvh, D, 0, 1.0 / D, window=window, rel=rel)
        base = band(k, v)
        last = tokens - 1
        for j, must_move in [(last - window, False), (last, True)]:
            kk, vv = k.copy(), v.copy()
            kk[j * kvh * D:(j + 1) * kvh * D] += 0.75
            vv[j * kvh * D:(j + 1) * kvh * D] -= 0.75
            moved = np.abs(band(kk, vv)[last] - base[last]).max()
            assert (moved > 1e-4) if must_move else (moved == 0.0), (tokens, j, moved)
    # banded.rs:462-500: a KV head reaches only the query heads of its own group
    tokens, heads, kvh, D, window = 24, 8, 2, 16, 12
    q, k, v, rel = _band_inputs(tokens, heads, kvh, D, window)
    base = orc.attention(q, k, v, heads, kvh, D, 0, 1.0 / D, window=window, rel=rel)
    at = tokens // 2
    for c in range(kvh):
        kk, vv = k.copy(), v.copy()
        kk[at * kvh * D + c * D: at * kvh * D + (c + 1) * D] += 0.5
        vv[at * kvh * D + c * D: at * kvh * D + (c + 1) * D] -= 0.5
        got = orc.attention(q, kk, vv, heads, kvh, D, 0, 1.0 / D, window=window, rel=rel)
        for h in range(heads):
            moved = np.abs(got[:, h * D:(h + 1) * D] - base[:, h * D:(h + 1) * D]).max()
            assert (moved > 1e-4) if h // (heads // kvh) == c else (moved == 0.0), (c, h, moved)


def test_attention_relative_bias_enters_by_distance(orc):
    # src/models/inkling/flash.rs:1966-1972: bias rel[(qi * heads + h) * eff + dist] for dist < eff, after the scale
    q = np.zeros((2, 1)); k = np.zeros((4, 1)); v = np.array([1.0, 10.0, 100.0, 1000.0])
    rel = np.array([[np.log(3.0), 0.0], [0.0, np.log(2.0)]], np.float32)     # [nq = 2, heads = 1, eff = 2]
    out = orc.attention(q, k, v, heads=1, kv_heads=1, D=1, q0=2, scale=1.0, rel=rel)
    # query 0 at position 2 sees keys 0..2: weights 1, 1, 3 (distance 0 carries log 3)
    assert np.isclose(out[0, 0], (1 + 10 + 3 * 100) / 5, rtol=1e-6)
    # query 1 at position 3 sees keys 0..3: distance 1 (key 2) carries log 2
    assert np.isclose(out[1, 0], (1 + 10 + 2 * 100 + 1000) / 5, rtol=1e-6)
    # with gaps the distance is in absolute positions: key rows 0..3 sit at 0, 1, 5, 6
    out = orc.attention(q, k, v, heads=1, kv_heads=1, D=1, q0=5, scale=1.0, key_pos=[0, 1, 5, 6], rel=rel)
    assert np.isclose(out[0, 0], (1 + 10 + 3 * 100) / 5, rtol=1e-6)           # position 5: key row 2 at distance 0
    assert np.isclose(out[1, 0], (1 + 10 + 2 * 100 + 1000) / 5, rtol=1e-6)    # position 6: key row 2 at distance 1


def test_attention_gqa_and_causality(orc):
    rng = np.random.default_rng(1)
    heads, kvh, D, nq, keys = 4, 2, 8, 3, 6
    q = rng.standard_normal((nq, heads * D)).astype(np.float32)
    k = rng.standard_normal((keys, kvh * D)).astype(np.float32)
    v = rng.standard_normal((keys, kvh * D)).astype(np.float32)
    out = orc.attention(q, k, v, heads, kvh, D, q0=3, scale=1 / np.sqrt(D))
    # numpy two-pass reference, kv head = h // (heads // kv_heads) (src/models/inkling/attn.rs:283-331)
    for qi in range(nq):
        for h in range(heads):
            g = h // (heads // kvh)
            vis = [j for j in range(keys) if j <= 3 + qi]
            s = np.array([q[qi, h * D:(h + 1) * D].astype(np.float64) @ k[j, g * D:(g + 1) * D] / np.sqrt(D) for j in vis])
            p = np.exp(s - s.max())
            p /= p.sum()
            want = sum(p[i] * v[j, g * D:(g + 1) * D].astype(np.float64) for i, j in enumerate(vis))
            assert np.allclose(out[qi, h * D:(h + 1) * D], want, atol=1e-12)
    # changing a masked (future) key must not move the answer
    k2 = k.copy()
    k2[5] += 100
    out2 = orc.attention(q, k2, v, heads, kvh, D, q0=3, scale=1 / np.sqrt(D))
    assert np.array_equal(out[:2], out2[:2])


def test_shards_tile_the_axis_and_gqa_cut(orc):
    # src/models/inkling/tp.rs:761-793
    for world in (1, 2, 4, 8):
        for extent in (32, 8, 256, 201024, 16384):
            if extent % world:
                continue
            seen = np.zeros(extent, np.uint8)
            for rank in range(world):
                lo, hi = orc.tp_shard(rank, world, extent)
                seen[lo:hi] += 1
            assert (seen == 1).all()
    assert orc.tp_shard(0, 2, 32) == (0, 16) and orc.tp_shard(1, 2, 32) == (16, 32)
    assert orc.tp_shard(0, 2, 8) == (0, 4) and orc.tp_shard(1, 2, 8) == (4, 8)
    assert orc.tp_shard(0, 1, 32) == (0, 32)          # the identity world shards nothing
    with pytest.raises(ValueError):
        orc.tp_shard(0, 3, 32)                        # Indivisible


def test_gate_up_silu_readings_and_ordered_scatter(orc):
    # src/models/inkling/fp4gemm.rs:472-507: interleaved vs halved; moegroup.rs:1690-1716: ascending fma
    both = np.arange(8, dtype=np.float32).reshape(1, 8) / 4
    inter = 4
    silu = lambda g: g / (1 + np.exp(-g))
    a = orc.gate_up_silu(both, 1, inter, halved=False)[0]
    assert np.allclose(a, [silu(both[0, 2 * i]) * both[0, 2 * i + 1] for i in range(inter)], rtol=1e-6)
    b = orc.gate_up_silu(both, 1, inter, halved=True)[0]
    assert np.allclose(b, [silu(both[0, i]) * both[0, inter + i] for i in range(inter)], rtol=1e-6)
    y = np.array([[1.0, 2.0], [10.0, 20.0], [100.0, 200.0]], np.float32)
    wgt = np.array([0.5, 0.25, 0.125], np.float32)
    out = orc.scatter_weighted(y, wgt, np.array([[0, 2], [1, 0]], np.uint32), np.array([2, 1], np.uint32), 2)
    assert np.array_equal(out, np.array([[13.0, 26.0], [2.5, 5.0]], np.float32))
