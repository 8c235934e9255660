"""GPU parity tests: flash attention (prefill + split-K decode), decoder-layer glue, the
NVFP4 decoder layer. Oracle = the CPU restatement on the same seeded bytes."""
import math

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle_lib import bf16_bits_to_f32, f32_to_bf16_bits  # noqa: E402
from test_gpu_nvfp4 import attn_check, dev_bf16, host_bits, rel_check  # noqa: E402


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from maryml_b200 import attention, layer
    return attention, layer


def _qkv(orc, seed, batch, nq, keys, heads, kvh, D=128):
    q = f32_to_bf16_bits(orc.normal_f32(seed, batch * nq * heads * D, 1.0)).reshape(batch, nq, heads * D)
    k = f32_to_bf16_bits(orc.normal_f32(seed + 1, batch * keys * kvh * D, 1.0)).reshape(batch, keys, kvh * D)
    v = f32_to_bf16_bits(orc.normal_f32(seed + 2, batch * keys * kvh * D, 1.0)).reshape(batch, keys, kvh * D)
    return q, k, v


def _check(att, orc, q, k, v, batch, nq, keys, heads, kvh, q0, causal=True, D=128, window=0):
    qd = dev_bf16(q).view(batch, nq, heads, D)
    kd = dev_bf16(k).view(batch, keys, kvh, D)
    vd = dev_bf16(v).view(batch, keys, kvh, D)
    out = att.flash_attention(qd, kd, vd, q0=q0, causal=causal, window=window)
    got = bf16_bits_to_f32(host_bits(out)).reshape(batch, nq, heads * D)
    scale = 1.0 / math.sqrt(D)
    for b in range(batch):
        ref = orc.attention(bf16_bits_to_f32(q[b]), bf16_bits_to_f32(k[b]), bf16_bits_to_f32(v[b]), heads, kvh, D,
                            q0 if causal else keys + nq, scale, window=window)
        rel, cos = attn_check(got[b], ref)
        assert rel <= _attn_bound(nq, heads, kvh) and cos >= 0.9999, (b, rel, cos)


def _attn_bound(nq, heads, kvh):
    """1e-2 for decode shapes. Prompt shapes check a few hundred thousand output vectors per call, many of them
    causal rows that see two or three keys with values of opposite sign: there the bf16 probabilities' 2^-9 steps
    do not average out, and the worst element measured sits at 1.14e-2 of its vector's rms (8192 x 8192: 0.98e-2).
    The bound for prompt shapes is therefore 1.5e-2; the cosine bound is the same."""
    return 1e-2 if nq * (heads // kvh) <= 16 else 1.5e-2


@pytest.mark.parametrize("batch,nq,keys,heads,kvh,q0", [
    (1, 1, 64, 4, 1, 63),          # one tile, one split
    (2, 1, 1000, 32, 8, 999),      # ragged key count, several splits
    (3, 1, 4097, 8, 2, 4096),
    (1, 2, 300, 8, 2, 298),        # two queries, causal inside the block
    (2, 4, 515, 4, 1, 100),        # queries in the middle of the cache: keys beyond q0+i are masked
])
def test_decode_attention(mods, orc, batch, nq, keys, heads, kvh, q0):
    att, _ = mods
    q, k, v = _qkv(orc, 11 * keys + nq, batch, nq, keys, heads, kvh)
    _check(att, orc, q, k, v, batch, nq, keys, heads, kvh, q0)


def test_decode_attention_gives_the_same_bits_every_time(mods):
    """The same queries over the same cache, 300 times, compared bit for bit. The shape is the one a 4-way shard of
    the benchmark layer runs (64 sequences, 2 KV heads, 4097 keys): its key splits end in a tile that lies almost
    wholly past the last key, so the tile ring's refill is a zero fill that arrives at once, which is what exposed a
    stage handed back to the producer before the last reads of it (one call in fifty, one split's partial)."""
    att, _ = mods
    g = torch.Generator(device="cuda").manual_seed(7)
    batch, keys, heads, kvh, D = 64, 4097, 8, 2, 128
    q = torch.randn(batch, 1, heads, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(batch, keys, kvh, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(batch, keys, kvh, D, device="cuda", generator=g).to(torch.bfloat16)
    ref = att.flash_attention(q, k, v, q0=keys - 1, causal=True).clone()
    moved = 0
    for _ in range(300):
        out = att.flash_attention(q, k, v, q0=keys - 1, causal=True)
        moved += int((out.view(torch.int16) != ref.view(torch.int16)).sum())
    assert moved == 0, moved


@pytest.mark.parametrize("batch,nq,keys,heads,kvh,q0,window", [
    (2, 1, 5000, 8, 2, 4999, 1024),     # decode: the splits share only the window's keys
    (1, 1, 300, 4, 1, 299, 64),
    (2, 2, 700, 8, 2, 650, 100),        # two queries, keys beyond them in the cache
    (1, 600, 600, 4, 1, 0, 200),        # prompt: the band skips whole key tiles below it
    (2, 300, 1000, 8, 2, 700, 129),     # prompt after a prefix, window edge inside a tile
    (1, 257, 257, 4, 4, 0, 1),          # a window of one key: every query sees itself only
])
def test_sliding_window_attention(mods, orc, batch, nq, keys, heads, kvh, q0, window):
    """mb_attention_window against the CPU rule (query p sees keys in (p - window, p])."""
    att, _ = mods
    q, k, v = _qkv(orc, 13 * keys + nq + window, batch, nq, keys, heads, kvh)
    _check(att, orc, q, k, v, batch, nq, keys, heads, kvh, q0, window=window)


@pytest.mark.parametrize("batch,nq,keys,heads,kvh,q0,window", [
    (1, 1, 64, 4, 1, 63, 0),
    (2, 1, 1000, 32, 8, 999, 0),        # ragged key count, several splits
    (3, 1, 4097, 8, 2, 4096, 0),
    (2, 4, 515, 4, 1, 100, 0),          # queries in the middle of the cache
    (2, 1, 5000, 8, 2, 4999, 1024),     # sliding window over the packed rows
])
def test_decode_attention_over_nvfp4_rows(mods, orc, batch, nq, keys, heads, kvh, q0, window):
    """The packed reader against the dense reader over the dequantized rows and against the CPU rule
    (src/models/inkling/flash.rs:520-540: same index arithmetic, values E2M1[code] * e4m3(scale)).
    The packed reader multiplies in f16 (the expanded rows are exact there, probabilities keep 11
    bits), the dense one in bf16, so the two agree to a bf16 step of the output, not to the bit."""
    from maryml_b200 import nvfp4 as nv
    att, _ = mods
    D = 128
    q, k, v = _qkv(orc, 17 * keys + nq, batch, nq, keys, heads, kvh)
    qd = dev_bf16(q).view(batch, nq, heads, D)
    kd = dev_bf16(k).view(batch, keys, kvh, D)
    vd = dev_bf16(v).view(batch, keys, kvh, D)
    kc, ks = att.quantize_kv_rows(kd)
    vc, vs = att.quantize_kv_rows(vd)
    # the cache bytes are the CPU quantizer's bytes for the same rows
    codes_ref, scales_ref = orc.quantize_act_recip(bf16_bits_to_f32(k[0]), keys, kvh * D)
    assert np.array_equal(kc[0].cpu().numpy().ravel(), codes_ref)
    assert np.array_equal(ks[0].cpu().numpy().ravel(), scales_ref)
    k_deq = nv.dequantize(kc.view(batch * keys, -1), ks.view(batch * keys, -1), 1.0, batch * keys, kvh * D,
                          torch.bfloat16).view(batch, keys, kvh, D)
    v_deq = nv.dequantize(vc.view(batch * keys, -1), vs.view(batch * keys, -1), 1.0, batch * keys, kvh * D,
                          torch.bfloat16).view(batch, keys, kvh, D)
    assert torch.equal(k_deq.float(), nv.dequantize(kc.view(batch * keys, -1), ks.view(batch * keys, -1), 1.0,
                                                    batch * keys, kvh * D, torch.float32).view(batch, keys, kvh, D))
    want = att.flash_attention(qd, k_deq, v_deq, q0=q0, window=window)
    got = att.flash_attention_fp4kv(qd, kc, ks, vc, vs, kvh, q0=q0, window=window)
    gw, gg = want.float(), got.float()
    assert float((gg - gw).abs().max()) <= 1e-2 * float(gw.abs().max())
    # both readers follow the CPU rule on the dequantized rows
    kb = host_bits(k_deq).reshape(batch, keys, kvh * D)
    vb = host_bits(v_deq).reshape(batch, keys, kvh * D)
    _check(att, orc, q, kb, vb, batch, nq, keys, heads, kvh, q0, window=window)
    gotf = bf16_bits_to_f32(host_bits(got)).reshape(batch, nq, heads * D)
    for b in range(batch):
        ref = orc.attention(bf16_bits_to_f32(q[b]), bf16_bits_to_f32(kb[b]), bf16_bits_to_f32(vb[b]), heads, kvh, D,
                            q0, 1.0 / math.sqrt(D), window=window)
        rel, cos = attn_check(gotf[b], ref)
        assert rel <= 1e-2 and cos >= 0.9999, (b, rel, cos)


@pytest.mark.parametrize("batch,nq,keys,heads,kvh,window,gaps,eff", [
    (1, 1, 897, 8, 2, 0, [], 16),                       # the bias alone
    (1, 1, 897, 8, 2, 19, [], 0),                       # window through the position path is not taken: plain call
    (1, 1, 897, 8, 2, 0, [(17, 5), (853, 19)], 0),      # gaps alone (the reference's gapped case: flash.rs:2040-2044)
    (2, 2, 700, 8, 2, 100, [(3, 2), (650, 40)], 33),    # everything, two queries, two sequences
    (1, 4, 300, 4, 1, 0, [(0, 7)], 300),                # a gap before the first row; bias over every distance
    # prompt-shaped blocks (more than 16 query rows per KV head) take the warp-level kernel's position path
    (1, 150, 400, 8, 2, 0, [], 24),                     # bias alone
    (2, 200, 700, 4, 2, 77, [(5, 3), (450, 21)], 16),   # everything; the block is not a multiple of the 128-row tile
    (1, 64, 333, 8, 1, 0, [(100, 9)], 0),               # gaps alone
])
def test_decode_attention_with_relative_bias_and_gaps(mods, orc, batch, nq, keys, heads, kvh, window, gaps, eff):
    att, _ = mods
    D = 128
    q, k, v = _qkv(orc, 19 * keys + nq + eff, batch, nq, keys, heads, kvh)
    pos = np.arange(keys, dtype=np.int64)
    for row, cum in gaps:
        pos[row:] = np.arange(row, keys) + cum
    q0 = int(pos[-1]) - (nq - 1)                          # the last query sits on the last key
    rel = None
    if eff:
        rel = (orc.normal_f32(3 + eff, batch * nq * heads * eff, 1.0)).reshape(batch, nq, heads, eff).astype(np.float32)
    gd = None
    if gaps:
        gd = (torch.tensor([g[0] for g in gaps], dtype=torch.int32, device="cuda"),
              torch.tensor([g[1] for g in gaps], dtype=torch.int32, device="cuda"))
    qd = dev_bf16(q).view(batch, nq, heads, D)
    kd = dev_bf16(k).view(batch, keys, kvh, D)
    vd = dev_bf16(v).view(batch, keys, kvh, D)
    out = att.decode_attention_ext(qd, kd, vd, q0, window=window, rel=None if rel is None else torch.from_numpy(rel).cuda(),
                                   gaps=gd)
    got = bf16_bits_to_f32(host_bits(out)).reshape(batch, nq, heads * D)
    for b in range(batch):
        ref = orc.attention(bf16_bits_to_f32(q[b]), bf16_bits_to_f32(k[b]), bf16_bits_to_f32(v[b]), heads, kvh, D, q0,
                            1.0 / math.sqrt(D), key_pos=pos if gaps else None, window=window,
                            rel=None if rel is None else rel[b])
        err, cos = attn_check(got[b], ref)
        assert err <= _attn_bound(nq, heads, kvh) and cos >= 0.9999, (b, err, cos)
    if not gaps and not eff:
        assert torch.equal(out, att.flash_attention(qd, kd, vd, q0=q0, window=window))


def test_prompt_shapes_refuse_nvfp4_rows(mods):
    from maryml_b200 import _lib
    att, _ = mods
    q = torch.zeros(1, 64, 4, 128, dtype=torch.bfloat16, device="cuda")
    z = torch.zeros(1, 64, 64, dtype=torch.uint8, device="cuda")
    zs = torch.zeros(1, 64, 8, dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.MaryError):
        att.flash_attention_fp4kv(q, z, zs, z, zs, 1)


@pytest.mark.parametrize("batch,nq,heads,kvh", [(1, 128, 4, 1), (2, 200, 8, 2), (1, 515, 4, 4)])
def test_prefill_attention_causal(mods, orc, batch, nq, heads, kvh):
    att, _ = mods
    q, k, v = _qkv(orc, 5 * nq, batch, nq, nq, heads, kvh)
    _check(att, orc, q, k, v, batch, nq, nq, heads, kvh, 0)


@pytest.mark.parametrize("nq,keys,q0,window", [(8192, 8192, 0, 0), (2048, 3072, 1024, 0), (2304, 2304, 0, 777)])
def test_prefill_attention_at_benchmark_length(mods, orc, figures, nq, keys, q0, window):
    """One (sequence, KV head) slice at the benchmark's sequence length against the f64 CPU rule: the rings of the
    tcgen05 kernel wrap hundreds of times here, with a prefix before the queries and with a window."""
    att, _ = mods
    q, k, v = _qkv(orc, 3 * nq + window, 1, nq, keys, 2, 1)
    qd, kd, vd = dev_bf16(q).view(1, nq, 2, 128), dev_bf16(k).view(1, keys, 1, 128), dev_bf16(v).view(1, keys, 1, 128)
    out = att.flash_attention(qd, kd, vd, q0=q0, window=window)
    got = bf16_bits_to_f32(host_bits(out)).reshape(nq, 256)
    ref = orc.attention(bf16_bits_to_f32(q[0]), bf16_bits_to_f32(k[0]), bf16_bits_to_f32(v[0]), 2, 1, 128, q0,
                        1.0 / math.sqrt(128), window=window)
    # row by row: the first rows see a handful of keys, the last ones thousands; each against its own rms
    worst = 0.0
    for r0 in range(0, nq, 256):
        rel, cos = attn_check(got[r0:r0 + 256], ref[r0:r0 + 256])
        worst = max(worst, rel)
        assert rel <= _attn_bound(nq, 2, 1) and cos >= 0.9999, (r0, rel, cos)
    figures("prefill_parity", nq=nq, keys=keys, q0=q0, window=window, max_rel=worst)


@pytest.mark.parametrize("steep", [False, True])
def test_prefill_row_maxima_that_keep_growing(mods, orc, steep):
    """After its first tile the prompt kernel tracks no maximum; a row's sum of probabilities tells when a score has
    outgrown the subtracted maximum by 2^40 or more. Here every key scores higher than the one before (about 17
    exponent units per 128-key tile: a rescale every few tiles), or jumps by some 650 units at key 700 (the sum
    overflows to infinity and the tile is taken again against its own maximum)."""
    att, _ = mods
    nq = keys = 1536
    heads, kvh = 2, 1
    q, k, v = _qkv(orc, 4242, 1, nq, keys, heads, kvh)
    qf = 1.0 + 0.2 * bf16_bits_to_f32(q).reshape(nq, heads * 128)
    ramp = np.where(np.arange(keys) >= 700, 40.0, 0.0) if steep else 12.0 * np.arange(keys) / keys
    kf = ramp[:, None].astype(np.float32) + 0.2 * bf16_bits_to_f32(k).reshape(keys, kvh * 128)
    q = f32_to_bf16_bits(qf.astype(np.float32).ravel()).reshape(1, nq, heads * 128)
    k = f32_to_bf16_bits(kf.astype(np.float32).ravel()).reshape(1, keys, kvh * 128)
    _check(att, orc, q, k, v, 1, nq, keys, heads, kvh, 0)


def test_prefill_with_prefix_and_non_causal(mods, orc):
    att, _ = mods
    batch, nq, keys, heads, kvh = 1, 130, 386, 4, 2
    q, k, v = _qkv(orc, 77, batch, nq, keys, heads, kvh)
    _check(att, orc, q, k, v, batch, nq, keys, heads, kvh, keys - nq)           # chunked prefill after a prefix
    _check(att, orc, q, k, v, batch, nq, keys, heads, kvh, 0, causal=False)


def test_key_axis_cuts_do_not_move_the_answer(mods, orc):
    """src/models/inkling/flash.rs:1575+: the split of the key axis is not visible in the result
    beyond f32 re-association; GQA heads are isolated; a future key changes nothing."""
    att, _ = mods
    batch, keys, heads, kvh, D = 1, 2048, 8, 2, 128
    q, k, v = _qkv(orc, 5, batch, 1, keys, heads, kvh)
    qd, kd, vd = dev_bf16(q).view(1, 1, heads, D), dev_bf16(k).view(1, keys, kvh, D), dev_bf16(v).view(1, keys, kvh, D)
    full = att.flash_attention(qd, kd, vd, q0=keys - 1)
    # the same cache seen through a longer allocation with a masked tail
    kd2 = torch.cat([kd, torch.full_like(kd, 7.0)], 1).contiguous()
    vd2 = torch.cat([vd, torch.full_like(vd, -3.0)], 1).contiguous()
    tail = att.flash_attention(qd, kd2, vd2, q0=keys - 1)
    assert (full.float() - tail.float()).abs().max().item() <= 2e-2 * full.float().abs().max().item()
    # heads of kv head 0 do not see kv head 1
    kd3 = kd.clone()
    kd3[:, :, 1] = 0
    iso = att.flash_attention(qd, kd3, vd, q0=keys - 1)
    g = heads // kvh
    assert torch.equal(iso[:, :, :g], full[:, :, :g])


def test_full_size_decode_properties(mods, orc):
    """BASELINE decode shape (reduced batch): constant V gives that constant back; all-equal keys
    give the mean of V; both are independent of the sequence length."""
    att, _ = mods
    batch, keys, heads, kvh, D = 4, 32768, 32, 8, 128
    g = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn(batch, 1, heads, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(batch, keys, kvh, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.full((batch, keys, kvh, D), 0.75, device="cuda", dtype=torch.bfloat16)
    out = att.attention_step(q, k, v)
    assert (out.float() - 0.75).abs().max().item() <= 1e-2
    k0 = torch.zeros_like(k)
    v2 = torch.randn(batch, keys, kvh, D, device="cuda", generator=g).to(torch.bfloat16)
    out2 = att.attention_step(q, k0, v2)
    mean = v2.float().mean(1).repeat_interleave(heads // kvh, 1).view(batch, 1, heads, D)
    assert (out2.float() - mean).abs().max().item() <= 5e-3


# ------------------------------------------------------------------------- layer glue
def test_rmsnorm_add_swiglu_rope_bit_exact(mods, orc):
    _, layer = mods
    rows, width = 37, 4096
    xb = f32_to_bf16_bits(orc.normal_f32(1, rows * width, 1.0))
    gb = f32_to_bf16_bits(1.0 + 0.1 * orc.normal_f32(2, width, 1.0))
    x, g = dev_bf16(xb).view(rows, width), dev_bf16(gb)
    y = layer.rmsnorm(x, g, 1e-6)
    ref = orc.rmsnorm_breeze(xb, gb, rows, width, 1e-6)
    got = host_bits(y).reshape(rows, width)
    # the sum of squares is re-associated (tree instead of a chain): at most an ulp of inv,
    # which can flip a bf16 rounding on a few elements
    diff = np.abs(bf16_bits_to_f32(got) - bf16_bits_to_f32(ref))
    assert (got != ref).mean() < 2e-3 and diff.max() <= 2 ** -6
    a = f32_to_bf16_bits(orc.normal_f32(3, 4096, 1.0))
    b = f32_to_bf16_bits(orc.normal_f32(4, 4096, 1.0))
    assert np.array_equal(host_bits(layer.add(dev_bf16(a), dev_bf16(b))), orc.add_bf16(a, b))
    sw = host_bits(layer.swiglu(dev_bf16(a), dev_bf16(b)))
    sw_ref = orc.swiglu_bf16(a, b)
    assert (sw != sw_ref).mean() < 5e-3       # expf differs from the host's by an ulp on a few inputs
    assert np.abs(bf16_bits_to_f32(sw) - bf16_bits_to_f32(sw_ref)).max() <= 2 ** -6
    p32 = orc.normal_f32(5, 4096, 1.0)
    got = host_bits(layer.add_f32(dev_bf16(a), torch.from_numpy(p32).cuda()))
    assert np.array_equal(got, orc.add_bf16(a, f32_to_bf16_bits(p32)))
    tokens, heads, d, past = 9, 4, 128, 17
    rb = f32_to_bf16_bits(orc.normal_f32(6, tokens * heads * d, 1.0))
    inv = layer.inv_freq(d, 1e6)
    r = host_bits(layer.rope(dev_bf16(rb), tokens, heads, d, past, torch.from_numpy(inv).cuda()))
    r_ref = orc.rope_bf16(rb, tokens, heads, d, past, inv)
    assert (r != r_ref).mean() < 5e-3
    assert np.abs(bf16_bits_to_f32(r) - bf16_bits_to_f32(r_ref)).max() <= 2 ** -5


def _layer_fixture(orc, layer, cfg, seed=100):
    import maryml_b200.nvfp4 as nv
    D = cfg.head_dim
    shapes = {"q": (cfg.heads * D, cfg.hidden), "k": (cfg.kv_heads * D, cfg.hidden), "v": (cfg.kv_heads * D, cfg.hidden),
              "o": (cfg.hidden, cfg.heads * D), "gate": (cfg.inter, cfg.hidden), "up": (cfg.inter, cfg.hidden),
              "down": (cfg.hidden, cfg.inter)}
    full = {}
    for i, (name, (n, k)) in enumerate(shapes.items()):
        bits = f32_to_bf16_bits(orc.normal_f32(seed + i, n * k, 0.02))
        c, s, s2 = orc.quantize_weight_bf16(bits, n, k)
        full[name] = (torch.from_numpy(c).view(n, k // 2), torch.from_numpy(s).view(n, k // 16), float(s2))
    g1 = f32_to_bf16_bits(1.0 + 0.05 * orc.normal_f32(seed + 20, cfg.hidden, 1.0))
    g2 = f32_to_bf16_bits(1.0 + 0.05 * orc.normal_f32(seed + 21, cfg.hidden, 1.0))
    return full, g1, g2


def _oracle_layer(orc, cfg, full, g1, g2, xbits, batch, t, past, kc, vc):
    """The Breeze layer (src/models/breeze/backbone.rs:287-333) from oracle pieces, W4A4 projections."""
    D = cfg.head_dim

    def lin(xb, name, rows):
        c, s, s2 = full[name]
        n, k = c.shape[0], c.shape[1] * 2
        ac, asc = orc.quantize_act_scaled(bf16_bits_to_f32(xb), rows, k, 1.0)
        y = orc.linear_w4a4(ac, asc, c.numpy().ravel(), s.numpy().ravel(), np.float32(s2), rows, n, k)
        return f32_to_bf16_bits(y)

    rows = batch * t
    n = orc.rmsnorm_breeze(xbits, g1, rows, cfg.hidden, cfg.eps)
    q, k, v = lin(n, "q", rows), lin(n, "k", rows), lin(n, "v", rows)
    from maryml_b200.layer import inv_freq
    inv = inv_freq(D, cfg.theta)
    q = np.concatenate([orc.rope_bf16(q.reshape(batch, -1)[b], t, cfg.heads, D, past, inv) for b in range(batch)])
    k = np.concatenate([orc.rope_bf16(k.reshape(batch, -1)[b], t, cfg.kv_heads, D, past, inv) for b in range(batch)])
    kc[:, past:past + t] = k.reshape(batch, t, cfg.kv_heads * D)
    vc[:, past:past + t] = v.reshape(batch, t, cfg.kv_heads * D)
    keys = past + t
    att = np.empty((batch, t, cfg.heads * D), np.float32)
    for b in range(batch):
        att[b] = orc.attention(bf16_bits_to_f32(q.reshape(batch, t, -1)[b]), bf16_bits_to_f32(kc[b, :keys]),
                               bf16_bits_to_f32(vc[b, :keys]), cfg.heads, cfg.kv_heads, D, past, 1.0 / math.sqrt(D))
    a = f32_to_bf16_bits(att)
    residual = orc.add_bf16(xbits, lin(a.reshape(-1), "o", rows))
    n = orc.rmsnorm_breeze(residual, g2, rows, cfg.hidden, cfg.eps)
    gate, up = lin(n, "gate", rows), lin(n, "up", rows)
    return orc.add_bf16(residual, lin(orc.swiglu_bf16(gate, up), "down", rows))


@pytest.mark.parametrize("batch,t,past", [(1, 40, 0), (3, 1, 21)])
def test_decoder_layer_against_oracle(mods, orc, batch, t, past):
    _, layer = mods
    cfg = layer.LayerConfig(hidden=512, heads=4, kv_heads=2, head_dim=128, inter=1024)
    full, g1, g2 = _layer_fixture(orc, layer, cfg)
    L = layer.DecoderLayer(cfg, full, dev_bf16(g1), dev_bf16(g2))
    cap = past + t
    xbits = f32_to_bf16_bits(orc.normal_f32(7, batch * t * cfg.hidden, 1.0))
    kc = f32_to_bf16_bits(orc.normal_f32(8, batch * cap * cfg.kv_heads * 128, 1.0)).reshape(batch, cap, -1)
    vc = f32_to_bf16_bits(orc.normal_f32(9, batch * cap * cfg.kv_heads * 128, 1.0)).reshape(batch, cap, -1)
    kd = dev_bf16(kc).view(batch, cap, cfg.kv_heads, 128).clone()
    vd = dev_bf16(vc).view(batch, cap, cfg.kv_heads, 128).clone()
    y = L.forward(dev_bf16(xbits).view(batch * t, cfg.hidden), batch, past, kd, vd)
    ref = _oracle_layer(orc, cfg, full, g1, g2, xbits, batch, t, past, kc.copy(), vc.copy())
    got = bf16_bits_to_f32(host_bits(y)).ravel()
    want = bf16_bits_to_f32(ref).ravel()
    _, cos = rel_check(got, want)
    # Seven quantised GEMMs in a row: where the GPU and CPU round an intermediate to different
    # bf16 neighbours, the next activation quantizer can flip an E2M1 code, so single outputs
    # move by a few percent of the output's rms. The layer-level bound is therefore stated
    # against the rms: max |err| <= 5e-2 rms, mean |err| <= 1e-2 rms (a bf16 ulp at 1.0 is 4e-3), cosine >= 0.9999.
    rms = np.sqrt(np.mean(want.astype(np.float64) ** 2))
    err = np.abs(got - want)
    assert cos >= 0.9999 and err.max() <= 5e-2 * rms and err.mean() <= 1e-2 * rms, (err.max() / rms, err.mean() / rms, cos)


# --------------------------------------------------------------------------- fused glue
@pytest.mark.parametrize("rows,width,with_partial", [(1, 64, False), (37, 4096, True), (64, 4096, False),
                                                     (5, 8192, True), (9, 1984, True)])
def test_residual_norm_quantize_equals_the_three_kernels(mods, orc, rows, width, with_partial):
    """One pass (add + norm + W4A4 quantizer) writes the bytes of mb_add_f32 -> mb_rmsnorm ->
    mb_nvfp4_quantize_act, and those are pinned to the oracle's quantizer above."""
    _, layer = mods
    from maryml_b200 import nvfp4 as nv, _lib
    x = dev_bf16(f32_to_bf16_bits(orc.normal_f32(1, rows * width, 1.0))).view(rows, width)
    gain = dev_bf16(f32_to_bf16_bits(1.0 + orc.normal_f32(2, width, 0.1)))
    partial = torch.from_numpy(orc.normal_f32(3, rows * width, 0.5).reshape(rows, width)).cuda() if with_partial else None
    r_ref = layer.add_f32(x, partial) if with_partial else x
    y_ref = layer.rmsnorm(r_ref, gain, 1e-6)
    c_ref, sf_ref, _ = nv.quantize_act(y_ref, _lib.QUANT_SCALED, 1.0, tiled=True)
    L = layer.DecoderLayer.__new__(layer.DecoderLayer)
    L.cfg = layer.LayerConfig(hidden=width, eps=1e-6)
    r, (codes, sf, n) = L._norm_quantize(x, partial, gain)
    assert n == rows
    assert torch.equal(r.view(torch.int16), r_ref.view(torch.int16))
    assert torch.equal(codes, c_ref)
    assert torch.equal(nv.untile_scales(sf, rows, width), nv.untile_scales(sf_ref, rows, width))
    # and against the oracle's norm + quantizer on the same bytes
    y_or = orc.rmsnorm_breeze(host_bits(r_ref).ravel(), host_bits(gain).ravel(), rows, width, 1e-6)
    c_or, s_or = orc.quantize_act_scaled(bf16_bits_to_f32(y_or), rows, width, 1.0)
    match = (codes.cpu().numpy().ravel() == c_or.ravel()).mean()
    assert match >= 0.999, match       # the f32 sum of squares is ordered differently on the two sides


@pytest.mark.parametrize("batch,t,hq,hkv,past,cap", [(3, 1, 4, 2, 21, 22), (2, 40, 4, 1, 0, 64), (1, 5, 8, 8, 7, 12),
                                                     # prompt sizes: eight heads per thread share their sines and cosines
                                                     (1, 1100, 4, 1, 3, 1200), (2, 600, 8, 2, 0, 600), (1, 1024, 32, 8, 0, 1024)])
def test_rope_append_equals_rope_and_copy(mods, orc, batch, t, hq, hkv, past, cap):
    _, layer = mods
    from maryml_b200 import _lib
    D = 128
    width = (hq + 2 * hkv) * D
    qkv = dev_bf16(f32_to_bf16_bits(orc.normal_f32(4, batch * t * width, 1.0))).view(batch * t, width)
    inv = torch.from_numpy(layer.inv_freq(D, 1e6)).cuda()
    kc = dev_bf16(f32_to_bf16_bits(orc.normal_f32(5, batch * cap * hkv * D, 1.0))).view(batch, cap, hkv, D).clone()
    vc = kc.clone() + 1
    kc2, vc2 = kc.clone(), vc.clone()
    # separate kernels: one rope call per sequence, then the cache writes
    q_sep = qkv[:, :hq * D].contiguous().view(batch, t * hq * D)
    k_sep = qkv[:, hq * D:(hq + hkv) * D].contiguous().view(batch, t * hkv * D)
    v_sep = qkv[:, (hq + hkv) * D:].contiguous().view(batch, t, hkv, D)
    q_ref = torch.stack([layer.rope(q_sep[b], t, hq, D, past, inv) for b in range(batch)]).view(batch, t, hq, D)
    k_ref = torch.stack([layer.rope(k_sep[b], t, hkv, D, past, inv) for b in range(batch)]).view(batch, t, hkv, D)
    kc[:, past:past + t].copy_(k_ref)
    vc[:, past:past + t].copy_(v_sep)
    q = torch.empty((batch, t, hq, D), dtype=torch.bfloat16, device="cuda")
    ctx = _lib.context(0)
    ctx.check(_lib.lib.mb_rope_append(ctx.handle, None, qkv.data_ptr(), batch, t, hq, hkv, D, past, inv.data_ptr(),
                                      q.data_ptr(), kc2.data_ptr(), vc2.data_ptr(), cap))
    assert torch.equal(q.view(torch.int16), q_ref.view(torch.int16))
    assert torch.equal(kc2.view(torch.int16), kc.view(torch.int16))
    assert torch.equal(vc2.view(torch.int16), vc.view(torch.int16))
    with pytest.raises(_lib.MaryError):
        ctx.check(_lib.lib.mb_rope_append(ctx.handle, None, qkv.data_ptr(), batch, t, hq, hkv, D, cap, inv.data_ptr(),
                                          q.data_ptr(), kc2.data_ptr(), vc2.data_ptr(), cap))


@pytest.mark.parametrize("m", [1, 64, 300])
def test_stacked_products_equal_the_separate_ones(mods, orc, m):
    """q|k|v as one product and gate/up + SwiGLU + quantizer as one product against the separate
    projections, the stand-alone SwiGLU and the stand-alone quantizer: the same bytes."""
    _, layer = mods
    from maryml_b200 import nvfp4 as nv, _lib
    k, nq, nkv, inter = 512, 512, 256, 768
    ws = [nv.Nvfp4.quantize(dev_bf16(f32_to_bf16_bits(orc.normal_f32(10 + i, n * k, 0.02 * (i + 1)))).view(n, k))
          for i, n in enumerate((nq, nkv, nkv, inter, inter))]
    x = dev_bf16(f32_to_bf16_bits(orc.normal_f32(3, m * k, 1.0))).view(m, k)
    codes, sf, _ = nv.quantize_act(x, _lib.QUANT_SCALED, 1.0, tiled=True)
    sep = [nv.gemm_w4a4(codes, sf, w.codes, w.sf_tiled(), w.scale2, m, w.n(), k) for w in ws]
    qkv = nv.gemm_w4a4_stacked(codes, sf, nv.Stacked(ws[:3]), m)
    assert torch.equal(qkv.view(torch.int16), torch.cat(sep[:3], 1).view(torch.int16))
    qkv32 = nv.gemm_w4a4_stacked(codes, sf, nv.Stacked(ws[:3]), m, out_dtype=torch.float32)
    assert torch.equal(qkv32.to(torch.bfloat16).view(torch.int16), qkv.view(torch.int16))
    gu = nv.Stacked(ws[3:], interleave=True)
    act_ref = layer.swiglu(sep[3], sep[4])
    act = nv.gemm_w4a4_stacked(codes, sf, gu, m, epilogue=_lib.EPI_SWIGLU_ROUNDED)
    assert torch.equal(act.view(torch.int16), act_ref.view(torch.int16))
    c_ref, sf_ref, _ = nv.quantize_act(act_ref, _lib.QUANT_SCALED, 1.0, tiled=True)
    c, s = nv.gemm_w4a4_stacked(codes, sf, gu, m, epilogue=_lib.EPI_SWIGLU_ROUNDED | _lib.EPI_QUANT_SCALED)
    assert torch.equal(c, c_ref)
    assert torch.equal(nv.untile_scales(s, m, inter), nv.untile_scales(sf_ref, m, inter))
    c_ref, sf_ref, _ = nv.quantize_act(act_ref, _lib.QUANT_RECIP, tiled=True)
    c, s = nv.gemm_w4a4_stacked(codes, sf, gu, m, epilogue=_lib.EPI_SWIGLU_ROUNDED | _lib.EPI_QUANT_RECIP)
    assert torch.equal(c, c_ref)
    assert torch.equal(nv.untile_scales(s, m, inter), nv.untile_scales(sf_ref, m, inter))
    ctx = _lib.context(0)
    with pytest.raises(_lib.MaryError):      # a quantized output without a SwiGLU epilogue is refused
        nv.gemm_w4a4_stacked(codes, sf, gu, m, epilogue=_lib.EPI_PLAIN | _lib.EPI_QUANT_RECIP)


@pytest.mark.parametrize("batch,t,past", [(1, 40, 0), (3, 1, 21), (2, 150, 10)])
def test_fused_layer_equals_the_kernel_by_kernel_layer(mods, orc, batch, t, past):
    _, layer = mods
    cfg = layer.LayerConfig(hidden=512, heads=4, kv_heads=2, head_dim=128, inter=1024)
    full, g1, g2 = _layer_fixture(orc, layer, cfg)
    cap = past + t
    x = dev_bf16(f32_to_bf16_bits(orc.normal_f32(7, batch * t * cfg.hidden, 1.0))).view(batch * t, cfg.hidden)
    kc = dev_bf16(f32_to_bf16_bits(orc.normal_f32(8, batch * cap * cfg.kv_heads * 128, 1.0))).view(batch, cap, cfg.kv_heads, 128)
    vc = dev_bf16(f32_to_bf16_bits(orc.normal_f32(9, batch * cap * cfg.kv_heads * 128, 1.0))).view(batch, cap, cfg.kv_heads, 128)
    outs = []
    for fuse in (False, True):
        L = layer.DecoderLayer(cfg, full, dev_bf16(g1), dev_bf16(g2), fuse=fuse)
        kd, vd = kc.clone(), vc.clone()
        outs.append((L.forward(x, batch, past, kd, vd), kd, vd))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_chunked_prompt_equals_the_whole_prompt(mods, orc):
    """The pipelined prompt path (token chunks on two streams, ordered by events) against one pass over the
    whole prompt, on one GPU: causal attention of a chunk sees exactly the keys earlier chunks appended."""
    _, layer = mods
    cfg = layer.LayerConfig(hidden=512, heads=4, kv_heads=2, head_dim=128, inter=1024)
    full, g1, g2 = _layer_fixture(orc, layer, cfg)
    L = layer.DecoderLayer(cfg, full, dev_bf16(g1), dev_bf16(g2))
    past, t = 256, 1024
    cap = past + t
    x = dev_bf16(f32_to_bf16_bits(orc.normal_f32(7, t * cfg.hidden, 1.0))).view(t, cfg.hidden)
    kc = dev_bf16(f32_to_bf16_bits(orc.normal_f32(8, cap * cfg.kv_heads * 128, 1.0))).view(1, cap, cfg.kv_heads, 128)
    vc = dev_bf16(f32_to_bf16_bits(orc.normal_f32(9, cap * cfg.kv_heads * 128, 1.0))).view(1, cap, cfg.kv_heads, 128)
    k1, v1, k2, v2 = kc.clone(), vc.clone(), kc.clone(), vc.clone()
    whole = L.forward(x, 1, past, k1, v1)
    torch.cuda.synchronize()
    parts = L.forward_chunked(x, past, k2, v2, chunk=256)
    torch.cuda.synchronize()
    assert torch.equal(k1.view(torch.int16), k2.view(torch.int16)) and torch.equal(v1.view(torch.int16), v2.view(torch.int16))
    a, b = whole.float(), parts.float()
    rms = a.pow(2).mean().sqrt()
    # the attention kernel may walk a row's key tiles in a different grouping when the query block starts elsewhere
    assert (a - b).abs().max() <= 2e-2 * rms and torch.nn.functional.cosine_similarity(a.ravel(), b.ravel(), dim=0) >= 0.99999
