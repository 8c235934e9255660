"""The allocation-free decode attention entry point against the ordinary one.

mb_attention_decode_static keeps its key-split scratch in an array inside the library, for
hosts that own all device memory through an arena of their own and may not allocate once
serving has begun. It must give what mb_attention gives, call after call, although every call
reuses the same scratch. Collected last so that a first-failure stop has already run the rest."""
import ctypes as C
import math

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu


def _p(t):
    return C.c_void_p(t.data_ptr())


def test_static_scratch_decode_matches_workspace_decode_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from maryml_b200 import _lib
    from maryml_b200.attention import flash_attention
    lib, ctx = _lib.lib, _lib.context(0)
    torch.cuda.set_device(0)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(11)
    # two different shapes in a row: the second call finds the first call's partials in the scratch
    for (batch, keys, heads, kvh) in [(4, 5000, 32, 8), (2, 1537, 8, 2)]:
        q = torch.randn(batch, 1, heads, 128, device="cuda", generator=g).to(torch.bfloat16)
        k = torch.randn(batch, keys, kvh, 128, device="cuda", generator=g).to(torch.bfloat16)
        v = torch.randn(batch, keys, kvh, 128, device="cuda", generator=g).to(torch.bfloat16)
        want = flash_attention(q, k, v, q0=keys - 1)
        for _ in range(2):
            out = torch.full_like(q, float("nan"))
            rc = lib.mb_attention_decode_static(ctx.handle, stream, _p(q), _p(k), _p(v), batch, 1, keys, heads, kvh,
                                                128, keys - 1, 1.0 / math.sqrt(128), 1, _p(out))
            assert rc == 0, lib.mb_last_error(ctx.handle)
            torch.cuda.synchronize()
            # the same kernels on the same inputs: the tolerance the other attention tests use
            assert (out.float() - want.float()).abs().max().item() <= 2e-2 * want.float().abs().max().item()
            assert torch.equal(out, want)
    # a shape whose preferred split count would not fit the array runs with fewer splits instead of being refused
    batch, keys, heads, kvh = 32, 4096, 32, 8
    q = torch.randn(batch, 1, heads, 128, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(batch, keys, kvh, 128, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(batch, keys, kvh, 128, device="cuda", generator=g).to(torch.bfloat16)
    assert lib.mb_attention_workspace(batch, 1, keys, heads, kvh, 128) > (16 << 20)
    want = flash_attention(q, k, v, q0=keys - 1)
    out = torch.full_like(q, float("nan"))
    rc = lib.mb_attention_decode_static(ctx.handle, stream, _p(q), _p(k), _p(v), batch, 1, keys, heads, kvh, 128,
                                        keys - 1, 1.0 / math.sqrt(128), 1, _p(out))
    assert rc == 0, lib.mb_last_error(ctx.handle)
    torch.cuda.synchronize()
    assert (out.float() - want.float()).abs().max().item() <= 2e-2 * want.float().abs().max().item()
    # a shape beyond the built-in scratch is refused before any launch, with a message
    big = 64
    q = torch.zeros(big, 1, 64, 128, device="cuda", dtype=torch.bfloat16)
    kv = torch.zeros(1, 64, 64, 128, device="cuda", dtype=torch.bfloat16)   # never read: the call must refuse first
    rc = lib.mb_attention_decode_static(ctx.handle, stream, _p(q), _p(kv), _p(kv), big, 1, 1 << 20, 64, 64, 128, 0,
                                        0.1, 1, _p(q))
    assert rc == _lib.ERR_INVALID and b"built-in array" in lib.mb_last_error(ctx.handle)
