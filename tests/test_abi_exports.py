"""The C-ABI shared object loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mary_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mb_[a-z0-9_]+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    from maryml_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 20
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    # the Python binding covers the same set
    assert sorted(_lib.SIGNATURES) == names
    assert b"sm_100a" in _lib.lib.mb_version()


def test_binding_argument_counts_match_the_header():
    """A ctypes table that disagrees with a prototype in the number of arguments is a stack of wrong
    values at run time; the header is the contract, so count its parameters."""
    from maryml_b200 import _lib
    text = open(os.path.join(ROOT, "include", "mary_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    protos = dict(re.findall(r"\b(mb_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", text, flags=re.S))
    assert set(protos) == set(_lib.SIGNATURES)
    wrong = {}
    for name, params in protos.items():
        params = " ".join(params.split())
        n = 0 if params in ("", "void") else params.count(",") + 1
        have = len(_lib.SIGNATURES[name][1])
        if n != have:
            wrong[name] = (n, have)
            continue
        # and the kind of each: pointer, size_t, int or float
        for i, (decl, ct) in enumerate(zip(params.split(","), _lib.SIGNATURES[name][1])):
            decl = decl.strip()
            if "*" in decl or "[" in decl or decl.startswith("mb_stream"):    # an array parameter is a pointer
                kind = "p"
            elif decl.startswith("size_t"):
                kind = "z"
            elif decl.startswith("float"):
                kind = "f"
            elif decl.startswith("int") or decl.startswith("uint32_t") or decl.startswith("int32_t"):
                kind = "i"
            else:
                kind = "?"
            if ct is ctypes.c_void_p or ct is ctypes.c_char_p or hasattr(ct, "contents"):
                got = "p"
            elif ct is ctypes.c_size_t:
                got = "z"
            elif ct is ctypes.c_float:
                got = "f"
            elif ct in (ctypes.c_int, ctypes.c_int32, ctypes.c_uint32):
                got = "i"
            else:
                got = "??"
            if kind != got:
                wrong[f"{name}[{i}]"] = (decl, str(ct))
    assert not wrong, wrong


def test_host_only_entry_points():
    from maryml_b200 import _lib
    lo, hi = ctypes.c_size_t(), ctypes.c_size_t()
    assert _lib.lib.mb_tp_shard(1, 2, 32, ctypes.byref(lo), ctypes.byref(hi)) == 0
    assert (lo.value, hi.value) == (16, 32)
    assert _lib.lib.mb_tp_shard(0, 3, 32, ctypes.byref(lo), ctypes.byref(hi)) == _lib.ERR_INVALID
    # tiled scale plane: 128-row x 4-scale atoms of 512 bytes, K padded to 256
    assert _lib.lib.mb_nvfp4_sf_bytes(128, 256) == 4 * 512
    assert _lib.lib.mb_nvfp4_sf_bytes(129, 320) == 2 * 8 * 512


def test_no_gpu_means_a_loud_failure_not_a_fallback():
    import pytest
    import torch
    from maryml_b200 import _lib
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(_lib.MaryError):
        _lib.Context(0)
