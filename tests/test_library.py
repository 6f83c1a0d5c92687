"""CPU-side checks of the C-ABI library: it builds, loads, and exports every symbol that
include/trb_kv.h declares; argument validation that needs no GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from tokenrush_b200 import build, _lib
    build.build()
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "trb_kv.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(trb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    from tokenrush_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_version_and_error_strings(lib):
    assert lib.trb_version() >= 100
    for code in range(0, -7, -1):
        assert lib.trb_strerror(code)
    assert b"unknown" in lib.trb_strerror(-99)


def test_argument_validation_needs_no_gpu(lib):
    from tokenrush_b200 import _lib as L
    cache = L.Cache(None, None, None, None, 4, 256, 1, 0, 128, 0, 0)
    cur = L.Cursor(None, 8, 0, 0)
    assert lib.trb_kv_append(C.byref(cache), None, None, 0, 0, 1, C.byref(cur), None, None) == -1          # null cache
    cache = L.Cache(4096, 8192, 4096, 4096, 4, 96, 1, 0, 128, 0, 0)
    assert lib.trb_kv_append(C.byref(cache), 4096, 4096, 256, 256, 1, C.byref(cur), None, None) == -5      # head_dim 96
    cache = L.Cache(4096, 8192, 4096, 4096, 4, 256, 1, 0, 128, 0, 0)
    cur = L.Cursor(None, 8, 0, 127)
    assert lib.trb_kv_append(C.byref(cache), 4096, 4096, 256, 256, 2, C.byref(cur), None, None) == -3      # past capacity
    assert lib.trb_kv_append(C.byref(cache), 4100, 4096, 256, 256, 1, C.byref(cur), None, None) == -2      # misaligned source
    assert lib.trb_decode_workspace_bytes(24, 4, 256, 8) > lib.trb_decode_workspace_bytes(24, 4, 256, 1) > 0
    assert lib.trb_decode_workspace_bytes(24, 4, 256, 9) == 0                                               # > 48 rows
    assert lib.trb_p2p_exchange_bytes(8, 24, 256) > lib.trb_p2p_exchange_bytes(2, 24, 256) > 0
    assert lib.trb_spec_commit(None, None, 3, None, None, None, 8, None) == -1


def test_host_wrappers_reject_cpu_tensors():
    import torch
    from tokenrush_b200 import fused
    k = torch.zeros(4, 1, 256, dtype=torch.bfloat16)
    cache = torch.zeros(4, 8, 256, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        fused.kv_append(k, k, cache, cache, 0)
