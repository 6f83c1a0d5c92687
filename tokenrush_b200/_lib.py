"""ctypes binding of libtrb_kv.so, the C-ABI CUDA library (include/trb_kv.h).

The library is the only implementation: there is no Triton, eager or CPU fallback.  If it
is missing or fails to load, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TRB_KV_LIB") or os.path.join(HERE, "libtrb_kv.so")

TRB_KV_BF16, TRB_KV_FP8 = 0, 1
ST_CURSOR_RANGE, ST_WAIT_TIMEOUT, ST_PEER_TIMEOUT, ST_WORKSPACE = 1, 2, 4, 8
IPC_HANDLE_BYTES = 64


class TrbError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: {lib().trb_strerror(code).decode()} (code {code})")
        self.code = code


class Cache(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
                ("hkv", C.c_int32), ("d", C.c_int32), ("kv_dtype", C.c_int32), ("sharded", C.c_int32),
                ("max_len", C.c_int64), ("ring", C.c_int64), ("shard_lo", C.c_int64)]


class Cursor(C.Structure):
    _fields_ = [("dev", C.c_void_p), ("width", C.c_int32), ("reserved", C.c_int32), ("host", C.c_int64)]


class DecodeArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("out", C.c_void_p), ("gate", C.c_void_p),
                ("gate_row_stride", C.c_int64), ("gate_head_stride", C.c_int64),
                ("m", C.c_int32), ("hq", C.c_int32), ("scale", C.c_float),
                ("new_rows", C.c_int32), ("window", C.c_int32), ("n_extra", C.c_int32),
                ("extra_ml", C.c_void_p), ("extra_acc", C.c_void_p),
                ("pos", Cursor), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("partial_ml", C.c_void_p), ("partial_acc", C.c_void_p),
                ("p2p_xchg", C.c_void_p), ("p2p_world", C.c_int32), ("p2p_rank", C.c_int32),
                ("ws_slot", C.c_int32), ("ws_slots", C.c_int32)]


class P2PMergeArgs(C.Structure):
    _fields_ = [("xchg", C.c_void_p), ("world", C.c_int32), ("rank", C.c_int32), ("seq", C.c_void_p),
                ("partial_ml", C.c_void_p), ("partial_acc", C.c_void_p),
                ("rows", C.c_int32), ("d", C.c_int32), ("hq", C.c_int32), ("reserved", C.c_int32),
                ("out", C.c_void_p), ("gate", C.c_void_p),
                ("gate_row_stride", C.c_int64), ("gate_head_stride", C.c_int64)]


# symbol -> (restype, argtypes); every function include/trb_kv.h declares
SIGNATURES = {
    "trb_version": (C.c_int, []),
    "trb_strerror": (C.c_char_p, [C.c_int]),
    "trb_set_programmatic_launch": (C.c_int, [C.c_int]),
    "trb_set_wait_limits": (C.c_int, [C.c_uint32, C.c_uint32, C.c_uint32]),
    "trb_launch_count": (C.c_ulonglong, []),
    "trb_set_decode_tensor_rows": (C.c_int, [C.c_int32]),
    "trb_device_status": (C.c_int, [C.POINTER(C.c_uint32)]),
    "trb_kv_append": (C.c_int, [C.POINTER(Cache), C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int32,
                                C.POINTER(Cursor), C.POINTER(Cursor), C.c_void_p]),
    "trb_attn_prep": (C.c_int, [C.POINTER(Cache), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64,
                                C.c_int32, C.c_float, C.c_int32, C.c_int32, C.POINTER(Cursor), C.c_void_p, C.c_void_p]),
    "trb_decode_workspace_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "trb_attn_decode": (C.c_int, [C.POINTER(Cache), C.POINTER(DecodeArgs), C.c_void_p]),
    "trb_attn_decode_static": (C.c_int, [C.POINTER(Cache), C.POINTER(DecodeArgs), C.c_void_p]),
    "trb_attn_block_partial": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                         C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]),
    "trb_lse_merge": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                C.c_int64, C.c_int64, C.c_int32, C.c_void_p]),
    "trb_spec_commit": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                  C.c_void_p]),
    "trb_cursor_advance": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64, C.c_void_p]),
    "trb_add_rmsnorm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_float, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                  C.c_void_p, C.c_void_p]),
    "trb_attn_prefill": (C.c_int, [C.POINTER(Cache), C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_float,
                                   C.c_void_p]),
    "trb_p2p_create": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]),
    "trb_p2p_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "trb_p2p_close": (C.c_int, [C.c_void_p]),
    "trb_p2p_destroy": (C.c_int, [C.c_void_p]),
    "trb_p2p_exchange_bytes": (C.c_size_t, [C.c_int32, C.c_int32, C.c_int32]),
    "trb_p2p_merge": (C.c_int, [C.POINTER(P2PMergeArgs), C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """Load libtrb_kv.so once.  Raises if the library has not been built
    (`python -m tokenrush_b200.build`)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m tokenrush_b200.build` "
                              "(there is no fallback implementation)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(code: int, what: str):
    if code != 0:
        raise TrbError(code, what)


def device_status() -> int:
    """Read and clear the device status word (synchronises; not inside graph capture)."""
    out = C.c_uint32(0)
    check(lib().trb_device_status(C.byref(out)), "trb_device_status")
    return out.value
