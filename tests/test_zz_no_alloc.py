"""trb_attn_decode_static: the decode entry point for callers that cannot hand over a scratch
buffer (their runtime owns device memory and offers plugins no way to allocate, or their FFI
binding only forwards the buffers it was given).  Its split scratch is a fixed array inside the
library, so the test calls it through the C ABI exactly as such a caller would, twice in a row
with different shapes, and compares each result with the oracle and with trb_attn_decode on a
caller-provided workspace.  Collected last on purpose: a failure here cannot hide the other tests' results."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from _util import HQ, HKV, D, to_dev

pytestmark = pytest.mark.gpu


def _args(tb, q, out, pos_t, m, workspace=None):
    L = tb._lib
    a = L.DecodeArgs()
    a.q, a.out, a.m, a.hq = q.data_ptr(), out.data_ptr(), m, HQ
    a.scale, a.new_rows = float(D ** -0.5), 1
    a.pos = L.Cursor(pos_t.data_ptr(), pos_t.element_size(), 0, 0)
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    return a


def test_static_scratch_decode_matches_workspace_decode_and_oracle():
    import tokenrush_b200 as tb
    from _util import f32_of, assert_attn_close, oracle_state_from
    L = tb._lib
    lib = L.lib()
    cfg = tb.AttnConfig(n_attn=1)
    stream = torch.cuda.current_stream().cuda_stream
    # four calls in a row on the shared array, shapes and queries changing from call to call
    for call, (rows, m) in enumerate([(2100, 1), (700, 4), (700, 2), (5000, 1)]):
        st = tb.State(cfg, rows + 64, "cuda", kv_dtype=torch.float8_e4m3fn)
        kb, vb = O.seeded_bf16(90 + call, HKV, rows + m, D), O.seeded_bf16(95 + call, HKV, rows + m, D)
        tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, 0, 0)
        st.set_pos(rows)
        qb = O.seeded_bf16(99 + call, m, HQ, D)
        q = to_dev(qb).reshape(m, -1)
        cache = tb.fused._cache(st.k[0], st.v[0], st.k_scale[0], st.v_scale[0])
        ws = torch.zeros(lib.trb_decode_workspace_bytes(HQ, HKV, D, m), device="cuda", dtype=torch.uint8)
        want = torch.zeros(m, HQ * D, device="cuda", dtype=torch.bfloat16)
        got = torch.zeros_like(want)
        a_ws = _args(tb, q, want, st.pos_t, m, ws)
        L.check(lib.trb_attn_decode(C.byref(cache), C.byref(a_ws), stream), "trb_attn_decode")
        a_st = _args(tb, q, got, st.pos_t, m)                                   # no workspace at all
        L.check(lib.trb_attn_decode_static(C.byref(cache), C.byref(a_st), stream), "trb_attn_decode_static")
        torch.cuda.synchronize()
        # against the oracle (fp32 math over the same cache bytes), at the bar of the other decode tests
        oracle = O.attn_rows_over_cache(oracle_state_from(st), 0, qb, rows)
        assert_attn_close(f32_of(got).reshape(m, HQ, D), oracle, f"static call {call}")
        # same kernel, same merge order as the workspace entry point: the bits agree
        assert torch.equal(got, want), call
    assert L.device_status() == 0


def test_static_scratch_refuses_the_exchange_between_gpus():
    import tokenrush_b200 as tb
    L = tb._lib
    lib = L.lib()
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, 256, "cuda", kv_dtype=torch.float8_e4m3fn)
    st.set_pos(100)
    q = torch.zeros(1, HQ * D, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    cache = tb.fused._cache(st.k[0], st.v[0], st.k_scale[0], st.v_scale[0])
    buf = torch.zeros(lib.trb_p2p_exchange_bytes(2, HQ, D), device="cuda", dtype=torch.uint8)
    ptrs = (C.c_void_p * 2)(buf.data_ptr(), buf.data_ptr())
    a = _args(tb, q, out, st.pos_t, 1)
    a.p2p_xchg, a.p2p_world, a.p2p_rank = C.cast(ptrs, C.c_void_p), 2, 0
    assert lib.trb_attn_decode_static(C.byref(cache), C.byref(a), torch.cuda.current_stream().cuda_stream) == -5
    torch.cuda.synchronize()
    assert L.device_status() == 0


def test_static_scratch_rejects_what_does_not_fit():
    import tokenrush_b200 as tb
    L = tb._lib
    lib = L.lib()
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, 256, "cuda", kv_dtype=torch.float8_e4m3fn)
    st.set_pos(100)
    m = 8                                                                       # 48 rows: beyond the 8 MiB array
    q = torch.zeros(m, HQ * D, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    cache = tb.fused._cache(st.k[0], st.v[0], st.k_scale[0], st.v_scale[0])
    assert lib.trb_decode_workspace_bytes(HQ, HKV, D, m) > (8 << 20)
    rc = lib.trb_attn_decode_static(C.byref(cache), C.byref(_args(tb, q, out, st.pos_t, m)), torch.cuda.current_stream().cuda_stream)
    assert rc == -7
    assert b"TRB_STATIC_SCRATCH_BYTES" in lib.trb_strerror(rc)
    torch.cuda.synchronize()
    assert L.device_status() == 0
