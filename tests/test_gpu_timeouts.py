"""The bounded device-side waits, made to run out without faulting anything: a fused exchange whose
"peer" buffer nobody writes, and a workspace whose ticket word was tampered with on the host.  Each
launch must return, the status word must name the problem, and the next ordinary call must work."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from _util import HQ, HKV, D, to_dev, f32_of, assert_attn_close, oracle_state_from

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


@pytest.fixture()
def tb():
    import tokenrush_b200 as tb
    yield tb
    tb._lib.lib().trb_set_wait_limits(0, 0, 0)                  # defaults again
    tb._lib.device_status()


def _state(tb, L):
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, L + 64, "cuda", kv_dtype=F8)
    tb.fused.kv_write_prefill(to_dev(O.seeded_bf16(1, HKV, L, D)), to_dev(O.seeded_bf16(2, HKV, L, D)), st, 0, 0)
    st.set_pos(L - 1)
    return cfg, st


def _check_ordinary_call(tb, cfg, st, L):
    qb = O.seeded_bf16(9, 1, HQ, D)
    o = tb.fused.attn_decode_fused(to_dev(qb).reshape(1, -1), None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
    torch.cuda.synchronize()
    assert_attn_close(f32_of(o).reshape(1, HQ, D), O.attn_rows_over_cache(oracle_state_from(st), 0, qb, L - 1), "after the timeout")
    assert tb._lib.device_status() == 0


def test_peer_wait_runs_out_and_reports(tb):
    L = 3000
    lib, Lb = tb._lib.lib(), tb._lib
    cfg, st = _state(tb, L)
    q = to_dev(O.seeded_bf16(3, 1, HQ, D)).reshape(1, -1)
    tb.fused.attn_decode_fused(q, None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])     # workspace exists
    nbytes = lib.trb_p2p_exchange_bytes(2, HQ, D)
    mine = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    other = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")   # stands for rank 1's buffer; rank 1 does not exist
    ptrs = (C.c_void_p * 2)(mine.data_ptr(), other.data_ptr())
    assert lib.trb_set_wait_limits(0, 0, 3000) == 0
    tb.fused.attn_decode_fused(q, None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0], p2p=(ptrs, 2, 0))
    torch.cuda.synchronize()                                     # the launch returned
    assert tb._lib.device_status() & Lb.ST_PEER_TIMEOUT
    # this GPU's packets went out all the same
    assert other.view(torch.int32).ne(0).any()
    lib.trb_set_wait_limits(0, 0, 0)
    _check_ordinary_call(tb, cfg, st, L)


def test_tail_wait_runs_out_on_a_stale_ticket_and_reports(tb):
    """A ticket word that already counts all splits but one.  The split ranges are chosen so that the
    last split of a kv head is a third shorter than the others: its CTA arrives first, completes the
    count and moves the word to the next epoch many microseconds before any other CTA arrives.  The
    others then tag their partials with that next epoch, so neither side ever sees the tags it polls
    for, and every helper's bounded wait runs out."""
    lib, Lb = tb._lib.lib(), tb._lib
    nsplit = torch.cuda.get_device_properties(0).multi_processor_count // HKV
    per = 101
    n_tiles = nsplit * (per - 1) + 1                            # -> `nsplit` active splits, the last one with few tiles
    active = -(-n_tiles // per)
    if active != nsplit or n_tiles - (active - 1) * per > per * 2 // 3:
        pytest.skip("split geometry of this GPU does not give one short split")
    L = n_tiles * 32
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, L + 64, "cuda", kv_dtype=F8)
    from _util import fill_cache_gpu
    fill_cache_gpu(tb, st, 0, L, seed=5)
    st.set_pos(L - 1)
    q = to_dev(O.seeded_bf16(3, 1, HQ, D)).reshape(1, -1)
    tb.fused.attn_decode_fused(q, None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
    torch.cuda.synchronize()
    assert tb._lib.device_status() == 0
    ws = tb.fused.workspace_tensor(q.device, HQ, HKV, D, 1)
    slot_bytes = ws.numel() // tb.fused.WORKSPACE_SLOTS
    for s_ in range(tb.fused.WORKSPACE_SLOTS):                   # whichever slot the next call gets
        ws[s_ * slot_bytes:s_ * slot_bytes + 8].view(torch.int64)[0] += active - 1
    assert lib.trb_set_wait_limits(0, 2000, 0) == 0
    tb.fused.attn_decode_fused(q, None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
    torch.cuda.synchronize()                                     # the launch returned
    assert tb._lib.device_status() & Lb.ST_WAIT_TIMEOUT
    ws.zero_()                                                   # what the header asks for after such a report
    lib.trb_set_wait_limits(0, 0, 0)
    _check_ordinary_call(tb, cfg, st, L)


def test_unzeroed_workspace_is_reported(tb):
    L = 5000
    Lb = tb._lib
    cfg, st = _state(tb, L)
    q = to_dev(O.seeded_bf16(3, 1, HQ, D)).reshape(1, -1)
    tb.fused.attn_decode_fused(q, None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
    torch.cuda.synchronize()
    ws = tb.fused.workspace_tensor(q.device, HQ, HKV, D, 1)
    slot_bytes = ws.numel() // tb.fused.WORKSPACE_SLOTS
    for s_ in range(tb.fused.WORKSPACE_SLOTS):                   # whichever slot the next call gets
        ws[s_ * slot_bytes + 8:s_ * slot_bytes + 16].view(torch.int64)[0] = 1000   # kv head 1: an arrival count no launch can produce
    tb.fused.attn_decode_fused(q, None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
    torch.cuda.synchronize()
    assert tb._lib.device_status() & Lb.ST_WORKSPACE
    ws.zero_()
    _check_ordinary_call(tb, cfg, st, L)
