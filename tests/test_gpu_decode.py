"""GPU parity of split-K decode, the M-row verify variant, window / ring attention and the
partial merge, through the C ABI, against the CPU oracle and the reference's golden vectors.
Bar: max-abs 2e-3 and rel 1e-2 against fp32 math over the same FP8 cache."""
import os

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from _util import HQ, HKV, D, to_dev, bits_of, f32_of, rel, assert_attn_close, oracle_state_from

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def tb():
    import tokenrush_b200 as tb
    return tb


def _filled_state(tb, L, max_len, seed=0, kv_dtype=F8, std=1.0):
    """A one-layer State holding L rows of N(0, std) K/V written by the append kernel, and the
    oracle's copy of the same cache."""
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, max_len, "cuda", kv_dtype=kv_dtype)
    kb, vb = O.seeded_bf16(seed + 1, HKV, max(L, 1), D, std=std), O.seeded_bf16(seed + 2, HKV, max(L, 1), D, std=std)
    if L:
        tb.fused.kv_write_prefill(to_dev(kb[:, :L]), to_dev(vb[:, :L]), st, 0, 0)
    st.set_pos(L)
    return cfg, st


def _step(tb, cfg, st, qb, kb, vb, gate_qkv=None):
    """append M rows at the cursor, attend; returns [M, HQ, D] fp32."""
    tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, 0, st.pos_t)
    ks, vs = (st.k_scale[0], st.v_scale[0]) if st.fp8 else (None, None)
    o = tb.fused.attn_decode_fused(to_dev(qb).reshape(qb.shape[0], -1), gate_qkv, st.k[0], st.v[0], st.pos_t, cfg, ks, vs)
    return o


def _oracle_step(st_gpu, qb, pos):
    ref = oracle_state_from(st_gpu)
    m = qb.shape[0]
    kd, vd = ref.dequant(0, pos + m)
    return O.attn_rows(O.bf16_bits_to_f32(qb), kd, vd, pos)


def test_decode_matches_reference_golden(tb, golden_dir):
    z = np.load(os.path.join(golden_dir, "decode_attn.npz"))
    L0 = int(z["L0"])
    kb, vb = O.seeded_bf16(201, HKV, L0 + 5, D), O.seeded_bf16(202, HKV, L0 + 5, D)
    qb, gb = O.seeded_bf16(203, 5, HQ, D), O.seeded_bf16(204, 5, HQ, D)
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, 128, "cuda", kv_dtype=F8)
    tb.fused.kv_write_prefill(to_dev(kb[:, :L0]), to_dev(vb[:, :L0]), st, 0, 0)
    st.set_pos(L0)
    o1 = _step(tb, cfg, st, qb[:1], kb[:, L0:L0 + 1], vb[:, L0:L0 + 1])
    assert_attn_close(f32_of(o1).reshape(1, HQ, D), z["out_m1"], "M=1 golden")
    for _ in range(3):                                         # a 5-row verify step, repeated on the same inputs
        o5 = _step(tb, cfg, st, qb, kb[:, L0:], vb[:, L0:])
        assert_attn_close(f32_of(o5).reshape(5, HQ, D), z["out_m5"], "M=5 golden")
    # output gate: qkv rows carry [q | gate] per head
    qkv = np.zeros((5, HQ * 2 * D + 2 * HKV * D), dtype=np.uint16)
    qkv[:, :HQ * 2 * D].reshape(5, HQ, 2 * D)[:, :, D:] = gb
    og = _step(tb, cfg, st, qb, kb[:, L0:], vb[:, L0:], gate_qkv=to_dev(qkv))
    want = O.bf16_bits_to_f32(z["gated_m5"])
    assert_attn_close(f32_of(og).reshape(5, HQ, D), want, "gated")
    assert tb._lib.device_status() == 0


@pytest.mark.parametrize("L", [0, 1, 15, 16, 31, 32, 33, 127, 128, 129, 300, 2100, 4096])
def test_decode_m1_lengths(tb, L):
    """Lengths around group (16), tile (32) and split edges; L = 4096 is the first workload
    of the benchmark family (4096 cached rows + 1 appended)."""
    cfg, st = _filled_state(tb, L, L + 64, seed=10 + L)
    qb = O.seeded_bf16(3, 1, HQ, D)
    kb, vb = O.seeded_bf16(4, HKV, 1, D), O.seeded_bf16(5, HKV, 1, D)
    o = _step(tb, cfg, st, qb, kb, vb)
    assert_attn_close(f32_of(o).reshape(1, HQ, D), _oracle_step(st, qb, L), f"L={L}")
    o2 = tb.fused.attn_decode_fused(to_dev(qb).reshape(1, -1), None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
    assert torch.equal(o, o2)                                  # replays are bit-identical
    # the same result before the bf16 rounding of the output (the partial a sequence shard emits)
    ml, acc = tb.fused.attn_decode_fused(to_dev(qb).reshape(1, -1), None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0],
                                         st.v_scale[0], partial=True)
    o32 = f32_of(acc) / f32_of(ml)[:, 1:2]
    assert_attn_close(o32.reshape(1, HQ, D), _oracle_step(st, qb, L), f"fp32 L={L}", out_ulp=0.0)


@pytest.fixture(params=["tensor", "mma"])
def verify_kernel(request, tb):
    """Runs a test once on each decode kernel for M > 1: the tcgen05 one (default from 12 query
    rows per kv head) and the mma.sync one (forced by raising the switch above the maximum)."""
    tb._lib.lib().trb_set_decode_tensor_rows(49 if request.param == "mma" else 0)
    yield request.param
    tb._lib.lib().trb_set_decode_tensor_rows(0)


@pytest.mark.parametrize("M", [2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("L", [5, 1100])
def test_verify_rows_match_oracle_and_sequential(tb, M, L, verify_kernel):
    cfg, st = _filled_state(tb, L, L + 64, seed=77)
    qb = O.seeded_bf16(6, M, HQ, D)
    kb, vb = O.seeded_bf16(7, HKV, M, D), O.seeded_bf16(8, HKV, M, D)
    o = f32_of(_step(tb, cfg, st, qb, kb, vb)).reshape(M, HQ, D)
    assert_attn_close(o, _oracle_step(st, qb, L), f"M={M} L={L}")
    # row i of the M-row step == a 1-row step at position L + i over the same cache
    for i in (0, M - 1):
        st.set_pos(L + i)
        oi = tb.fused.attn_decode_fused(to_dev(qb[i:i + 1]).reshape(1, -1), None, st.k[0], st.v[0], st.pos_t, cfg,
                                        st.k_scale[0], st.v_scale[0])
        assert rel(f32_of(oi).reshape(HQ, D), o[i]) < 5e-3


@pytest.mark.parametrize("M,L", [(8, 0), (8, 120), (8, 121), (8, 127), (8, 128), (4, 255), (2, 383), (8, 4736), (5, 20000), (8, 40000)])
def test_verify_tile_edges_and_many_splits(tb, M, L, verify_kernel):
    """Lengths around the 128-key tiles of the tensor-core kernel, one tile per split up to many
    tiles per split; the un-rounded fp32 (max, sum, acc) output is checked at the flat 2e-3 bar.
    (The tensor-core kernel carries its softmax weights with 8 significant bits, as the bf16
    output does; with fewer than a few dozen keys per row nothing averages that out, and the bar
    there is the one of the bf16 output.)"""
    cfg, st = _filled_state(tb, L, L + 64, seed=300 + M)
    qb = O.seeded_bf16(31, M, HQ, D)
    kb, vb = O.seeded_bf16(32, HKV, M, D), O.seeded_bf16(33, HKV, M, D)
    o = f32_of(_step(tb, cfg, st, qb, kb, vb)).reshape(M, HQ, D)
    want = _oracle_step(st, qb, L)
    assert_attn_close(o, want, f"{verify_kernel} M={M} L={L}")
    ml, acc = tb.fused.attn_decode_fused(to_dev(qb).reshape(M, -1), None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0],
                                         st.v_scale[0], partial=True)
    o32 = (acc / ml[:, 1:2]).float().cpu().numpy().reshape(M, HQ, D)
    assert_attn_close(o32, want, f"{verify_kernel} fp32 M={M} L={L}", out_ulp=2.0 ** -8 if (verify_kernel == "tensor" and L < 64) else 0.0)
    assert tb._lib.device_status() == 0


def test_verify_peaked_rows_and_gate(tb, verify_kernel):
    """Eight rows with queries scaled x6 (peaked softmax, row maxima that keep moving between
    tiles) and planted keys in the first, a middle and the last tile; the sigmoid gate fused in
    the tail."""
    M, L = 8, 6000
    cfg, st = _filled_state(tb, L, L + 64, seed=41)
    qb = O.f32_to_bf16_bits(O.bf16_bits_to_f32(O.seeded_bf16(34, M, HQ, D)) * 6.0)
    q = O.bf16_bits_to_f32(qb)
    for n, pos_plant in enumerate((3, 2900, 5999)):
        krow = np.stack([q[n, j * 6 + n] * 0.5 for j in range(HKV)])[:, None, :]
        tb.fused.kv_write_prefill(to_dev(O.f32_to_bf16_bits(krow)), to_dev(O.seeded_bf16(35 + n, HKV, 1, D)), st, 0, pos_plant)
    kb, vb = O.seeded_bf16(38, HKV, M, D), O.seeded_bf16(39, HKV, M, D)
    o = f32_of(_step(tb, cfg, st, qb, kb, vb)).reshape(M, HQ, D)
    want = _oracle_step(st, qb, L)
    assert_attn_close(o, want, f"{verify_kernel} peaked M=8")
    gb = O.seeded_bf16(40, M, HQ, D)
    qkv = np.zeros((M, HQ * 2 * D + 2 * HKV * D), dtype=np.uint16)
    qkv[:, :HQ * 2 * D].reshape(M, HQ, 2 * D)[:, :, D:] = gb
    og = tb.fused.attn_decode_fused(to_dev(qb).reshape(M, -1), to_dev(qkv), st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0],
                                    st.v_scale[0])
    # the gate is applied to the bf16-rounded output, as the oracle composes it
    assert_attn_close(f32_of(og).reshape(M, HQ, D), O.bf16_bits_to_f32(O.gate_output(o, gb)), f"{verify_kernel} gated", out_ulp=2.0 ** -7)
    assert tb._lib.device_status() == 0


def test_verify_graph_replay_is_reproducible(tb, verify_kernel):
    """An 8-row verify step captured once and replayed at growing lengths read from the device
    cursor: every replay matches the oracle, and the same length gives the same bits."""
    M, L0 = 8, 700
    cfg, st = _filled_state(tb, L0, 2048, seed=55)
    qb = O.seeded_bf16(45, M, HQ, D)
    kb, vb = O.seeded_bf16(46, HKV, M, D), O.seeded_bf16(47, HKV, M, D)
    dq, dk, dv = to_dev(qb).reshape(M, -1), to_dev(kb), to_dev(vb)
    out = torch.empty(M, HQ * D, dtype=torch.bfloat16, device="cuda")

    def step():
        tb.fused.kv_write_prefill(dk, dv, st, 0, st.pos_t)
        tb.fused.attn_decode_fused(dq, None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0], out=out)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        step()
        torch.cuda.current_stream().synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            step()
    seen = {}
    for L in (L0, L0 + 3, L0 + 120, L0 + 3):
        st.set_pos(L)
        g.replay()
        torch.cuda.synchronize()
        o = out.clone()
        assert_attn_close(f32_of(o).reshape(M, HQ, D), _oracle_step(st, qb, L), f"{verify_kernel} replay L={L}")
        if L in seen:
            assert torch.equal(seen[L], o)
        seen[L] = o
    assert tb._lib.device_status() == 0


def test_decode_peaked_distribution_and_planted_keys(tb):
    """q scaled x8 makes the softmax peaked; planted keys sit in the last partial tile and in
    a split of their own, so masking / merge errors cannot hide in a flat average."""
    L = 3000
    cfg, st = _filled_state(tb, L, 4096, seed=5)
    qb = O.f32_to_bf16_bits(O.bf16_bits_to_f32(O.seeded_bf16(9, 1, HQ, D)) * 8.0)
    q = O.bf16_bits_to_f32(qb)
    kb, vb = O.seeded_bf16(11, HKV, 1, D), O.seeded_bf16(12, HKV, 1, D)
    for pos_plant in (2999, 17, 1500):
        krow = np.stack([q[0, j * 6] * 0.5 for j in range(HKV)])[:, None, :]          # aligned with head j*6's query
        tb.fused.kv_write_prefill(to_dev(O.f32_to_bf16_bits(krow)), to_dev(O.seeded_bf16(13, HKV, 1, D)), st, 0, pos_plant)
    o = _step(tb, cfg, st, qb, kb, vb)
    want = _oracle_step(st, qb, L)
    assert_attn_close(f32_of(o).reshape(1, HQ, D), want, "peaked")


def test_rollback_then_overwrite(tb):
    """An 8-row verify step, commit c of them on the device, next step overwrites the rest."""
    L = 500
    cfg, st = _filled_state(tb, L, 1024, seed=21)
    qb = O.seeded_bf16(14, 8, HQ, D)
    kb, vb = O.seeded_bf16(15, HKV, 8, D), O.seeded_bf16(16, HKV, 8, D)
    _step(tb, cfg, st, qb, kb, vb)
    pred = torch.tensor([3, 1, 4, 1, 5, 9, 2, 6], device="cuda"); drafts = torch.tensor([3, 1, 4, 7, 5, 9, 2], device="cuda")
    na = torch.zeros(1, device="cuda", dtype=torch.long); tk = torch.zeros(1, device="cuda", dtype=torch.long)
    tb.fused.spec_commit(pred, drafts, na, tk, st.pos_t)
    assert (int(na), int(tk), int(st.pos_t)) == (3, 1, L + 4)
    before = oracle_state_from(st)
    qb2 = O.seeded_bf16(17, 2, HQ, D)
    kb2, vb2 = O.seeded_bf16(18, HKV, 2, D), O.seeded_bf16(19, HKV, 2, D)
    o = _step(tb, cfg, st, qb2, kb2, vb2)
    after = oracle_state_from(st)
    ref = O.OracleState(1, HKV, 1024, D)
    ref.k[:], ref.v[:], ref.k_scale[:], ref.v_scale[:] = before.k, before.v, before.k_scale, before.v_scale
    O.kv_write(ref, 0, L + 4, kb2, vb2)
    assert np.array_equal(after.k, ref.k) and np.array_equal(after.k_scale.view(np.uint32), ref.k_scale.view(np.uint32))
    assert_attn_close(f32_of(o).reshape(2, HQ, D), _oracle_step(st, qb2, L + 4), "after rollback")


def test_device_cursor_in_cuda_graph(tb):
    """append + attend captured once; the live length advances on the device between replays."""
    L = 200
    cfg, st = _filled_state(tb, L, 512, seed=31)
    steps = 40
    qs = O.seeded_bf16(20, steps, HQ, D)
    kbs, vbs = O.seeded_bf16(21, HKV, steps, D), O.seeded_bf16(22, HKV, steps, D)
    q_in = torch.zeros(1, HQ * D, device="cuda", dtype=torch.bfloat16)
    k_in = torch.zeros(HKV, 1, D, device="cuda", dtype=torch.bfloat16); v_in = torch.zeros_like(k_in)
    out = torch.zeros(1, HQ * D, device="cuda", dtype=torch.bfloat16)

    def body():
        tb.fused.kv_write_prefill(k_in, v_in, st, 0, st.pos_t)
        o = tb.fused.attn_decode_fused(q_in, None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
        out.copy_(o)
        tb.fused.cursor_advance(st.pos_t, 1)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        body()                                                 # warm-up: builds the workspace outside capture
    torch.cuda.current_stream().wait_stream(s)
    st.set_pos(L)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=s):
        body()
    st.set_pos(L)
    for t in range(steps):
        q_in.copy_(to_dev(qs[t:t + 1]).reshape(1, -1)); k_in.copy_(to_dev(kbs[:, t:t + 1])); v_in.copy_(to_dev(vbs[:, t:t + 1]))
        graph.replay()
        if t % 13 == 0 or t == steps - 1:
            torch.cuda.synchronize()
            assert int(st.pos_t) == L + t + 1
            ref = oracle_state_from(st)
            kd, vd = ref.dequant(0, L + t + 1)
            want = O.attn_rows(O.bf16_bits_to_f32(qs[t:t + 1]), kd, vd, L + t)
            assert_attn_close(f32_of(out).reshape(1, HQ, D), want, f"replay {t}")
    assert tb._lib.device_status() == 0


def test_bf16_cache_decode(tb):
    L = 700
    cfg, st = _filled_state(tb, L, 1024, seed=41, kv_dtype=torch.bfloat16)
    for M in (1, 4):
        st.set_pos(L)
        qb = O.seeded_bf16(23, M, HQ, D)
        kb, vb = O.seeded_bf16(24, HKV, M, D), O.seeded_bf16(25, HKV, M, D)
        o = _step(tb, cfg, st, qb, kb, vb)
        assert_attn_close(f32_of(o).reshape(M, HQ, D), _oracle_step(st, qb, L), f"bf16 M={M}")


def test_window_block_matches_reference_golden_and_ring(tb, golden_dir):
    z = np.load(os.path.join(golden_dir, "window_block.npz"))
    pos, W, R, B = int(z["pos"]), int(z["window"]), int(z["ring"]), int(z["B"])
    hq, hkv, d = 32, 8, 128
    kfb, vfb = O.seeded_bf16(401, hkv, pos, d), O.seeded_bf16(402, hkv, pos, d)
    qb = O.seeded_bf16(403, B, hq, d)
    kbb, vbb = O.seeded_bf16(404, hkv, B, d), O.seeded_bf16(405, hkv, B, d)
    pos_t = torch.full((1,), pos, device="cuda", dtype=torch.long)
    q = to_dev(qb).reshape(B, hq * d)
    # (a) full-length cache, no ring
    kc = torch.zeros(hkv, 256, d, device="cuda", dtype=torch.bfloat16); vc = torch.zeros_like(kc)
    tb.fused.kv_append(to_dev(kfb), to_dev(vfb), kc, vc, 0)
    o = tb.fused.attn_window_block(q, kc, vc, pos_t, to_dev(kbb), to_dev(vbb), hq, hkv, d, W)
    assert_attn_close(f32_of(o).reshape(B, hq, d), z["out"], "window, full cache")
    # (b) the same history written through a ring in 7-row appends
    kr = torch.zeros(hkv, R, d, device="cuda", dtype=torch.bfloat16); vr = torch.zeros_like(kr)
    p = 0
    while p < pos:
        t = min(7, pos - p)
        tb.fused.ring_write(to_dev(kfb[:, p:p + t]), to_dev(vfb[:, p:p + t]), kr, vr, p, R)
        p += t
    o = tb.fused.attn_window_block(q, kr, vr, pos_t, to_dev(kbb), to_dev(vbb), hq, hkv, d, W, ring=R)
    assert_attn_close(f32_of(o).reshape(B, hq, d), z["out"], "window, ring")


@pytest.mark.parametrize("pos", [60, 3000, 9000])
def test_window_block_reference_test_geometry(tb, pos):
    """The geometry of the reference's own tests (tests/test_fused.py:343-380): W = 2048,
    ring 4096, positions inside the window, beyond it, and beyond the ring size."""
    hq, hkv, d, B, W, R = 32, 8, 128, 8, 2048, 4096
    kfb, vfb = O.seeded_bf16(51, hkv, pos, d), O.seeded_bf16(52, hkv, pos, d)
    qb = O.seeded_bf16(53, B, hq, d)
    kbb, vbb = O.seeded_bf16(54, hkv, B, d), O.seeded_bf16(55, hkv, B, d)
    kr = torch.zeros(hkv, R, d, device="cuda", dtype=torch.bfloat16); vr = torch.zeros_like(kr)
    lo = max(0, pos - (R - 8))
    rows = np.arange(lo, pos)
    idx = torch.from_numpy(rows % R).cuda()
    kr[:, idx] = to_dev(kfb[:, lo:pos]); vr[:, idx] = to_dev(vfb[:, lo:pos])
    pos_t = torch.full((1,), pos, device="cuda", dtype=torch.long)
    o = tb.fused.attn_window_block(to_dev(qb).reshape(B, hq * d), kr, vr, pos_t, to_dev(kbb), to_dev(vbb), hq, hkv, d, W, ring=R)
    f = O.bf16_bits_to_f32
    want = O.window_block_attention(f(qb), f(kfb), f(vfb), f(kbb), f(vbb), pos, W)
    assert_attn_close(f32_of(o).reshape(B, hq, d), want, f"pos={pos}")


def test_ring_wraparound_600_steps(tb):
    """Ring capacity 4096, window 2048: 7-row block appends across 600 steps (4200 rows, one
    wrap), attention checked on the steps around the wrap and at the end."""
    hq, hkv, d, B, W, R = 32, 8, 128, 8, 2048, 4096
    steps, blk = 600, 7
    total = steps * blk
    kfb, vfb = O.seeded_bf16(61, hkv, total, d), O.seeded_bf16(62, hkv, total, d)
    kr = torch.zeros(hkv, R, d, device="cuda", dtype=torch.bfloat16); vr = torch.zeros_like(kr)
    pos_t = torch.zeros(1, device="cuda", dtype=torch.long)
    kdev, vdev = to_dev(kfb), to_dev(vfb)
    f = O.bf16_bits_to_f32
    check = {584, 585, 586, 599}                               # 585 * 7 = 4095 -> the append that straddles row 4096
    for s in range(steps):
        tb.fused.ring_write(kdev[:, s * blk:(s + 1) * blk], vdev[:, s * blk:(s + 1) * blk], kr, vr, pos_t, R)
        tb.fused.cursor_advance(pos_t, blk)
        if s in check:
            pos = (s + 1) * blk
            qb = O.seeded_bf16(63 + s, B, hq, d)
            kbb, vbb = O.seeded_bf16(64 + s, hkv, B, d), O.seeded_bf16(65 + s, hkv, B, d)
            o = tb.fused.attn_window_block(to_dev(qb).reshape(B, hq * d), kr, vr, pos_t, to_dev(kbb), to_dev(vbb), hq, hkv, d, W, ring=R)
            want = O.window_block_attention(f(qb), f(kfb[:, :pos]), f(vfb[:, :pos]), f(kbb), f(vbb), pos, W)
            assert_attn_close(f32_of(o).reshape(B, hq, d), want, f"step {s}")
    assert int(pos_t) == total


@pytest.mark.parametrize("M", [1, 4, 8])
def test_sequence_shards_merge_to_unsharded(tb, M):
    """Two and four contiguous shards of one cache (as separate caches on this GPU): per-shard
    partials merged by the LSE formula equal the unsharded result; the appended rows land in
    the shard that owns their positions.  M = 1 runs the mma.sync kernel, M = 4 and 8 the tcgen05
    kernel (rows that straddle a shard boundary included: L + M crosses 1536 for M = 8 below)."""
    S = 2048                                                   # window size, sharded equally
    L = 1500 if M < 8 else 1531
    kb, vb = O.seeded_bf16(71, HKV, L + M, D), O.seeded_bf16(72, HKV, L + M, D)
    qb = O.seeded_bf16(73, M, HQ, D)
    cfg = tb.AttnConfig(n_attn=1)
    whole = tb.State(cfg, S, "cuda", kv_dtype=F8)
    tb.fused.kv_write_prefill(to_dev(kb[:, :L]), to_dev(vb[:, :L]), whole, 0, 0)
    whole.set_pos(L)
    o_ref = _step(tb, cfg, whole, qb, kb[:, L:], vb[:, L:])
    for G in (2, 4):
        per = S // G
        shards = [tb.State(cfg, per, "cuda", kv_dtype=F8, shard_lo=g * per) for g in range(G)]
        mls, accs = [], []
        for g, sh in enumerate(shards):
            lo, hi = g * per, min((g + 1) * per, L)
            if hi > lo:
                tb.fused.kv_append(to_dev(kb[:, lo:hi]), to_dev(vb[:, lo:hi]), sh.k[0], sh.v[0], lo, sh.k_scale[0], sh.v_scale[0],
                                   shard_lo=sh.shard_lo)
            sh.set_pos(L)
            tb.fused.kv_write_prefill(to_dev(kb[:, L:]), to_dev(vb[:, L:]), sh, 0, sh.pos_t)      # only the owners write
            ml, acc = tb.fused.attn_decode_fused(to_dev(qb).reshape(M, -1), None, sh.k[0], sh.v[0], sh.pos_t, cfg,
                                                 sh.k_scale[0], sh.v_scale[0], shard_lo=sh.shard_lo, partial=True)
            mls.append(ml); accs.append(acc)
        for t in range(M):                                     # every new row is in exactly one shard
            owner = (L + t) // per
            for g, sh in enumerate(shards):
                if g * per <= L + t < (g + 1) * per:
                    assert g == owner and bool((sh.k_scale[0][:, L + t - g * per] != 1).all())
        o = tb.fused.lse_merge(torch.stack(mls), torch.stack(accs), hq=HQ)
        assert_attn_close(f32_of(o).reshape(M, HQ, D), f32_of(o_ref).reshape(M, HQ, D), f"M={M} G={G}")
        assert_attn_close(f32_of(o).reshape(M, HQ, D), _oracle_step(whole, qb, L), f"M={M} G={G} vs oracle")
    assert tb._lib.device_status() == 0
