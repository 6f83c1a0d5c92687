"""GPU parity of the chunked prefill attention (tcgen05 kernel, through the C ABI) against the
reference's golden vectors and the CPU oracle; new rows are appended (FP8) first and attended in
quantised form, as the reference does (tokenrush/model.py:136-137)."""
import os

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from _util import HQ, HKV, D, to_dev, f32_of, assert_attn_close, assert_attn_close_bf16_p, oracle_state_from

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def tb():
    import tokenrush_b200 as tb
    return tb


def _prefill(tb, cfg, st, qb, kb, vb, pos):
    """append the chunk at pos (host int, as the reference's eager prefill) then attend."""
    tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, 0, pos)
    return tb.fused.attn_prefill_fused(to_dev(qb), st.k[0], st.v[0], pos, cfg, st.k_scale[0], st.v_scale[0])


def test_prefill_matches_reference_golden(tb, golden_dir):
    z = np.load(os.path.join(golden_dir, "prefill.npz"))
    pos, T, rows = int(z["pos"]), int(z["T"]), z["rows"]
    kb, vb = O.seeded_bf16(501, HKV, pos + T, D), O.seeded_bf16(502, HKV, pos + T, D)
    qb = O.seeded_bf16(503, T, HQ, D)
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, 128, "cuda", kv_dtype=F8)
    tb.fused.kv_write_prefill(to_dev(kb[:, :pos]), to_dev(vb[:, :pos]), st, 0, 0)
    for _ in range(2):
        o = _prefill(tb, cfg, st, qb, kb[:, pos:], vb[:, pos:], pos)
        assert_attn_close(f32_of(o)[rows], z["out"], "prefill golden")
    assert tb._lib.device_status() == 0


@pytest.mark.parametrize("pos,T", [(0, 1), (0, 64), (0, 130), (37, 150), (300, 300), (1000, 257)])
def test_prefill_vs_oracle(tb, pos, T):
    """Chunks that start at 0 and mid-cache, sizes around the 128-row query block and the
    64-key tile; every row is compared."""
    kb, vb = O.seeded_bf16(601 + pos, HKV, pos + T, D), O.seeded_bf16(602 + pos, HKV, pos + T, D)
    qb = O.seeded_bf16(603 + T, T, HQ, D)
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, pos + T + 40, "cuda", kv_dtype=F8)
    if pos:
        tb.fused.kv_write_prefill(to_dev(kb[:, :pos]), to_dev(vb[:, :pos]), st, 0, 0)
    o = _prefill(tb, cfg, st, qb, kb[:, pos:], vb[:, pos:], pos)
    ref = oracle_state_from(st)
    kd, vd = ref.dequant(0, pos + T)
    want = O.attn_prefill(O.bf16_bits_to_f32(qb), kd, vd, pos)
    assert_attn_close(f32_of(o), want, f"pos={pos} T={T}")
    assert tb._lib.device_status() == 0


def test_prefill_then_decode_consistency(tb):
    """The last row of a prefill chunk equals a 1-row decode at the same position over the same
    cache (the reference's tests/test_ops.py:139-146 self-consistency, here across two kernels)."""
    pos, T = 200, 96
    kb, vb = O.seeded_bf16(701, HKV, pos + T, D), O.seeded_bf16(702, HKV, pos + T, D)
    qb = O.seeded_bf16(703, T, HQ, D)
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, 512, "cuda", kv_dtype=F8)
    tb.fused.kv_write_prefill(to_dev(kb[:, :pos]), to_dev(vb[:, :pos]), st, 0, 0)
    o = f32_of(_prefill(tb, cfg, st, qb, kb[:, pos:], vb[:, pos:], pos))
    st.set_pos(pos + T - 1)
    od = tb.fused.attn_decode_fused(to_dev(qb[T - 1:T]).reshape(1, -1), None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
    a, b = o[T - 1].reshape(-1), f32_of(od).reshape(-1)
    assert np.linalg.norm(a - b) / np.linalg.norm(b) < 5e-3


def test_prefill_peaked_scores(tb):
    """q scaled x8: peaked softmax, running maximum changes often (exercises the correction of O)."""
    pos, T = 64, 200
    kb, vb = O.seeded_bf16(801, HKV, pos + T, D), O.seeded_bf16(802, HKV, pos + T, D)
    qb = O.f32_to_bf16_bits(O.bf16_bits_to_f32(O.seeded_bf16(803, T, HQ, D)) * 8.0)
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, 512, "cuda", kv_dtype=F8)
    tb.fused.kv_write_prefill(to_dev(kb[:, :pos]), to_dev(vb[:, :pos]), st, 0, 0)
    o = _prefill(tb, cfg, st, qb, kb[:, pos:], vb[:, pos:], pos)
    ref = oracle_state_from(st)
    kd, vd = ref.dequant(0, pos + T)
    want = O.attn_prefill(O.bf16_bits_to_f32(qb), kd, vd, pos)
    assert_attn_close(f32_of(o), want, "peaked prefill")


@pytest.mark.parametrize("hq,hkv,d,pos,T", [(24, 4, 256, 37, 150), (32, 8, 128, 37, 150), (24, 4, 256, 0, 9), (24, 4, 256, 4113, 520), (8, 8, 256, 0, 1)])
def test_prefill_over_a_bf16_cache(tb, hq, hkv, d, pos, T):
    """The reference's attn_prefill_fused defaults to a bf16 cache and its own test pins that mode at
    pos 37, T 150 (tests/test_fused.py:265-276).  The same call on a bf16 State, at both head
    geometries of the reference's tests, against fp32 oracle attention over the bf16 rows.  256-dim heads
    take the tensor-core kernel (bf16 MMAs; the longer case spans 73 key tiles and 5 query blocks),
    128-dim heads the M-row decode kernel."""
    from types import SimpleNamespace
    cfg = SimpleNamespace(n_heads=hq, n_kv_heads=hkv, head_dim=d, attn_layers=[0])
    kb, vb = O.seeded_bf16(701, hkv, pos + T, d), O.seeded_bf16(702, hkv, pos + T, d)
    qb = O.seeded_bf16(703, T, hq, d)
    st = tb.State(cfg, pos + T + 40, "cuda", kv_dtype=torch.bfloat16)
    tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, 0, 0)      # bf16 cache: rows stored as they are
    o = tb.fused.attn_prefill_fused(to_dev(qb), st.k[0], st.v[0], pos, cfg)
    assert o.shape == (T, hq, d) and o.dtype == torch.bfloat16
    want = O.attn_prefill(O.bf16_bits_to_f32(qb), O.bf16_bits_to_f32(kb), O.bf16_bits_to_f32(vb), pos)
    assert_attn_close_bf16_p(f32_of(o), want, "prefill over a bf16 cache")
    assert tb._lib.device_status() == 0


def test_prefill_over_an_fp8_cache_of_128_dim_heads(tb):
    """The reference's second test geometry (32 query heads, 8 kv heads, 128 dims: tests/test_fused.py:265-276)
    on an e4m3 cache: the tensor-core prefill kernel is built for 256-dim heads, so the chunk goes through the
    M-row decode kernel in groups of rows; same call, same bar."""
    from types import SimpleNamespace
    hq, hkv, d, pos, T = 32, 8, 128, 37, 150
    cfg = SimpleNamespace(n_heads=hq, n_kv_heads=hkv, head_dim=d, attn_layers=[0])
    kb, vb = O.seeded_bf16(711, hkv, pos + T, d), O.seeded_bf16(712, hkv, pos + T, d)
    qb = O.seeded_bf16(713, T, hq, d)
    st = tb.State(cfg, pos + T + 40, "cuda", kv_dtype=F8)
    tb.fused.kv_write_prefill(to_dev(kb[:, :pos]), to_dev(vb[:, :pos]), st, 0, 0)
    o = _prefill(tb, cfg, st, qb, kb[:, pos:], vb[:, pos:], pos)
    ref = oracle_state_from(st)
    kd, vd = ref.dequant(0, pos + T)
    want = O.attn_prefill(O.bf16_bits_to_f32(qb), kd, vd, pos)
    assert_attn_close(f32_of(o), want, "fp8 cache, 128-dim heads")
    assert tb._lib.device_status() == 0
