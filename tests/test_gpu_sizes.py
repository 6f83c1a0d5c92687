"""Parity at the sizes the benchmark runs, one layer each: M = 1 over 32768 and 262144 live rows,
the M = 8 verify step over 65536 rows on both decode kernels with commit and the overwriting step,
and an 8192-token prefill chunk over 131072 cached rows.  The cache is filled on the GPU by the
product's append; the oracle reads the device's bytes back, dequantises them and computes fp32
attention (one kv head at a time).  Rows appended in the measured step are also compared bit for bit
with the oracle's quantiser."""
import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from _util import HQ, HKV, D, to_dev, f32_of, rel, assert_attn_close, oracle_state_from, fill_cache_gpu, rows_bit_exact

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def tb():
    import tokenrush_b200 as tb
    return tb


@pytest.mark.parametrize("L", [32768, 262144])
@pytest.mark.parametrize("q_std", [1.0, 6.0])
def test_decode_m1_at_benchmark_sizes(tb, L, q_std):
    """q_std = 6 makes the softmax peaked (a few keys carry most of the weight), so that a masking or
    merge error cannot hide in a flat average over a quarter of a million keys."""
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, L + 64, "cuda", kv_dtype=F8)
    fill_cache_gpu(tb, st, 0, L - 1, seed=L)
    st.set_pos(L - 1)
    qb = O.seeded_bf16(11, 1, HQ, D, std=q_std)
    kb, vb = O.seeded_bf16(12, HKV, 1, D), O.seeded_bf16(13, HKV, 1, D)
    tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, 0, st.pos_t)
    o = tb.fused.attn_decode_fused(to_dev(qb).reshape(1, -1), None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
    torch.cuda.synchronize()
    rows_bit_exact(st, 0, L - 1, kb, vb)
    ref = oracle_state_from(st)
    want = O.attn_rows_over_cache(ref, 0, qb, L - 1)
    assert_attn_close(f32_of(o).reshape(1, HQ, D), want, f"M=1 L={L} q_std={q_std}")
    assert tb._lib.device_status() == 0


@pytest.mark.parametrize("kernel", ["tensor", "mma"])
def test_verify_m8_at_benchmark_size_with_commit_and_overwrite(tb, kernel):
    lib = tb._lib.lib()
    lib.trb_set_decode_tensor_rows(49 if kernel == "mma" else 0)
    try:
        L, M = 65536, 8
        cfg = tb.AttnConfig(n_attn=1)
        st = tb.State(cfg, L + 64, "cuda", kv_dtype=F8)
        fill_cache_gpu(tb, st, 0, L - M, seed=7)
        st.set_pos(L - M)
        pos = L - M
        for step, commit in enumerate((3, 8)):
            qb = O.seeded_bf16(21 + step, M, HQ, D)
            kb, vb = O.seeded_bf16(31 + step, HKV, M, D), O.seeded_bf16(41 + step, HKV, M, D)
            tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, 0, st.pos_t)
            o = tb.fused.attn_decode_fused(to_dev(qb).reshape(M, -1), None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
            torch.cuda.synchronize()
            rows_bit_exact(st, 0, pos, kb, vb)                   # step 1 overwrites the rows step 0 rejected
            ref = oracle_state_from(st)
            want = O.attn_rows_over_cache(ref, 0, qb, pos)
            assert_attn_close(f32_of(o).reshape(M, HQ, D), want, f"M=8 {kernel} step {step}")
            # commit `commit` of the M rows on the device (commit - 1 drafts accepted)
            drafts = torch.arange(M - 1, dtype=torch.int64, device="cuda")
            pred = torch.cat([drafts, torch.tensor([99], device="cuda")])
            if commit - 1 < M - 1:
                pred[commit - 1] += 1
            nacc, tok = torch.zeros(1, dtype=torch.int64, device="cuda"), torch.zeros(1, dtype=torch.int64, device="cuda")
            tb.fused.spec_commit(pred, drafts, nacc, tok, st.pos_t)
            pos += commit
            assert int(st.pos_t.item()) == pos and int(nacc.item()) == commit - 1
        assert tb._lib.device_status() == 0
    finally:
        lib.trb_set_decode_tensor_rows(0)


def test_prefill_8192_over_131072(tb):
    pos, T = 131072, 8192
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, pos + T + 64, "cuda", kv_dtype=F8)
    fill_cache_gpu(tb, st, 0, pos, seed=3)
    kb, vb = O.seeded_bf16(51, HKV, T, D), O.seeded_bf16(52, HKV, T, D)
    qb = O.seeded_bf16(53, T, HQ, D)
    tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, 0, pos)
    o = tb.fused.attn_prefill_fused(to_dev(qb), st.k[0], st.v[0], pos, cfg, st.k_scale[0], st.v_scale[0])
    torch.cuda.synchronize()
    rows_bit_exact(st, 0, pos, kb, vb)                           # the chunk's 8192 rows, every byte and scale
    # 64 query rows: the ends of the chunk, the edges of the 128-row query blocks and of the 64-key
    # tiles, and a spread of others; all 24 heads each
    rows = sorted(set([0, 1, 63, 64, 127, 128, 129, 4095, 4096, T - 129, T - 128, T - 2, T - 1] +
                      list(np.linspace(5, T - 7, 51).astype(int))))[:64]
    ref = oracle_state_from(st)
    got = f32_of(o)
    want = O.attn_rows_over_cache(ref, 0, qb[rows], pos, row_pos=pos + np.asarray(rows))   # each row has its own causal limit
    assert_attn_close(got[rows], want, "prefill 8192 over 131072")
    assert tb._lib.device_status() == 0


def test_prefill_2048_over_65536_bf16_cache(tb):
    """The bf16-cache instance of the prefill kernel (kind::f16 MMAs, 64-key tiles, query block in tensor
    memory) at a long context: 1056 key tiles per query block, 16 query blocks; the chunk's rows are stored
    as they are, sampled query rows x all heads against fp32 oracle attention over the device's rows."""
    pos, T = 65536, 2048
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, pos + T + 64, "cuda", kv_dtype=torch.bfloat16)
    fill_cache_gpu(tb, st, 0, pos, seed=4)
    kb, vb = O.seeded_bf16(61, HKV, T, D), O.seeded_bf16(62, HKV, T, D)
    qb = O.seeded_bf16(63, T, HQ, D)
    tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, 0, pos)
    o = tb.fused.attn_prefill_fused(to_dev(qb), st.k[0], st.v[0], pos, cfg)
    torch.cuda.synchronize()
    from _util import bits_of
    assert np.array_equal(bits_of(st.k[0][:, pos:pos + T]), kb) and np.array_equal(bits_of(st.v[0][:, pos:pos + T]), vb)
    rows = sorted(set([0, 1, 63, 64, 127, 128, 129, 1023, 1024, T - 129, T - 128, T - 2, T - 1] +
                      list(np.linspace(5, T - 7, 19).astype(int))))[:32]
    ref = oracle_state_from(st)
    want = O.attn_rows_over_cache(ref, 0, qb[rows], pos, row_pos=pos + np.asarray(rows))
    assert_attn_close(f32_of(o)[rows], want, "bf16 prefill 2048 over 65536")
    assert tb._lib.device_status() == 0
