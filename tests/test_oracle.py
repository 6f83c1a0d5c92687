"""The CPU oracle against the golden vectors produced by the reference's own torch code
(tests/golden/make_golden.py) and against torch's e4m3 cast."""
import hashlib
import os

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O

HQ, HKV, D = 24, 4, 256


def sha(*arrs):
    h = hashlib.sha256()
    for a in arrs:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest(), dtype=np.uint8)


def load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def test_e4m3_codec_matches_torch_cast():
    g = torch.Generator().manual_seed(7)
    x = torch.cat([torch.randn(200000, generator=g) * 100, torch.randn(200000, generator=g),
                   torch.randn(100000, generator=g) * 0.01,
                   torch.tensor([0.0, -0.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9, 2.5 * 2.0 ** -9, 448.0, 449.0, 464.0,
                                 464.5, 480.0, -500.0, 2.0 ** -6, 0.0175, 1e-8, float("inf"), float("nan")])])
    want = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = O.e4m3_encode(x.numpy())
    nan_w = (want & 0x7F) == 0x7F
    assert np.array_equal(got[~nan_w], want[~nan_w])
    assert np.array_equal((got & 0x7F) == 0x7F, nan_w)
    codes = np.arange(256, dtype=np.uint8)
    back = torch.from_numpy(codes).view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.nan_to_num(O.e4m3_decode(codes), nan=123.0), np.nan_to_num(back, nan=123.0))


def test_bf16_bit_helpers_round_trip():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(10000, generator=g) * 37
    assert np.array_equal(O.f32_to_bf16_bits(x.numpy()), O.torch_bf16_to_bits(x.to(torch.bfloat16)))
    bits = O.seeded_bf16(5, 4, 7)
    assert np.array_equal(O.torch_bf16_to_bits(O.bits_to_torch_bf16(bits)), bits)


def test_fp8_append_bit_exact_vs_reference(golden_dir):
    z = load(golden_dir, "fp8_append.npz")
    pos = int(z["pos"])
    st = O.OracleState(1, HKV, 64, D)
    O.kv_write(st, 0, pos, z["k_bits"], z["v_bits"])
    assert np.array_equal(st.k[0], z["k_codes"]) and np.array_equal(st.v[0], z["v_codes"])
    assert np.array_equal(st.k_scale[0].view(np.uint32), z["k_scale"].view(np.uint32))
    assert np.array_equal(st.v_scale[0].view(np.uint32), z["v_scale"].view(np.uint32))
    assert st.kv_bytes_per_token == int(z["bytes_per_token"]) == 2080
    # untouched rows keep the reference's initial state: zero codes, unit scales
    assert (st.k[0][:, :pos] == 0).all() and (st.k_scale[0][:, :pos] == 1).all()
    # the all-zero row takes the floor scale 1e-6 / 448
    assert st.k_scale[0, 0, pos] == np.float32(1e-6) / np.float32(448.0) and (st.k[0, 0, pos] == 0).all()


def test_decode_and_verify_attention_vs_reference(golden_dir):
    z = load(golden_dir, "decode_attn.npz")
    L0 = int(z["L0"])
    kb, vb = O.seeded_bf16(201, HKV, L0 + 5, D), O.seeded_bf16(202, HKV, L0 + 5, D)
    qb, gb = O.seeded_bf16(203, 5, HQ, D), O.seeded_bf16(204, 5, HQ, D)
    assert np.array_equal(sha(kb, vb, qb, gb), z["in_sha"])
    st = O.OracleState(1, HKV, 128, D)
    O.kv_write(st, 0, 0, kb[:, :L0], vb[:, :L0])
    o1 = O.decode_step_cpu(st, 0, qb[:1], kb[:, L0:L0 + 1], vb[:, L0:L0 + 1], L0)
    np.testing.assert_allclose(o1, z["out_m1"], rtol=0, atol=1e-6)
    o5 = O.decode_step_cpu(st, 0, qb, kb[:, L0:], vb[:, L0:], L0)
    np.testing.assert_allclose(o5, z["out_m5"], rtol=0, atol=1e-6)
    # the threaded form that the CPU baseline is timed on gives the same numbers
    o5t = O.decode_step_cpu_threaded(st, 0, qb, kb[:, L0:], vb[:, L0:], L0)
    np.testing.assert_allclose(o5t, z["out_m5"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(o5t, o5, rtol=0, atol=1e-6)
    # row i of an M-row step equals a 1-row step at position L0 + i (tests/test_fused.py:97-122)
    kd, vd = st.dequant(0, L0 + 5)
    for i in range(5):
        oi = O.attn_rows(O.bf16_bits_to_f32(qb[i:i + 1]), kd[:, :L0 + i + 1], vd[:, :L0 + i + 1], L0 + i)
        np.testing.assert_allclose(oi[0], o5[i], rtol=0, atol=2e-6)
    # output gate, bf16 bit patterns: allow one rounding step where o sat on a bf16 tie
    got = O.gate_output(o5, gb).astype(np.int32)
    want = z["gated_m5"].astype(np.int32)
    assert (np.abs(got - want) <= 1).all() and (got != want).mean() < 1e-3
    # split-K partials merged by the LSE formula reproduce the unsplit result
    q32 = O.bf16_bits_to_f32(qb)
    for nsplit in (1, 4, 32):
        m, l, acc = O.split_partials(q32, kd, vd, L0, 5, nsplit, block_n=8)
        np.testing.assert_allclose(O.lse_merge(m, l, acc).reshape(5, HQ, D), o5, rtol=0, atol=3e-6)


def test_prep_norm_rope_vs_reference(golden_dir):
    z = load(golden_dir, "prep.npz")
    M, pos = int(z["M"]), int(z["pos"])
    qkvb = O.seeded_bf16(301, M, HQ * 2 * D + 2 * HKV * D)
    qwb, kwb = O.seeded_bf16(302, D, std=0.5), O.seeded_bf16(303, D, std=0.5)
    assert np.array_equal(sha(qkvb, qwb, kwb), z["in_sha"])
    cos, sin = O.rope_table(2048, 64, 1e7)
    rows = z["table_rows"]
    assert np.array_equal(O.torch_bf16_to_bits(cos[rows]), z["cos_bits"])
    assert np.array_equal(O.torch_bf16_to_bits(sin[rows]), z["sin_bits"])
    q, gate, k, v = O.attn_prep(O.bits_to_torch_bf16(qkvb), O.bits_to_torch_bf16(qwb), O.bits_to_torch_bf16(kwb),
                                cos, sin, pos, HQ, HKV, D, 1e-6)
    assert np.array_equal(O.torch_bf16_to_bits(q), z["q_bits"])
    assert np.array_equal(O.torch_bf16_to_bits(k), z["k_bits"])
    # v and gate are views of the projection row, untouched
    assert np.array_equal(O.torch_bf16_to_bits(v[2, 1]), qkvb[1, HQ * 2 * D + HKV * D + 2 * D: HQ * 2 * D + HKV * D + 3 * D])
    assert np.array_equal(O.torch_bf16_to_bits(gate[1, 3]), qkvb[1, 3 * 2 * D + D: 3 * 2 * D + 2 * D])


def test_window_block_ring_vs_reference(golden_dir):
    z = load(golden_dir, "window_block.npz")
    pos, W, R, B = int(z["pos"]), int(z["window"]), int(z["ring"]), int(z["B"])
    hq, hkv, d = 32, 8, 128
    kfb, vfb = O.seeded_bf16(401, hkv, pos, d), O.seeded_bf16(402, hkv, pos, d)
    qb = O.seeded_bf16(403, B, hq, d)
    kbb, vbb = O.seeded_bf16(404, hkv, B, d), O.seeded_bf16(405, hkv, B, d)
    assert np.array_equal(sha(kfb, vfb, qb, kbb, vbb), z["in_sha"])
    assert O.ring_size(W, B) == R and O.ring_size(2048, 8) == 4096
    f = O.bf16_bits_to_f32
    full = O.window_block_attention(f(qb), f(kfb), f(vfb), f(kbb), f(vbb), pos, W)
    np.testing.assert_allclose(full, z["out"], rtol=0, atol=1e-6)
    # the same history written through a ring (row = position mod ring) in 7-row appends
    st = O.OracleState(1, hkv, R, d, fp8=False)
    p = 0
    while p < pos:
        t = min(7, pos - p)
        O.kv_write(st, 0, p, kfb[:, p:p + t], vfb[:, p:p + t], ring=R)
        p += t
    ringed = O.window_block_attention(f(qb), f(st.k[0]), f(st.v[0]), f(kbb), f(vbb), pos, W, ring=R)
    assert np.array_equal(ringed, full)


def test_prefill_vs_reference(golden_dir):
    z = load(golden_dir, "prefill.npz")
    pos, T, rows = int(z["pos"]), int(z["T"]), z["rows"]
    kb, vb = O.seeded_bf16(501, HKV, pos + T, D), O.seeded_bf16(502, HKV, pos + T, D)
    qb = O.seeded_bf16(503, T, HQ, D)
    assert np.array_equal(sha(kb, vb, qb), z["in_sha"])
    st = O.OracleState(1, HKV, 128, D)
    O.kv_write(st, 0, 0, kb[:, :pos], vb[:, :pos])
    O.kv_write(st, 0, pos, kb[:, pos:], vb[:, pos:])
    kd, vd = st.dequant(0, pos + T)
    out = O.attn_prefill(O.bf16_bits_to_f32(qb), kd, vd, pos, rows=rows)
    np.testing.assert_allclose(out, z["out"], rtol=0, atol=1e-6)


def test_commit_vs_reference(golden_dir):
    cases = load(golden_dir, "commit.npz")["cases"]
    for row in cases:
        K, pos0, n, tok, pos1 = (int(x) for x in row[:5])
        got = O.spec_commit(row[5:5 + K + 1], row[13:13 + K], pos0)
        assert got == (n, tok, pos1)


@pytest.mark.parametrize("L", [0, 1, 31, 32, 33])
def test_attention_edge_lengths(L):
    """Lengths around a block edge, and an empty history (only the new row is visible)."""
    kb, vb = O.seeded_bf16(11, HKV, L + 1, D), O.seeded_bf16(12, HKV, L + 1, D)
    qb = O.seeded_bf16(13, 1, HQ, D)
    st = O.OracleState(1, HKV, 64, D)
    if L:
        O.kv_write(st, 0, 0, kb[:, :L], vb[:, :L])
    o = O.decode_step_cpu(st, 0, qb, kb[:, L:], vb[:, L:], L)
    assert np.isfinite(o).all()
    if L == 0:      # one visible key: the output is that key's dequantised V row
        _, vd = st.dequant(0, 1)
        np.testing.assert_allclose(o[0].reshape(HKV, 6, D), np.repeat(vd[:, 0][:, None], 6, axis=1), atol=1e-6)


def test_add_rmsnorm_matches_reference_golden(golden_dir):
    """The residual add + RMSNorm chain (the step after the attention output projection) against what
    the reference's torch functions returned: every bf16 bit."""
    z = np.load(os.path.join(golden_dir, "add_rmsnorm.npz"))
    B = O.bits_to_torch_bf16
    x, h, w = B(z["x_bits"]), B(z["h_bits"]), B(z["w_bits"])
    xo, y = O.add_rmsnorm(x, h, w, 1e-6)
    assert np.array_equal(O.torch_bf16_to_bits(xo), z["xo_bits"]) and np.array_equal(O.torch_bf16_to_bits(y), z["y_bits"])
    xo, y = O.add_rmsnorm(x, None, w, 1e-6)
    assert xo is x and np.array_equal(O.torch_bf16_to_bits(y), z["y_noh_bits"])
    xo, y = O.add_rmsnorm(x, h, w + 1, 1e-6, plain=True)
    assert np.array_equal(O.torch_bf16_to_bits(y), z["y_plain_bits"])
    xo, y = O.add_rmsnorm(x, torch.from_numpy(z["h_parts"]), w, 1e-6)
    assert np.array_equal(O.torch_bf16_to_bits(xo), z["xo_parts_bits"]) and np.array_equal(O.torch_bf16_to_bits(y), z["y_parts_bits"])
