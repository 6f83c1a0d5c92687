"""The call patterns on either side of the kernels (through the host shim): the fused decode branch
of `attn_forward` (prep -> decode with gate, tokenrush/model.py:116-120), the MTP head's rewind
(`set_pos`, tokenrush/mtp.py:84-87), a graph-captured DFlash draft step (ring write with a device
valid count + window attention, tokenrush/dflash.py:293-299), and the `ops.py` callables."""
import os

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from _util import HQ, HKV, D, to_dev, bits_of, f32_of, rel, assert_attn_close, assert_attn_close_bf16_p, oracle_state_from

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def tb():
    import tokenrush_b200 as tb
    return tb


def test_attn_forward_fused_branch_over_steps(tb):
    """prep (norm + rope + append) then gated decode, six steps from T0 = 5 and 2100, fp8 cache:
    against the oracle's prep + append + fp32 attention + gate (tests/test_fused.py:200-227 pattern)."""
    cfg = tb.AttnConfig(n_attn=1)
    max_len = 4096
    cos, sin = O.rope_table(max_len, 64, 1e7)
    qw, kw = O.seeded_bf16(41, D, std=0.5), O.seeded_bf16(42, D, std=0.5)
    for T0 in (5, 2100):
        st = tb.State(cfg, max_len, "cuda", kv_dtype=F8)
        ref = O.OracleState(1, HKV, max_len, D)
        kb, vb = O.seeded_bf16(43 + T0, HKV, T0, D), O.seeded_bf16(44 + T0, HKV, T0, D)
        tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, 0, 0)
        O.kv_write(ref, 0, 0, kb, vb)
        st.set_pos(T0)
        for t in range(T0, T0 + 6):
            qkvb = O.seeded_bf16(1000 + t, 1, HQ * 2 * D + 2 * HKV * D)
            qkv = to_dev(qkvb)
            q = tb.fused.attn_prep(qkv, to_dev(qw), to_dev(kw), cos.cuda(), sin.cuda(), st.pos_t, st.k[0], st.v[0], cfg,
                                   st.k_scale[0], st.v_scale[0])
            o = tb.fused.attn_decode_fused(q, qkv, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
            st.advance(1)
            # oracle on the GPU's own cache bytes and its own q (the norm may differ by one bf16 step)
            mine = oracle_state_from(st)
            kd, vd = mine.dequant(0, t + 1)
            want = O.attn_rows(O.bf16_bits_to_f32(bits_of(q).reshape(1, HQ, D)), kd, vd, t)
            gate = qkvb[:, :HQ * 2 * D].reshape(1, HQ, 2 * D)[:, :, D:]
            want_g = O.bf16_bits_to_f32(O.gate_output(want, np.ascontiguousarray(gate)))
            # the gated output is rounded to bf16 twice (o, then o * sigmoid(gate)): two rounding steps
            assert_attn_close(f32_of(o).reshape(1, HQ, D), want_g, f"T0={T0} t={t}", out_ulp=2.0 ** -7)
            # and the cache row against the oracle's own prep (K within the reference's 5e-3, V exact)
            qo, _, ko, vo = O.attn_prep(O.bits_to_torch_bf16(qkvb), O.bits_to_torch_bf16(qw), O.bits_to_torch_bf16(kw), cos, sin,
                                        t, HQ, HKV, D, 1e-6)
            O.kv_write(ref, 0, t, O.torch_bf16_to_bits(ko), O.torch_bf16_to_bits(vo))
            assert np.array_equal(mine.v[0, :, t], ref.v[0, :, t])
            kr, _ = ref.dequant(0, t + 1)
            assert rel(kd[:, t], kr[:, t]) < 5e-3
    assert tb._lib.device_status() == 0


def test_rewind_then_recompute_is_bit_identical(tb):
    """MTP-style rewind: decode three steps, set_pos back, recompute the same steps: identical bits
    (tests/test_mtp.py:25-45), and rows beyond the cursor are simply overwritten."""
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, 512, "cuda", kv_dtype=F8)
    L = 300
    kb, vb = O.seeded_bf16(51, HKV, L + 3, D), O.seeded_bf16(52, HKV, L + 3, D)
    qb = O.seeded_bf16(53, 3, HQ, D)
    tb.fused.kv_write_prefill(to_dev(kb[:, :L]), to_dev(vb[:, :L]), st, 0, 0)

    def three_steps():
        outs = []
        st.set_pos(L)
        for t in range(3):
            tb.fused.kv_write_prefill(to_dev(kb[:, L + t:L + t + 1]), to_dev(vb[:, L + t:L + t + 1]), st, 0, st.pos_t)
            outs.append(tb.fused.attn_decode_fused(to_dev(qb[t:t + 1]).reshape(1, -1), None, st.k[0], st.v[0], st.pos_t, cfg,
                                                   st.k_scale[0], st.v_scale[0]).clone())
            st.advance(1)
        return torch.stack(outs), st.k[0].view(torch.uint8).clone()

    a, ka = three_steps()
    b, kb2 = three_steps()
    assert torch.equal(a, b) and torch.equal(ka, kb2)


def test_draft_step_in_cuda_graph(tb):
    """One captured draft step: 8 context rows offered, the first n_valid (device) written into the
    ring at the device cursor, window + block attention at the new block start; replayed with
    different accept counts."""
    hq, hkv, d, B, W, R = 32, 8, 128, 8, 2048, 4096
    total = 400
    kfb, vfb = O.seeded_bf16(61, hkv, total + 8, d), O.seeded_bf16(62, hkv, total + 8, d)
    kr = torch.zeros(hkv, R, d, device="cuda", dtype=torch.bfloat16); vr = torch.zeros_like(kr)
    ctx_t = torch.zeros(1, device="cuda", dtype=torch.long)      # end of the draft cache
    n_ctx = torch.ones(1, device="cuda", dtype=torch.long)
    p0 = torch.zeros(1, device="cuda", dtype=torch.long)         # block start = ctx_t + n_ctx
    k_in = torch.zeros(hkv, 8, d, device="cuda", dtype=torch.bfloat16); v_in = torch.zeros_like(k_in)
    q_in = torch.zeros(B, hq * d, device="cuda", dtype=torch.bfloat16)
    kb_in = torch.zeros(hkv, B, d, device="cuda", dtype=torch.bfloat16); vb_in = torch.zeros_like(kb_in)
    out = torch.zeros(B, hq * d, device="cuda", dtype=torch.bfloat16)

    def body():
        tb.fused.ring_write(k_in, v_in, kr, vr, ctx_t, R, n_valid=n_ctx)
        p0.copy_(ctx_t + n_ctx)
        out.copy_(tb.fused.attn_window_block(q_in, kr, vr, p0, kb_in, vb_in, hq, hkv, d, W, ring=R))
        ctx_t.copy_(p0)

    s = torch.cuda.Stream(); s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        body()
    torch.cuda.current_stream().wait_stream(s); torch.cuda.synchronize()
    kr.zero_(); vr.zero_(); ctx_t.zero_()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        body()
    kr.zero_(); vr.zero_(); ctx_t.zero_()
    f = O.bf16_bits_to_f32
    pos, rng = 0, np.random.default_rng(3)
    for step in range(40):
        n = int(rng.integers(1, 9))
        n_ctx.fill_(n)
        k_in.copy_(to_dev(kfb[:, pos:pos + 8])); v_in.copy_(to_dev(vfb[:, pos:pos + 8]))
        qb = O.seeded_bf16(70 + step, B, hq, d)
        kbb, vbb = O.seeded_bf16(170 + step, hkv, B, d), O.seeded_bf16(270 + step, hkv, B, d)
        q_in.copy_(to_dev(qb).reshape(B, -1)); kb_in.copy_(to_dev(kbb)); vb_in.copy_(to_dev(vbb))
        g.replay()
        pos += n
        if step % 9 == 0 or step == 39:
            torch.cuda.synchronize()
            assert int(ctx_t) == pos
            want = O.window_block_attention(f(qb), f(kfb[:, :pos]), f(vfb[:, :pos]), f(kbb), f(vbb), pos, W)
            assert_attn_close(f32_of(out).reshape(B, hq, d), want, f"draft step {step}")
    assert tb._lib.device_status() == 0


def test_ops_callables_over_bf16_cache(tb):
    """ops.attn_decode / attn_decode_bucket / attn_prefill on slices of a bf16 cache, against the
    oracle (tests/test_ops.py:139-146: prefill == per-token decode)."""
    cfg = tb.AttnConfig(n_attn=1)
    max_len, pos, T = 256, 37, 20
    st = tb.State(cfg, max_len, "cuda")                                          # bf16 cache
    kb, vb = O.seeded_bf16(81, HKV, pos + T, D), O.seeded_bf16(82, HKV, pos + T, D)
    tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, 0, 0)
    qb = O.seeded_bf16(83, T, HQ, D)
    q = to_dev(qb).transpose(0, 1).contiguous()                                  # [Hq, T, D]
    f = O.bf16_bits_to_f32
    want = O.attn_prefill(f(qb), f(kb), f(vb), pos)                             # [T, HQ, D]
    got = tb.ops.attn_prefill(q, st.k[0, :, :pos + T], st.v[0, :, :pos + T], pos)
    assert_attn_close_bf16_p(f32_of(got.transpose(0, 1)), want, "ops.attn_prefill")       # tensor-core prefill kernel, bf16 P
    i = 7
    o1 = tb.ops.attn_decode(q[:, i:i + 1], st.k[0, :, :pos + i + 1], st.v[0, :, :pos + i + 1])
    assert_attn_close(f32_of(o1)[:, 0], want[i], "ops.attn_decode")
    pos_t = torch.tensor([pos + i], device="cuda")
    o2 = tb.ops.attn_decode_bucket(q[:, i:i + 1], st.k[0, :, :128], st.v[0, :, :128], pos_t)
    assert torch.equal(o1, o2)


def test_add_rmsnorm_after_the_output_projection(tb, golden_dir):
    """The step after attention: the decode output is [M, HQ*D] bf16, the rows the output projection
    reads; its (split-K) result goes through add_rmsnorm.  Against the reference's golden vectors:
    the residual sum bit for bit, the normed rows within one bf16 step (the fp32 mean of squares is
    summed in another order than torch's CPU reduction) and mostly bit for bit."""
    z = np.load(os.path.join(golden_dir, "add_rmsnorm.npz"))
    x, h, w = to_dev(z["x_bits"]), to_dev(z["h_bits"]), to_dev(z["w_bits"])

    def close(got_bits, want_bits, what):
        g, wv = O.bf16_bits_to_f32(got_bits), O.bf16_bits_to_f32(want_bits)
        assert (np.abs(g - wv) <= 2.0 ** -7 * np.abs(wv) + 1e-6).all(), what
        assert (got_bits == want_bits).mean() > 0.99, (what, float((got_bits == want_bits).mean()))
    xo, y = tb.fused.add_rmsnorm(x, h, w, 1e-6)
    assert np.array_equal(bits_of(xo), z["xo_bits"])
    close(bits_of(y), z["y_bits"], "bf16 h")
    xo, y = tb.fused.add_rmsnorm(x, None, w, 1e-6)
    assert xo is x
    close(bits_of(y), z["y_noh_bits"], "no h")
    xo, y = tb.fused.add_rmsnorm(x, h, (w.float() + 1).to(torch.bfloat16), 1e-6, plain=True)
    close(bits_of(y), z["y_plain_bits"], "plain gain")
    xo, y = tb.fused.add_rmsnorm(x, torch.from_numpy(z["h_parts"]).cuda(), w, 1e-6)
    assert np.array_equal(bits_of(xo), z["xo_parts_bits"])                       # split partials summed in split order
    close(bits_of(y), z["y_parts_bits"], "fp32 partials")
    # hand-off: what attn_decode_fused returns is what a projection over [M, HQ*D] rows takes as it is
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, 128, "cuda", kv_dtype=torch.float8_e4m3fn)
    st.set_pos(7)
    o = tb.fused.attn_decode_fused(torch.zeros(2, HQ * D, device="cuda", dtype=torch.bfloat16), None, st.k[0], st.v[0], st.pos_t, cfg,
                                   st.k_scale[0], st.v_scale[0])
    assert o.shape == (2, HQ * D) and o.is_contiguous() and o.dtype == torch.bfloat16
    assert tb._lib.device_status() == 0


def test_launch_count_counts_the_library_kernels(tb):
    """trb_launch_count: one per kernel the library launches (append, decode, cursor update), nothing for
    calls that fail their argument checks."""
    lib = tb._lib.lib()
    cfg = tb.AttnConfig(n_attn=1)
    st = tb.State(cfg, 512, "cuda", kv_dtype=F8)
    k = to_dev(O.seeded_bf16(91, HKV, 40, D))
    tb.fused.kv_write_prefill(k, k, st, 0, 0)                       # the workspace of the decode below exists afterwards
    st.set_pos(39)
    q = to_dev(O.seeded_bf16(92, 1, HQ * D))
    tb.fused.attn_decode_fused(q, None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
    n0 = lib.trb_launch_count()
    tb.fused.kv_write_prefill(k[:, :1], k[:, :1], st, 0, st.pos_t)
    tb.fused.attn_decode_fused(q, None, st.k[0], st.v[0], st.pos_t, cfg, st.k_scale[0], st.v_scale[0])
    tb.fused.cursor_advance(st.pos_t, 1)
    assert lib.trb_launch_count() - n0 == 3
    with pytest.raises(Exception):
        tb.fused.kv_append(k[:, :1].float(), k[:, :1].float(), st.k[0], st.v[0], 0, st.k_scale[0], st.v_scale[0])
    assert lib.trb_launch_count() - n0 == 3
    torch.cuda.synchronize()
    assert tb._lib.device_status() == 0
