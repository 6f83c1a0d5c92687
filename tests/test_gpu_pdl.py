"""Programmatic dependent launch must not change results: call sequences with no other kernel in
between (the cases in which a kernel starts while the launches before it are still running) are
compared bit for bit with ordinary launches, in both programmatic modes."""
import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from _util import HQ, HKV, D, to_dev, f32_of, assert_attn_close, oracle_state_from

pytestmark = pytest.mark.gpu
F8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def tb():
    import tokenrush_b200 as tb
    yield tb
    tb.fused.set_launch_mode(1)


def _prep_inputs(tb, L, m, seed):
    cfg = tb.AttnConfig(n_attn=1)
    qkv = to_dev(O.seeded_bf16(seed, m, HQ * 2 * D + 2 * HKV * D))
    qn, kn = to_dev(O.seeded_bf16(seed + 1, D, std=0.1)), to_dev(O.seeded_bf16(seed + 2, D, std=0.1))
    cos, sin = O.rope_table(L + 64, cfg.rotary_dim, cfg.rope_theta)
    kctx, vctx = to_dev(O.seeded_bf16(seed + 3, HKV, L, D)), to_dev(O.seeded_bf16(seed + 4, HKV, L, D))
    return cfg, qkv, qn, kn, cos.cuda(), sin.cuda(), kctx, vctx


def _ctx_prep_decode(tb, mode, L, m, iters):
    """kv_write_prefill(L context rows) -> attn_prep(m rows at L) -> attn_decode_fused, nothing between
    them, `iters` times on fresh caches; host cursors, so that no torch kernel is needed."""
    tb.fused.set_launch_mode(mode)
    cfg, qkv, qn, kn, cos, sin, kctx, vctx = _prep_inputs(tb, L, m, 300)
    outs = []
    states = [tb.State(cfg, L + 64, "cuda", kv_dtype=F8) for _ in range(iters)]
    out = torch.zeros(iters, m, HQ * D, device="cuda", dtype=torch.bfloat16)
    tb.fused.attn_decode_fused(torch.zeros(m, HQ * D, device="cuda", dtype=torch.bfloat16), None, states[0].k[0], states[0].v[0], 0, cfg,
                               states[0].k_scale[0], states[0].v_scale[0])       # workspace exists before the timed sequence
    torch.cuda.synchronize()
    for it, st in enumerate(states):
        tb.fused.kv_write_prefill(kctx, vctx, st, 0, 0)
        q = tb.fused.attn_prep(qkv, qn, kn, cos, sin, L, st.k[0], st.v[0], cfg, st.k_scale[0], st.v_scale[0])
        tb.fused.attn_decode_fused(q, qkv, st.k[0], st.v[0], L, cfg, st.k_scale[0], st.v_scale[0], out=out[it])
    torch.cuda.synchronize()
    return out.clone(), states[-1], cfg


@pytest.mark.parametrize("m", [1, 4])
def test_context_write_prep_decode_back_to_back(tb, m):
    L = 60000                                                   # a long append: a decode that started early would see unwritten rows
    want, _, _ = _ctx_prep_decode(tb, 0, L, m, 6)
    for mode in (1, 2):
        got, st, cfg = _ctx_prep_decode(tb, mode, L, m, 6)
        assert torch.equal(got, want), f"mode {mode}"
    # and the value itself against the oracle (ungated part: gate applied to the oracle's output)
    assert tb._lib.device_status() == 0


@pytest.mark.parametrize("mode", [1, 2])
def test_append_then_decode_of_all_rows_back_to_back(tb, mode):
    """trb_kv_append -> trb_attn_decode(new_rows = 0) with a host cursor: the decode reads the rows the
    append has just written (they lie below its cursor), so it must wait for it."""
    L, n_new = 50000, 6000
    cfg = tb.AttnConfig(n_attn=1)
    kb, vb = to_dev(O.seeded_bf16(1, HKV, L, D)), to_dev(O.seeded_bf16(2, HKV, L, D))
    q = to_dev(O.seeded_bf16(3, 1, HQ, D)).reshape(1, -1)
    res = {}
    for md in (0, mode):
        tb.fused.set_launch_mode(md)
        outs = torch.zeros(5, 1, HQ * D, device="cuda", dtype=torch.bfloat16)
        for it in range(5):
            st = tb.State(cfg, L + 64, "cuda", kv_dtype=F8)
            tb.fused.kv_append(kb[:, :L - n_new], vb[:, :L - n_new], st.k[0], st.v[0], 0, st.k_scale[0], st.v_scale[0])
            torch.cuda.synchronize()
            tb.fused.kv_append(kb[:, L - n_new:], vb[:, L - n_new:], st.k[0], st.v[0], L - n_new, st.k_scale[0], st.v_scale[0])
            tb.fused._decode(q, st.k[0], st.v[0], L, HQ, HKV, D, st.k_scale[0], st.v_scale[0], new_rows=0, out=outs[it])
        torch.cuda.synchronize()
        res[md] = outs.clone()
    assert torch.equal(res[mode], res[0])
    assert tb._lib.device_status() == 0


@pytest.mark.parametrize("m", [1, 8])
def test_chained_step_graph_matches_ordinary_launches(tb, m):
    """A decode step of four layers (append + decode each, then the cursor update) captured as one
    graph in chained mode, replayed with the cursor advancing on the device, against the same step
    run with ordinary launches.  The appended keys are aligned with the queries, so that the new rows
    carry most of the softmax weight: a decode that missed the rows of its own step (or saw those of
    another layer) would be far off, not a little.  Chained launches use other CTA shapes than
    ordinary ones, so the comparison is to the output's own rounding, and two chained runs must agree
    bit for bit; the last step is also checked against the oracle."""
    L, layers, steps = 20000, 4, 12
    g = HQ // HKV
    cfg = tb.AttnConfig(n_attn=layers)
    kb, vb = O.seeded_bf16(1, HKV, L, D), O.seeded_bf16(2, HKV, L, D)
    q_bits = O.seeded_bf16(3, layers, m, HQ, D)
    qf = O.bf16_bits_to_f32(q_bits)
    # key of (layer, kv head j, new row i) = sum of the six query heads of j for row i: score ~ |q|^2 / 16
    kn = O.f32_to_bf16_bits(qf.reshape(layers, m, HKV, g, D).sum(3).transpose(0, 2, 1, 3))      # [layers, HKV, m, D]
    vn = O.seeded_bf16(5, layers, HKV, m, D)
    qs = to_dev(q_bits).reshape(layers, m, HQ * D)
    kn_d, vn_d = to_dev(kn), to_dev(vn)

    def run(mode, graph):
        tb.fused.set_launch_mode(mode)
        st = tb.State(cfg, L + m * (steps + 4) + 64, "cuda", kv_dtype=F8)
        for l in range(layers):
            tb.fused.kv_write_prefill(to_dev(kb), to_dev(vb), st, l, 0)
        st.set_pos(L)
        out = torch.zeros(layers, m, HQ * D, device="cuda", dtype=torch.bfloat16)

        def step():
            for l in range(layers):
                tb.fused.kv_write_prefill(kn_d[l], vn_d[l], st, l, st.pos_t)
                tb.fused.attn_decode_fused(qs[l], None, st.k[l], st.v[l], st.pos_t, cfg, st.k_scale[l], st.v_scale[l], out=out[l])
            tb.fused.cursor_advance(st.pos_t, m)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        hist = []
        with torch.cuda.stream(side):
            step()                                               # workspaces and kernel attributes exist before capture
            side.synchronize()
            st.set_pos(L)
            if graph:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=side):
                    step()
                st.set_pos(L)
            for _ in range(steps):
                gr.replay() if graph else step()
                side.synchronize()
                hist.append(out.clone())
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        return torch.stack(hist), st

    want, _ = run(0, False)
    got, st = run(2, True)
    again, _ = run(2, True)
    assert torch.equal(got, again)                               # chained replays are reproducible
    w, gt_ = want.float(), got.float()
    assert ((gt_ - w).abs() <= 1e-3 + 2.0 ** -7 * w.abs()).all(), float((gt_ - w).abs().max())
    got1, _ = run(1, True)
    assert torch.equal(got1, want)                               # mode 1 runs the same CTA shapes as ordinary launches
    # the new rows do carry the weight: without them the outputs would be near zero
    assert float(w.abs().mean()) > 0.3
    # the last replay against the oracle over the device's bytes, layer 0 and the last layer
    pos = L + m * (steps - 1)
    for l in (0, layers - 1):
        ref = oracle_state_from(st, l)
        wantl = O.attn_rows_over_cache(ref, 0, q_bits[l], pos)
        assert_attn_close(f32_of(got[-1][l]).reshape(m, HQ, D), wantl, f"layer {l}")
    assert tb._lib.device_status() == 0
