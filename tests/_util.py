"""Helpers shared by the GPU parity tests: numpy bit patterns <-> CUDA tensors, error metrics."""
import numpy as np
import torch

from oracle import kv_oracle as O

HQ, HKV, D = 24, 4, 256


def to_dev(bits: np.ndarray) -> torch.Tensor:
    """bf16 bit patterns -> CUDA bf16 tensor (identical bits)."""
    return O.bits_to_torch_bf16(bits).cuda()


def bits_of(t: torch.Tensor) -> np.ndarray:
    return O.torch_bf16_to_bits(t.detach().cpu())


def f32_of(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def rel(a: np.ndarray, b: np.ndarray) -> float:
    """||a - b|| / ||b|| over the whole tensor (the reference's metric, tests/test_fused.py:17-18)."""
    a = a.astype(np.float64).ravel(); b = b.astype(np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def assert_attn_close(got: np.ndarray, want: np.ndarray, what="", out_ulp=2.0 ** -8):
    """The parity bar of the attention outputs against fp32 math over the same cache: rel 1e-2
    over the tensor, and every element within 2e-3 plus one rounding step of the bf16 output
    itself (2^-8 relative; at short contexts |o| is O(1) and that step alone exceeds 2e-3).
    out_ulp=0 for outputs that were never rounded to bf16."""
    assert np.isfinite(got).all(), what
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    tol = 2e-3 + out_ulp * np.abs(want.astype(np.float64))
    r = rel(got, want)
    assert (err <= tol).all() and r <= 1e-2, (what, float((err - tol).max()), float(err.max()), r)


def assert_attn_close_bf16_p(got: np.ndarray, want: np.ndarray, what=""):
    """The bar for prefill attention over a bf16 cache: the probabilities enter the PV product as bf16 (as in
    the reference's kernel: `p.to(tl.bfloat16)`, tokenrush/fused.py:515).  With only a few visible keys of
    mixed signs that rounding does not average out and is proportional to sum p |v|, not to |o|: the
    north_star's rel 1e-2 over the tensor plus 2^-7 of the largest output per element."""
    assert np.isfinite(got).all(), what
    r = rel(got, want)
    err = float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max())
    assert r <= 1e-2 and err <= 2e-3 + 2.0 ** -7 * float(np.abs(want).max()), (what, err, r)


def oracle_state_from(state, slot=0) -> O.OracleState:
    """Copy one layer of a CUDA State into an OracleState (bytes and scales)."""
    hkv, max_len, d = state.k[slot].shape
    st = O.OracleState(1, hkv, max_len, d, fp8=state.fp8)
    if state.fp8:
        st.k[0] = state.k[slot].view(torch.uint8).cpu().numpy()
        st.v[0] = state.v[slot].view(torch.uint8).cpu().numpy()
        st.k_scale[0] = state.k_scale[slot].cpu().numpy()
        st.v_scale[0] = state.v_scale[slot].cpu().numpy()
    else:
        st.k[0] = bits_of(state.k[slot])
        st.v[0] = bits_of(state.v[slot])
    return st


def fill_cache_gpu(tb, state, slot: int, rows: int, seed: int, start: int = 0, chunk: int = 16384):
    """Rows [start, start + rows) of one layer <- N(0,1) bf16 drawn on the GPU and written by the
    product's own append (the oracle later reads the bytes back, so the CPU never has to quantise
    hundreds of thousands of rows)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    hkv, _, d = state.k[slot].shape
    ks, vs = (state.k_scale[slot], state.v_scale[slot]) if state.fp8 else (None, None)
    for p0 in range(start, start + rows, chunk):
        t = min(chunk, start + rows - p0)
        k = torch.randn(hkv, t, d, device="cuda", generator=g).to(torch.bfloat16)
        v = torch.randn(hkv, t, d, device="cuda", generator=g).to(torch.bfloat16)
        tb.fused.kv_append(k, v, state.k[slot], state.v[slot], p0, ks, vs)
    torch.cuda.synchronize()


def rows_bit_exact(state, slot: int, pos: int, k_bits: np.ndarray, v_bits: np.ndarray):
    """The codes and scales of cache rows pos.. equal what the oracle's quantiser makes of the bf16 rows."""
    t = k_bits.shape[1]
    for src, cache, scale, what in ((k_bits, state.k, state.k_scale, "K"), (v_bits, state.v, state.v_scale, "V")):
        codes, sc = O.quantize_rows(O.bf16_bits_to_f32(src))
        got_c = cache[slot][:, pos:pos + t].view(torch.uint8).cpu().numpy()
        got_s = scale[slot][:, pos:pos + t].cpu().numpy()
        assert np.array_equal(got_c, codes), f"{what} codes differ"
        assert np.array_equal(got_s.view(np.uint32), sc.view(np.uint32)), f"{what} scales differ"
