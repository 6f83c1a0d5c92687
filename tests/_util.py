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
