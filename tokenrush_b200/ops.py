"""The three attention callables of the reference's `tokenrush/ops.py` (its torch reference math,
:166-195), same names and shapes, served by the CUDA decode kernel over bf16 keys / values:

    attn_decode(q, K, V)                 tokenrush/ops.py:166-168
    attn_decode_bucket(q, K, V, pos_t)   tokenrush/ops.py:171-176
    attn_prefill(q, K, V, pos, block)    tokenrush/ops.py:179-195

K, V are views `[Hkv, S, D]` of a bf16 cache (rows contiguous; the head stride may be larger than
S * D, as for `state.k[slot, :, :pos + 1]`).  Outputs are bf16 like the inputs.  CUDA only.
"""
from __future__ import annotations

import torch

from . import fused


class _Geom:
    def __init__(self, hq, hkv, d):
        self.n_heads, self.n_kv_heads, self.head_dim = hq, hkv, d


def _as_cache(K: torch.Tensor, V: torch.Tensor):
    """A [Hkv, S, D] view -> the contiguous [Hkv, rows, D] tensor over the same memory that the C ABI
    takes (rows = head stride / D), without copying."""
    if K.dtype != torch.bfloat16 or V.dtype != torch.bfloat16:
        raise TypeError("ops.* take bf16 K / V (use fused.* for the fp8 cache)")
    if K.stride(2) != 1 or K.stride(1) != K.shape[2] or K.stride() != V.stride():
        raise ValueError("K / V rows must be contiguous and share strides")
    hkv, s, d = K.shape
    rows = K.stride(0) // d if hkv > 1 else s
    if rows < s:
        raise ValueError("unexpected head stride")
    if rows == s:
        return K, V
    return torch.as_strided(K, (hkv, rows, d), (rows * d, d, 1)), torch.as_strided(V, (hkv, rows, d), (rows * d, d, 1))


def attn_decode(q, K, V):
    """q [Hq, 1, D]; K, V [Hkv, S, D] -> [Hq, 1, D]. Every cached key is visible."""
    hq, _, d = q.shape
    kc, vc = _as_cache(K, V)
    o = fused._decode(q.reshape(1, hq * d).contiguous(), kc, vc, K.shape[1], hq, K.shape[0], d, None, None, new_rows=0)
    return o.view(hq, 1, d)


def attn_decode_bucket(q, K, V, pos_t):
    """q [Hq, 1, D]; K, V [Hkv, S, D] where S is a fixed bucket >= pos+1; keys beyond pos_t (a device
    tensor) are not visible.  Shape-static, so it captures into a graph."""
    hq, _, d = q.shape
    kc, vc = _as_cache(K, V)
    cur = fused._cursor(pos_t)
    cur.host = 1                                            # live length = pos_t + 1
    o = fused._decode(q.reshape(1, hq * d).contiguous(), kc, vc, cur, hq, K.shape[0], d, None, None, new_rows=0)
    return o.view(hq, 1, d)


def attn_prefill(q, K, V, pos: int, block: int = 1024):
    """q [Hq, T, D] for positions pos..pos+T-1; K, V [Hkv, pos+T, D].  Causal over the whole cache:
    query i sees keys <= pos+i.  256-dim heads take the tensor-core prefill kernel (bf16 MMAs over the
    rows as they are); other head sizes go through the M-row decode kernel in groups of rows."""
    hq, t, d = q.shape
    hkv = K.shape[0]
    assert K.shape[1] == pos + t
    kc, vc = _as_cache(K, V)
    qt = q.transpose(0, 1).contiguous()                      # [T, Hq, D]
    if d == 256:
        return fused.attn_prefill_fused(qt, kc, vc, pos, _Geom(hq, hkv, d)).transpose(0, 1)
    m_max = max(1, 48 // (hq // hkv))
    out = torch.empty_like(q)
    for s0 in range(0, t, m_max):
        m = min(m_max, t - s0)
        o = fused._decode(qt[s0:s0 + m].reshape(m, hq * d), kc, vc, pos + s0, hq, hkv, d, None, None, new_rows=1)
        out[:, s0:s0 + m] = o.view(m, hq, d).transpose(0, 1)
    return out
