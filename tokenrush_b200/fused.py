"""The attention / KV entry points of the reference's `tokenrush/fused.py`, same names and
argument meaning, backed by the sm_100a CUDA library through its C ABI.

    attn_prep            tokenrush/fused.py:314-324
    kv_write_prefill     tokenrush/fused.py:327-340
    attn_decode_fused    tokenrush/fused.py:449-470
    attn_prefill_fused   tokenrush/fused.py:523-533
    attn_window_block    tokenrush/fused.py:600-622
    add_rmsnorm          tokenrush/fused.py:48-60    (the step after the attention output projection)

plus the cursor arithmetic the reference does with small torch ops (`spec_commit`,
tokenrush/model.py:306-312) and the ring write of the DFlash draft cache (`ring_write`,
tokenrush/dflash.py:293-294).  Every call launches on torch's current stream, allocates
only its outputs (with torch, so it is legal under graph capture) and never synchronises.
There is no fallback: a CUDA tensor and the built library are required.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L

FP8_MAX = 448.0            # float8_e4m3fn (tokenrush/fused.py:243)

_workspaces: dict = {}
_extras: dict = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("tokenrush_b200 runs on CUDA tensors only (there is no CPU path)")


def _cursor(pos) -> L.Cursor:
    """A python int, or a device tensor of one int32 / int64 (State.pos_t)."""
    if isinstance(pos, L.Cursor):
        return pos
    if isinstance(pos, torch.Tensor):
        if pos.dtype not in (torch.int32, torch.int64) or pos.numel() < 1:
            raise TypeError("position tensor must be int32 or int64")
        _need_cuda(pos)
        return L.Cursor(pos.data_ptr(), pos.element_size(), 0, 0)
    return L.Cursor(None, 8, 0, int(pos))


def _cache(k_cache, v_cache, k_scale, v_scale, ring: int = 0, shard_lo=None) -> L.Cache:
    """Per-layer cache views [HKV, MAXLEN, D] (+ scales [HKV, MAXLEN] for fp8).  shard_lo: None for
    a whole cache, else the first position this shard of a longer sequence holds."""
    _need_cuda(k_cache, v_cache, k_scale, v_scale)
    if k_cache.dim() != 3 or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise ValueError("cache views must be contiguous [HKV, MAXLEN, D]")
    fp8 = k_cache.dtype == torch.float8_e4m3fn
    if not fp8 and k_cache.dtype != torch.bfloat16:
        raise TypeError("KV cache must be float8_e4m3fn or bfloat16")
    if fp8 and (k_scale is None or v_scale is None):
        raise ValueError("an fp8 cache needs k_scale and v_scale")
    hkv, max_len, d = k_cache.shape
    return L.Cache(k_cache.data_ptr(), v_cache.data_ptr(), k_scale.data_ptr() if fp8 else None,
                   v_scale.data_ptr() if fp8 else None, hkv, d, L.TRB_KV_FP8 if fp8 else L.TRB_KV_BF16,
                   0 if shard_lo is None else 1, max_len, ring, 0 if shard_lo is None else int(shard_lo))


def set_launch_mode(mode: int):
    """0: ordinary launches; 1 (default): programmatic dependent launch, every kernel waits before
    it releases the next one; 2: chained - a decode step made of calls of this module only (as in a
    captured graph) overlaps each layer's scan with the tail of the layer before it.  In mode 2 the
    caller promises that nothing else writes the caches, cursors or query rows between two calls
    of this module on one stream.  See trb_set_programmatic_launch in include/trb_kv.h."""
    L.check(L.lib().trb_set_programmatic_launch(int(mode)), "trb_set_programmatic_launch")


WORKSPACE_SLOTS = 16       # decode workspaces per (device, stream, geometry), used in rotation


def _workspace(device, hq: int, hkv: int, d: int, m: int):
    """Split-partial scratch + ticket words for one decode call: (device pointer, bytes, slot, slots).  Every
    (device, stream, geometry) owns WORKSPACE_SLOTS workspaces, zeroed once, and hands them out in
    rotation: consecutive decode calls of a step then never share one, which lets a call in a
    chain of library launches (launch mode 2) publish its partials without waiting for the call
    before it.  Calls that get the same slot are ordered by the stream."""
    key = (device.index, _stream(), hq, hkv, d, m)
    ent = _workspaces.get(key)
    if ent is None:
        if torch.cuda.is_current_stream_capturing():
            # a zero-fill recorded into the graph would wipe the launch counts at every replay
            raise RuntimeError("the first decode call of a (device, stream, geometry) allocates and zeroes its workspaces: "
                               "make it outside graph capture (run the step once on the capture stream first)")
        n = L.lib().trb_decode_workspace_bytes(hq, hkv, d, m)
        if n == 0:
            raise ValueError(f"unsupported geometry hq={hq} hkv={hkv} d={d} m={m}")
        n = (n + 255) // 256 * 256
        # rotation only pays for the calls that can run ahead of the call before them (one 8-row slice:
        # two of their CTAs share an SM); the partials of wider calls are large, and one workspace
        # that stays in L2 serves them better than sixteen that do not
        slots = WORKSPACE_SLOTS if (hq // hkv) * m <= 8 else 1
        ent = [torch.zeros(slots * n, device=device, dtype=torch.uint8), n, 0]
        _workspaces[key] = ent
    buf, n, count = ent
    ent[2] = count + 1
    slots = buf.numel() // n
    return buf.data_ptr() + (count % slots) * n, n, count % slots, slots


def workspace_tensor(device, hq: int, hkv: int, d: int, m: int):
    """The tensor that holds the WORKSPACE_SLOTS workspaces of the current stream for this geometry
    (None before the first decode call); zero it after a call reported a workspace problem."""
    ent = _workspaces.get((device.index, _stream(), hq, hkv, d, m))
    return None if ent is None else ent[0]


# ------------------------------------------------------------------------------ append

def kv_append(k, v, k_cache, v_cache, pos, k_scale=None, v_scale=None, ring: int = 0, shard_lo=None, n_valid=None):
    """k, v [HKV, T, D] bf16 (any strides with a contiguous last dim) -> cache rows at positions
    pos..pos+T-1; pos and n_valid may be device tensors.  FP8 caches are quantised on write."""
    _need_cuda(k, v)
    if k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("k, v must be bfloat16")
    if k.stride(-1) != 1 or v.stride(-1) != 1 or k.stride() != v.stride() or k.shape != v.shape:
        raise ValueError("k and v must share shape and strides, last dim contiguous")
    cache = _cache(k_cache, v_cache, k_scale, v_scale, ring, shard_lo)
    cur = _cursor(pos)
    nv = _cursor(n_valid) if n_valid is not None else None
    L.check(L.lib().trb_kv_append(C.byref(cache), k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), k.shape[1],
                                  C.byref(cur), C.byref(nv) if nv is not None else None, _stream()), "trb_kv_append")


def kv_write_prefill(k, v, state, slot, pos):
    """Prefill-side cache write. k, v [Hkv, T, D] bf16 -> cache rows pos..pos+T-1 of layer `slot`,
    quantised to fp8 with per-(head, position) scales when the cache is fp8."""
    ks = state.k_scale[slot] if state.fp8 else None
    vs = state.v_scale[slot] if state.fp8 else None
    kv_append(k, v, state.k[slot], state.v[slot], pos, ks, vs, shard_lo=getattr(state, "shard_lo", None))


def ring_write(k, v, k_cache, v_cache, pos, ring: int, n_valid=None):
    """Write rows at positions pos.. into a ring cache, row = position mod ring
    (tokenrush/dflash.py:197-198,256-257,293-294)."""
    kv_append(k, v, k_cache, v_cache, pos, ring=ring, n_valid=n_valid)


def attn_prep(qkv, q_norm_w, k_norm_w, cos, sin, pos_t, k_cache, v_cache, cfg, k_scale=None, v_scale=None, shard_lo=None):
    """qkv [M, HQ*2D + 2*HKV*D] -> q [M, HQ*D] normed + roped; writes K, V (and their fp8
    scales when the cache is fp8) at pos_t + i."""
    _need_cuda(qkv, q_norm_w, k_norm_w, cos, sin)
    HQ, HKV, D = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    M = qkv.shape[0]
    if qkv.dtype != torch.bfloat16 or not qkv.is_contiguous() or qkv.shape[1] != HQ * 2 * D + 2 * HKV * D:
        raise ValueError("qkv must be contiguous bf16 [M, HQ*2D + 2*HKV*D]")
    if not (cos.is_contiguous() and sin.is_contiguous()) or cos.dtype != torch.bfloat16:
        raise ValueError("cos / sin must be contiguous bf16 [rows, rotary_dim]")
    cache = _cache(k_cache, v_cache, k_scale, v_scale, shard_lo=shard_lo)
    q = torch.empty(M, HQ * D, device=qkv.device, dtype=qkv.dtype)
    cur = _cursor(pos_t)
    L.check(L.lib().trb_attn_prep(C.byref(cache), qkv.data_ptr(), q_norm_w.data_ptr(), k_norm_w.data_ptr(), cos.data_ptr(),
                                  sin.data_ptr(), cos.shape[0], cos.shape[1], float(cfg.eps), M, HQ, C.byref(cur),
                                  q.data_ptr(), _stream()), "trb_attn_prep")
    return q


# ------------------------------------------------------------------------------ decode

def _decode(q, k_cache, v_cache, pos, HQ, HKV, D, k_scale, v_scale, *, gate=None, gate_rs=0, gate_hs=0, new_rows=1,
            window=0, ring=0, shard_lo=None, extra=None, partial=False, scale=None, out=None, p2p=None):
    _need_cuda(q)
    if q.dtype != torch.bfloat16 or not q.is_contiguous():
        raise ValueError("q must be contiguous bf16 [M, HQ*D]")
    M = q.shape[0]
    cache = _cache(k_cache, v_cache, k_scale, v_scale, ring, shard_lo)
    ws_ptr, ws_bytes, ws_slot, ws_slots = _workspace(q.device, HQ, HKV, D, M)
    a = L.DecodeArgs()
    a.q = q.data_ptr()
    a.m, a.hq = M, HQ
    a.scale = float(D ** -0.5 if scale is None else scale)
    a.new_rows, a.window = int(new_rows), int(window)
    a.pos = _cursor(pos)
    a.workspace, a.workspace_bytes = ws_ptr, ws_bytes
    a.ws_slot, a.ws_slots = ws_slot, ws_slots
    if gate is not None:
        a.gate, a.gate_row_stride, a.gate_head_stride = gate, gate_rs, gate_hs
    if extra is not None:
        a.n_extra, a.extra_ml, a.extra_acc = 1, extra[0].data_ptr(), extra[1].data_ptr()
    if p2p is not None:                                   # (host ctypes array of exchange-buffer pointers, world, rank)
        a.p2p_xchg, a.p2p_world, a.p2p_rank = C.cast(p2p[0], C.c_void_p), int(p2p[1]), int(p2p[2])
    if partial:
        ml = torch.empty(M * HQ, 2, device=q.device, dtype=torch.float32)
        acc = torch.empty(M * HQ, D, device=q.device, dtype=torch.float32)
        a.partial_ml, a.partial_acc = ml.data_ptr(), acc.data_ptr()
        out = (ml, acc)
    else:
        if out is None:
            out = torch.empty(M, HQ * D, device=q.device, dtype=q.dtype)
        elif out.dtype != torch.bfloat16 or not out.is_contiguous() or out.numel() != M * HQ * D:
            raise ValueError("out must be contiguous bf16 [M, HQ*D]")
        a.out = out.data_ptr()
    L.check(L.lib().trb_attn_decode(C.byref(cache), C.byref(a), _stream()), "trb_attn_decode")
    return out


def attn_decode_fused(q, qkv, k_cache, v_cache, pos_t, cfg, k_scale=None, v_scale=None, NSPLIT=32, BLOCK_N=32,
                      shard_lo=None, partial: bool = False, out=None, p2p=None):
    """q [M, HQ*D] (from attn_prep) for the M new tokens at pos.., qkv [M, ..] (for the gates;
    None: ungated) -> gated attention output [M, HQ*D]; query i sees cache rows <= pos + i.
    NSPLIT / BLOCK_N are accepted for signature compatibility; the split count is chosen
    from the SM count and the split ranges from the live length on the device.
    partial=True (sequence shards): returns this cache's (ml [M*HQ, 2], acc [M*HQ, D]).
    out (optional): a preallocated [M, HQ*D] bf16 tensor to write instead of a new one.
    p2p (sequence shards, fused exchange): (ctypes array of the GPUs' exchange-buffer
    pointers, world, rank); the kernel's tail then merges the partials of all GPUs itself."""
    HQ, HKV, D = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    gate = None
    rs = hs = 0
    if qkv is not None and not partial:
        _need_cuda(qkv)
        gate, rs, hs = qkv.data_ptr() + D * qkv.element_size(), qkv.stride(0), 2 * D
    return _decode(q, k_cache, v_cache, pos_t, HQ, HKV, D, k_scale, v_scale, gate=gate, gate_rs=rs, gate_hs=hs,
                   new_rows=1, shard_lo=shard_lo, partial=partial, out=out, p2p=p2p)


def attn_window_block(q, k_cache, v_cache, pos_t, k_blk, v_blk, HQ, HKV, D, window, NSPLIT=15, BLOCK_N=32, ring=0):
    """DFlash draft attention: q [B, HQ*D] for a block of B queries at positions pos..
    over (a) the cache rows < pos within `window` of each query and (b) the B block keys
    k_blk/v_blk [HKV, B, D] (bidirectional). Ungated. Returns [B, HQ*D].
    ring > 0: the cache is a ring of `ring` rows, row = position mod ring."""
    _need_cuda(q, k_blk, v_blk)
    B = q.shape[0]
    if not (k_blk.is_contiguous() and v_blk.is_contiguous()) or k_blk.dtype != torch.bfloat16:
        raise ValueError("k_blk / v_blk must be contiguous bf16 [HKV, B, D]")
    ml = torch.empty(B * HQ, 2, device=q.device, dtype=torch.float32)
    acc = torch.empty(B * HQ, D, device=q.device, dtype=torch.float32)
    L.check(L.lib().trb_attn_block_partial(q.data_ptr(), k_blk.data_ptr(), v_blk.data_ptr(), B, HQ, HKV, D,
                                           float(D ** -0.5), ml.data_ptr(), acc.data_ptr(), _stream()),
            "trb_attn_block_partial")
    return _decode(q, k_cache, v_cache, pos_t, HQ, HKV, D, None, None, new_rows=0, window=window, ring=ring,
                   extra=(ml, acc))


def lse_merge(ml, acc, out_dtype=torch.bfloat16, hq: int = 1):
    """ml [P, R, 2] (max in log2 units, sum), acc [P, R, D] fp32 -> [R, D]: the split merge
    of tokenrush/fused.py:432-438 over the leading axis, in index order."""
    _need_cuda(ml, acc)
    P, R, D = acc.shape
    out = torch.empty(R, D, device=acc.device, dtype=out_dtype)
    L.check(L.lib().trb_lse_merge(ml.contiguous().data_ptr(), acc.contiguous().data_ptr(), P, R, D, out.data_ptr(), None, 0, 0,
                                  hq, _stream()), "trb_lse_merge")
    return out


# ------------------------------------------------------------------------------ prefill

def attn_prefill_fused(q, k_cache, v_cache, pos, cfg, k_scale=None, v_scale=None, BM=64, BN=32):
    """q [T, HQ, D] bf16 (normed, roped) for positions pos.. ; cache holds rows 0..pos+T-1
    -> o [T, HQ, D] bf16."""
    _need_cuda(q)
    T, HQ, D = q.shape
    if q.dtype != torch.bfloat16 or not q.is_contiguous():
        raise ValueError("q must be contiguous bf16 [T, HQ, D]")
    cache = _cache(k_cache, v_cache, k_scale, v_scale)
    if D != 256:
        # The tensor-core prefill kernel is built for 256-dim heads (e4m3 or bf16 cache; the reference's
        # default is bf16, tokenrush/fused.py:523-533 with FP8 = False).  Caches of another head size
        # go through the M-row decode kernel, in groups of as many rows as one launch takes.
        HKV = k_cache.shape[0]
        m_max = max(1, 48 // (HQ // HKV))
        o = torch.empty_like(q)
        for s0 in range(0, T, m_max):
            m = min(m_max, T - s0)
            _decode(q[s0:s0 + m].reshape(m, HQ * D), k_cache, v_cache, int(pos) + s0, HQ, HKV, D, k_scale, v_scale, new_rows=1,
                    out=o[s0:s0 + m].view(m, HQ * D))
        return o
    o = torch.empty_like(q)
    L.check(L.lib().trb_attn_prefill(C.byref(cache), q.data_ptr(), o.data_ptr(), T, HQ, int(pos), float(D ** -0.5), _stream()),
            "trb_attn_prefill")
    return o


# ------------------------------------------------------------------------------ after attention

def add_rmsnorm(x: torch.Tensor, h, weight: torch.Tensor, eps: float, plain: bool = False):
    """x [T, N] bf16; h None, [T, N] bf16, or [S, T, N] fp32 partials ->
    (x + h as bf16, rmsnorm(x + h)); with h None -> (x, rmsnorm(x)).
    plain: Qwen3's weight * x gain (the DFlash draft) instead of Qwen3.5's (1 + weight).
    (tokenrush/fused.py:48-60; the attention output of attn_decode_fused reaches it through the
    output projection: tokenrush/model.py:119-120.)"""
    _need_cuda(x, h, weight)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous() or x.dim() != 2:
        raise ValueError("x must be contiguous bf16 [T, N], weight bf16 [N]")
    T, N = x.shape
    y = torch.empty_like(x)
    if h is None:
        xo, splits, hp = x, 0, None
    else:
        if not h.is_contiguous():
            raise ValueError("h must be contiguous")
        if h.dim() == 2 and h.dtype == torch.bfloat16 and h.shape == x.shape:
            splits = -1
        elif h.dim() == 3 and h.dtype == torch.float32 and tuple(h.shape[1:]) == (T, N):
            splits = h.shape[0]
        else:
            raise ValueError("h must be [T, N] bf16 or [S, T, N] fp32")
        xo, hp = torch.empty_like(x), h.data_ptr()
    L.check(L.lib().trb_add_rmsnorm(x.data_ptr(), hp, splits, weight.data_ptr(), float(eps), int(plain), T, N,
                                    xo.data_ptr() if h is not None else None, y.data_ptr(), _stream()), "trb_add_rmsnorm")
    return xo, y


# ------------------------------------------------------------------------------ cursors

def spec_commit(pred, drafts, n_accepted, tok, pos_t):
    """Device-side commit of a verify step (tokenrush/model.py:306-312): n = leading drafts
    that match; n_accepted <- n; tok <- pred[n]; pos_t += n + 1.  All tensors stay on the
    device; nothing in the cache moves."""
    _need_cuda(pred, drafts, n_accepted, tok, pos_t)
    if pred.dtype != torch.int64 or drafts.dtype != torch.int64:
        raise TypeError("pred / drafts must be int64")
    L.check(L.lib().trb_spec_commit(pred.data_ptr(), drafts.data_ptr(), drafts.numel(), n_accepted.data_ptr(), tok.data_ptr(),
                                    pos_t.data_ptr(), pos_t.element_size(), _stream()), "trb_spec_commit")


def cursor_advance(pos_t, delta: int):
    """pos_t += delta on the device, as one tiny launch (State.advance's device half)."""
    _need_cuda(pos_t)
    L.check(L.lib().trb_cursor_advance(pos_t.data_ptr(), pos_t.element_size(), int(delta), _stream()), "trb_cursor_advance")
