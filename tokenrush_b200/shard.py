"""Sequence-sharded decode over the GPUs of one box (one process per GPU).

The reference is single-GPU; its split kernel already reduces (max, sum, acc) triples over
32 key ranges of one cache (tokenrush/fused.py:417-420 write, :432-438 merge).  Here the same
reduction runs one level up: GPU g owns positions [g*S/G, (g+1)*S/G) of every layer's cache,
scans its live rows, and the per-GPU partials are merged in rank order on every GPU.

Three exchange paths:
  * "fused" (default): the decode kernel's tail pushes each row's partial into every GPU's
    exchange buffer (plain peer stores over NVLink, buffers shared with CUDA IPC handles),
    waits (bounded) for the peers' flags and merges: scan, exchange and merge are one launch;
  * "p2p": the same exchange as a separate kernel after the scan (trb_p2p_merge);
  * "nccl": torch.distributed all_gather of the partials, then trb_lse_merge.  The baseline.
All produce the same bits: the merge order is the rank order.

The appended row is written by the GPU that owns its position; every rank issues the same
launches, the kernels skip positions they do not hold, so one captured graph is valid on
all ranks.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L
from . import fused
from .state import State


def shard_range(rank: int, world: int, window: int) -> tuple[int, int]:
    """Contiguous equal shards of a window of `window` positions."""
    if window % world:
        raise ValueError("window must be a multiple of the number of GPUs")
    per = window // world
    return rank * per, (rank + 1) * per


def owner_of(pos: int, world: int, window: int) -> int:
    """Rank that holds position pos; positions past the window stay with the last rank."""
    return min(pos // (window // world), world - 1)


def live_rows(rank: int, world: int, window: int, live: int, headroom: int = 0) -> int:
    """Rows of this rank's shard that are live when the sequence holds `live` positions."""
    lo, hi = shard_range(rank, world, window)
    cap = hi - lo + (headroom if rank == world - 1 else 0)
    return max(0, min(live - lo, cap))


def resume_plan(pos: int, world: int, window: int, headroom: int = 0) -> dict:
    """What resuming a sharded sequence at position `pos` (a prefix-reuse restore or a rewind after
    rejected drafts: tokenrush/session.py:92-103, tokenrush/mtp.py:84-87) means for every rank.  The
    cursor is replicated, so every rank sets the same value; nothing in any cache moves:

      owner  - the rank that holds position `pos`, i.e. the one whose append writes the next row;
      live   - live rows per rank afterwards (rank r keeps min(max(pos - lo_r, 0), rows_r));
      dead   - rows per rank that held positions >= pos of the old sequence and are dead data from
               now on (given the old live length `old_live` via resume_rows_dropped); they are
               overwritten by later appends, as the rejected rows of a verify step are.
    A rewind across a shard boundary therefore empties the later ranks completely (live 0: their
    kernels see no tile and publish an empty partial) and shortens the owner's shard."""
    if not 0 <= pos <= window + headroom:
        raise ValueError(f"position {pos} outside the sharded sequence (window {window} + headroom {headroom})")
    return {"pos": pos, "owner": owner_of(pos, world, window),
            "live": [live_rows(r, world, window, pos, headroom) for r in range(world)]}


def resume_rows_dropped(old_live: int, pos: int, world: int, window: int, headroom: int = 0) -> list:
    """Rows per rank that stop being live when a sequence of `old_live` positions resumes at `pos`."""
    return [live_rows(r, world, window, old_live, headroom) - live_rows(r, world, window, min(pos, old_live), headroom)
            for r in range(world)]


def ring_snapshot_valid(snap_pos: int, cur_pos: int, ring: int, window: int, block: int) -> bool:
    """Can a snapshot taken at `snap_pos` still be resumed when the draft's ring cache has been
    written up to `cur_pos`?  Resuming needs the `window` rows before snap_pos; the ring has
    ring - window - block - 8 rows of slack beyond what one step reads, and rows older than that
    have been overwritten (tokenrush/session.py:282-285: the prompt-end snapshot is dropped once
    P - snap.pos exceeds that slack; ring size: tokenrush/dflash.py:139-146)."""
    return cur_pos - snap_pos <= ring - window - block - 8


class ShardedState(State):
    """One rank's shard of the KV state.  The last rank carries `headroom` extra rows so that
    the sequence can grow past the window."""

    def __init__(self, cfg, window: int, rank: int, world: int, device="cuda", kv_dtype=torch.float8_e4m3fn,
                 headroom: int = 0, pos_dtype=torch.long):
        lo, hi = shard_range(rank, world, window)
        rows = hi - lo + (headroom if rank == world - 1 else 0)
        super().__init__(cfg, rows, device, kv_dtype=kv_dtype, shard_lo=lo, pos_dtype=pos_dtype)
        self.rank, self.world, self.window, self.headroom = rank, world, window, headroom

    def resume_at(self, pos: int) -> dict:
        """Resume (or rewind to) position `pos` on this rank: sets the replicated cursor and returns the
        plan of `resume_plan`, plus this rank's own live rows.  Every rank makes the same call."""
        plan = resume_plan(pos, self.world, self.window, self.headroom)
        self.set_pos(pos)
        plan["live_here"] = plan["live"][self.rank]
        return plan


class PartialExchange:
    """Exchange buffers for the per-layer merge of (max, sum, acc) partials of `rows` query rows."""

    def __init__(self, rows: int, d: int, hq: int, group=None, mode: str = "fused", device=None):
        import torch.distributed as dist
        self.rows, self.d, self.hq, self.mode = rows, d, hq, mode
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._local = None
        self._peers = []
        if mode in ("p2p", "fused"):
            lib = L.lib()
            nbytes = lib.trb_p2p_exchange_bytes(self.world, rows, d)
            if nbytes == 0:
                raise ValueError("unsupported exchange geometry")
            local = C.c_void_p()
            handle = C.create_string_buffer(L.IPC_HANDLE_BYTES)
            L.check(lib.trb_p2p_create(nbytes, C.byref(local), handle), "trb_p2p_create")
            self._local = local.value
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
            else:
                handles[0] = bytes(handle.raw)
            ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    ptrs.append(self._local)
                else:
                    peer = C.c_void_p()
                    L.check(lib.trb_p2p_open(handles[r], C.byref(peer)), "trb_p2p_open")
                    self._peers.append(peer.value)
                    ptrs.append(peer.value)
            self.xchg = torch.tensor(ptrs, dtype=torch.int64, device=self.device)     # device array (separate merge kernel)
            self.xchg_host = (C.c_void_p * self.world)(*ptrs)                            # host array (fused tail)
            self.seq = torch.zeros(1, dtype=torch.int32, device=self.device)
            if self.world > 1:
                dist.barrier(group=group)
        elif mode != "nccl":
            raise ValueError("mode must be 'fused', 'p2p' or 'nccl'")

    def merge(self, ml: torch.Tensor, acc: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
        """ml [rows, 2], acc [rows, d] of this rank -> merged attention output [rows, d] bf16
        (identical on every rank)."""
        if out is None:
            out = torch.empty(self.rows, self.d, device=acc.device, dtype=torch.bfloat16)
        if self.mode == "p2p":
            a = L.P2PMergeArgs(self.xchg.data_ptr(), self.world, self.rank, self.seq.data_ptr(), ml.data_ptr(), acc.data_ptr(),
                               self.rows, self.d, self.hq, 0, out.data_ptr(), None, 0, 0)
            L.check(L.lib().trb_p2p_merge(C.byref(a), torch.cuda.current_stream().cuda_stream), "trb_p2p_merge")
            return out
        import torch.distributed as dist
        mls = torch.empty(self.world, self.rows, 2, device=acc.device, dtype=torch.float32)
        accs = torch.empty(self.world, self.rows, self.d, device=acc.device, dtype=torch.float32)
        if self.world > 1:
            dist.all_gather_into_tensor(mls, ml.contiguous(), group=self.group)
            dist.all_gather_into_tensor(accs, acc.contiguous(), group=self.group)
        else:
            mls[0], accs[0] = ml, acc
        res = fused.lse_merge(mls, accs, hq=self.hq)
        if out is not None:
            out.view(self.rows, self.d).copy_(res)
            return out
        return res

    def close(self):
        if self.mode in ("p2p", "fused") and self._local is not None:
            torch.cuda.synchronize()
            lib = L.lib()
            for p in self._peers:
                lib.trb_p2p_close(p)
            lib.trb_p2p_destroy(self._local)
            self._local, self._peers = None, []


def sharded_decode_layer(state: ShardedState, slot: int, q, k_new, v_new, cfg, xchg: PartialExchange, out=None) -> torch.Tensor:
    """One layer of a sharded decode step: append the new rows (only the owner writes), scan
    this shard, exchange and merge.  q [M, HQ*D]; k_new, v_new [HKV, M, D].  Returns [M, HQ*D]."""
    ks = state.k_scale[slot] if state.fp8 else None
    vs = state.v_scale[slot] if state.fp8 else None
    fused.kv_append(k_new, v_new, state.k[slot], state.v[slot], state.pos_t, ks, vs, shard_lo=state.shard_lo)
    if xchg.mode == "fused":
        return fused.attn_decode_fused(q, None, state.k[slot], state.v[slot], state.pos_t, cfg, ks, vs, shard_lo=state.shard_lo,
                                       out=out, p2p=(xchg.xchg_host, xchg.world, xchg.rank))
    ml, acc = fused.attn_decode_fused(q, None, state.k[slot], state.v[slot], state.pos_t, cfg, ks, vs,
                                      shard_lo=state.shard_lo, partial=True)
    res = xchg.merge(ml, acc, out=out)
    return res.view(q.shape[0], -1)
