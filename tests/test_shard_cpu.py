"""Host-side logic of the sequence-sharded decode on CPU ranks (gloo, world_size 2 and 4):
shard ranges, ownership of the appended position, live rows per shard, and the rank-order LSE
merge of per-shard partials gathered with torch.distributed, against the unsharded oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import kv_oracle as O
from tokenrush_b200 import shard

HQ, HKV, D = 24, 4, 256


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _partial(q, kd, vd, lo, hi, pos):
    """(m, l, acc) of the keys [lo, hi) for one query row at position pos, natural-log units."""
    g = HQ // HKV
    m = np.full(HQ, -np.inf, np.float32); l = np.zeros(HQ, np.float32); acc = np.zeros((HQ, D), np.float32)
    hi = min(hi, pos + 1)
    if hi > lo:
        for h in range(HQ):
            s = (kd[h // g, lo:hi] @ q[h]) * np.float32(D ** -0.5)
            m[h] = s.max(); p = np.exp(s - m[h]); l[h] = p.sum(); acc[h] = p @ vd[h // g, lo:hi]
    return m, l, acc


def _worker(rank, world, port, window, L, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        kb, vb = O.seeded_bf16(1, HKV, L + 1, D), O.seeded_bf16(2, HKV, L + 1, D)
        qb = O.seeded_bf16(3, 1, HQ, D)
        lo, hi = shard.shard_range(rank, world, window)
        head = 16 if rank == world - 1 else 0
        st = O.OracleState(1, HKV, hi - lo + head, D)
        n_old = shard.live_rows(rank, world, window, L, head)
        if n_old:
            O.kv_write(st, 0, 0, kb[:, lo:lo + n_old], vb[:, lo:lo + n_old])
        if shard.owner_of(L, world, window) == rank:            # only the owner appends the new row
            O.kv_write(st, 0, L - lo, kb[:, L:], vb[:, L:])
        n_live = shard.live_rows(rank, world, window, L + 1, head)
        kd, vd = st.dequant(0, max(n_live, 1))
        q = O.bf16_bits_to_f32(qb)[0]
        m, l, acc = _partial(q, kd, vd, 0, n_live, L - lo)
        mine = torch.from_numpy(np.concatenate([m[:, None], l[:, None], acc], axis=1))
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        parts = np.stack([t.numpy() for t in gathered], axis=1)                    # [HQ, world, 2 + D]
        merged = O.lse_merge(parts[:, :, 0], parts[:, :, 1], parts[:, :, 2:])
        total = torch.tensor([n_live]); dist.all_reduce(total)
        if rank == 0:
            out_q.put((merged, int(total)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,L", [(2, 700), (2, 1024), (4, 1500), (4, 2047)])
def test_sharded_merge_equals_unsharded(world, L):
    window = 2048
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, window, L, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    merged, total = out_q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert total == L + 1                                        # every live row is held by exactly one rank
    kb, vb = O.seeded_bf16(1, HKV, L + 1, D), O.seeded_bf16(2, HKV, L + 1, D)
    qb = O.seeded_bf16(3, 1, HQ, D)
    st = O.OracleState(1, HKV, window + 16, D)
    O.kv_write(st, 0, 0, kb[:, :L], vb[:, :L])
    want = O.decode_step_cpu(st, 0, qb, kb[:, L:], vb[:, L:], L)
    np.testing.assert_allclose(merged, want[0], rtol=0, atol=3e-6)


def test_shard_partition_helpers():
    assert shard.shard_range(1, 4, 2048) == (512, 1024)
    with pytest.raises(ValueError):
        shard.shard_range(0, 3, 2048)
    assert [shard.owner_of(p, 4, 2048) for p in (0, 511, 512, 2047, 2048, 5000)] == [0, 0, 1, 3, 3, 3]
    for live in (0, 1, 512, 513, 2048, 2060):
        rows = [shard.live_rows(r, 4, 2048, live, headroom=32) for r in range(4)]
        assert sum(rows) == min(live, 2048 + 32) and all(0 <= x for x in rows)


def test_resume_plan_and_ring_validity():
    # owner of the resume position and live rows after a rewind across shard boundaries
    plan = shard.resume_plan(1300, 4, 2048, headroom=32)
    assert plan["owner"] == 2 and plan["live"] == [512, 512, 276, 0]
    assert shard.resume_rows_dropped(2060, 1300, 4, 2048, headroom=32) == [0, 0, 236, 524]
    assert shard.resume_plan(0, 4, 2048)["live"] == [0, 0, 0, 0] and shard.resume_plan(0, 4, 2048)["owner"] == 0
    assert shard.resume_plan(2048, 4, 2048, headroom=8)["owner"] == 3          # past the window: the last rank's headroom
    with pytest.raises(ValueError):
        shard.resume_plan(2100, 4, 2048, headroom=8)
    # the reference's draft geometry: ring 4096 = smallest power of two >= 2048 + 8 + 8, slack 2032
    ring = O.ring_size(2048, 8)
    assert ring == 4096
    assert shard.ring_snapshot_valid(1000, 1000 + 2032, ring, 2048, 8)
    assert not shard.ring_snapshot_valid(1000, 1000 + 2033, ring, 2048, 8)


def _resume_worker(rank, world, port, window, L, P, out_q):
    """Fill to L, decode; rewind to P (across shard boundaries), append other rows, decode again: the
    merged result must equal an unsharded sequence that was rewound the same way."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        kb, vb = O.seeded_bf16(1, HKV, L, D), O.seeded_bf16(2, HKV, L, D)
        k2, v2 = O.seeded_bf16(4, HKV, 1, D), O.seeded_bf16(5, HKV, 1, D)
        qb = O.seeded_bf16(3, 1, HQ, D)
        lo, hi = shard.shard_range(rank, world, window)
        st = O.OracleState(1, HKV, hi - lo, D)
        n_old = shard.live_rows(rank, world, window, L)
        if n_old:
            O.kv_write(st, 0, 0, kb[:, lo:lo + n_old], vb[:, lo:lo + n_old])
        plan = shard.resume_plan(P, world, window)                # every rank computes the same plan
        if plan["owner"] == rank:                                # the owner of P writes the next row over dead data
            O.kv_write(st, 0, P - lo, k2, v2)
        n_live = shard.live_rows(rank, world, window, P + 1)
        assert n_live == plan["live"][rank] + (1 if plan["owner"] == rank else 0)
        m, l, acc = O.partial_rows_over_cache(st, 0, qb, P, n_live, key_offset=lo)
        mine = torch.from_numpy(np.concatenate([m[0][:, None], l[0][:, None], acc[0]], axis=1))
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        if rank == 0:
            parts = np.stack([t.numpy() for t in gathered], axis=1)
            out_q.put(O.lse_merge(parts[:, :, 0], parts[:, :, 1], parts[:, :, 2:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,L,P", [(2, 1900, 700), (4, 2000, 513), (4, 2000, 1024)])
def test_resume_across_shard_boundary(world, L, P):
    window = 2048
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_resume_worker, args=(r, world, port, window, L, P, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    merged = out_q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    kb, vb = O.seeded_bf16(1, HKV, L, D), O.seeded_bf16(2, HKV, L, D)
    st = O.OracleState(1, HKV, window, D)
    O.kv_write(st, 0, 0, kb, vb)                                 # the old sequence, L rows
    want = O.decode_step_cpu(st, 0, O.seeded_bf16(3, 1, HQ, D), O.seeded_bf16(4, HKV, 1, D), O.seeded_bf16(5, HKV, 1, D), P)
    np.testing.assert_allclose(merged, want[0], rtol=0, atol=3e-6)
