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
