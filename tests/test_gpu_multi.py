"""Sequence-sharded decode on 2+ GPUs of one box (one process per GPU): per-GPU partials merged
over NVLink peer memory (and, as the baseline, with an NCCL all-gather) must equal the unsharded
oracle.  Skipped on a single GPU; the same arithmetic is covered there by
test_gpu_decode.py::test_sequence_shards_merge_to_unsharded and on CPU by test_shard_cpu.py."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HQ, HKV, D = 24, 4, 256


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    import tokenrush_b200 as tb
    from tokenrush_b200 import shard
    from oracle import kv_oracle as O
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        window, L, steps = 4096, 3000, 3
        cfg = tb.AttnConfig(n_attn=2)
        kb, vb = O.seeded_bf16(1, HKV, L + steps, D), O.seeded_bf16(2, HKV, L + steps, D)
        qb = O.seeded_bf16(3, steps, HQ, D)
        dev = lambda bits: O.bits_to_torch_bf16(bits).cuda()
        st = shard.ShardedState(cfg, window, rank, world, "cuda", headroom=64)
        lo, hi = shard.shard_range(rank, world, window)
        n_old = shard.live_rows(rank, world, window, L, 64)
        if n_old:
            tb.fused.kv_append(dev(kb[:, lo:lo + n_old]), dev(vb[:, lo:lo + n_old]), st.k[1], st.v[1], lo, st.k_scale[1], st.v_scale[1],
                               shard_lo=st.shard_lo)
        results = {}
        for mode in ("fused", "p2p", "nccl"):
            xchg = shard.PartialExchange(HQ, D, HQ, mode=mode)
            st.set_pos(L)
            outs = []
            for t in range(steps):                             # consecutive calls: sequence numbers, slot reuse
                o = shard.sharded_decode_layer(st, 1, dev(qb[t:t + 1]).reshape(1, -1), dev(kb[:, L + t:L + t + 1]),
                                               dev(vb[:, L + t:L + t + 1]), cfg, xchg)
                outs.append(o.float().cpu().numpy())
                st.advance(1)
            torch.cuda.synchronize()
            results[mode] = np.stack(outs)
            xchg.close()
        status = tb._lib.device_status()
        if rank == 0:
            out_q.put((results, status))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_decode_over_nvlink(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    from oracle import kv_oracle as O
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    results, status = out_q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert status == 0
    L, steps = 3000, 3
    kb, vb = O.seeded_bf16(1, HKV, L + steps, D), O.seeded_bf16(2, HKV, L + steps, D)
    qb = O.seeded_bf16(3, steps, HQ, D)
    ref = O.OracleState(1, HKV, 4096 + 64, D)
    O.kv_write(ref, 0, 0, kb[:, :L], vb[:, :L])
    for t in range(steps):
        want = O.decode_step_cpu(ref, 0, qb[t:t + 1], kb[:, L + t:L + t + 1], vb[:, L + t:L + t + 1], L + t)
        for mode in ("fused", "p2p", "nccl"):
            got = results[mode][t].reshape(1, HQ, D)
            err = np.abs(got - want)
            rel = np.linalg.norm(got - want) / np.linalg.norm(want)
            assert (err <= 2e-3 + 2.0 ** -8 * np.abs(want)).all() and rel <= 1e-2, (mode, t, float(err.max()), float(rel))
    assert np.array_equal(results["p2p"], results["nccl"])      # same merge order, same bits
    assert np.array_equal(results["fused"], results["nccl"])
