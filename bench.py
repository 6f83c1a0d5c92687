#!/usr/bin/env python
"""Benchmark of the full-attention KV-cache decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Metric: effective KV bandwidth of decode attention (GB/s) and the step time behind it.
A step is one decode step of all 16 full-attention layers: per layer, append one new K/V row
(FP8 quantise-on-write) and attend one query token (24 query heads x 256, 4 KV heads) over the
live FP8 cache.  The live length is read from a device integer and advanced on the device, and
the whole step is one captured CUDA graph.  Algorithmic bytes of a step = layers x live rows x
2080 (every live K and V code byte and every fp32 scale once).

Workloads (synthetic: N(0,1) values quantised into the FP8 cache layout, seeded):
    window256k   16 layers x 262144 live rows (8.72 GB of KV): the default; on N > 1 GPUs the
                 window is sharded by sequence in contiguous equal shards, per-GPU partials are
                 merged per layer over NVLink peer memory (strong scaling, fixed total work)
    ctx32k       16 layers x 32768 rows
    ctx4k        16 layers x 4096 rows
    verify64k    M = 8 query rows over 65536 rows (speculative verify)
    prefill8k    chunked prefill: 8192 new tokens over 131072 cached rows, 16 layers (metric:
                 attention TFLOP/s against the dense bf16 peak; the chunk's K/V rows are appended to
                 the FP8 cache in the same step)
Inputs are far larger than L2 (126 MB), so consecutive steps cannot be served from cache.

`--impl reference` times the CPU restatement of the reference's torch path (append + dequantise +
fp32 attention) on the host cores for the same workload, one bounded sample per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HQ, HKV, D, LAYERS = 24, 4, 256, 16
ROW_BYTES = 2 * HKV * D + 2 * HKV * 4            # 2080 B of K+V codes and scales per layer per position
WORKLOADS = {
    "window256k": dict(ctx=262144, m=1),
    "ctx32k": dict(ctx=32768, m=1),
    "ctx4k": dict(ctx=4096, m=1),
    "verify64k": dict(ctx=65536, m=8),
    "prefill8k": dict(ctx=131072, t=8192),
}
# DRAM bytes per live row per layer-launch of the decode kernels (dram__bytes_read.sum +
# dram__bytes_write.sum of one ncu capture, divided by the rows of that launch), by query rows M:
# profiles/decode_kernel_fp8_m1_window256k.md (131072 rows) and profiles/decode_tc_kernel_m8_verify64k.md (65536 rows)
NCU_TRAFFIC_BYTES_PER_ROW = {1: 2109, 8: 2158}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            parts = [x.strip() for x in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0])); mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def fill_cache_(state, seed: int):
    """Fill the whole cache with what the append kernel produces for N(0,1) rows, without holding a
    bf16 copy of 262144 x 16 layers: quantise chunk by chunk through the product's own append."""
    import tokenrush_b200 as tb
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_layers, hkv, max_len, d = state.k.shape
    chunk = 16384
    for slot in range(n_layers):
        for p0 in range(0, max_len, chunk):
            t = min(chunk, max_len - p0)
            k = torch.randn(hkv, t, d, device="cuda", generator=g).to(torch.bfloat16)
            v = torch.randn(hkv, t, d, device="cuda", generator=g).to(torch.bfloat16)
            tb.fused.kv_append(k, v, state.k[slot], state.v[slot], state.shard_lo + p0 if state.shard_lo is not None else p0,
                               state.k_scale[slot], state.v_scale[slot], shard_lo=state.shard_lo)
    torch.cuda.synchronize()


def run_product(args):
    import torch.distributed as dist
    import tokenrush_b200 as tb
    from tokenrush_b200 import shard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    wl = WORKLOADS[args.workload]
    ctx, m = wl["ctx"], wl["m"]
    steps, warmup = args.steps, max(args.warmup, 3)
    headroom = m * (steps + warmup + 8) * 3 + 64
    cfg = tb.AttnConfig(n_attn=LAYERS)
    f8 = torch.float8_e4m3fn

    if world > 1:
        state = shard.ShardedState(cfg, ctx, rank, world, "cuda", kv_dtype=f8, headroom=headroom)
        xchg = shard.PartialExchange(m * HQ, D, HQ, mode=args.exchange)
    else:
        state = tb.State(cfg, ctx + headroom, "cuda", kv_dtype=f8)
        xchg = None
    fill_cache_(state, seed=rank)
    pos0 = ctx - m                                            # live length of the first step = ctx
    state.set_pos(pos0)

    # pinned host inputs of one step and the device buffers the graph reads
    gen = torch.Generator().manual_seed(0)
    h_q = torch.randn(LAYERS, m, HQ * D, generator=gen).to(torch.bfloat16).pin_memory()
    h_k = torch.randn(LAYERS, HKV, m, D, generator=gen).to(torch.bfloat16).pin_memory()
    h_v = torch.randn(LAYERS, HKV, m, D, generator=gen).to(torch.bfloat16).pin_memory()
    h_out = torch.empty(LAYERS, m, HQ * D, dtype=torch.bfloat16).pin_memory()
    d_q, d_k, d_v = h_q.cuda(), h_k.cuda(), h_v.cuda()
    d_out = torch.zeros(LAYERS, m, HQ * D, device="cuda", dtype=torch.bfloat16)
    launches_per_step = 0
    # M-row verify: after the step, c ~ U{1..M} of the rows are committed on the device (drafts
    # accepted up to the first mismatch); the rejected rows stay as dead data and the next step's
    # append overwrites them.  The draft / prediction tokens of step s come from a seeded table that
    # the captured graph indexes with a device counter.
    TAB = 64
    commit = torch.randint(1, m + 1, (TAB,), generator=torch.Generator().manual_seed(0)).tolist() if m > 1 else [1] * TAB
    if m > 1:
        drafts_tab = torch.arange(TAB * (m - 1), dtype=torch.int64).reshape(TAB, m - 1) % 1000
        pred_tab = torch.cat([drafts_tab, torch.full((TAB, 1), 7, dtype=torch.int64)], 1)
        for s_, c_ in enumerate(commit):
            if c_ - 1 < m - 1:
                pred_tab[s_, c_ - 1] = drafts_tab[s_, c_ - 1] + 1     # first mismatch after c - 1 accepted drafts
        drafts_tab, pred_tab = drafts_tab.cuda(), pred_tab.cuda()
        d_counter = torch.zeros(1, dtype=torch.int64, device="cuda")
        d_idx = torch.zeros(1, dtype=torch.int64, device="cuda")
        d_drafts = torch.zeros(1, m - 1, dtype=torch.int64, device="cuda")
        d_pred = torch.zeros(1, m, dtype=torch.int64, device="cuda")
        d_nacc = torch.zeros(1, dtype=torch.int64, device="cuda")
        d_tok = torch.zeros(1, dtype=torch.int64, device="cuda")
    replays = 0                                               # graph replays since the cursor was set: indexes `commit`

    def live_after(n_replays):
        """Sum of the live lengths of the next n_replays steps, advancing the host's copy of the schedule."""
        nonlocal replays, pos_host
        total = 0
        for _ in range(n_replays):
            total += pos_host + m
            pos_host += commit[replays % TAB] if m > 1 else m
            replays += 1
        return total
    pos_host = pos0

    def step_body(count=False):
        nonlocal launches_per_step
        n = 0
        for l in range(LAYERS):
            if world > 1:
                shard.sharded_decode_layer(state, l, d_q[l], d_k[l], d_v[l], cfg, xchg, out=d_out[l])
                n += 2 if args.exchange == "fused" else 3      # append, shard scan (+ exchange and merge in its tail, or as a third launch)
            else:
                tb.fused.kv_write_prefill(d_k[l], d_v[l], state, l, state.pos_t)
                tb.fused.attn_decode_fused(d_q[l], None, state.k[l], state.v[l], state.pos_t, cfg, state.k_scale[l], state.v_scale[l],
                                           out=d_out[l])
                n += 2                                        # append, decode (combine fused in its tail)
        if m > 1:
            torch.remainder(d_counter, TAB, out=d_idx)
            torch.index_select(drafts_tab, 0, d_idx, out=d_drafts)
            torch.index_select(pred_tab, 0, d_idx, out=d_pred)
            tb.fused.spec_commit(d_pred[0], d_drafts[0], d_nacc, d_tok, state.pos_t)
            d_counter.add_(1)
        else:
            tb.fused.cursor_advance(state.pos_t, m)
        n += 1
        if count:
            launches_per_step = n

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step_body(count=True)                                 # builds workspaces outside capture
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    state.set_pos(pos0)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step_body()
    state.set_pos(pos0)
    if m > 1:
        d_counter.zero_()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms

    # ---- device-resident number: K graph replays, inputs already in HBM ---------------------
    for _ in range(warmup):
        graph.replay()
    live_after(warmup)
    with ClockSampler(local_rank) as clocks:
        ms = timed(graph.replay, steps)
    bytes_total = LAYERS * ROW_BYTES * live_after(steps)
    value = bytes_total / (ms * 1e-3) / 1e9

    # ---- end to end: pinned host inputs in, outputs back, every step ------------------------
    def e2e_step():
        d_q.copy_(h_q, non_blocking=True); d_k.copy_(h_k, non_blocking=True); d_v.copy_(h_v, non_blocking=True)
        graph.replay()
        h_out.copy_(d_out, non_blocking=True)
        torch.cuda.current_stream().synchronize()             # the caller reads the step's result
    e2e_steps = max(10, steps // 4)
    ms_e2e = timed(e2e_step, e2e_steps)
    e2e_bytes = LAYERS * ROW_BYTES * live_after(e2e_steps)
    e2e_value = e2e_bytes / (ms_e2e * 1e-3) / 1e9
    h2d = (h_q.numel() + h_k.numel() + h_v.numel()) * 2
    d2h = h_out.numel() * 2

    # ---- the dominant kernel alone: decode launches of all layers, CUDA events on their stream
    roofline = None
    cpu_baseline = None
    if world == 1:
        def decode_only():
            for l in range(LAYERS):
                tb.fused.attn_decode_fused(d_q[l], None, state.k[l], state.v[l], state.pos_t, cfg, state.k_scale[l], state.v_scale[l])
        with torch.cuda.stream(side):
            decode_only()
        torch.cuda.synchronize()
        kgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(kgraph, stream=side):
            decode_only()
        for _ in range(3):
            kgraph.replay()
        reps = max(10, steps // 4)
        ms_k = timed(kgraph.replay, reps)
        live_now = int(state.pos_t.item()) + m
        us_launch = ms_k * 1e3 / (reps * LAYERS)
        achieved = live_now * ROW_BYTES / (us_launch * 1e-6) / 1e9
        peaks, how = measured_peaks()
        roofline = {"bound": "hbm", "kernel": "decode_kernel<256, fp8>" if m == 1 else "decode_tc_kernel (tcgen05)", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                    "peak_source": how, "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                    "us_per_launch": round(us_launch, 2), "algorithmic_bytes_per_launch": live_now * ROW_BYTES,
                    "traffic": (NCU_TRAFFIC_BYTES_PER_ROW[m] * live_now) if m in NCU_TRAFFIC_BYTES_PER_ROW else None}
        cpu_baseline = run_cpu_sample(ctx, m, budget_s=args.cpu_seconds)

    status = tb._lib.device_status()
    if rank == 0:
        line = {
            "metric": "decode_attn_effective_kv_bandwidth", "value": round(value, 1), "unit": "GB/s",
            "us_per_step": round(ms * 1e3 / steps, 2), "ms_per_step": round(ms / steps, 5),
            "n_gpus": world, "steps": steps, "warmup": warmup, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 cache, f16 MMA, fp32 softmax/accumulate" if m == 1 else "fp8_e4m3 cache and operands (q, p as hi+lo pairs), fp32 accumulate in TMEM",
            "data": "synthetic",
            "config": {"workload": args.workload, "layers": LAYERS, "context_rows": ctx, "query_rows": m,
                       "heads": f"{HQ}q/{HKV}kv x {D}", "kv_bytes_per_step": round(bytes_total / steps),
                       "commit": "all rows" if m == 1 else f"c ~ U{{1..{m}}} per step, seeded, on the device (trb_spec_commit)",
                       "cuda_graph": True, "cursor": "device int64", "l2": "inputs larger than L2 (no flush needed)",
                       "sharding": f"sequence x{world}" if world > 1 else "none",
                       "exchange": args.exchange if world > 1 else None},
            "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "us_per_step": round(ms_e2e * 1e3 / e2e_steps, 2),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * steps,
            "clocks": clocks.summary(),
            "roofline": roofline, "cpu_baseline": cpu_baseline,
            "device_status": status,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing NCCL down: destroying a communicator whose collectives were captured
        # into a still-live CUDA graph can block forever.  Everything is flushed and every rank has
        # finished its timed work before the processes exit.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def prefill_flops(t: int, pos: int) -> float:
    """2 GEMMs x 2 flop/MAC over the causal region, all query heads, one layer."""
    return 4.0 * HQ * D * (t * pos + t * (t + 1) / 2)


def run_prefill(args):
    """Chunked prefill (BASELINE config 4): per layer, append the chunk's K/V rows to the FP8 cache
    and attend the chunk's queries causally over cache + chunk.  Single GPU."""
    import tokenrush_b200 as tb
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if int(os.environ.get("RANK", "0")) != 0:
        return
    wl = WORKLOADS[args.workload]
    pos, t = wl["ctx"], wl["t"]
    steps, warmup = max(1, min(args.steps, 10)), max(1, min(args.warmup, 3))
    cfg = tb.AttnConfig(n_attn=LAYERS)
    state = tb.State(cfg, pos + t + 64, "cuda", kv_dtype=torch.float8_e4m3fn)
    fill_cache_(state, seed=0)
    gen = torch.Generator().manual_seed(0)
    h_q = torch.randn(t, HQ, D, generator=gen).to(torch.bfloat16).pin_memory()
    h_k = torch.randn(HKV, t, D, generator=gen).to(torch.bfloat16).pin_memory()
    h_v = torch.randn(HKV, t, D, generator=gen).to(torch.bfloat16).pin_memory()
    h_out = torch.empty(t, HQ, D, dtype=torch.bfloat16).pin_memory()
    d_q, d_k, d_v = h_q.cuda(), h_k.cuda(), h_v.cuda()
    outs = [None] * LAYERS

    def step():
        for l in range(LAYERS):
            tb.fused.kv_write_prefill(d_k, d_v, state, l, pos)
            outs[l] = tb.fused.attn_prefill_fused(d_q, state.k[l], state.v[l], pos, cfg, state.k_scale[l], state.v_scale[l])

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    for _ in range(warmup):
        step()
    with ClockSampler(torch.cuda.current_device()) as clocks:
        ms = timed(step, steps)
    flops = LAYERS * prefill_flops(t, pos)
    value = flops * steps / (ms * 1e-3) / 1e12

    def e2e_step():
        for l in range(LAYERS):                                  # every layer's chunk comes from the host
            d_q.copy_(h_q, non_blocking=True); d_k.copy_(h_k, non_blocking=True); d_v.copy_(h_v, non_blocking=True)
            tb.fused.kv_write_prefill(d_k, d_v, state, l, pos)
            o = tb.fused.attn_prefill_fused(d_q, state.k[l], state.v[l], pos, cfg, state.k_scale[l], state.v_scale[l])
            h_out.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_steps = max(1, steps // 2)
    ms_e2e = timed(e2e_step, e2e_steps)
    e2e_value = flops * e2e_steps / (ms_e2e * 1e-3) / 1e12

    def attn_only():
        for l in range(LAYERS):
            tb.fused.attn_prefill_fused(d_q, state.k[l], state.v[l], pos, cfg, state.k_scale[l], state.v_scale[l])
    ms_k = timed(attn_only, 1)
    peaks, how = measured_peaks()
    peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    achieved = flops / (ms_k * 1e-3) / 1e12
    # CPU sample: the oracle port on 32 query rows of one layer
    import numpy as np
    from oracle import kv_oracle as O
    rows = np.linspace(0, t - 1, 32).astype(np.int64)
    rng = np.random.default_rng(0)
    kd = rng.standard_normal((HKV, pos + t, D), dtype=np.float32); vd = rng.standard_normal((HKV, pos + t, D), dtype=np.float32)
    qf = rng.standard_normal((t, HQ, D), dtype=np.float32)
    t0 = time.perf_counter()
    O.attn_prefill(qf, kd, vd, pos, rows=rows)
    dt = time.perf_counter() - t0
    cpu_flops = float(sum(4.0 * HQ * D * (pos + r + 1) for r in rows))
    line = {
        "metric": "prefill_attn_tflops", "value": round(value, 1), "unit": "TFLOP/s", "ms_per_step": round(ms / steps, 3),
        "n_gpus": 1, "steps": steps, "warmup": warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3 operands (q and p as hi+lo pairs), fp32 accumulate in TMEM", "data": "synthetic",
        "config": {"workload": args.workload, "layers": LAYERS, "cached_rows": pos, "new_tokens": t, "heads": f"{HQ}q/{HKV}kv x {D}",
                   "flop_per_step": flops, "l2": "inputs larger than L2 (no flush needed)"},
        "e2e": {"value": round(e2e_value, 1), "unit": "TFLOP/s", "ms_per_step": round(ms_e2e / e2e_steps, 3),
                "h2d_bytes_per_step": LAYERS * (h_q.numel() + h_k.numel() + h_v.numel()) * 2, "d2h_bytes_per_step": LAYERS * h_out.numel() * 2},
        "gpu_launches": 2 * LAYERS * steps,
        "clocks": clocks.summary(),
        "roofline": {"bound": "tensor", "kernel": "prefill_kernel", "achieved": round(achieved, 1), "peak": peak, "peak_source": how,
                     "unit": "TFLOP/s", "frac": round(achieved / peak, 4), "traffic": None,
                     "note": "algorithmic flops (each product counted once); the kernel issues two e4m3 MMAs per product at the FP8 rate"},
        "cpu_baseline": {"value": round(cpu_flops / dt / 1e12, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"32 query rows of one layer over {pos + t} keys ({dt:.2f} s)"},
        "device_status": tb._lib.device_status(),
    }
    print(json.dumps(line), flush=True)


def run_cpu_sample(ctx: int, m: int, budget_s: float = 15.0):
    """The oracle (a CPU port of the reference's torch path: append + dequantise + fp32 attention)
    on all host cores (torch's intra-op threads): layer-steps at the full context until the time
    budget is spent."""
    import numpy as np
    from oracle import kv_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(0)
    st = O.OracleState(1, HKV, ctx + m, D)
    # random codes and scales with the distribution of quantised N(0,1) rows (filling through the
    # oracle's own quantiser would take minutes at this size)
    st.k[:] = rng.integers(0, 0x7F, st.k.shape, dtype=np.uint8) | (rng.integers(0, 2, st.k.shape, dtype=np.uint8) << 7)
    st.v[:] = rng.integers(0, 0x7F, st.v.shape, dtype=np.uint8) | (rng.integers(0, 2, st.v.shape, dtype=np.uint8) << 7)
    st.k_scale[:] = rng.uniform(0.006, 0.011, st.k_scale.shape).astype(np.float32)
    st.v_scale[:] = rng.uniform(0.006, 0.011, st.v_scale.shape).astype(np.float32)
    qb = O.seeded_bf16(1, m, HQ, D)
    kb, vb = O.seeded_bf16(2, HKV, m, D), O.seeded_bf16(3, HKV, m, D)
    times, busy = [], []
    t_end = time.perf_counter() + budget_s
    while True:
        t0, c0 = time.perf_counter(), time.process_time()
        O.decode_step_cpu_threaded(st, 0, qb, kb, vb, ctx - m)
        times.append(time.perf_counter() - t0)
        busy.append((time.process_time() - c0) / max(times[-1], 1e-9))
        if time.perf_counter() > t_end or len(times) >= 16:
            break
    best = min(times)
    return {"value": round(ctx * ROW_BYTES / best / 1e9, 4), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "cores_busy_avg": round(sum(busy) / len(busy), 1), "seconds_per_layer_step": round(best, 4),
            "sample": f"{len(times)} layer-steps of 1 layer x {ctx} rows, M={m} (best of {len(times)}); a step of the workload is 16 such layer-steps"}


def run_reference(args):
    """The reference arm: its CPU path (restated in oracle/, parity-pinned to the reference's own
    torch functions) on the host cores.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    wl = WORKLOADS[args.workload]
    if "t" in wl:
        print(json.dumps({"impl": "reference", "unavailable": "the reference arm covers the decode workloads; the prefill CPU sample is in the product line's cpu_baseline"}), flush=True)
        return
    steps = max(1, min(args.steps, 8))
    base = run_cpu_sample(wl["ctx"], wl["m"], budget_s=min(60.0, 4.0 * steps))
    sec_step = base["seconds_per_layer_step"] * LAYERS
    value = LAYERS * wl["ctx"] * ROW_BYTES / sec_step / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_effective_kv_bandwidth", "value": round(value, 4), "unit": "GB/s",
        "us_per_step": round(sec_step * 1e6, 1), "ms_per_step": round(sec_step * 1e3, 3), "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32 math over the fp8 cache (CPU)", "data": "synthetic",
        "config": {"workload": args.workload, "layers": LAYERS, "context_rows": wl["ctx"], "query_rows": wl["m"],
                   "heads": f"{HQ}q/{HKV}kv x {D}"},
        "cpu_baseline": dict(base, value=round(value, 4)),
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="product", choices=["product", "reference"])
    ap.add_argument("--workload", default="window256k", choices=sorted(WORKLOADS))
    ap.add_argument("--exchange", default="fused", choices=["fused", "p2p", "nccl"])
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif "t" in WORKLOADS[args.workload]:
        run_prefill(args)
    else:
        run_product(args)


if __name__ == "__main__":
    main()
