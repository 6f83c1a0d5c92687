#!/usr/bin/env python
"""Benchmark of the full-attention KV-cache decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Metric: effective KV bandwidth of decode attention (GB/s) and the step time behind it.
A step is one decode step of all 16 full-attention layers: per layer, append the new K/V rows
(FP8 quantise-on-write) and attend the query rows (24 query heads x 256, 4 KV heads) over the
live FP8 cache.  The live length is read from a device integer and advanced on the device, and
the whole step is one captured CUDA graph.  Algorithmic bytes of a step = layers x live rows x
2080 (every live K and V code byte and every fp32 scale once).

Workloads (synthetic: N(0,1) values quantised into the FP8 cache layout, seeded):
    window256k   16 layers x 262144 live rows (8.72 GB of KV): the default; on N > 1 GPUs the
                 window is sharded by sequence in contiguous equal shards, per-GPU partials are
                 merged per layer over NVLink peer memory (strong scaling, fixed total work)
    ctx32k       16 layers x 32768 rows
    ctx4k        16 layers x 4096 rows
    verify64k    M = 8 query rows over 65536 rows (speculative verify, commit on the device)
    prefill8k    chunked prefill: 8192 new tokens over 131072 cached rows, 16 layers (metric:
                 attention TFLOP/s against the dense bf16 peak; the chunk's K/V rows are appended to
                 the FP8 cache in the same step)
    profile-decode / profile-prefill
                 small, self-ending cases of one kernel for a profiler (--rows, --m, --t)
    timeline     per-phase time stamps of the M = 1 decode kernel's CTAs (needs the diagnostic
                 library: python -m tokenrush_b200.build --timeline), --rows live rows, 16 layers
    timeline-prefill   clock stamps of the prefill kernel's softmax and MMA warps over 32 key tiles of one
                 query block (same library), --rows cached rows, --t new tokens, --kv fp8|bf16
Inputs are far larger than L2 (126 MB), so consecutive steps cannot be served from cache.

The default single-GPU run reports window256k as the headline and attaches short runs of ctx32k,
verify64k and prefill8k under `workloads`.  Every line carries a `parity` object: one extra step,
outside the timed region, whose outputs are compared with the CPU oracle (fp32 attention over the
device's own cache bytes; appended rows bit for bit); on N > 1 GPUs every rank evaluates the
oracle partial of its own shard and rank 0 merges them.

`--impl reference` times the reference's own CPU path (its torch functions from an installed copy
of the reference when one is found, else the restatement in oracle/) on the host cores, one
layer of the workload per step, and - when a GPU and the reference's Triton kernels are available
- those kernels on the same GPU as an extra record.
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
    "profile-decode": dict(profile="decode"),
    "profile-prefill": dict(profile="prefill"),
    "timeline-prefill": dict(profile="prefill-timeline"),
    "timeline": dict(profile="timeline"),
}
# DRAM bytes moved per live row by one launch of the decode kernels (dram__bytes_read.sum +
# dram__bytes_write.sum of one ncu capture divided by the rows of that launch; the traffic is
# proportional to the rows streamed), by query rows M: a 131072-row launch of decode_kernel (M = 1)
# and a 65536-row launch of decode_tc_kernel (M = 8).
NCU_TRAFFIC_BYTES_PER_ROW = {1: 2111, 8: 2163}
PARITY_BAR = "rel <= 1e-2 and |err| <= 2e-3 + 2^-8 |o| (bf16 output)"


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML queries from a thread
    every 20 ms (read-only), or `nvidia-smi -lms 100` where the NVML binding is missing."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc, self.nvml, self.stop = index, [], None, None, threading.Event()

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def __enter__(self):
        try:
            self.nvml = self._nvml_handle()
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _poll(self):
        nv, h = self.nvml
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        while True:
            try:
                mhz, mx = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
                r = int(get_reasons(h))
                self.samples.append(",".join([str(mhz), str(mx)] + ["Active" if r & bits[n] else "Not Active" for n in self.NAMES]))
            except Exception:
                pass
            if self.stop.wait(0.02):
                return

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def __exit__(self, *exc):
        self.stop.set()
        if self.nvml is not None:
            self.thread.join(timeout=1)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        for s in self.samples:
            parts = [x.strip() for x in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0])); mx = max(mx, float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(self.NAMES, parts[2:6]):
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
                               state.k_scale[slot] if state.fp8 else None, state.v_scale[slot] if state.fp8 else None, shard_lo=state.shard_lo)
    torch.cuda.synchronize()


def random_fill_(state):
    """Random e4m3 codes and plausible scales (no quantisation pass, so few launches precede the
    kernel of interest in a profile)."""
    for t in (state.k, state.v):
        codes = torch.randint(0, 0x7E, t.shape, device="cuda", dtype=torch.uint8)
        sign = torch.randint(0, 2, t.shape, device="cuda", dtype=torch.uint8) << 7
        t.view(torch.uint8).copy_(codes | sign)
    state.k_scale.uniform_(0.006, 0.011)
    state.v_scale.uniform_(0.006, 0.011)


# ------------------------------------------------------------------------------ parity helpers

def _oracle_layer(state, slot: int, heads, n_rows: int):
    """One layer of a CUDA State as an OracleState holding rows [0, n_rows) of the kv heads listed
    (the other heads stay zero: they are not evaluated)."""
    from oracle import kv_oracle as O
    st = O.OracleState(1, HKV, max(n_rows, 1), D, fp8=state.fp8)
    for j in heads:
        if not state.fp8:
            st.k[0, j] = state.k[slot, j, :n_rows].view(torch.int16).cpu().numpy().view("uint16")
            st.v[0, j] = state.v[slot, j, :n_rows].view(torch.int16).cpu().numpy().view("uint16")
            continue
        st.k[0, j] = state.k[slot, j, :n_rows].view(torch.uint8).cpu().numpy()
        st.v[0, j] = state.v[slot, j, :n_rows].view(torch.uint8).cpu().numpy()
        st.k_scale[0, j] = state.k_scale[slot, j, :n_rows].cpu().numpy()
        st.v_scale[0, j] = state.v_scale[slot, j, :n_rows].cpu().numpy()
    return st


def _bits(t):
    from oracle import kv_oracle as O
    return O.torch_bf16_to_bits(t.detach().cpu())


def _compare(got, want):
    import numpy as np
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    tol = 2e-3 + 2.0 ** -8 * np.abs(want.astype(np.float64))
    rel = float(np.linalg.norm(got.astype(np.float64) - want) / max(float(np.linalg.norm(want)), 1e-30))
    return bool((err <= tol).all() and rel <= 1e-2 and np.isfinite(got).all()), float(err.max()), rel


def decode_parity(state, d_q, d_k, d_v, d_out, pos: int, m: int, world: int, rank: int, layers=(0, LAYERS - 1), heads=(0, HKV - 1)):
    """After one step at cursor `pos` (rows pos..pos+m-1 appended, d_out written): the appended rows bit
    for bit against the oracle's quantiser, and the outputs of the query heads of `heads` against fp32
    oracle attention over the device's cache bytes.  Sharded: each rank evaluates its shard's partial,
    rank 0 merges them in rank order (the merge formula of the reference's reduce kernel)."""
    import numpy as np
    import torch.distributed as dist
    from oracle import kv_oracle as O
    lo = state.shard_lo or 0
    rows_here = state.k.shape[2]
    n_live = max(0, min(pos + m - lo, rows_here))
    g = HQ // HKV
    exact = True
    parts = {}
    for l in layers:
        # appended rows held by this rank
        for i in range(m):
            r = pos + i - lo
            if 0 <= r < rows_here:
                for src, cache, scale in ((d_k, state.k, state.k_scale), (d_v, state.v, state.v_scale)):
                    codes, sc = O.quantize_rows(O.bf16_bits_to_f32(_bits(src[l][:, i])))
                    exact &= bool(np.array_equal(cache[l, :, r].view(torch.uint8).cpu().numpy(), codes))
                    exact &= bool(np.array_equal(scale[l, :, r].cpu().numpy().view(np.uint32), sc.view(np.uint32)))
        ref = _oracle_layer(state, l, heads, n_live)
        qb = _bits(d_q[l]).reshape(m, HQ, D)
        parts[l] = O.partial_rows_over_cache(ref, 0, qb, pos, n_live, kv_heads=heads, key_offset=lo)
    gathered = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, (parts, exact, {l: _bits(d_out[l]) for l in layers}))
    else:
        gathered[0] = (parts, exact, None)
    if rank != 0:
        return None
    ok, max_abs, max_rel, identical = True, 0.0, 0.0, True
    hq_sel = [j * g + x for j in heads for x in range(g)]
    for l in layers:
        ms = np.stack([gathered[r][0][l][0] for r in range(world)], -1).reshape(m * HQ, world)
        ls = np.stack([gathered[r][0][l][1] for r in range(world)], -1).reshape(m * HQ, world)
        accs = np.stack([gathered[r][0][l][2] for r in range(world)], -2).reshape(m * HQ, world, D)
        sel = np.array([i * HQ + h for i in range(m) for h in hq_sel])
        want = O.lse_merge(ms[sel], ls[sel], accs[sel])
        got = d_out[l].float().cpu().numpy().reshape(m * HQ, D)[sel]
        o, a, r_ = _compare(got, want)
        ok &= o; max_abs = max(max_abs, a); max_rel = max(max_rel, r_)
        if world > 1:
            identical &= all(np.array_equal(gathered[r][2][l], gathered[0][2][l]) for r in range(1, world))
    exact_all = all(gathered[r][1] for r in range(world))
    return {"ok": bool(ok and exact_all and identical), "layers": list(layers), "kv_heads": list(heads), "max_abs_err": max_abs, "rel_err": max_rel,
            "appended_rows_bit_exact": bool(exact_all), "outputs_identical_on_all_ranks": bool(identical), "bar": PARITY_BAR,
            "against": "fp32 oracle attention over the device's cache bytes, at the benchmarked size"}


# ------------------------------------------------------------------------------ decode workloads

def run_decode(name: str, args, steps: int, warmup: int, blocks: int, cpu_seconds: float):
    import torch.distributed as dist
    import tokenrush_b200 as tb
    from tokenrush_b200 import shard

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = WORKLOADS[name]
    ctx, m = wl["ctx"], wl["m"]
    warmup = max(warmup, 3)
    e2e_steps = max(10, steps // 4)
    n_replays = warmup + blocks * steps + e2e_steps + 64
    headroom = m * n_replays + 64
    cfg = tb.AttnConfig(n_attn=LAYERS)
    f8 = torch.float8_e4m3fn
    tb.fused.set_launch_mode(args.launch_mode)

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
    pos_host = pos0

    def live_after(n):
        """Sum of the live lengths of the next n steps, advancing the host's copy of the schedule."""
        nonlocal replays, pos_host
        total = 0
        for _ in range(n):
            total += pos_host + m
            pos_host += commit[replays % TAB] if m > 1 else m
            replays += 1
        return total

    def step_body(count=False):
        nonlocal launches_per_step
        n = 0
        lib_before = tb._lib.lib().trb_launch_count()
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
            # the library's own count of what this step launched (a decode call may be two kernels: the scan
            # and the merge of its rows); n, the number of calls, is the floor
            launches_per_step = max(n, int(tb._lib.lib().trb_launch_count() - lib_before))

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

    # ---- device-resident number: blocks of K graph replays, inputs already in HBM ------------
    for _ in range(warmup):
        graph.replay()
    live_after(warmup)
    block_ms, block_gbs = [], []
    with ClockSampler(local_rank) as clocks:
        for _ in range(blocks):
            ms_b = timed(graph.replay, steps)
            bytes_b = LAYERS * ROW_BYTES * live_after(steps)
            block_ms.append(ms_b)
            block_gbs.append(bytes_b / (ms_b * 1e-3) / 1e9)
    order = sorted(range(blocks), key=lambda i: block_ms[i])
    mid = order[len(order) // 2]                              # the median block is the one reported
    ms, value = block_ms[mid], block_gbs[mid]
    bytes_per_step = value * 1e9 * ms * 1e-3 / steps

    # ---- end to end: pinned host inputs in, outputs back, every step ------------------------
    def e2e_step():
        d_q.copy_(h_q, non_blocking=True); d_k.copy_(h_k, non_blocking=True); d_v.copy_(h_v, non_blocking=True)
        graph.replay()
        h_out.copy_(d_out, non_blocking=True)
        torch.cuda.current_stream().synchronize()             # the caller reads the step's result
    ms_e2e = timed(e2e_step, e2e_steps)
    e2e_bytes = LAYERS * ROW_BYTES * live_after(e2e_steps)
    e2e_value = e2e_bytes / (ms_e2e * 1e-3) / 1e9
    h2d = (h_q.numel() + h_k.numel() + h_v.numel()) * 2
    d2h = h_out.numel() * 2

    # ---- parity of one more step, outside the timed region -----------------------------------
    torch.cuda.synchronize()
    pos_p = int(state.pos_t.item())
    graph.replay()
    live_after(1)
    torch.cuda.synchronize()
    parity = decode_parity(state, d_q, d_k, d_v, d_out, pos_p, m, world, rank)

    # ---- the dominant kernel alone: decode launches of all layers, CUDA events on their stream
    roofline = None
    cpu_baseline = None
    if world == 1:
        def decode_only():
            for l in range(LAYERS):
                tb.fused.attn_decode_fused(d_q[l], None, state.k[l], state.v[l], state.pos_t, cfg, state.k_scale[l], state.v_scale[l],
                                           out=d_out[l])
        with torch.cuda.stream(side):
            decode_only()
        torch.cuda.synchronize()
        kgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(kgraph, stream=side):
            decode_only()
        for _ in range(3):
            kgraph.replay()
        reps = max(10, steps // 4)
        ms_k = statistics.median(timed(kgraph.replay, reps) for _ in range(3))
        live_now = int(state.pos_t.item()) + m
        us_launch = ms_k * 1e3 / (reps * LAYERS)
        achieved = live_now * ROW_BYTES / (us_launch * 1e-6) / 1e9
        peaks, how = measured_peaks()
        roofline = {"bound": "hbm", "kernel": "decode_kernel<256, fp8>" if m == 1 else "decode_tc_kernel (tcgen05)", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"],
                    "peak_source": how, "unit": "GB/s", "frac": round(achieved / peaks["hbm_gbs"], 4),
                    "us_per_launch": round(us_launch, 2), "algorithmic_bytes_per_launch": live_now * ROW_BYTES,
                    "traffic": (NCU_TRAFFIC_BYTES_PER_ROW[m] * live_now) if m in NCU_TRAFFIC_BYTES_PER_ROW else None,
                    "how": "CUDA events around a graph of the 16 decode launches alone, median of 3"}
        if cpu_seconds > 0:
            cpu_baseline = run_cpu_sample(ctx, m, budget_s=cpu_seconds)

    status = tb._lib.device_status()
    if world > 1:
        t = torch.tensor([status], device="cuda", dtype=torch.int64)
        gl = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(gl, t)
        status = 0
        for x in gl:
            status |= int(x.item())
    line = None
    if rank == 0:
        line = {
            "metric": "decode_attn_effective_kv_bandwidth", "value": round(value, 1), "unit": "GB/s",
            "us_per_step": round(ms * 1e3 / steps, 2), "ms_per_step": round(ms / steps, 5),
            "n_gpus": world, "steps": steps, "warmup": warmup, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 cache, f16 MMA, fp32 softmax/accumulate" if m == 1 else "fp8_e4m3 cache and operands (q, p as hi+lo pairs), fp32 accumulate in TMEM",
            "data": "synthetic",
            "blocks": {"n": blocks, "steps_each": steps, "us_per_step": [round(x * 1e3 / steps, 2) for x in block_ms],
                       "value": [round(x, 1) for x in block_gbs], "reported": "median block"},
            "config": {"workload": name, "layers": LAYERS, "context_rows": ctx, "query_rows": m,
                       "heads": f"{HQ}q/{HKV}kv x {D}", "kv_bytes_per_step": round(bytes_per_step),
                       "commit": "all rows" if m == 1 else f"c ~ U{{1..{m}}} per step, seeded, on the device (trb_spec_commit)",
                       "cuda_graph": True, "cursor": "device int64", "l2": "inputs larger than L2 (no flush needed)",
                       "programmatic_launch": {0: "off", 1: "on", 2: "chained"}[args.launch_mode],
                       "sharding": f"sequence x{world}" if world > 1 else "none",
                       "exchange": args.exchange if world > 1 else None},
            "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "us_per_step": round(ms_e2e * 1e3 / e2e_steps, 2),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * steps,
            "clocks": clocks.summary(),
            "roofline": roofline, "cpu_baseline": cpu_baseline,
            "parity": parity,
            "device_status": status,
        }
    del graph
    if xchg is not None and world == 1:
        xchg.close()
    return line


def prefill_flops(t: int, pos: int) -> float:
    """2 GEMMs x 2 flop/MAC over the causal region, all query heads, one layer."""
    return 4.0 * HQ * D * (t * pos + t * (t + 1) / 2)


def run_prefill(name: str, args, steps: int, warmup: int):
    """Chunked prefill: per layer, append the chunk's K/V rows to the FP8 cache and attend the chunk's
    queries causally over cache + chunk.  Single GPU."""
    import numpy as np
    import tokenrush_b200 as tb
    from oracle import kv_oracle as O
    wl = WORKLOADS[name]
    pos, t = wl["ctx"], wl["t"]
    steps, warmup = max(1, min(steps, 10)), max(1, min(warmup, 3))
    cfg = tb.AttnConfig(n_attn=LAYERS)
    fp8 = args.kv == "fp8"
    state = tb.State(cfg, pos + t + 64, "cuda", kv_dtype=torch.float8_e4m3fn if fp8 else torch.bfloat16)
    fill_cache_(state, seed=0)
    scales = (lambda l: (state.k_scale[l], state.v_scale[l])) if fp8 else (lambda l: (None, None))
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
            outs[l] = tb.fused.attn_prefill_fused(d_q, state.k[l], state.v[l], pos, cfg, *scales(l))

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
            o = tb.fused.attn_prefill_fused(d_q, state.k[l], state.v[l], pos, cfg, *scales(l))
            h_out.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e2e_steps = max(1, steps // 2)
    ms_e2e = timed(e2e_step, e2e_steps)
    e2e_value = flops * e2e_steps / (ms_e2e * 1e-3) / 1e12

    def attn_only():
        for l in range(LAYERS):
            tb.fused.attn_prefill_fused(d_q, state.k[l], state.v[l], pos, cfg, *scales(l))
    ms_k = timed(attn_only, 1)
    peaks, how = measured_peaks()
    peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    achieved = flops / (ms_k * 1e-3) / 1e12

    # ---- parity, outside the timed region: the chunk's rows bit for bit (first and last layer) and 64
    # sampled query rows x the heads of the first and last kv head of the last layer against the oracle
    kb, vb, qb = _bits(d_k), _bits(d_v), _bits(d_q)
    exact = True
    for l in (0, LAYERS - 1):
        for src, cache, scale in ((kb, state.k, state.k_scale), (vb, state.v, state.v_scale)):
            if not fp8:
                exact &= bool(np.array_equal(cache[l, :, pos:pos + t].view(torch.int16).cpu().numpy().view(np.uint16), src))
                continue
            codes, sc = O.quantize_rows(O.bf16_bits_to_f32(src))
            exact &= bool(np.array_equal(cache[l, :, pos:pos + t].view(torch.uint8).cpu().numpy(), codes))
            exact &= bool(np.array_equal(scale[l, :, pos:pos + t].cpu().numpy().view(np.uint32), sc.view(np.uint32)))
    rows = sorted(set([0, 1, 63, 64, 127, 128, 129, t // 2 - 1, t // 2, t - 129, t - 128, t - 2, t - 1] + list(np.linspace(5, t - 7, 51).astype(int))))[:64]
    heads = (0, HKV - 1)
    g = HQ // HKV
    l = LAYERS - 1
    t0 = time.perf_counter()
    ref = _oracle_layer(state, l, heads, pos + t)
    want = O.attn_rows_over_cache(ref, 0, qb[rows], pos, kv_heads=heads, row_pos=pos + np.asarray(rows))
    cpu_dt = time.perf_counter() - t0
    hq_sel = [j * g + x for j in heads for x in range(g)]
    got = outs[l].float().cpu().numpy()[rows][:, hq_sel]
    ok, max_abs, rel = _compare(got, want[:, hq_sel])
    cpu_flops = float(sum(4.0 * len(hq_sel) * D * (pos + r + 1) for r in rows))
    line = {
        "metric": "prefill_attn_tflops", "value": round(value, 1), "unit": "TFLOP/s", "ms_per_step": round(ms / steps, 3),
        "n_gpus": 1, "steps": steps, "warmup": warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": ("fp8_e4m3 operands (q and p as hi+lo pairs)" if fp8 else "bf16 operands") + ", fp32 accumulate in TMEM", "data": "synthetic",
        "config": {"workload": name, "layers": LAYERS, "cached_rows": pos, "new_tokens": t, "heads": f"{HQ}q/{HKV}kv x {D}", "kv_cache": args.kv,
                   "flop_per_step": flops, "l2": "inputs larger than L2 (no flush needed)"},
        "e2e": {"value": round(e2e_value, 1), "unit": "TFLOP/s", "ms_per_step": round(ms_e2e / e2e_steps, 3),
                "h2d_bytes_per_step": LAYERS * (h_q.numel() + h_k.numel() + h_v.numel()) * 2, "d2h_bytes_per_step": LAYERS * h_out.numel() * 2},
        "gpu_launches": 2 * LAYERS * steps,
        "clocks": clocks.summary(),
        "roofline": {"bound": "tensor", "kernel": "prefill_kernel", "achieved": round(achieved, 1), "peak": peak, "peak_source": how,
                     "unit": "TFLOP/s", "frac": round(achieved / peak, 4), "traffic": None,
                     "note": "algorithmic flops (each product counted once); " + ("the kernel issues two e4m3 MMAs per product at the FP8 rate" if fp8 else "one bf16 MMA per product")},
        "cpu_baseline": {"value": round(cpu_flops / cpu_dt / 1e12, 5), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{len(rows)} query rows x {len(hq_sel)} heads of one layer over {pos + t} keys incl. dequantisation ({cpu_dt:.2f} s); it is also the parity check"},
        "parity": {"ok": bool(ok and exact), "layers": [0, LAYERS - 1], "kv_heads": list(heads), "sampled_query_rows": len(rows), "max_abs_err": max_abs,
                   "rel_err": rel, "appended_rows_bit_exact": bool(exact), "bar": PARITY_BAR,
                   "against": "fp32 oracle attention over the device's cache bytes, at the benchmarked size"},
        "device_status": tb._lib.device_status(),
    }
    return line


def run_profile_case(args):
    """Small, self-ending cases of one kernel for a profiler: few launches before the kernel of
    interest, inputs beyond L2 for the decode case, a few GB on the device at most."""
    import tokenrush_b200 as tb
    kind = WORKLOADS[args.workload]["profile"]
    f8 = torch.float8_e4m3fn
    tb.fused.set_launch_mode(args.launch_mode)              # chained: every launch after the first takes the half-size CTAs
    if kind == "decode":
        rows = args.rows or 131072
        cfg = tb.AttnConfig(n_attn=args.layers)
        st = tb.State(cfg, rows + 64, "cuda", kv_dtype=f8)
        random_fill_(st)
        st.set_pos(rows - args.m)
        q = torch.randn(args.m, HQ * D, device="cuda").to(torch.bfloat16)
        for _ in range(args.iters):
            for l in range(args.layers):
                tb.fused.attn_decode_fused(q, None, st.k[l], st.v[l], st.pos_t, cfg, st.k_scale[l], st.v_scale[l])
    else:
        rows = args.rows or 16384
        cfg = tb.AttnConfig(n_attn=1)
        st = tb.State(cfg, rows + args.t + 64, "cuda", kv_dtype=f8 if args.kv == "fp8" else torch.bfloat16)
        if st.fp8:
            random_fill_(st)
        else:
            st.k.normal_(); st.v.normal_()
        q = torch.randn(args.t, HQ, D, device="cuda").to(torch.bfloat16)
        for _ in range(min(args.iters, 2)):
            tb.fused.attn_prefill_fused(q, st.k[0], st.v[0], rows, cfg, st.k_scale[0] if st.fp8 else None, st.v_scale[0] if st.fp8 else None)
    torch.cuda.synchronize()
    if kind == "prefill-timeline":
        import ctypes as C
        import numpy as np
        lib = tb._lib.lib()
        if not hasattr(lib, "trb_dbg_timeline"):
            raise SystemExit("the loaded library has no timeline: build it with `python -m tokenrush_b200.build --timeline`")
        lib.trb_dbg_timeline.argtypes, lib.trb_dbg_timeline.restype = [C.c_void_p, C.c_size_t], C.c_int
        buf = np.zeros((64, 256, 16), dtype=np.uint64)
        assert lib.trb_dbg_timeline(buf.ctypes.data, buf.nbytes) == 0
        a = buf[63, :32].astype(np.int64)
        t0 = a[0, 0]
        names = ["sm pass start", "sm S ready", "sm S loaded", "sm max done", "sm barrier passed", "sm PV(i-1) done", "sm P written", "sm P published",
                 "mma qk entry", "mma K landed", "mma K landed (again)", "mma QK issued", "mma pv entry", "mma V landed", "mma P ready", "mma PV issued"]
        print("clock64 cycles relative to the first stamp; one line per key tile (softmax warp 0, then the MMA warp)")
        print(" | ".join(names))
        for r in a:
            print(" ".join(f"{int(v - t0):7d}" for v in r))
        d = np.diff(a[:, 0])
        print(json.dumps({"cycles_per_tile_median": float(np.median(d)), "softmax_pass_cycles_median": float(np.median(a[:, 7] - a[:, 0])),
                          "kv": args.kv}))
        return
    print(json.dumps({"profile_case": kind, "rows": rows, "device_status": tb._lib.device_status()}), flush=True)


TL_NAMES = ["cta start", "ranges known, barriers set", "first tiles requested", "query staged", "first tile landed", "last tile consumed",
            "dependency wait passed", "all warps in the epilogue", "partial on its way", "tail: start", "tail: (max, sum) of all splits here",
            "tail: accumulators merged", "cta leaves"]


def run_timeline(args):
    """Where the time of a decode launch goes: thread 0 of every CTA stamps %globaltimer at fixed points
    (diagnostic build of the library); this prints, for the last launches of a captured step, every
    stamp relative to the first CTA start of its launch, and how launches overlap."""
    import ctypes as C
    import numpy as np
    import tokenrush_b200 as tb
    lib = tb._lib.lib()
    if not hasattr(lib, "trb_dbg_timeline"):
        raise SystemExit("the loaded library has no timeline: build it with `python -m tokenrush_b200.build --timeline`")
    lib.trb_dbg_timeline.argtypes, lib.trb_dbg_timeline.restype = [C.c_void_p, C.c_size_t], C.c_int
    rows, m = args.rows or 32768, args.m
    tb.fused.set_launch_mode(args.launch_mode)
    cfg = tb.AttnConfig(n_attn=LAYERS)
    st = tb.State(cfg, rows + 256, "cuda", kv_dtype=torch.float8_e4m3fn)
    random_fill_(st)
    st.set_pos(rows - m)
    q = torch.randn(LAYERS, m, HQ * D, device="cuda").to(torch.bfloat16)
    kn = torch.randn(LAYERS, HKV, m, D, device="cuda").to(torch.bfloat16)
    out = torch.zeros(LAYERS, m, HQ * D, device="cuda", dtype=torch.bfloat16)

    def step():
        for l in range(LAYERS):
            if not args.decode_only:
                tb.fused.kv_write_prefill(kn[l], kn[l], st, l, st.pos_t)
            tb.fused.attn_decode_fused(q[l], None, st.k[l], st.v[l], st.pos_t, cfg, st.k_scale[l], st.v_scale[l], out=out[l])
        if not args.decode_only:
            tb.fused.cursor_advance(st.pos_t, m)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        step()
    for _ in range(5):
        g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(3):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    us_step = e0.elapsed_time(e1) * 1e3 / 3
    buf = np.zeros((64, 256, 16), dtype=np.uint64)
    assert lib.trb_dbg_timeline(buf.ctypes.data, buf.nbytes) == 0
    t = buf.astype(np.int64)
    # the 16 launches of the last replay: the 16 ring slots with the latest start stamps
    starts = np.where(t[:, :, 0] > 0, t[:, :, 0], 0).max(axis=1)
    order = [int(i) for i in np.argsort(starts) if starts[i] > 0][-LAYERS:]
    launches = []
    prev_end = None
    for slot in order:
        a = t[slot]
        valid = (a[:, 0] > starts[slot] - 2_000_000) & (a[:, 12] > 0)
        a = a[valid]
        t0 = a[:, 0].min()
        rec = {"ctas": int(valid.sum()), "first_start_to_last_leave_us": round((a[:, 12].max() - t0) / 1e3, 2),
               "cta_start_spread_us": round((a[:, 0].max() - t0) / 1e3, 2)}
        if prev_end is not None:
            rec["first_start_minus_previous_launch_end_us"] = round((t0 - prev_end) / 1e3, 2)
        prev_end = a[:, 12].max()
        helpers = a[:, 13].astype(np.int32) >= 0
        phases = {}
        for i, nm in enumerate(TL_NAMES):
            col = a[:, i]
            sel = col > 0
            if i in (9, 10, 11):
                sel &= helpers
            if sel.any():
                c = (col[sel] - t0) / 1e3
                phases[nm] = [round(float(c.min()), 2), round(float(np.median(c)), 2), round(float(c.max()), 2)]
        rec["stamps_us_min_median_max"] = phases
        # per CTA: time between consecutive stamps (median over CTAs)
        seg = {}
        for (i, j2, nm) in ((0, 4, "start -> first tile landed"), (4, 5, "streaming"), (5, 7, "last tile -> all warps done"),
                            (7, 8, "CTA merge + partial store"), (8, 12, "helpers: partial -> leave")):
            sel = (a[:, i] > 0) & (a[:, j2] > 0)
            if nm.startswith("helpers"):
                sel &= helpers
            if sel.any():
                seg[nm] = round(float(np.median((a[sel, j2] - a[sel, i]) / 1e3)), 2)
        rec["per_cta_median_us"] = seg
        launches.append(rec)
    print(json.dumps({"timeline": {"rows": rows, "query_rows": m, "layers": LAYERS, "launch_mode": args.launch_mode, "decode_only": bool(args.decode_only),
                                   "us_per_step": round(us_step, 2), "us_per_layer": round(us_step / LAYERS, 2), "stamp_names": TL_NAMES,
                                   "launches": launches[-4:], "device_status": tb._lib.device_status()}}), flush=True)


def summary_of(line):
    """The part of a workload's line that the headline line carries under `workloads`."""
    keys = ("metric", "value", "unit", "us_per_step", "ms_per_step", "steps", "warmup", "blocks", "e2e", "clocks", "gpu_launches", "device_status")
    out = {k: line[k] for k in keys if k in line}
    out["roofline"] = {k: line["roofline"][k] for k in ("kernel", "bound", "achieved", "peak", "unit", "frac", "us_per_launch") if k in line["roofline"]}
    out["parity"] = {k: line["parity"][k] for k in ("ok", "max_abs_err", "rel_err", "appended_rows_bit_exact") if k in line["parity"]}
    out["config"] = line["config"]
    return out


def run_product(args):
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if int(os.environ.get("RANK", "0")) != 0 and "t" in WORKLOADS[args.workload]:
        return
    if "t" in WORKLOADS[args.workload]:
        line = run_prefill(args.workload, args, args.steps, args.warmup)
    else:
        line = run_decode(args.workload, args, args.steps, args.warmup, args.blocks, args.cpu_seconds)
    if world == 1 and args.workload == "window256k" and not args.no_extra:
        # the other configurations, a few steps each, on the same line
        extra = {}
        torch.cuda.empty_cache()
        for name, st_, wu in (("ctx32k", 100, 5), ("verify64k", 50, 5)):
            extra[name] = summary_of(run_decode(name, args, st_, wu, 3, 0.0))
            torch.cuda.empty_cache()
        extra["prefill8k"] = summary_of(run_prefill("prefill8k", args, 2, 1))
        line["workloads"] = extra
    if line is not None:
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


# ------------------------------------------------------------------------------ CPU baselines

def _random_codes(shape, rng):
    import numpy as np
    return rng.integers(0, 0x7F, shape, dtype=np.uint8) | (rng.integers(0, 2, shape, dtype=np.uint8) << 7)


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
    st.k[:] = _random_codes(st.k.shape, rng)
    st.v[:] = _random_codes(st.v.shape, rng)
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


def find_reference():
    """An importable copy of the reference (its `tokenrush` package): the in-tree install location,
    then the path that BASELINE.json names.  Returns (fused, ops, state, config modules, where) or None."""
    cands = [os.path.join(ROOT, "baseline", "_ref")]
    try:
        with open(os.path.join(ROOT, "BASELINE.json")) as f:
            cands.append(json.load(f).get("reference_path") or "")
    except OSError:
        pass
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "tokenrush", "fused.py")):
            sys.dont_write_bytecode = True
            sys.path.insert(0, c)
            try:
                from tokenrush import config as rcfg, fused as rfused, ops as rops, state as rstate
                return rfused, rops, rstate, rcfg, c
            except Exception as e:                                  # noqa: BLE001 - any import problem means "not available"
                sys.path.remove(c)
                sys.stderr.write(f"reference at {c} does not import: {e!r}\n")
    return None


def _reference_cfg(rcfg, n_layers: int):
    """The reference's ModelConfig with the attention geometry of the benchmark and minimal sizes for
    the layers that are not on this path."""
    return rcfg.ModelConfig(hidden=HQ * D, n_layers=n_layers, layer_types=("full_attention",) * n_layers, vocab=8, ffn=8,
                            n_heads=HQ, n_kv_heads=HKV, head_dim=D, rotary_dim=64, rope_theta=1e7,
                            gdn_k_heads=1, gdn_v_heads=1, gdn_k_dim=8, gdn_v_dim=8, conv_k=4, eps=1e-6, max_pos=1 << 20, eos_ids=(0,))


def run_reference(args):
    """The reference arm: the reference's CPU path on the host cores, one layer of the workload per
    step (a bounded sample: the metric is a rate, so a layer gives the same figure as a step of 16).
    Its own torch functions when an installed copy is found, else the restatement in oracle/.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    wl = WORKLOADS[args.workload]
    if "t" in wl or "profile" in wl:
        print(json.dumps({"impl": "reference", "unavailable": "the reference arm covers the decode workloads; the prefill CPU sample is in the product line's cpu_baseline"}), flush=True)
        return
    import numpy as np
    ctx, m = wl["ctx"], wl["m"]
    steps, warmup = max(1, min(args.steps, 24)), max(1, min(args.warmup, 3))
    torch.set_num_threads(os.cpu_count() or 1)
    ref = find_reference()
    rng = np.random.default_rng(0)
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(m, HQ, D, generator=gen).to(torch.bfloat16)
    kn = torch.randn(HKV, m, D, generator=gen).to(torch.bfloat16)
    vn = torch.randn(HKV, m, D, generator=gen).to(torch.bfloat16)
    pos = ctx - m
    if ref is not None:
        rfused, rops, rstate, rcfg, where = ref
        st = rstate.State(_reference_cfg(rcfg, 1), ctx + m, "cpu", kv_dtype=torch.float8_e4m3fn)
        st.k.view(torch.uint8).copy_(torch.from_numpy(_random_codes(tuple(st.k.shape), rng)))
        st.v.view(torch.uint8).copy_(torch.from_numpy(_random_codes(tuple(st.v.shape), rng)))
        st.k_scale.uniform_(0.006, 0.011); st.v_scale.uniform_(0.006, 0.011)

        def layer_step():
            # the composition of the reference's own tests: write, dequantise, fp32 attention
            rfused.kv_write_prefill(kn, vn, st, 0, pos)
            n = pos + m
            kd = st.k[0, :, :n].float() * st.k_scale[0, :, :n, None]
            vd = st.v[0, :, :n].float() * st.v_scale[0, :, :n, None]
            qf = q.float().transpose(0, 1).contiguous()
            return rops.attn_decode(qf, kd, vd) if m == 1 else rops.attn_prefill(qf, kd, vd, pos)
        kind, what = "reference", f"tokenrush.fused.kv_write_prefill + dequantise + tokenrush.ops.attn_{'decode' if m == 1 else 'prefill'} (fp32) from {os.path.relpath(where, ROOT) if where.startswith(ROOT) else where}"
    else:
        from oracle import kv_oracle as O
        ost = O.OracleState(1, HKV, ctx + m, D)
        ost.k[:] = _random_codes(ost.k.shape, rng); ost.v[:] = _random_codes(ost.v.shape, rng)
        ost.k_scale[:] = rng.uniform(0.006, 0.011, ost.k_scale.shape).astype(np.float32)
        ost.v_scale[:] = rng.uniform(0.006, 0.011, ost.v_scale.shape).astype(np.float32)
        qb, kb, vb = O.torch_bf16_to_bits(q), O.torch_bf16_to_bits(kn), O.torch_bf16_to_bits(vn)

        def layer_step():
            return O.decode_step_cpu_threaded(ost, 0, qb, kb, vb, pos)
        kind, what = "port", "oracle.kv_oracle.decode_step_cpu_threaded (no installed copy of the reference was found)"
    for _ in range(warmup):
        layer_step()
    c0, t0 = time.process_time(), time.perf_counter()
    for _ in range(steps):
        layer_step()
    wall = time.perf_counter() - t0
    busy = (time.process_time() - c0) / max(wall, 1e-9)
    sec_step = wall / steps
    value = ctx * ROW_BYTES / sec_step / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_effective_kv_bandwidth", "value": round(value, 4), "unit": "GB/s",
        "us_per_step": round(sec_step * 1e6, 1), "ms_per_step": round(sec_step * 1e3, 3), "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": steps, "warmup": warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp32 math over the fp8 cache (CPU)", "data": "synthetic",
        "config": {"workload": args.workload, "layers": LAYERS, "context_rows": ctx, "query_rows": m,
                   "heads": f"{HQ}q/{HKV}kv x {D}", "kv_bytes_per_step": ctx * ROW_BYTES,
                   "sample": "each step is ONE of the workload's 16 layers (a full step is 16 of these); the rate is the same"},
        "cpu_baseline": {"value": round(value, 4), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": kind,
                         "cores_busy_avg": round(busy, 1), "sample": f"{steps} layer-steps of 1 layer x {ctx} rows, M={m}, mean of all: {what}"},
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    if torch.cuda.is_available() and not args.no_triton:
        line["reference_gpu_kernels"] = run_reference_triton(ref, ctx, m)
    print(json.dumps(line), flush=True)


def run_reference_triton(ref, ctx: int, m: int):
    """The reference's own Triton kernels (attn_prep + attn_decode_fused, launch constants as shipped)
    on this GPU, on a cache of the same shape and value distribution, timed like the product: a
    captured graph of the 16 layers, CUDA events."""
    if ref is None:
        return {"unavailable": "no installed copy of the reference on this box"}
    try:
        import triton  # noqa: F401
        rfused, rops, rstate, rcfg, where = ref
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        cfg = _reference_cfg(rcfg, LAYERS)
        st = rstate.State(cfg, ctx + 64 * m + 64, "cuda", kv_dtype=torch.float8_e4m3fn)
        random_fill_(st)
        st.pos_t.fill_(ctx - m)
        qkv = torch.randn(m, HQ * 2 * D + 2 * HKV * D, device="cuda").to(torch.bfloat16)
        qn = torch.zeros(D, device="cuda", dtype=torch.bfloat16)
        kn = torch.zeros(D, device="cuda", dtype=torch.bfloat16)
        cos, sin = rops.rope_table(ctx + 64 * m + 64, cfg.rotary_dim, cfg.rope_theta, "cuda") if hasattr(rops, "rope_table") else (None, None)
        q_fixed = torch.randn(m, HQ * D, device="cuda").to(torch.bfloat16)

        def decode_only():
            for l in range(LAYERS):
                rfused.attn_decode_fused(q_fixed, qkv, st.k[l], st.v[l], st.pos_t, cfg, st.k_scale[l], st.v_scale[l])

        def full_step():
            for l in range(LAYERS):
                qq = rfused.attn_prep(qkv, qn, kn, cos, sin, st.pos_t, st.k[l], st.v[l], cfg, st.k_scale[l], st.v_scale[l])
                rfused.attn_decode_fused(qq, qkv, st.k[l], st.v[l], st.pos_t, cfg, st.k_scale[l], st.v_scale[l])

        def timed_graph(fn, reps):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()                                                 # compiles
                fn()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                fn()
            for _ in range(3):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(reps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / reps
        out = {"kernels": "tokenrush.fused.attn_decode_fused (NSPLIT=32, BLOCK_N=32) / attn_prep, Triton " + __import__("triton").__version__,
               "context_rows": ctx, "query_rows": m, "layers": LAYERS, "timing": "captured graph of the 16 layers, CUDA events, 20 replays"}
        us = timed_graph(decode_only, 20)
        out["decode_only_us_per_step"] = round(us, 1)
        out["decode_only_gbs"] = round(LAYERS * ctx * ROW_BYTES / (us * 1e-6) / 1e9, 1)
        if cos is not None:
            us2 = timed_graph(full_step, 20)
            out["prep_plus_decode_us_per_step"] = round(us2, 1)
            out["prep_plus_decode_gbs"] = round(LAYERS * ctx * ROW_BYTES / (us2 * 1e-6) / 1e9, 1)
        return out
    except Exception as e:                                          # noqa: BLE001 - report whatever stopped it
        return {"unavailable": f"unavailable on this box: {type(e).__name__}: {str(e)[:300]}"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--blocks", type=int, default=5, help="timed blocks of --steps steps; the median block is reported")
    ap.add_argument("--impl", default="product", choices=["product", "reference"])
    ap.add_argument("--workload", default="window256k", choices=sorted(WORKLOADS))
    ap.add_argument("--exchange", default="fused", choices=["fused", "p2p", "nccl"])
    ap.add_argument("--launch-mode", type=int, default=2, choices=[0, 1, 2],
                    help="programmatic dependent launch: 0 off, 1 on, 2 chained (the step is a graph of library calls only)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-extra", action="store_true", help="headline workload only (no `workloads` object)")
    ap.add_argument("--no-triton", action="store_true", help="reference arm: skip the reference's GPU kernels")
    ap.add_argument("--kv", default="fp8", choices=["fp8", "bf16"], help="prefill workloads: cache dtype")
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--t", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--decode-only", action="store_true", help="timeline: a graph of the 16 decode launches without appends")
    args = ap.parse_args()
    if args.workload.startswith("timeline"):
        os.environ["TRB_KV_LIB"] = os.path.join(ROOT, "tokenrush_b200", "libtrb_kv_timeline.so")   # read when the package is imported
    if args.workload == "timeline":
        run_timeline(args)
    elif args.impl == "reference":
        run_reference(args)
    elif "profile" in WORKLOADS[args.workload]:
        run_profile_case(args)
    else:
        run_product(args)


if __name__ == "__main__":
    main()
