// Split-K flash-decoding for several query rows per kv head (speculative verify, M >= 2) on the
// 5th-generation tensor cores.  Included by decode.cu after DecodeParams and decode_tail.
//
// With 6 M query rows per kv head, converting every e4m3 tile to f16 once per 8-row slice (the
// mma.sync kernel) costs more issue slots than the stream leaves; tcgen05.mma reads the e4m3
// codes of the cache straight from the TMA tile.  The products are laid out transposed, so
// that the 128-row operand is always the cache tile and the few query rows are the N extent:
//     S^T[128 keys x 2N]  = K . [Qhi ; Qlo]^T      A = K tile (K-major),  B = stacked query block
//     O^T[128 dims x 2N] += V^T . [Phi ; Plo]^T    A = V tile (MN-major), B = probabilities, keys x rows
// (two O^T accumulators for the 256 dims).  The probability tile is stored [key][row] (MN-major
// B operand): a thread owns one key, so its 16 rows are one 16-byte store.  hi + lo are two e4m3 terms of a value (8 significant
// bits, what bf16 carries); stacking them as 2N operand rows reads each cache tile once per
// product, and the two partial results are added after the tensor-memory load.
//
// Warp roles: one softmax warpgroup per 16 query rows (thread = key of the tile = TMEM lane of
// S^T; for the O^T correction and the epilogue the same thread = head dim), then one TMA
// producer warp and one MMA issuer warp: 192, 320 or 448 threads for up to 16, 32, 48 rows.  The
// warpgroups work independently on their rows (own named barrier, own statistics), so the work
// per thread does not grow with M.  S^T and P are double-buffered.  Row maxima over the keys of
// a row follow lazily: the stored probability is 2^(t - ref + 7), and ref moves only when a score
// exceeds it by more than 1.75 (one barrier with an OR reduction per tile detects that); only
// then the exact tile maxima are found (redux.sync.max.f32 + a 4-warp exchange) and the row's O^T
// column and sum are rescaled.  The CTA's result goes to the split workspace in the layout of decode_kernel, and the
// same ticket + tail finishes the launch.  Every wait is bounded.
#pragma once
#include "tc.cuh"

namespace trb {

constexpr int TC_BN = 128;                     // keys per tile = M of every MMA
constexpr int TC_D = 256;
constexpr int TC_MAX_THREADS = 448;           // 4 softmax warps per 16 query rows + TMA warp + MMA warp
constexpr int TC_KSLOTS = 3, TC_VSLOTS = 2;
constexpr int TC_TILE = TC_BN * TC_D;          // 32 KB of e4m3 codes
constexpr int TC_MAX_N2 = 96;                  // stacked rows: 2 x (query rows rounded up to 16)
constexpr int TC_OFF_K = 0;
constexpr int TC_OFF_V = TC_OFF_K + TC_KSLOTS * TC_TILE;
constexpr int TC_OFF_Q = TC_OFF_V + TC_VSLOTS * TC_TILE;          // [2 column blocks][2N rows][128 B]
constexpr int TC_Q_BYTES = 2 * TC_MAX_N2 * 128;
constexpr int TC_OFF_P = TC_OFF_Q + TC_Q_BYTES;                    // 2 buffers of [128 keys][128 B: hi rows | lo rows | zeros]
constexpr int TC_P_BYTES = TC_BN * 128;
constexpr int TC_OFF_SC = TC_OFF_P + 2 * TC_P_BYTES;               // [KSLOTS][2][128] floats
constexpr int TC_OFF_ST = TC_OFF_SC + TC_KSLOTS * 2 * TC_BN * 4;   // per-row statistics, see below
constexpr int TC_ST_FLOATS = 2 * 4 * 48 + 2 * 48 + 8;
constexpr int TC_OFF_BAR = TC_OFF_ST + TC_ST_FLOATS * 4;
constexpr int TC_OFF_TL = TC_OFF_BAR + 256;                        // timeline stamps (diagnostic build only)
constexpr int TC_SMEM = TC_OFF_TL + 128 + 1024;
constexpr int TC_TMEM_COLS = 512;
constexpr int TC_TMEM_S = 0;                   // S^T buffers at columns 0 and 128
constexpr int TC_TMEM_O = 256;                 // O^T accumulators (dims 0-127, 128-255) at columns 256 and 384

__device__ __forceinline__ float redux_max(float v) {
    float r;
    asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
    return r;
}
constexpr float TC_LAG = 1.75f;                // a score may exceed its row's reference exponent by this much
// bar.red: barrier over `threads` threads of barrier `id`, returning the OR of their predicates
__device__ __forceinline__ bool barrier_or(int id, int threads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\t"
        "bar.red.or.pred q, %2, %3, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r) : "r"((uint32_t)pred), "r"(id), "r"(threads) : "memory");
    return r != 0;
}
template <int NROW>
__global__ void __launch_bounds__(8 * NROW + 64, 1)
decode_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const DecodeParams p) {
    constexpr int D = TC_D, N2 = 2 * NROW, NCH = NROW / 16;
    constexpr int NTHREADS = 8 * NROW + 64, W_TMA = 4 * NCH, W_MMA = 4 * NCH + 1;
    extern __shared__ uint8_t tc_smem_raw[];
    uint8_t *smem = tc_smem_raw + ((1024u - (smem_u32(tc_smem_raw) & 1023u)) & 1023u);
    float *sm_sc = reinterpret_cast<float *>(smem + TC_OFF_SC);
    float *sm_wmax = reinterpret_cast<float *>(smem + TC_OFF_ST);        // [2 buffers][row group][4 quarters][16] warp maxima / sums
    float *sm_qinv = sm_wmax + 2 * 4 * 48;                                // [48] inverse of the query row scale
    int *sm_hi = reinterpret_cast<int *>(sm_qinv + 48);                   // [48] last visible key of a row
    int *sm_flag = sm_hi + 48;                                            // [3] used by decode_tail
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(sm_flag + 3);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + TC_OFF_BAR);
    uint64_t *k_full = bars, *k_free = bars + 3, *v_full = bars + 6, *v_free = bars + 8;
    uint64_t *s_full = bars + 10, *s_free = bars + 12, *p_full = bars + 14, *pv_done = bars + 16;

    const int split = blockIdx.x, j = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    unsigned long long *sm_tl = reinterpret_cast<unsigned long long *>(smem + TC_OFF_TL);
    (void)sm_tl;
    TRB_TL(sm_tl, 0);

    // ---- dependency plan (see decode_kernel) ----
    const int flags = p.pdl_flags;
    bool waited = false;
    auto dep_wait = [&]() {
        if (!waited) {
            pdl_wait();
            waited = true;
            if (!(flags & PDL_TRIGGER_TOP)) pdl_launch_dependents();
        }
    };
    if (flags & PDL_TRIGGER_TOP) pdl_launch_dependents();
    if (!(flags & PDL_PRE_CURSOR)) dep_wait();

    // ---- ranges, all derived from the device cursor (as in decode_kernel, in 128-key tiles) ----
    const long long pos = load_cursor(p.pos);
    const long long live = pos + (p.new_rows ? p.m : 0);
    long long lloc = live - p.shard_lo;
    if (lloc < 0) lloc = 0;
    if (lloc > p.max_len) {
        if (!p.sharded && tid == 0 && split == 0 && j == 0) raise_status(TRB_ST_CURSOR_RANGE);
        lloc = p.max_len;
    }
    const int n_tiles = (int)((lloc + TC_BN - 1) / TC_BN);
    int per = (n_tiles + p.nsplit - 1) / p.nsplit;
    if (per < 1) per = 1;
    int active = (n_tiles + per - 1) / per;
    if (active < 1) active = 1;
    if (split >= active) return;
    const int t0 = split * per;
    int my_tiles = (t0 + per < n_tiles ? t0 + per : n_tiles) - t0;
    if (my_tiles < 0) my_tiles = 0;
    const int lloc_i = (int)lloc;
    const int pos_loc = (int)(pos - p.shard_lo);

    if (tid == 0) {
        for (int s = 0; s < TC_KSLOTS; ++s) { mbar_init(&k_full[s], 33u); mbar_init(&k_free[s], 1u + 4u * NCH); }
        for (int s = 0; s < TC_VSLOTS; ++s) { mbar_init(&v_full[s], 1u); mbar_init(&v_free[s], 1u); }
        for (int b = 0; b < 2; ++b) { mbar_init(&s_full[b], 1u); mbar_init(&s_free[b], 4u * NCH); mbar_init(&p_full[b], 4u * NCH); mbar_init(&pv_done[b], 1u); }
        mbar_fence_init();
        tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
    }
    if (warp == 0) { tmem_alloc(tmem_slot, TC_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    TRB_TL(sm_tl, 1);

    // producer helpers (the TMA warp)
    auto issue_k = [&](int i) {
        const int s = i % TC_KSLOTS;
        const int row0 = (t0 + i) * TC_BN;
        uint8_t *kt = smem + TC_OFF_K + s * TC_TILE;
        if (lane == 0) {
            mbar_arrive_expect_tx(&k_full[s], TC_TILE);
            tma_load_4d(kt, &tm_k, &k_full[s], 0, 0, row0, j);
            tma_load_4d(kt + TC_BN * 128, &tm_k, &k_full[s], 0, 1, row0, j);
        }
#pragma unroll
        for (int hh = 0; hh < 4; ++hh) {
            const long long r = (long long)row0 + lane + 32 * hh;
            const bool ok = r < p.max_len;
            const long long off = (long long)j * p.max_len + (ok ? r : 0);
            cp_async_4(&sm_sc[(s * 2 + 0) * TC_BN + lane + 32 * hh], p.ks + off, ok ? 4u : 0u);
            cp_async_4(&sm_sc[(s * 2 + 1) * TC_BN + lane + 32 * hh], p.vs + off, ok ? 4u : 0u);
        }
        cp_async_mbar_arrive_noinc(&k_full[s]);
    };
    auto issue_v = [&](int i) {
        const int s = i % TC_VSLOTS;
        const int row0 = (t0 + i) * TC_BN;
        uint8_t *vt = smem + TC_OFF_V + s * TC_TILE;
        if (lane == 0) {
            mbar_arrive_expect_tx(&v_full[s], TC_TILE);
            tma_load_4d(vt, &tm_v, &v_full[s], 0, 0, row0, j);
            tma_load_4d(vt + TC_BN * 128, &tm_v, &v_full[s], 0, 1, row0, j);
        }
    };
    // Tiles below the rows that a launch still in flight may be writing are complete: they stream
    // before the dependency wait (the producer warp waits when it reaches the first other tile).
    const long long fresh_from = (flags & PDL_ALL_STABLE) ? (1LL << 62) : (p.new_rows ? pos - p.shard_lo : 0);
    int n_stable = my_tiles;
    if (!waited) {
        long long ns = fresh_from / TC_BN - t0;
        if (ns < 0) ns = 0;
        if (ns < n_stable) n_stable = (int)ns;
    }
    // with a workspace of its own the CTA takes its ticket at its start (see decode_kernel)
    if (warp == W_TMA && lane == 0 && (flags & PDL_PRIVATE_WS))
        decode_ticket(p, j, active, NTHREADS / (D / 4), sm_flag, decode_ticket_take(p, j));
    int pre = 0;
    if (warp == W_TMA)
        while (pre < my_tiles && pre < 2 && pre < n_stable) { issue_k(pre); issue_v(pre); ++pre; }
    if (!(flags & PDL_PRE_Q)) dep_wait();                      // the query rows may come from the launch before this one

    // ---- query block: rows r of this kv head (query r / g, head j g + r % g) as two stacked e4m3
    // copies with a power-of-two row scale; thread = (row, 32-dim eighth).  (The bytes of a
    // probability row beyond its 2N codes are never written: they only feed O^T columns that
    // nobody reads.)
    {
        const int row = tid >> 3, part = tid & 7;
        const bool in_block = row < NROW, valid = row < p.rows && in_block;
        const int qi = valid ? row / p.g : 0, hq = valid ? j * p.g + row % p.g : 0;
        const __nv_bfloat16 *qp = p.q + ((long long)qi * p.hq + hq) * D + part * 32;
        uint4 raw[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) raw[c] = valid ? __ldg(reinterpret_cast<const uint4 *>(qp) + c) : make_uint4(0u, 0u, 0u, 0u);
        float amax = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const __nv_bfloat162 *b2 = reinterpret_cast<const __nv_bfloat162 *>(&raw[c]);
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(b2[e]); amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y))); }
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        int e = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
        if (amax == 0.f || e < -90 || !valid) e = 7;
        if (e > 90) e = 90;
        const float sc = valid ? __uint_as_float((uint32_t)(127 + 7 - e) << 23) : 0.f;
        if (in_block) {
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {                                  // 16 dims per chunk
                const int c = part * 2 + cc;
                uint32_t hw[4], lw[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint32_t *rw = reinterpret_cast<const uint32_t *>(&raw[2 * cc + (w >> 1)]) + 2 * (w & 1);
                    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(rw));
                    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(rw + 1));
                    const float y[4] = {a.x * sc, a.y * sc, b.x * sc, b.y * sc};
                    pf_split4(y, hw[w], lw[w]);
                }
                const uint32_t off = (c >> 3) * (N2 * 128) + sw128(row, (c & 7) * 16);
                *reinterpret_cast<uint4 *>(smem + TC_OFF_Q + off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                *reinterpret_cast<uint4 *>(smem + TC_OFF_Q + off + NROW * 128) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
            }
            if (part == 0) {
                sm_qinv[row] = __uint_as_float((uint32_t)(127 - 7 + e) << 23);
                int hi = lloc_i - 1;
                if (p.new_rows && pos_loc + qi < hi) hi = pos_loc + qi;
                sm_hi[row] = hi;
            }
        }
    }
    fence_async_smem();
    __syncthreads();
    TRB_TL(sm_tl, 3);

    bool ok = true;
    if (warp == W_TMA) {
        // ================================ TMA producer ================================
        for (int i = pre; i < my_tiles; ++i) {
            if (i >= n_stable) dep_wait();                     // rows that were still being written when this launch began
            if (i >= TC_KSLOTS && !mbar_wait(&k_free[i % TC_KSLOTS], ((i / TC_KSLOTS) & 1) ^ 1)) break;
            issue_k(i);
            if (i >= TC_VSLOTS && !mbar_wait(&v_free[i % TC_VSLOTS], ((i / TC_VSLOTS) & 1) ^ 1)) break;
            issue_v(i);
        }
        // this warp is idle from here on: it takes the kv head's ticket (a workspace that an earlier
        // launch may still use: after the wait)
        if (!(flags & PDL_PRIVATE_WS)) {
            dep_wait();
            if (lane == 0) decode_ticket(p, j, active, NTHREADS / (D / 4), sm_flag, decode_ticket_take(p, j));
        }
        named_barrier(15, NTHREADS);
    } else if (warp == W_MMA) {
        // ================================ MMA issuer ==================================
        // order on the tensor pipe: QK(0), QK(1), PV(0), QK(2), PV(1), ...
        const uint32_t q_sm = smem_u32(smem + TC_OFF_Q), p_sm = smem_u32(smem + TC_OFF_P);
        constexpr uint32_t IDESC_QK = umma_idesc_f8(TC_BN, N2, false, false), IDESC_PV = umma_idesc_f8(128, 128, true, true);
        auto issue_qk = [&](int i) -> bool {
            const int s = i % TC_KSLOTS, b = i & 1;
            if (!mbar_wait(&k_full[s], (i / TC_KSLOTS) & 1)) return false;
            if (i >= 2 && !mbar_wait(&s_free[b], ((i >> 1) & 1) ^ 1)) return false;      // S^T of tile i-2 has been read
            tc_fence_after();
            if (lane == 0) {
                const uint32_t kt = smem_u32(smem + TC_OFF_K + s * TC_TILE);
#pragma unroll
                for (int sg = 0; sg < 2; ++sg)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t a = umma_desc(kt + sg * (TC_BN * 128) + k * 32, 16, 1024);
                        const uint64_t bd = umma_desc(q_sm + sg * (N2 * 128) + k * 32, 16, 1024);
                        tc_mma_f8(tmem + TC_TMEM_S + b * 128, a, bd, IDESC_QK, (sg | k) ? 1u : 0u);
                    }
                tc_commit(&s_full[b]);
                tc_commit(&k_free[s]);
            }
            __syncwarp();
            return true;
        };
        if (my_tiles > 0) ok = issue_qk(0);
        for (int i = 0; i < my_tiles && ok; ++i) {
            const int b = i & 1;
            if (i + 1 < my_tiles && !(ok = issue_qk(i + 1))) break;
            if (!(ok = mbar_wait(&p_full[b], (i >> 1) & 1))) break;                       // P of tile i staged, O^T corrected
            if (!(ok = mbar_wait(&v_full[b], (i >> 1) & 1))) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t vt = smem_u32(smem + TC_OFF_V + b * TC_TILE), pb = p_sm + b * TC_P_BYTES;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t a = umma_desc(vt + h * (TC_BN * 128) + k * (32 * 128), TC_BN * 128, 1024);
                        const uint64_t bd = umma_desc(pb + k * (32 * 128), TC_BN * 128, 1024);
                        tc_mma_f8(tmem + TC_TMEM_O + h * 128, a, bd, IDESC_PV, (i | k) ? 1u : 0u);
                    }
                tc_commit(&v_free[b]);
                tc_commit(&pv_done[b]);
            }
            __syncwarp();
        }
        named_barrier(15, NTHREADS);
    } else if (warp < 4 * NCH) {
        // ====== softmax / correction / epilogue: one warpgroup per 16 query rows; thread = key lane = dim lane ======
        const int rg = warp >> 2, qw = warp & 3;                               // row group, lane quarter
        const int kl = qw * 32 + lane;                                         // 0..127
        const int r0 = rg * 16;                                                // first row of this group
        const uint32_t lane_addr = tmem + ((uint32_t)(qw * 32) << 16);
        const int all_hi = p.new_rows ? (pos_loc < lloc_i - 1 ? pos_loc : lloc_i - 1) : lloc_i - 1;
        const float *g_qinv = sm_qinv + r0;
        const int *g_hi = sm_hi + r0;
        const int bar_id = 1 + rg;
        // this thread's two 16-byte slots in a probability row: hi codes of rows r0.., lo codes of rows r0..
        const uint32_t p_hi_off = (uint32_t)kl * 128u + ((((uint32_t)rg) ^ ((uint32_t)kl & 7u)) << 4);
        const uint32_t p_lo_off = (uint32_t)kl * 128u + ((((uint32_t)(NCH + rg)) ^ ((uint32_t)kl & 7u)) << 4);
        // Reference exponent of a row: probabilities are stored as 2^(t - ref + 7).  ref follows the
        // row maximum lazily: it moves (and the row's O^T column and sum are rescaled) only when a
        // score exceeds it by more than TC_LAG, so that the stored value stays below the e4m3
        // maximum (2^(7 + 1.75) = 430 < 448).  cref = 7 - ref, identical in every thread of the group;
        // a row is `unset` until its first visible key.
        float lsum[16], cref[16];
#pragma unroll
        for (int r = 0; r < 16; ++r) { lsum[r] = 0.f; cref[r] = 0.f; }
        uint32_t unset = 0xffffu;
        float *g_wmax = sm_wmax + rg * 64;                                     // [4 quarters][16 rows], slow path only

        // A warp whose bounded wait ran out is `dead`: it stops waiting and computing, but still takes
        // part in its group's named barriers, which the three sibling warps keep reaching.
        bool dead = false;
        for (int i = 0; i < my_tiles; ++i) {
            const int s = i % TC_KSLOTS, b = i & 1;
            const int kv = (t0 + i) * TC_BN + kl;                              // virtual row of this thread's key
            if (!dead && !mbar_wait(&k_full[s], (i / TC_KSLOTS) & 1)) dead = true;
            float ksc = 0.f, vsc = 0.f;
            if (!dead) {
                ksc = sm_sc[(s * 2 + 0) * TC_BN + kl]; vsc = sm_sc[(s * 2 + 1) * TC_BN + kl];
                __syncwarp();
                if (lane == 0) mbar_arrive(&k_free[s]);                        // the scale slot may be refilled
            }
            const bool key_ok = kv < lloc_i && vsc > 0.f;
            const float kfac = ksc * p.scale_log2;
            const float vlog = key_ok ? __log2f(vsc) : 0.f;
            const float vinv = key_ok ? __fdividef(0.0078125f, vsc) : 0.f;      // 1 / (128 v_scale)
            if (!dead && !mbar_wait(&s_full[b], (i >> 1) & 1)) dead = true;
            if (dead) {
                if (barrier_or(bar_id, 128, false)) named_barrier(bar_id, 128);
                continue;
            }
            if (i == 0) TRB_TL(sm_tl, 4);
            tc_fence_after();
            float tv[16];
            {
                float hi[16], lo[16];
                tmem_ld16_nowait(lane_addr + TC_TMEM_S + b * 128 + r0, hi);
                tmem_ld16_nowait(lane_addr + TC_TMEM_S + b * 128 + NROW + r0, lo);
                tmem_wait_ld();
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const float4 qv = *reinterpret_cast<const float4 *>(&g_qinv[q4 * 4]);
                    tv[q4 * 4 + 0] = fmaf((hi[q4 * 4 + 0] + lo[q4 * 4 + 0]) * kfac, qv.x, vlog + cref[q4 * 4 + 0]);
                    tv[q4 * 4 + 1] = fmaf((hi[q4 * 4 + 1] + lo[q4 * 4 + 1]) * kfac, qv.y, vlog + cref[q4 * 4 + 1]);
                    tv[q4 * 4 + 2] = fmaf((hi[q4 * 4 + 2] + lo[q4 * 4 + 2]) * kfac, qv.z, vlog + cref[q4 * 4 + 2]);
                    tv[q4 * 4 + 3] = fmaf((hi[q4 * 4 + 3] + lo[q4 * 4 + 3]) * kfac, qv.w, vlog + cref[q4 * 4 + 3]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_free[b]);                            // tile i+2 may overwrite this buffer
            if (!((t0 + i) * TC_BN + TC_BN - 1 <= all_hi)) {                   // the tiles at the end of the live range
#pragma unroll
                for (int r = 0; r < 16; ++r)
                    if (!(key_ok && kv <= g_hi[r])) tv[r] = -INFINITY;
            }
            // ---- does any score of the group exceed its row's reference by more than the lag (or reach a
            // row that has none yet)?  One barrier with an OR reduction answers for the four warps.
            float tmax = tv[0];
#pragma unroll
            for (int r = 1; r < 16; ++r) tmax = fmaxf(tmax, tv[r]);
            bool danger = tmax > 7.f + TC_LAG;
            if (unset) {
#pragma unroll
                for (int r = 0; r < 16; ++r) danger |= ((unset >> r) & 1u) && tv[r] > -INFINITY;
            }
            if (barrier_or(bar_id, 128, danger)) {
                // slow path: exact row maxima of this tile (warp reduction, the four quarters through
                // shared memory); rows beyond the lag get the tile maximum as their new reference
                {
                    float wm[16];
#pragma unroll
                    for (int r = 0; r < 16; ++r) wm[r] = redux_max(tv[r]);
                    if (lane == 0) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4)
                            *reinterpret_cast<float4 *>(&g_wmax[qw * 16 + q4 * 4]) = make_float4(wm[q4 * 4], wm[q4 * 4 + 1], wm[q4 * 4 + 2], wm[q4 * 4 + 3]);
                    }
                }
                named_barrier(bar_id, 128);
                float al[16];
                uint32_t upd = 0u;
#pragma unroll
                for (int r = 0; r < 16; ++r) {
                    const float gm = fmaxf(fmaxf(g_wmax[r], g_wmax[16 + r]), fmaxf(g_wmax[32 + r], g_wmax[48 + r]));
                    const bool u = gm > 7.f + TC_LAG || (((unset >> r) & 1u) && gm > -INFINITY);
                    const float delta = u ? gm - 7.f : 0.f;                    // new reference = the tile maximum
                    al[r] = ((unset >> r) & 1u) ? 0.f : fast_exp2(-delta);     // a row without reference has no sum and a zero column yet
                    cref[r] -= delta;
                    tv[r] -= delta;
                    lsum[r] *= al[r];
                    upd |= (u ? 1u : 0u) << r;
                }
                unset &= ~upd;
                if (i > 0) {
                    // correct the O^T columns of the updated rows; PV(i-1) must have landed
                    if (!mbar_wait(&pv_done[b ^ 1], ((i - 1) >> 1) & 1)) { dead = true; continue; }
                    tc_fence_after();
#pragma unroll 1
                    for (uint32_t mk = upd; mk; mk &= mk - 1) {
                        const int rr = __ffs(mk) - 1;
                        const float a_r = al[rr];
                        const uint32_t a0 = lane_addr + TC_TMEM_O + r0 + rr, a1 = a0 + NROW, a2 = a0 + 128, a3 = a2 + NROW;
                        float o0 = tmem_ld1(a0), o1 = tmem_ld1(a1), o2 = tmem_ld1(a2), o3 = tmem_ld1(a3);
                        tmem_wait_ld();
                        tmem_st1(a0, o0 * a_r); tmem_st1(a1, o1 * a_r); tmem_st1(a2, o2 * a_r); tmem_st1(a3, o3 * a_r);
                    }
                    tmem_wait_st();
                }
            }
            // the P buffer of tile i-2 must have been consumed
            if (i >= 2 && !mbar_wait(&pv_done[b], ((i >> 1) & 1) ^ 1)) { dead = true; continue; }
            // ---- probabilities 2^(t - ref + 7) as hi + lo e4m3 codes: this key's 16 rows are 16 + 16 bytes
            uint32_t hw[4], lw[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                uint32_t hc[2], lc[2];
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    const int r = w * 4 + 2 * h2;
                    const float p0 = fast_exp2(tv[r]), p1 = fast_exp2(tv[r + 1]);
                    const float2 pq = pf_split2_hq(p0, p1, hc[h2], lc[h2]);    // the weights as the MMA sees them
                    lsum[r] = fmaf(pq.x, vinv, lsum[r]);
                    lsum[r + 1] = fmaf(pq.y, vinv, lsum[r + 1]);
                }
                hw[w] = hc[0] | (hc[1] << 16);
                lw[w] = lc[0] | (lc[1] << 16);
            }
            uint8_t *pb = smem + TC_OFF_P + b * TC_P_BYTES;
            *reinterpret_cast<uint4 *>(pb + p_hi_off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
            *reinterpret_cast<uint4 *>(pb + p_lo_off) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
            fence_async_smem();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[b]);
        }
        // ---- epilogue: this CTA's partial rows.  acc[row][dim] = (hi + lo part of O^T[dim][row]) / 128
        ok = !dead;
        TRB_TL(sm_tl, 5);
        if (ok && my_tiles > 0) ok = mbar_wait(&pv_done[(my_tiles - 1) & 1], ((my_tiles - 1) >> 1) & 1);
        tc_fence_after();
        TRB_TL(sm_tl, 6);
        if (!(flags & PDL_PRIVATE_WS)) dep_wait();                             // the workspace belongs to this launch now
        named_barrier(15, NTHREADS);                                           // the ticket (taken by the producer warp) is in sm_flag
        TRB_TL(sm_tl, 7);
        const unsigned int tag = (unsigned int)sm_flag[2] + 1u;
        const long long part_base = ((long long)j * p.nsplit + split) * p.rows_pad;
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
            float hi[16], lo[16];
            if (my_tiles > 0) {
                tmem_ld16_nowait(lane_addr + TC_TMEM_O + h * 128 + r0, hi);
                tmem_ld16_nowait(lane_addr + TC_TMEM_O + h * 128 + NROW + r0, lo);
                tmem_wait_ld();
            } else {
#pragma unroll
                for (int e = 0; e < 16; ++e) hi[e] = lo[e] = 0.f;
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const int r = r0 + e;
                if (r < p.rows) p.part_acc[(part_base + r) * D + h * 128 + kl] = make_uint2(__float_as_uint((hi[e] + lo[e]) * 0.0078125f), tag);
            }
        }
        tc_fence_before();
        // row sums over the 128 key lanes: a butterfly that halves the rows a lane carries per step
        // (lane L ends with row L & 15 summed over the lanes of its half-warp), then one more step
        float v8[8], v4[4], v2[2], v1;
        {
            const bool up = lane & 16;
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float send = up ? lsum[r] : lsum[8 + r], keep = up ? lsum[8 + r] : lsum[r];
                v8[r] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
            }
        }
        {
            const bool up = lane & 8;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float send = up ? v8[r] : v8[4 + r], keep = up ? v8[4 + r] : v8[r];
                v4[r] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
            }
        }
        {
            const bool up = lane & 4;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float send = up ? v4[r] : v4[2 + r], keep = up ? v4[2 + r] : v4[r];
                v2[r] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
            }
        }
        {
            const bool up = lane & 2;
            const float send = up ? v2[0] : v2[1], keep = up ? v2[1] : v2[0];
            v1 = keep + __shfl_xor_sync(0xffffffffu, send, 2);
        }
        v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
        // lane L now holds the warp's sum of row 8 b4 + 4 b3 + 2 b2 + b1 (b = bits of L), twice (b0)
        const int my_row = ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
        float *g_sum = sm_wmax + 4 * 48 + rg * 64;                              // not the slow path's buffer
        if (!(lane & 1)) g_sum[qw * 16 + my_row] = v1;
        named_barrier(bar_id, 128);
        if (kl < 16 && r0 + kl < p.rows) {
            const float l = (g_sum[kl] + g_sum[16 + kl]) + (g_sum[32 + kl] + g_sum[48 + kl]);
            float cr = 0.f;                                                    // cref[kl] without dynamic register indexing
#pragma unroll
            for (int r = 0; r < 16; ++r) cr = kl == r ? cref[r] : cr;
            st_volatile_v4(p.part_ml + part_base + r0 + kl,
                           make_uint4(__float_as_uint(((unset >> kl) & 1u) ? -INFINITY : 7.f - cr), tag, __float_as_uint(l), tag));
        }
    }
    if (!(flags & PDL_PRIVATE_WS)) dep_wait();
    __syncthreads();
    if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, TC_TMEM_COLS); }
    TRB_TL(sm_tl, 8);
    TRB_TL_SET(sm_tl, 13, sm_flag[0]);
    TRB_TL_SET(sm_tl, 14, my_tiles);
    decode_tail_teams<D, NTHREADS>(p, smem, sm_flag, j, active, sm_tl);
    TRB_TL_FLUSH(sm_tl, (unsigned int)sm_flag[2], j * p.nsplit + split);
}

}  // namespace trb
