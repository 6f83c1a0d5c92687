// Split-K flash-decoding over the live length of an FP8 (e4m3 + per-row scale) or bf16 KV
// cache, with the split partial-combine fused into the tail of the same launch.
//
// Shape of the kernel (one CTA per (split, kv head), one CTA per SM):
//   * 32-key tiles of K and V stream into a ring of shared-memory stages with TMA
//     (cp.async.bulk.tensor, 128-byte swizzle), the two scale vectors with cp.async; one
//     mbarrier per stage tracks arrival, a second one the release of the stage;
//   * twelve warps, no dedicated producer.  The (query row x query head) rows of this kv head
//     are cut into slices of 8; a warp owns one slice and every KW-th tile, and the slice-0
//     warp of a tile refills its stage as soon as every slice has left it.  Per tile: S^T = K Q^T and
//     O^T += V^T P^T on mma.sync with the KEYS (resp. head dims) as the 16-row operand, so
//     the 6..48 query rows fill n = 8 columns instead of padding a 16-row tile;
//   * FP8 caches: e4m3 codes become f16 in registers (one cvt per pair, exact) and feed f16
//     MMAs (m16n8k16) against an f16 copy of the query and f16 probabilities; the per-key
//     scales are applied to the fp32 scores, and the V scale is moved into the exponent of
//     the probability, so the codes themselves are never scaled.  (mma.sync with e4m3
//     operands is not native on sm_100: it compiles to conversions plus f16 MMAs plus
//     separate fp32 adds, several times the instruction count of converting once.)
//   * bf16 caches: bf16 MMAs (m16n8k16), operands straight from ldmatrix;
//   * online softmax in registers with warp shuffles; every warp keeps its own running
//     (max, sum, acc) and the warps of a CTA, the CTAs of a kv head and (for sequence
//     shards) the GPUs are all merged with the same log-sum-exp formula in a fixed order;
//   * every CTA writes one (max, sum, acc) partial per row and takes an atomic ticket of its
//     kv head; the last arrival publishes an epoch and resets the ticket (so the launch
//     replays inside a CUDA graph).  The last arrivals, as many as there are output rows (or
//     row pairs), stay until the ticket shows that every split has arrived (bounded) and take
//     the rows that their arrival number assigns them: a row's split partials are fetched in
//     one round trip, merged in split order, gated if asked, and written as bf16 - or, for a
//     sequence shard, pushed to the peers' exchange buffers and merged in rank order.
//   * programmatic dependent launch: tiles that the preceding append cannot touch are
//     requested before griddepcontrol.wait, so the prologue overlaps the append's tail.
//
// The live length and all split ranges are derived on the device from the cursor, so the
// grid is static and one captured graph serves every length.
#include "common.cuh"
#include "tmap.h"

namespace trb {

constexpr int DEC_BN = 32;                       // keys per pipeline stage = one unit of work
constexpr int DEC_CONSUMERS = 12;                // warps per CTA (all consume; the slice-0 warps also issue their stream's loads)
constexpr int DEC_HALF_WARPS = 6;                // ... of the half-size CTA, two of which fit one SM (see launch_decode)
constexpr int DEC_MAX_ROWS = 48;                 // (hq / hkv) * m
constexpr int DEC_MAX_NT = DEC_MAX_ROWS / 8;
constexpr int DEC_MIN_TILES = 4;                 // a split is not made smaller than this
constexpr int DEC_STAGE_BYTES_PER_WARP = 16 * 1024;   // pipeline stages: 192 KB for 12 warps, 96 KB for 6
constexpr int DEC_MAX_SPLITS = 148;              // bounds the tail's weight table in shared memory
constexpr int DEC_EPI_PAD = 4;                   // floats of padding per staged output row

struct DecodeParams {
    const __nv_bfloat16 *q;
    __nv_bfloat16 *out;
    const __nv_bfloat16 *gate;
    long long gate_rs, gate_hs;
    const float *ks, *vs;
    int m, hq, hkv, g, rows;      // rows = g * m
    int nt, kw;                   // 8-row slices, tiles in flight per slice (nt * kw <= 12)
    int nsplit, rows_pad;
    float scale_log2;             // softmax scale * log2(e)
    int new_rows, window, n_extra;
    const float *extra_ml, *extra_acc;
    Cursor pos;
    long long max_len, ring, shard_lo;
    int sharded;
    int tail_rows_per_helper;     // output rows merged by one helper CTA (several when its shared memory holds two rows' partials)
    int tail_teams;               // the launch ends with decode_tail_teams (tensor-core kernel)
    unsigned int xtag_mul, xtag_add;  // exchange tag = workspace epoch * xtag_mul + xtag_add + 1 (rotation of workspaces)
    int pdl_flags;                // PDL_*: what this launch may touch before its dependency wait
    // rows pos .. pos + m - 1 taken from the source rows of the append that is still writing them
    // (fresh_k == nullptr: they are read from the cache like every other row)
    const __nv_bfloat16 *fresh_k, *fresh_v;
    long long fresh_hs, fresh_rs; // element strides of the source: head, row
    unsigned long long *word;     // [hkv] ticket words: launch epoch << 16 | CTAs arrived
    uint4 *part_ml;               // [hkv][nsplit][rows_pad] (max, tag, sum, tag)
    uint2 *part_acc;              // [hkv][nsplit][rows_pad][D] (value, tag)
    float *shard_ml, *shard_acc;
    void *p2p_ptr[8];             // sequence shards: every GPU's exchange buffer as mapped here
    int p2p_world, p2p_rank;      // p2p_world == 0: no exchange
};

template <int D, bool FP8, int NW = DEC_CONSUMERS>
struct DecodeCfg {
    static constexpr int MAXNT = NW == DEC_CONSUMERS ? DEC_MAX_NT : 1;   // the half-size CTA serves one 8-row slice (M = 1)
    static constexpr int ROWB = D * (FP8 ? 1 : 2);
    static constexpr int SEGS = ROWB / 128;
    static constexpr int TILE = DEC_BN * ROWB;
    static constexpr int NSTAGE_RAW = NW * DEC_STAGE_BYTES_PER_WARP / (2 * TILE);
    static constexpr int NSTAGE = NSTAGE_RAW > 16 ? 16 : NSTAGE_RAW;
    static constexpr int NCP = ROWB / 32;                        // 32-byte chunk pairs per row
    static constexpr int ACC = FP8 ? NCP * 2 : NCP;              // m16n8 accumulator tiles
    static constexpr int QF_WORDS = FP8 ? 4 : 2;                 // query-fragment words per (slice, cp, lane)
    static constexpr int SCALE_OFF = NSTAGE * 2 * TILE;          // [NSTAGE][2][BN] floats
    static constexpr int BAR_OFF = SCALE_OFF + NSTAGE * 2 * DEC_BN * 4;
    static constexpr int QF_OFF = BAR_OFF + 2 * NSTAGE * 8;      // [MAXNT][NCP][32][QF_WORDS] words
    static constexpr int QF_BYTES = MAXNT * NCP * 32 * QF_WORDS * 4;
    static constexpr int MISC_OFF = QF_OFF + QF_BYTES;
    static constexpr int ML_BYTES = NW * 8 * 2 * 4;              // per-warp (max, sum) of 8 columns
    static constexpr int QINV_OFF = MISC_OFF + ML_BYTES;         // [MAXNT][8] floats
    static constexpr int FLAG_OFF = QINV_OFF + MAXNT * 8 * 4;
    static constexpr int TL_OFF = FLAG_OFF + 64;                 // timeline stamps (diagnostic build only)
    static constexpr int SMEM = TL_OFF + 128 + 1024;             // + slack to align the base
    static_assert(SMEM <= (NW == DEC_CONSUMERS ? 227 : 113) * 1024, "shared memory budget (two half-size CTAs per SM)");
};

// Byte offset of (row, byte_in_row) inside a K or V tile in shared memory.  A tile is stored as
// ROWB / 128 column blocks of [DEC_BN rows][128 bytes], each written by one TMA copy with the
// 128-byte swizzle (16-byte chunk index XOR row mod 8), so the eight rows that one ldmatrix
// phase reads fall into eight different bank groups.
__device__ __forceinline__ uint32_t tile_off(uint32_t row, uint32_t byte_in_row) {
    return (byte_in_row >> 7) * (DEC_BN * 128u) + row * 128u + (((((byte_in_row >> 4) & 7u) ^ (row & 7u)) << 4) | (byte_in_row & 15u));
}

// dim of accumulator element (tile a, element i) held by lane (g, t); the query column is 2t + (i & 1)
template <bool FP8>
__device__ __forceinline__ int acc_dim(int a, int i, int g) {
    if (FP8) return 32 * (a >> 1) + 16 * (i >> 1) + 2 * g + (a & 1);
    return 16 * a + 8 * (i >> 1) + g;
}

// ---- ticket, partials and tail shared by the decode kernels ------------------------------------
// Every CTA of a kv head publishes one (max, sum, acc) partial per query row in the workspace and
// the last CTAs to arrive merge them.  Nothing in this exchange is ordered by a fence or a flag:
// every 8 bytes of a partial are a (value, tag) pair, the tag being the launch's epoch + 1, and a
// reader polls the data itself until the tags are those of its own launch (bounded).  The epoch
// and the arrival number of a CTA come from ONE atomic on the kv head's ticket word
// (epoch << 16 | arrived): the CTA that completes the count adds what makes the count zero and
// the epoch one more, so the word is ready for the next launch on this workspace (which touches
// it only after its dependency wait, i.e. after this launch has completed).

// Both called by one thread of the CTA, after the dependency wait: the first issues the atomic,
// the second (as late as the caller can afford, the round trip runs in between) turns its result
// into sm_flag[0] <- helper number of this CTA (or -1: not a helper), sm_flag[2] <- epoch.
__device__ __forceinline__ unsigned long long decode_ticket_take(const DecodeParams &p, const int j) {
    return atomicAdd(p.word + j, 1ull);
}
__device__ __forceinline__ void decode_ticket(const DecodeParams &p, const int j, const int active, const int groups, int *sm_flag,
                                              const unsigned long long old) {
    const unsigned int arrival = (unsigned int)(old & 0xffffull);
    if (arrival == (unsigned int)(active - 1)) atomicAdd(p.word + j, (1ull << 16) - (unsigned long long)active);
    // More arrivals than splits: the word was not zeroed, or two launches overlap on one workspace.
    if (arrival >= (unsigned int)active) raise_status(TRB_ST_WORKSPACE);
    // The rows are merged by the last CTAs of this kv head to arrive, a helper taking every
    // helpers-th row: arrival number a makes a CTA helper a - (active - helpers); earlier arrivals
    // leave after writing their partial and free their SM for the next kernel in the stream.  Few
    // helpers, several rows each: the helpers are the CTAs that wait (for the slowest partial, and
    // for the launches before this one), so the fewer they are the fewer SMs stand still.
    int want;
    if (p.tail_teams) {                                       // decode_tail_teams: claims of two rows when there are more rows than splits
        const int rc = (p.rows > active && p.p2p_world == 0 && groups >= 2) ? 2 : 1;
        want = (p.rows + rc - 1) / rc;
    } else {
        want = (p.rows + p.tail_rows_per_helper - 1) / p.tail_rows_per_helper;
    }
    const int helpers = want < active ? want : active;
    const int h = (int)arrival - (active - helpers);
    sm_flag[0] = (h >= 0 && h < helpers) ? h : -1;
    sm_flag[2] = (int)(unsigned int)(old >> 16);
}

__device__ __forceinline__ void st_tagged4(uint2 *dst, const float4 v, const unsigned int tag) {
    st_volatile_v4(reinterpret_cast<uint4 *>(dst), make_uint4(__float_as_uint(v.x), tag, __float_as_uint(v.y), tag));
    st_volatile_v4(reinterpret_cast<uint4 *>(dst) + 1, make_uint4(__float_as_uint(v.z), tag, __float_as_uint(v.w), tag));
}

// Poll a (value, tag, value, tag) packet until both tags are `tag`; false after the limit (or,
// once a wait of this process has run out, after a short while: one stale workspace costs one
// limit, not one per row).
__device__ __forceinline__ bool poll_tagged(const uint4 *src, const unsigned int tag, uint4 &v, const unsigned int limit) {
    for (unsigned int it = 0; it < limit; ++it) {
        if (v.y == tag && v.w == tag) return true;
        if (it > 16) __nanosleep(it < 256 ? 40 : 200);
        if (it == 2048 && (*(volatile unsigned int *)&g_status & TRB_ST_WAIT_TIMEOUT)) break;
        v = ld_volatile_v4(src);
    }
    return v.y == tag && v.w == tag;
}

// Bulk copy global -> shared (size a multiple of 16 bytes, both addresses 16-byte aligned);
// completes on the mbarrier with its byte count.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Tail: LSE merge of the output rows over the active splits (+ extra partials), in split order,
// by the helper CTAs.  Called by every thread of the CTA after the CTA's own partial rows are
// on their way to the workspace and sm_flag is visible.  `smem` .. `smem + smem_bytes` is scratch
// once every thread has passed the first barrier below.
//
// A row's partials (one per active split: 2 KB at D = 256, plus the (max, sum) entries) are fetched
// into shared memory with bulk copies, all in flight at once on one mbarrier: one round trip for
// the whole row and no registers tied up.  The tags of what arrived are then checked; splits
// whose partial had not been written yet are fetched again (bounded), and only then the row is
// merged, in split order, from shared memory.  With room for two rows the next row's copies are
// in flight while this one is merged.
template <int D, int NTHREADS>
__device__ __forceinline__ void decode_tail(const DecodeParams &p, uint8_t *smem, const int smem_bytes, const int *sm_flag, const int j,
                                            const int active, unsigned long long *tl = nullptr) {
    (void)tl;
    const int helper = sm_flag[0];
    if (helper < 0) return;
    TRB_TL(tl, 9);
    const unsigned int tag = (unsigned int)sm_flag[2] + 1u;
    const int tid = threadIdx.x, lane = threadIdx.x & 31;
    constexpr int ITEMS = D / 4, GROUPS = NTHREADS / ITEMS;
    const int want = (p.rows + p.tail_rows_per_helper - 1) / p.tail_rows_per_helper;       // as in decode_ticket
    const int helpers = want < active ? want : active;
    const int max_rounds = (int)(c_wait_limit[1] >> 8) + 4;            // fetch rounds before a row gives up

    // Thread (item, group) sums the splits of its group, the groups are added in group order
    // through shared memory.
    const int n_parts = active + p.n_extra;
    const int item = tid % ITEMS, tgrp = tid / ITEMS, d4 = item * 4;
    const bool in_team = tgrp < GROUPS;                                 // (threads beyond the last whole group idle)
    constexpr int gt = GROUPS;
    // ---- shared memory of the tail
    float *sm_m = reinterpret_cast<float *>(smem);                      // [n_parts]
    float *sm_l = sm_m + (DEC_MAX_SPLITS + 4);                          // [n_parts]
    constexpr int RED_OFF = 2 * (DEC_MAX_SPLITS + 4) * 4;
    float4 *sm_red = reinterpret_cast<float4 *>(smem + RED_OFF);        // [GROUPS][ITEMS]
    constexpr int BAR_OFF = RED_OFF + GROUPS * ITEMS * 16;
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + BAR_OFF);       // [2]
    uint8_t *sm_bad_all = smem + BAR_OFF + 16;                          // [2][DEC_MAX_SPLITS + 4] split's partial not here yet
    constexpr int BAD_STRIDE = DEC_MAX_SPLITS + 4;
    constexpr int FRESH_OFF = (BAR_OFF + 16 + 2 * BAD_STRIDE + 127) / 128 * 128;
    const int n_fresh = p.fresh_k ? p.m : 0;
    float *fr_k = reinterpret_cast<float *>(smem + FRESH_OFF);          // [n_fresh][D]
    float *fr_v = fr_k + n_fresh * D;                                   // [n_fresh][D]
    float *fr_s = fr_v + n_fresh * D;                                   // [8] scores of the current row, log2 units
    int *fr_held = reinterpret_cast<int *>(fr_s + 8);                   // [8] this cache holds the row's position
    const int bulk_off = (FRESH_OFF + 2 * n_fresh * D * 4 + 64 + 127) / 128 * 128;
    const int ml_bytes = (active * 16 + 127) / 128 * 128;
    const int buf_bytes = ml_bytes + active * D * 8;                    // one row: (max, sum) entries, then the accumulators
    const int nbuf = (smem_bytes - bulk_off >= 2 * buf_bytes) ? 2 : 1;  // (the host sized the splits so that one row always fits)
    bool all_ok = true;
    uint32_t phase[2] = {0u, 0u};

    // ---- the m rows that the append of this step is still writing, from its source rows: quantised
    // and dequantised exactly as the append does (tokenrush/fused.py:336-340), kept as fp32 rows of
    // this kv head in shared memory.  They enter the merge below as one more partial.
    constexpr int EPL = D / 32;
    const int fr_row = tid >> 5;                                        // the fresh row this warp prepares (rows beyond the warp count: below)
    __nv_bfloat16 fr_raw[2][EPL];
    if (fr_row < n_fresh) {                                             // requested now, used once the partial copies are out
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            const __nv_bfloat16 *src = (which ? p.fresh_v : p.fresh_k) + (long long)j * p.fresh_hs + (long long)fr_row * p.fresh_rs + lane * EPL;
            if (EPL == 8) *reinterpret_cast<uint4 *>(fr_raw[which]) = *reinterpret_cast<const uint4 *>(src);
            else *reinterpret_cast<uint2 *>(fr_raw[which]) = *reinterpret_cast<const uint2 *>(src);
        }
    }
    // quantise + dequantise one source row held as EPL values per lane, into shared memory
    auto fresh_store = [&](int r, int which, const __nv_bfloat16 (&raw)[EPL]) {
        float f[EPL];
#pragma unroll
        for (int e = 0; e < EPL; ++e) f[e] = __bfloat162float(raw[e]);
        if (p.ks) {
            float amax = 0.f;
#pragma unroll
            for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(f[e]));
            amax = warp_max(amax);
            const float sc = __fdiv_rn(fmaxf(amax, 1e-6f), 448.0f);
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const __nv_fp8_storage_t code = __nv_cvt_float_to_fp8(__fdiv_rn(f[e], sc), __NV_SATFINITE, __NV_E4M3);
                f[e] = __half2float(__half(__nv_cvt_fp8_to_halfraw(code, __NV_E4M3))) * sc;
            }
        }
#pragma unroll
        for (int e = 0; e < EPL; ++e) (which ? fr_v : fr_k)[r * D + lane * EPL + e] = f[e];
    };

    __syncthreads();                                                    // the CTA's own partial has left shared memory: it is scratch now
    if (tid == 0) { mbar_init(&bar[0], 1u); mbar_init(&bar[1], 1u); mbar_fence_init(); }
    for (int i = tid; i < 2 * BAD_STRIDE; i += NTHREADS) sm_bad_all[i] = 1;   // nothing fetched yet
    __syncthreads();

    const long long ws_row0 = (long long)j * p.nsplit * p.rows_pad;     // first workspace row of this kv head
    // warp 0: request every split of `row` that is marked missing into buffer b (all copies on one barrier)
    auto fetch = [&](int row, int b) {
        if (tid < 32) {
            uint8_t *bad = sm_bad_all + b * BAD_STRIDE;
            uint8_t *buf = smem + bulk_off + b * buf_bytes;
            uint32_t bytes = 0;
            for (int sp = lane; sp < active; sp += 32)
                if (bad[sp]) bytes += D * 8 + 16;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) bytes += __shfl_xor_sync(0xffffffffu, bytes, off);
            if (lane == 0) { fence_proxy_async_smem(); mbar_arrive_expect_tx(&bar[b], bytes); }
            __syncwarp();
            for (int sp = lane; sp < active; sp += 32)
                if (bad[sp]) {
                    const long long wrow = ws_row0 + (long long)sp * p.rows_pad + row;
                    bulk_g2s(buf + ml_bytes + (size_t)sp * D * 8, p.part_acc + wrow * D, D * 8, &bar[b]);
                    bulk_g2s(buf + sp * 16, p.part_ml + wrow, 16, &bar[b]);
                }
        }
    };
    int nk = 0;
    for (int row = helper; row < p.rows; row += helpers) ++nk;
    if (nk > 0) fetch(helper, 0);
    if (n_fresh) {                                                      // the fresh rows of this kv head into shared memory
        const long long pos = load_cursor(p.pos);
        for (int r = fr_row; r < n_fresh; r += NTHREADS / 32) {
            if (r != fr_row) {                                          // more fresh rows than warps: fetched here
#pragma unroll
                for (int which = 0; which < 2; ++which) {
                    const __nv_bfloat16 *src = (which ? p.fresh_v : p.fresh_k) + (long long)j * p.fresh_hs + (long long)r * p.fresh_rs + lane * EPL;
                    if (EPL == 8) *reinterpret_cast<uint4 *>(fr_raw[which]) = *reinterpret_cast<const uint4 *>(src);
                    else *reinterpret_cast<uint2 *>(fr_raw[which]) = *reinterpret_cast<const uint2 *>(src);
                }
            }
            fresh_store(r, 0, fr_raw[0]);
            fresh_store(r, 1, fr_raw[1]);
            const long long loc = pos + r - p.shard_lo;                 // a sequence shard holds a range of positions
            if (lane == 0) fr_held[r] = (loc >= 0 && loc < p.max_len) ? 1 : 0;
        }
    }
    for (int k = 0; k < nk; ++k) {
        const int row = helper + k * helpers, b = nbuf == 2 ? (k & 1) : 0;
        const bool row_on = in_team;
        const int qi = row / p.g, hq = j * p.g + row % p.g;
        const long long grow = (long long)qi * p.hq + hq;
        uint8_t *bad = sm_bad_all + b * BAD_STRIDE;
        const uint4 *bk_ml = reinterpret_cast<const uint4 *>(smem + bulk_off + b * buf_bytes);
        const uint4 *bk_acc = reinterpret_cast<const uint4 *>(smem + bulk_off + b * buf_bytes + ml_bytes);
        if (nbuf == 2 && k + 1 < nk) fetch(row + helpers, b ^ 1);      // the next row's copies fly while this row is merged
        // ---- fetch rounds of this row
        for (int round = 0;; ++round) {
            const bool landed = mbar_wait(&bar[b], phase[b]);
            phase[b] ^= 1u;
            __syncthreads();                                            // warp 0 has read the old marks
            for (int i = tid; i < BAD_STRIDE; i += NTHREADS) bad[i] = 0;
            __syncthreads();
            // check the tags of everything this thread will use
            bool miss = !landed;
            if (in_team)
                for (int sp = tgrp; sp < active; sp += gt) {
                    const uint4 a0 = bk_acc[(size_t)sp * (D / 2) + item * 2], a1 = bk_acc[(size_t)sp * (D / 2) + item * 2 + 1];
                    if (!(a0.y == tag && a0.w == tag && a1.y == tag && a1.w == tag)) { bad[sp] = 1; miss = true; }
                }
            for (int sp = tid; sp < active; sp += NTHREADS) {
                const uint4 w = bk_ml[sp];
                if (!(w.y == tag && w.w == tag)) { bad[sp] = 1; miss = true; }
            }
            if (!__syncthreads_or(miss ? 1 : 0)) break;                 // the whole row is here
            // give up after the limit (or soon, once a wait of this process has run out: a stale workspace
            // costs one limit, not one per row); one thread decides for all
            const bool stop = tid == 0 && (round >= max_rounds || (round >= 8 && (*(volatile unsigned int *)&g_status & TRB_ST_WAIT_TIMEOUT)));
            if (__syncthreads_or(stop ? 1 : 0)) {
                all_ok = false;                                         // the missing splits count as empty
                break;
            }
            __nanosleep(round < 4 ? 100 : 500);
            fetch(row, b);
        }
        // ---- (max, sum) of all splits, the scores of the fresh keys, the weights' reference
        for (int sp = tid; sp < n_parts; sp += NTHREADS) {
            float2 v;
            if (sp < active) {
                const uint4 w = bk_ml[sp];
                v = (w.y == tag && w.w == tag) ? make_float2(__uint_as_float(w.x), __uint_as_float(w.z)) : make_float2(-INFINITY, 0.f);
            } else {
                v = *reinterpret_cast<const float2 *>(&p.extra_ml[(grow * p.n_extra + (sp - active)) * 2]);
            }
            sm_m[sp] = v.x; sm_l[sp] = v.y;
        }
        if (n_fresh) {                                                  // one warp per fresh key
            const __nv_bfloat16 *qp = p.q + grow * D + lane * EPL;
            for (int r = tid >> 5; r < n_fresh; r += NTHREADS / 32) {
                float dot = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) dot = fmaf(__bfloat162float(qp[e]), fr_k[r * D + lane * EPL + e], dot);
                dot = warp_sum(dot);
                if (lane == 0) fr_s[r] = dot * p.scale_log2;
            }
        }
        __syncthreads();
        TRB_TL(tl, 10);
        float mmax = -INFINITY, lsum = 0.f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row_on) {
            for (int sp = lane; sp < n_parts; sp += 32) mmax = fmaxf(mmax, sm_m[sp]);
            mmax = warp_max(mmax);
            // fresh keys 0..qi are visible to query row qi (tokenrush/fused.py:382: keys <= pos + qi)
            const int n_vis = n_fresh ? (qi + 1 < n_fresh ? qi + 1 : n_fresh) : 0;
            for (int r = 0; r < n_vis; ++r)
                if (fr_held[r]) mmax = fmaxf(mmax, fr_s[r]);
            for (int sp = lane; sp < n_parts; sp += 32) lsum += sm_m[sp] == -INFINITY ? 0.f : fast_exp2(sm_m[sp] - mmax) * sm_l[sp];
            lsum = warp_sum(lsum);
            for (int r = 0; r < n_vis; ++r)
                if (fr_held[r]) {
                    const float w = fast_exp2(fr_s[r] - mmax);
                    lsum += w;
                    if (tgrp == 0) {
                        const float4 v = *reinterpret_cast<const float4 *>(&fr_v[r * D + d4]);
                        o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
                    }
                }
            // the accumulators, split order within the group: ascending
            for (int sp = tgrp; sp < active; sp += gt) {
                const uint4 a0 = bk_acc[(size_t)sp * (D / 2) + item * 2], a1 = bk_acc[(size_t)sp * (D / 2) + item * 2 + 1];
                const bool here = a0.y == tag && a0.w == tag && a1.y == tag && a1.w == tag;
                const float w = (sm_m[sp] == -INFINITY || !here) ? 0.f : fast_exp2(sm_m[sp] - mmax);
                o.x = fmaf(w, __uint_as_float(a0.x), o.x); o.y = fmaf(w, __uint_as_float(a0.z), o.y);
                o.z = fmaf(w, __uint_as_float(a1.x), o.z); o.w = fmaf(w, __uint_as_float(a1.z), o.w);
            }
            if (tgrp == 0)
                for (int e = 0; e < p.n_extra; ++e) {
                    const float4 v = *reinterpret_cast<const float4 *>(&p.extra_acc[(grow * p.n_extra + e) * D + d4]);
                    const float w = sm_m[active + e] == -INFINITY ? 0.f : fast_exp2(sm_m[active + e] - mmax);
                    o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
                }
            sm_red[tgrp * ITEMS + item] = o;
        }
        for (int i = tid; i < BAD_STRIDE; i += NTHREADS) bad[i] = 1;   // the buffer's next row: nothing fetched yet
        __syncthreads();                                                // ... and the buffer may be refilled
        TRB_TL(tl, 11);
        if (nbuf == 1 && k + 1 < nk) fetch(row + helpers, 0);
        const bool lead = row_on && tgrp == 0;                           // these threads hold the row from here on
        if (lead) {
            for (int kk = 1; kk < gt; ++kk) {
                const float4 v = sm_red[kk * ITEMS + item];
                o.x += v.x; o.y += v.y; o.z += v.z; o.w += v.w;
            }
        }
        // Outputs (and the exchange with other GPUs) only once every earlier launch is complete.  The
        // helpers are the CTAs of a launch that always wait, so a launch never completes before
        // the launches it follows; with a private workspace the other CTAs have left without waiting.
        pdl_wait();
        if (p.shard_acc) {
            if (lead) {
                *reinterpret_cast<float4 *>(&p.shard_acc[grow * D + d4]) = o;
                if (item == 0) { p.shard_ml[grow * 2] = mmax; p.shard_ml[grow * 2 + 1] = lsum; }
            }
            continue;
        }
        if (p.p2p_world > 1 && lead) {
            // ---- sequence shards: exchange this row's (max, sum, acc) with the other GPUs by peer
            // stores, wait (bounded) for theirs, merge in rank order.  Every 8 bytes that cross the
            // link are (value, tag): the receiver polls the data itself, so there is no flag, no fence
            // and no second message.  The tag is this kv head's launch epoch + 1, identical on all GPUs
            // because they make the same calls on their workspaces; slots rotate over P2P_SLOTS calls
            // (a GPU cannot be more than one call ahead of a peer whose packets it waits for).  This
            // GPU's own partial stays in registers.
            const P2PLayout xl = p2p_layout(p.p2p_world, p.m * p.hq, D);
            // the exchange counts the calls on this GPU's rotation of workspaces: every GPU makes the same calls
            const unsigned int xtag = ((unsigned int)sm_flag[2]) * p.xtag_mul + p.xtag_add + 1u;
            const size_t slot = xtag % P2P_SLOTS;
            const size_t nrow = (size_t)(p.m * p.hq);
            const uint4 k0 = make_uint4(__float_as_uint(o.x), xtag, __float_as_uint(o.y), xtag);
            const uint4 k1 = make_uint4(__float_as_uint(o.z), xtag, __float_as_uint(o.w), xtag);
            const uint4 k2 = make_uint4(__float_as_uint(mmax), xtag, __float_as_uint(lsum), xtag);
            for (int r = 0; r < p.p2p_world; ++r) {
                if (r == p.p2p_rank) continue;
                uint4 *dst = reinterpret_cast<uint4 *>((uint8_t *)p.p2p_ptr[r] + xl.ll) +
                             (((slot * p.p2p_world + p.p2p_rank) * nrow + grow) * ITEMS + item) * 3;
                st_volatile_v4(dst, k0); st_volatile_v4(dst + 1, k1); st_volatile_v4(dst + 2, k2);
            }
            const uint4 *local = reinterpret_cast<const uint4 *>((const uint8_t *)p.p2p_ptr[p.p2p_rank] + xl.ll);
            // one polling loop over all peers: a peer's three packets are taken when all six tags match
            const unsigned int plimit = c_wait_limit[2];
            uint4 pk[P2P_MAX_WORLD][3];
            unsigned int pending = 0u;
            for (int r = 0; r < p.p2p_world; ++r)
                if (r != p.p2p_rank) pending |= 1u << r;
            for (unsigned int it = 0; it < plimit && pending; ++it) {
#pragma unroll
                for (int r = 0; r < P2P_MAX_WORLD; ++r) {
                    if (!((pending >> r) & 1u)) continue;
                    const uint4 *src = local + (((slot * p.p2p_world + r) * nrow + grow) * ITEMS + item) * 3;
                    const uint4 b0 = ld_volatile_v4(src), b1 = ld_volatile_v4(src + 1), b2 = ld_volatile_v4(src + 2);
                    if (b0.y == xtag && b0.w == xtag && b1.y == xtag && b1.w == xtag && b2.y == xtag && b2.w == xtag) {
                        pk[r][0] = b0; pk[r][1] = b1; pk[r][2] = b2;
                        pending &= ~(1u << r);
                    }
                }
                if (it > 64) __nanosleep(100);
                // once a wait of this process has run out, later ones give up early: a lost peer costs
                // one limit, not one limit per row and layer
                if (it == 4096 && (*(volatile unsigned int *)&g_status & TRB_ST_PEER_TIMEOUT)) break;
            }
            if (pending) {
                raise_status(TRB_ST_PEER_TIMEOUT);
            } else {
                float gm = mmax;
#pragma unroll
                for (int r = 0; r < P2P_MAX_WORLD; ++r)
                    if (r < p.p2p_world && r != p.p2p_rank) gm = fmaxf(gm, __uint_as_float(pk[r][2].x));
                // weights and sums in rank order, own partial from registers
                float gl = 0.f;
                float4 go = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int r = 0; r < P2P_MAX_WORLD; ++r) {
                    if (r >= p.p2p_world) continue;
                    float2 mlr = make_float2(mmax, lsum);
                    float4 v = o;
                    if (r != p.p2p_rank) {
                        v = make_float4(__uint_as_float(pk[r][0].x), __uint_as_float(pk[r][0].z), __uint_as_float(pk[r][1].x), __uint_as_float(pk[r][1].z));
                        mlr = make_float2(__uint_as_float(pk[r][2].x), __uint_as_float(pk[r][2].z));
                    }
                    const float w = mlr.x == -INFINITY ? 0.f : fast_exp2(mlr.x - gm);
                    gl = fmaf(w, mlr.y, gl);
                    go.x = fmaf(w, v.x, go.x); go.y = fmaf(w, v.y, go.y); go.z = fmaf(w, v.z, go.z); go.w = fmaf(w, v.w, go.w);
                }
                o = go; lsum = gl;
            }
        }
        if (!lead) continue;
        const float inv = 1.f / lsum;
        float r[4] = {o.x * inv, o.y * inv, o.z * inv, o.w * inv};
        __nv_bfloat16 ob[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) ob[e] = __float2bfloat16_rn(r[e]);
        if (p.gate) {
            const __nv_bfloat16 *gp = p.gate + (long long)qi * p.gate_rs + (long long)hq * p.gate_hs + d4;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float gv = __bfloat162float(gp[e]);
                const float sg = __bfloat162float(__float2bfloat16_rn(1.f / (1.f + __expf(-gv))));
                ob[e] = __float2bfloat16_rn(__bfloat162float(ob[e]) * sg);
            }
        }
        *reinterpret_cast<uint2 *>(&p.out[grow * D + d4]) = *reinterpret_cast<const uint2 *>(ob);
    }
    if (!all_ok) raise_status(TRB_ST_WAIT_TIMEOUT);
}

// The tail of the tensor-core kernel (M-row verify): the same merge as decode_tail, with the
// partials loaded straight into registers and two rows per claim.  That kernel fills an SM alone and
// all its CTAs finish together, so many helpers with one short claim each (one round trip) cost less
// SM time than few helpers that fetch row after row.
// LSE merge of the output rows over the active splits (+ extra partials), in split order,
// by the helper CTAs.  Called by every thread of the CTA after the CTA's own partial rows are
// on their way to the workspace and sm_flag is visible.  `smem` is scratch from its start (at
// least 16 KB) once every thread has passed the barrier below.
template <int D, int NTHREADS>
__device__ __forceinline__ void decode_tail_teams(const DecodeParams &p, uint8_t *smem, const int *sm_flag, const int j, const int active,
                                            unsigned long long *tl = nullptr) {
    (void)tl;
    const int helper = sm_flag[0];
    if (helper < 0) return;
    TRB_TL(tl, 9);
    const unsigned int tag = (unsigned int)sm_flag[2] + 1u;
    const int tid = threadIdx.x, lane = threadIdx.x & 31;
    constexpr int ITEMS = D / 4, GROUPS = NTHREADS / ITEMS;
    const int rc = (p.rows > active && p.p2p_world == 0 && GROUPS >= 2) ? 2 : 1;     // as in decode_ticket
    const int nclaims = (p.rows + rc - 1) / rc;
    const int helpers = nclaims < active ? nclaims : active;
    const unsigned int limit = c_wait_limit[1];

    // Thread (item, group) sums the splits of its group, the groups are added in group order
    // through shared memory.  With more rows than splits (M-row verify) a claim takes two rows and
    // the thread groups form two teams, one per row, so that one round of claims covers all rows.
    const int n_parts = active + p.n_extra;
    const int gt = GROUPS / rc;                                         // groups per team
    const int item = tid % ITEMS, grp = tid / ITEMS, d4 = item * 4;
    const int team = grp / gt, tgrp = grp - team * gt;                 // team >= rc: idle threads
    const int ttid = tid - team * gt * ITEMS, team_threads = gt * ITEMS;
    const bool in_team = team < rc;
    float *sm_m = reinterpret_cast<float *>(smem) + (in_team ? team : 0) * 2 * (DEC_MAX_SPLITS + 4);   // [n_parts] per team
    float *sm_l = sm_m + (DEC_MAX_SPLITS + 4);                          // [n_parts]
    float4 *sm_red = reinterpret_cast<float4 *>(reinterpret_cast<float *>(smem) + 4 * (DEC_MAX_SPLITS + 4)) +
                     (in_team ? team : 0) * gt * ITEMS;                 // [gt][ITEMS] per team
    constexpr int PRE = NTHREADS >= 384 ? 8 : 13;                       // splits per thread requested together
    bool all_ok = true;

    // ---- the m rows that the append of this step is still writing, from its source rows: quantised
    // and dequantised exactly as the append does (tokenrush/fused.py:336-340), kept as fp32 rows of
    // this kv head in shared memory.  They enter the merge below as one more partial.
    float *fr_k = reinterpret_cast<float *>(smem + 16384);              // [8][D]
    float *fr_v = fr_k + 8 * D;                                         // [8][D]
    float *fr_s = fr_v + 8 * D;                                         // [2 teams][8] scores, log2 units
    int *fr_held = reinterpret_cast<int *>(fr_s + 16);                  // [8] this cache holds the row's position
    const int n_fresh = p.fresh_k ? p.m : 0;
    if (n_fresh) {
        __syncthreads();                                                // the CTA's own partial has left shared memory
        const long long pos = load_cursor(p.pos);
        constexpr int EPL = D / 32;
        for (int r = tid >> 5; r < n_fresh; r += NTHREADS / 32) {
            const long long loc = pos + r - p.shard_lo;
            for (int which = 0; which < 2; ++which) {
                const __nv_bfloat16 *src = (which ? p.fresh_v : p.fresh_k) + (long long)j * p.fresh_hs + (long long)r * p.fresh_rs;
                float f[EPL];
                __nv_bfloat16 raw[EPL];
                load_row<EPL>(src, lane, f, raw);
                if (p.ks) {
                    float amax = 0.f;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(f[e]));
                    amax = warp_max(amax);
                    const float sc = __fdiv_rn(fmaxf(amax, 1e-6f), 448.0f);
#pragma unroll
                    for (int e = 0; e < EPL; ++e) {
                        const __nv_fp8_storage_t code = __nv_cvt_float_to_fp8(__fdiv_rn(f[e], sc), __NV_SATFINITE, __NV_E4M3);
                        f[e] = __half2float(__half(__nv_cvt_fp8_to_halfraw(code, __NV_E4M3))) * sc;
                    }
                }
#pragma unroll
                for (int e = 0; e < EPL; ++e) (which ? fr_v : fr_k)[r * D + lane * EPL + e] = f[e];
            }
            if (lane == 0) fr_held[r] = (p.ring > 0 || (loc >= 0 && loc < p.max_len)) ? 1 : 0;
        }
    }
    for (int c = helper; c < nclaims; c += helpers) {
        __syncthreads();                                                // the shared memory below is free (first claim: the CTA's own partial has left it)
        const int row = c * rc + team;
        const bool row_on = in_team && row < p.rows;
        const int qi = row_on ? row / p.g : 0, hq = row_on ? j * p.g + row % p.g : 0;
        const long long grow = (long long)qi * p.hq + hq;
        // one round trip: the (max, sum) pairs of all splits and this thread's first slices of the
        // accumulators are requested together; whatever has not arrived yet is polled afterwards
        const uint4 *pa = reinterpret_cast<const uint4 *>(p.part_acc + ((long long)j * p.nsplit * p.rows_pad + (row_on ? row : 0)) * D + d4);
        const long long pstride = (long long)p.rows_pad * D / 2;        // uint4 (two pairs) per split
        uint4 a0[PRE], a1[PRE];
#pragma unroll
        for (int u = 0; u < PRE; ++u) {
            const int sp = tgrp + u * gt;
            if (row_on && sp < active) { a0[u] = ld_volatile_v4(pa + sp * pstride); a1[u] = ld_volatile_v4(pa + sp * pstride + 1); }
            else { a0[u] = make_uint4(0u, tag, 0u, tag); a1[u] = a0[u]; }
        }
        if (row_on)
            for (int sp = ttid; sp < n_parts; sp += team_threads) {
                float2 v;
                if (sp < active) {
                    const uint4 *src = p.part_ml + ((long long)j * p.nsplit + sp) * p.rows_pad + row;
                    uint4 w = ld_volatile_v4(src);
                    if (!poll_tagged(src, tag, w, limit)) { all_ok = false; w.x = __float_as_uint(-INFINITY); w.z = 0u; }
                    v = make_float2(__uint_as_float(w.x), __uint_as_float(w.z));
                } else {
                    v = *reinterpret_cast<const float2 *>(&p.extra_ml[(grow * p.n_extra + (sp - active)) * 2]);
                }
                sm_m[sp] = v.x; sm_l[sp] = v.y;
            }
        if (n_fresh && row_on) {                                        // scores of this row against the fresh keys, one warp per key
            constexpr int EPL = D / 32;
            const __nv_bfloat16 *qp = p.q + grow * D + lane * EPL;
            for (int r = ttid >> 5; r < n_fresh; r += team_threads / 32) {
                float dot = 0.f;
#pragma unroll
                for (int e = 0; e < EPL; ++e) dot = fmaf(__bfloat162float(qp[e]), fr_k[r * D + lane * EPL + e], dot);
                dot = warp_sum(dot);
                if (lane == 0) fr_s[team * 8 + r] = dot * p.scale_log2;
            }
        }
        __syncthreads();
        TRB_TL(tl, 10);
        float mmax = -INFINITY, lsum = 0.f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row_on) {
            for (int sp = lane; sp < n_parts; sp += 32) mmax = fmaxf(mmax, sm_m[sp]);
            mmax = warp_max(mmax);
            // fresh keys 0..qi are visible to query row qi (tokenrush/fused.py:382: keys <= pos + qi)
            const int n_vis = n_fresh ? (qi + 1 < n_fresh ? qi + 1 : n_fresh) : 0;
            for (int r = 0; r < n_vis; ++r)
                if (fr_held[r]) mmax = fmaxf(mmax, fr_s[team * 8 + r]);
            for (int sp = lane; sp < n_parts; sp += 32) lsum += sm_m[sp] == -INFINITY ? 0.f : fast_exp2(sm_m[sp] - mmax) * sm_l[sp];
            lsum = warp_sum(lsum);
            for (int r = 0; r < n_vis; ++r)
                if (fr_held[r]) {
                    const float w = fast_exp2(fr_s[team * 8 + r] - mmax);
                    lsum += w;
                    if (tgrp == 0) {
                        const float4 v = *reinterpret_cast<const float4 *>(&fr_v[r * D + d4]);
                        o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
                    }
                }
            for (int sp0 = tgrp; sp0 < active; sp0 += PRE * gt) {         // split order within the group: ascending
                if (sp0 != tgrp) {
#pragma unroll
                    for (int u = 0; u < PRE; ++u) {
                        const int sp = sp0 + u * gt;
                        if (sp < active) { a0[u] = ld_volatile_v4(pa + sp * pstride); a1[u] = ld_volatile_v4(pa + sp * pstride + 1); }
                    }
                }
#pragma unroll
                for (int u = 0; u < PRE; ++u) {
                    const int sp = sp0 + u * gt;
                    if (sp < active) {
                        const bool here = poll_tagged(pa + sp * pstride, tag, a0[u], limit) && poll_tagged(pa + sp * pstride + 1, tag, a1[u], limit);
                        if (!here) all_ok = false;
                        const float w = (sm_m[sp] == -INFINITY || !here) ? 0.f : fast_exp2(sm_m[sp] - mmax);
                        o.x = fmaf(w, __uint_as_float(a0[u].x), o.x); o.y = fmaf(w, __uint_as_float(a0[u].z), o.y);
                        o.z = fmaf(w, __uint_as_float(a1[u].x), o.z); o.w = fmaf(w, __uint_as_float(a1[u].z), o.w);
                    }
                }
            }
            if (tgrp == 0)
                for (int e = 0; e < p.n_extra; ++e) {
                    const float4 v = *reinterpret_cast<const float4 *>(&p.extra_acc[(grow * p.n_extra + e) * D + d4]);
                    const float w = sm_m[active + e] == -INFINITY ? 0.f : fast_exp2(sm_m[active + e] - mmax);
                    o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
                }
            sm_red[tgrp * ITEMS + item] = o;
        }
        __syncthreads();
        TRB_TL(tl, 11);
        const bool lead = row_on && tgrp == 0;                           // these threads hold the row from here on
        if (lead) {
            for (int k = 1; k < gt; ++k) {
                const float4 v = sm_red[k * ITEMS + item];
                o.x += v.x; o.y += v.y; o.z += v.z; o.w += v.w;
            }
        }
        // Outputs (and the exchange with other GPUs) only once every earlier launch is complete.  The
        // helpers are the CTAs of a launch that always wait, so a launch never completes before
        // the launches it follows; with a private workspace the other CTAs have left without waiting.
        pdl_wait();
        if (p.shard_acc) {
            if (lead) {
                *reinterpret_cast<float4 *>(&p.shard_acc[grow * D + d4]) = o;
                if (item == 0) { p.shard_ml[grow * 2] = mmax; p.shard_ml[grow * 2 + 1] = lsum; }
            }
            continue;
        }
        if (p.p2p_world > 1 && lead) {
            // ---- sequence shards: exchange this row's (max, sum, acc) with the other GPUs by peer
            // stores, wait (bounded) for theirs, merge in rank order.  Every 8 bytes that cross the
            // link are (value, tag): the receiver polls the data itself, so there is no flag, no fence
            // and no second message.  The tag is this kv head's launch epoch + 1, identical on all GPUs
            // because they make the same calls on their workspaces; slots rotate over P2P_SLOTS calls
            // (a GPU cannot be more than one call ahead of a peer whose packets it waits for).  This
            // GPU's own partial stays in registers.
            const P2PLayout xl = p2p_layout(p.p2p_world, p.m * p.hq, D);
            // the exchange counts the calls on this GPU's rotation of workspaces: every GPU makes the same calls
            const unsigned int xtag = ((unsigned int)sm_flag[2]) * p.xtag_mul + p.xtag_add + 1u;
            const size_t slot = xtag % P2P_SLOTS;
            const size_t nrow = (size_t)(p.m * p.hq);
            const uint4 k0 = make_uint4(__float_as_uint(o.x), xtag, __float_as_uint(o.y), xtag);
            const uint4 k1 = make_uint4(__float_as_uint(o.z), xtag, __float_as_uint(o.w), xtag);
            const uint4 k2 = make_uint4(__float_as_uint(mmax), xtag, __float_as_uint(lsum), xtag);
            for (int r = 0; r < p.p2p_world; ++r) {
                if (r == p.p2p_rank) continue;
                uint4 *dst = reinterpret_cast<uint4 *>((uint8_t *)p.p2p_ptr[r] + xl.ll) +
                             (((slot * p.p2p_world + p.p2p_rank) * nrow + grow) * ITEMS + item) * 3;
                st_volatile_v4(dst, k0); st_volatile_v4(dst + 1, k1); st_volatile_v4(dst + 2, k2);
            }
            const uint4 *local = reinterpret_cast<const uint4 *>((const uint8_t *)p.p2p_ptr[p.p2p_rank] + xl.ll);
            // one polling loop over all peers: a peer's three packets are taken when all six tags match
            const unsigned int plimit = c_wait_limit[2];
            uint4 pk[P2P_MAX_WORLD][3];
            unsigned int pending = 0u;
            for (int r = 0; r < p.p2p_world; ++r)
                if (r != p.p2p_rank) pending |= 1u << r;
            for (unsigned int it = 0; it < plimit && pending; ++it) {
#pragma unroll
                for (int r = 0; r < P2P_MAX_WORLD; ++r) {
                    if (!((pending >> r) & 1u)) continue;
                    const uint4 *src = local + (((slot * p.p2p_world + r) * nrow + grow) * ITEMS + item) * 3;
                    const uint4 b0 = ld_volatile_v4(src), b1 = ld_volatile_v4(src + 1), b2 = ld_volatile_v4(src + 2);
                    if (b0.y == xtag && b0.w == xtag && b1.y == xtag && b1.w == xtag && b2.y == xtag && b2.w == xtag) {
                        pk[r][0] = b0; pk[r][1] = b1; pk[r][2] = b2;
                        pending &= ~(1u << r);
                    }
                }
                if (it > 64) __nanosleep(100);
                // once a wait of this process has run out, later ones give up early: a lost peer costs
                // one limit, not one limit per row and layer
                if (it == 4096 && (*(volatile unsigned int *)&g_status & TRB_ST_PEER_TIMEOUT)) break;
            }
            if (pending) {
                raise_status(TRB_ST_PEER_TIMEOUT);
            } else {
                float gm = mmax;
#pragma unroll
                for (int r = 0; r < P2P_MAX_WORLD; ++r)
                    if (r < p.p2p_world && r != p.p2p_rank) gm = fmaxf(gm, __uint_as_float(pk[r][2].x));
                // weights and sums in rank order, own partial from registers
                float gl = 0.f;
                float4 go = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int r = 0; r < P2P_MAX_WORLD; ++r) {
                    if (r >= p.p2p_world) continue;
                    float2 mlr = make_float2(mmax, lsum);
                    float4 v = o;
                    if (r != p.p2p_rank) {
                        v = make_float4(__uint_as_float(pk[r][0].x), __uint_as_float(pk[r][0].z), __uint_as_float(pk[r][1].x), __uint_as_float(pk[r][1].z));
                        mlr = make_float2(__uint_as_float(pk[r][2].x), __uint_as_float(pk[r][2].z));
                    }
                    const float w = mlr.x == -INFINITY ? 0.f : fast_exp2(mlr.x - gm);
                    gl = fmaf(w, mlr.y, gl);
                    go.x = fmaf(w, v.x, go.x); go.y = fmaf(w, v.y, go.y); go.z = fmaf(w, v.z, go.z); go.w = fmaf(w, v.w, go.w);
                }
                o = go; lsum = gl;
            }
        }
        if (!lead) continue;
        const float inv = 1.f / lsum;
        float r[4] = {o.x * inv, o.y * inv, o.z * inv, o.w * inv};
        __nv_bfloat16 ob[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) ob[e] = __float2bfloat16_rn(r[e]);
        if (p.gate) {
            const __nv_bfloat16 *gp = p.gate + (long long)qi * p.gate_rs + (long long)hq * p.gate_hs + d4;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float gv = __bfloat162float(gp[e]);
                const float sg = __bfloat162float(__float2bfloat16_rn(1.f / (1.f + __expf(-gv))));
                ob[e] = __float2bfloat16_rn(__bfloat162float(ob[e]) * sg);
            }
        }
        *reinterpret_cast<uint2 *>(&p.out[grow * D + d4]) = *reinterpret_cast<const uint2 *>(ob);
    }
    if (!all_ok) raise_status(TRB_ST_WAIT_TIMEOUT);
}

}  // namespace trb

#include "decode_tc.cuh"

namespace trb {

template <int D, bool FP8, int GS, int NW>
__global__ void __launch_bounds__(NW * 32, NW == DEC_CONSUMERS ? 1 : 2)
decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const DecodeParams p) {
    using C = DecodeCfg<D, FP8, NW>;
    constexpr int DEC_CTHREADS = NW * 32;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    float *sm_scale = reinterpret_cast<float *>(smem + C::SCALE_OFF);
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(smem + C::BAR_OFF);
    uint64_t *bar_empty = bar_full + C::NSTAGE;
    uint32_t *sm_qf = reinterpret_cast<uint32_t *>(smem + C::QF_OFF);
    float *sm_ml = reinterpret_cast<float *>(smem + C::MISC_OFF);                 // [12][8][2]
    float *sm_qinv = reinterpret_cast<float *>(smem + C::QINV_OFF);               // [6][8]
    int *sm_flag = reinterpret_cast<int *>(smem + C::FLAG_OFF);
    unsigned long long *sm_tl = reinterpret_cast<unsigned long long *>(smem + C::TL_OFF);
    (void)sm_tl;

    const int split = blockIdx.x, j = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    TRB_TL(sm_tl, 0);

    // ---- dependency plan: what may be touched before the wait was decided on the host -----
    const int flags = p.pdl_flags;
    bool waited = false;
    // wait for the launches before this one (once per thread); unless the dependents were released
    // at the top, they are released as soon as this launch's own dependencies are complete
    auto dep_wait = [&]() {
        if (!waited) {
            pdl_wait();
            waited = true;
            if (!(flags & PDL_TRIGGER_TOP)) pdl_launch_dependents();
        }
    };
    if (flags & PDL_TRIGGER_TOP) pdl_launch_dependents();
    if (!(flags & PDL_PRE_CURSOR)) dep_wait();

    // ---- ranges, all derived from the device cursor -------------------------------------
    const long long pos = load_cursor(p.pos);
    const long long live = pos + (p.new_rows ? p.m : 0);
    long long lloc = live - p.shard_lo;                       // live rows held here (virtual)
    if (lloc < 0) lloc = 0;
    if (p.ring == 0 && lloc > p.max_len) {
        if (!p.sharded && threadIdx.x == 0 && split == 0 && j == 0) raise_status(TRB_ST_CURSOR_RANGE);
        lloc = p.max_len;
    }
    long long lo_all = p.window > 0 ? live - p.window - p.m : 0;
    if (lo_all < 0) lo_all = 0;
    long long row_lo = lo_all - p.shard_lo;
    if (row_lo < 0) row_lo = 0;
    const int first_tile = (int)(row_lo / DEC_BN);
    const int n_tiles = (int)((lloc + DEC_BN - 1) / DEC_BN);
    const int nt_total = n_tiles > first_tile ? n_tiles - first_tile : 0;
    int per = (nt_total + p.nsplit - 1) / p.nsplit;
    if (per < DEC_MIN_TILES) per = DEC_MIN_TILES;
    int active = (nt_total + per - 1) / per;
    if (active < 1) active = 1;
    if (split >= active) return;
    const int t0 = first_tile + split * per;
    int my_tiles = (t0 + per < n_tiles ? t0 + per : n_tiles) - t0;
    if (my_tiles < 0) my_tiles = 0;

    // With a workspace of its own the CTA takes its ticket now: the order of STARTING then decides
    // who merges the output rows.  All CTAs do the same work, so the last to start are the last to
    // finish, and a helper finds (nearly) all partials written when it gets to them - it never sits
    // on its SM waiting for CTAs that have not even been scheduled yet.
    unsigned long long ticket = 0ull;
    if (threadIdx.x == 0 && (flags & PDL_PRIVATE_WS)) ticket = decode_ticket_take(p, j);
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::NSTAGE; ++s) {
            mbar_init(&bar_full[s], FP8 ? 33u : 1u);
            mbar_init(&bar_empty[s], (uint32_t)(p.nt * (2 / GS)));
        }
        mbar_fence_init();
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
    }
    __syncthreads();

    // =============================== consumer warps ======================================
    const int g = lane >> 2, t = lane & 3;

    // warp -> (slice, 16-key group of a tile when a tile is shared by two warps, tile stream)
    constexpr int GPT = 2 / GS;                                // warps per tile and slice
    const bool warp_on = warp < p.nt * p.kw * GPT;
    const int nt_idx = warp_on ? warp % p.nt : 0;
    const int grp_idx = warp_on ? (warp / p.nt) % GPT : 0;
    const int kw_idx = warp_on ? warp / (p.nt * GPT) : 0;
    const int gb = grp_idx * 16;                               // first key row of this warp's group(s) in a tile
    // Loads of tile i into stage i % NSTAGE: issued by the slice-0 warp of the group that owns
    // the stage at that moment (TMA by lane 0, one scale pair per lane with cp.async).
    auto issue_tile = [&](int i) {
        const int s = i % C::NSTAGE;
        const long long vrow0 = (long long)(t0 + i) * DEC_BN;
        const int prow0 = (int)(p.ring > 0 ? vrow0 % p.ring : vrow0);
        if (lane == 0) {
            mbar_arrive_expect_tx(&bar_full[s], 2 * C::TILE);
#pragma unroll
            for (int sg = 0; sg < C::SEGS; ++sg) {              // one 128-byte column of the rows per copy
                tma_load_4d(smem + s * 2 * C::TILE + sg * (DEC_BN * 128), &tm_k, &bar_full[s], 0, sg, prow0, j);
                tma_load_4d(smem + s * 2 * C::TILE + C::TILE + sg * (DEC_BN * 128), &tm_v, &bar_full[s], 0, sg, prow0, j);
            }
        }
        if (FP8) {
            const long long r = (long long)prow0 + lane;
            const bool ok = r < p.max_len;
            const long long off = (long long)j * p.max_len + (ok ? r : 0);
            cp_async_4(&sm_scale[(s * 2 + 0) * DEC_BN + lane], p.ks + off, ok ? 4u : 0u);
            cp_async_4(&sm_scale[(s * 2 + 1) * DEC_BN + lane], p.vs + off, ok ? 4u : 0u);
            cp_async_mbar_arrive_noinc(&bar_full[s]);
        }
    };
    const bool issuer = warp_on && nt_idx == 0 && grp_idx == 0;
    // Rows that a launch still in flight may be writing (the append of this step) start at pos;
    // tiles entirely below them are complete and stream at once, so that this launch overlaps the
    // tail of the one before it.  The other tiles are requested only after the dependency wait,
    // by their stream's issuer when it reaches them (they are the last tiles of the last split).
    const long long fresh_from = (flags & PDL_ALL_STABLE) ? (1LL << 62) : (p.new_rows ? pos - p.shard_lo : 0);
    int n_stable = my_tiles;                                   // tiles [0, n_stable) of this split are complete
    if (!waited) {
        long long ns = fresh_from / DEC_BN - t0;
        if (ns < 0) ns = 0;
        if (ns < n_stable) n_stable = (int)ns;
    }
    int next_issue = kw_idx;                                   // next tile of this warp's stream to request
    bool pipe_ok = true;
    auto issue_more = [&](int upto) {                          // request this stream's tiles below `upto`, in order
        while (next_issue < upto && next_issue < my_tiles && (waited || next_issue < n_stable)) {
            if (next_issue >= C::NSTAGE && !mbar_wait(&bar_empty[next_issue % C::NSTAGE], ((next_issue / C::NSTAGE) - 1) & 1)) {
                pipe_ok = false;
                break;
            }
            issue_tile(next_issue);
            next_issue += p.kw;
        }
    };
    TRB_TL(sm_tl, 1);
    if (issuer) issue_more(C::NSTAGE);
    TRB_TL(sm_tl, 2);
    if (!(flags & PDL_PRE_Q)) {                                // the query rows may come from the launch before this one
        dep_wait();
        if (issuer) issue_more(C::NSTAGE);                     // ... and every row of the cache is complete now
    }

    // ---- query fragments (the B operand of S^T = K Q^T) into shared memory, once per CTA:
    // warp w < nt prepares slice w; lane (g, t) owns column n = g (row 8w + g) and the dims
    // that its k-slots cover.
    if (warp < p.nt) {
        const int r = 8 * warp + g;
        const bool valid = r < p.rows;
        const int qi = valid ? r / p.g : 0, hq = valid ? j * p.g + r % p.g : 0;
        const __nv_bfloat16 *qp = p.q + ((long long)qi * p.hq + hq) * D;
        if (FP8) {
            // f16 copies of the bf16 query (exact for |q| < 65504): word [h][w] of chunk pair cp holds
            // dims 32cp + 16w + 4t + 2h, +1, the k-slots that the low / high half-words of the
            // ldmatrix registers of K map to
            // all loads first (one round trip), then the conversions
            uint2 raw[C::NCP][2];
#pragma unroll
            for (int cp = 0; cp < C::NCP; ++cp)
#pragma unroll
                for (int w = 0; w < 2; ++w)
                    raw[cp][w] = valid ? __ldg(reinterpret_cast<const uint2 *>(qp + 32 * cp + 16 * w + 4 * t)) : make_uint2(0u, 0u);
#pragma unroll
            for (int cp = 0; cp < C::NCP; ++cp) {
                uint32_t f[2][2];
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw[cp][w].x));
                    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw[cp][w].y));
                    f[0][w] = pack_f16x2(a.x, a.y);
                    f[1][w] = pack_f16x2(b.x, b.y);
                }
                *reinterpret_cast<uint4 *>(&sm_qf[((warp * C::NCP + cp) * 32 + lane) * 4]) = make_uint4(f[0][0], f[0][1], f[1][0], f[1][1]);
            }
            if (t == 0) sm_qinv[warp * 8 + g] = 1.f;
        } else {
#pragma unroll
            for (int cp = 0; cp < C::NCP; ++cp) {
                uint32_t w0 = 0u, w1 = 0u;
                if (valid) {
                    w0 = *reinterpret_cast<const uint32_t *>(qp + 16 * cp + 2 * t);
                    w1 = *reinterpret_cast<const uint32_t *>(qp + 16 * cp + 8 + 2 * t);
                }
                *reinterpret_cast<uint2 *>(&sm_qf[((warp * C::NCP + cp) * 32 + lane) * 2]) = make_uint2(w0, w1);
            }
            if (t == 0) sm_qinv[warp * 8 + g] = 1.f;
        }
    }
    __syncthreads();

    TRB_TL(sm_tl, 3);
    const uint32_t *qf = sm_qf + (size_t)nt_idx * C::NCP * 32 * C::QF_WORDS + lane * C::QF_WORDS;

    // Visibility window of this lane's two query columns, in virtual rows of this cache
    // (32-bit: the host rejects caches of 2^31 rows or more).
    const int lloc_i = (int)lloc, row_lo_i = (int)row_lo;
    const int pos_loc = (int)(pos - p.shard_lo);               // may be negative on a later shard
    float qfac[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) qfac[c] = sm_qinv[nt_idx * 8 + 2 * t + c] * p.scale_log2;
    // bounds within which a whole tile needs no masking for any column of the slice
    int all_hi = lloc_i - 1, all_lo = 0;
    if (p.new_rows) {
        const int h0 = pos_loc + (8 * nt_idx < p.rows ? (8 * nt_idx) / p.g : 0);
        if (h0 < all_hi) all_hi = h0;
    }
    if (p.window > 0) {
        int rmax = 8 * nt_idx + 7;
        if (rmax >= p.rows) rmax = p.rows - 1;
        all_lo = pos_loc + (rmax >= 0 ? rmax / p.g : 0) - p.window + 1;
    }

    float mx[2] = {-INFINITY, -INFINITY}, ls[2] = {0.f, 0.f};
    float acc[C::ACC][4];
#pragma unroll
    for (int a = 0; a < C::ACC; ++a)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[a][i] = 0.f;

    // ldmatrix lane roles; the byte offset of a lane's row inside a tile splits into a lane part
    // (row * 128 and the swizzle XOR, which depends on chunk mod 8 only) and compile-time parts
    // (128-byte column block, 16-key group), so one address per chunk-pair-mod-4 serves a tile.
    const int mi = lane >> 3, rr = lane & 7;
    // K (plain): matrices (keys 0-7 | 8-15) x (chunk c | c+1)
    const uint32_t k_lane = (uint32_t)(rr + 8 * (mi & 1)) * 128u, k_chunk = (uint32_t)(mi >> 1);
    // V (transposed): (keys 0-7 | 8-15) x (chunk c | c+1) as a0..a3 of one m16n8k16
    const uint32_t v_lane = (uint32_t)(rr + 8 * (mi >> 1)) * 128u, v_chunk = (uint32_t)(mi & 1);
    const uint32_t urr = (uint32_t)rr;
    constexpr int NSEG = C::NCP / 4 > 0 ? C::NCP / 4 : 1;      // 128-byte column blocks per row
    constexpr int NQ = C::NCP < 4 ? C::NCP : 4;                 // chunk pairs per column block

    if (warp_on) {
#pragma unroll 1
        for (int i = kw_idx; i < my_tiles; i += p.kw) {
            const int s = i % C::NSTAGE;
            if (issuer && next_issue <= i) {                   // tile i was held back: its rows were still being written
                dep_wait();
                issue_more(i + C::NSTAGE);
            }
            if (!pipe_ok || !mbar_wait(&bar_full[s], (i / C::NSTAGE) & 1)) break;
            if (i == 0) TRB_TL(sm_tl, 4);
            const int key0 = (t0 + i) * DEC_BN;                                    // virtual row of the tile
            if (key0 + gb < lloc_i && key0 + gb + 16 * GS - 1 >= row_lo_i) {
                const uint32_t kt = smem_u32(smem + s * 2 * C::TILE);
                const uint32_t vt = kt + C::TILE;
                const float *scl = sm_scale + s * 2 * DEC_BN;
                // ---- S^T[16 GS keys, 8 columns] = K Q^T per 16-key group, two accumulation chains each
                float sc4[GS][2][4];
#pragma unroll
                for (int a = 0; a < GS; ++a)
#pragma unroll
                    for (int b = 0; b < 2; ++b)
#pragma unroll
                        for (int e = 0; e < 4; ++e) sc4[a][b][e] = 0.f;
#pragma unroll
                for (int q = 0; q < NQ; ++q) {
                    const uint32_t ka = kt + k_lane + gb * 128 + (((2u * q + k_chunk) ^ urr) << 4);
#pragma unroll
                    for (int sg = 0; sg < NSEG; ++sg) {
                        const int cp = 4 * sg + q;
                        uint32_t qw[4];
                        if (FP8) {
                            const uint4 qv = *reinterpret_cast<const uint4 *>(qf + cp * 32 * 4);
                            qw[0] = qv.x; qw[1] = qv.y; qw[2] = qv.z; qw[3] = qv.w;
                        } else {
                            const uint2 qv = *reinterpret_cast<const uint2 *>(qf + cp * 32 * 2);
                            qw[0] = qv.x; qw[1] = qv.y; qw[2] = 0u; qw[3] = 0u;
                        }
#pragma unroll
                        for (int a = 0; a < GS; ++a) {
                            uint32_t r0[4];
                            ldmatrix_x4(r0, ka + sg * (DEC_BN * 128) + a * (16 * 128));
                            if (FP8) {
                                // e4m3 -> f16 in registers (exact); low half-words feed one MMA, high ones the next
                                uint32_t af[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) af[e] = e4m3x2_to_f16x2((uint16_t)(r0[e] & 0xffffu));
                                mma_f16(sc4[a][0], af, qw[0], qw[1]);
#pragma unroll
                                for (int e = 0; e < 4; ++e) af[e] = e4m3x2_to_f16x2((uint16_t)(r0[e] >> 16));
                                mma_f16(sc4[a][1], af, qw[2], qw[3]);
                            } else {
                                mma_bf16(sc4[a][sg & 1], r0, qw[0], qw[1]);
                            }
                        }
                    }
                }
                // tv[grp][e], e = 2*h + c -> key gb + 16*grp + g + 8h, column 2t + c
                float tv[GS][4];
#pragma unroll
                for (int a = 0; a < GS; ++a)
#pragma unroll
                    for (int e = 0; e < 4; ++e) tv[a][e] = sc4[a][0][e] + sc4[a][1][e];

                // ---- per-key factors: score scale, and the V scale moved into the exponent
                float vr[GS][2];
#pragma unroll
                for (int a = 0; a < GS; ++a)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (FP8) {
                            const float ksc = scl[gb + a * 16 + g + 8 * h];
                            const float vsc = scl[DEC_BN + gb + a * 16 + g + 8 * h];
                            const float vb = __log2f(vsc);
                            vr[a][h] = __fdividef(1.f, vsc);
                            tv[a][2 * h + 0] = fmaf(tv[a][2 * h + 0], ksc * qfac[0], vb);
                            tv[a][2 * h + 1] = fmaf(tv[a][2 * h + 1], ksc * qfac[1], vb);
                        } else {
                            vr[a][h] = 1.f;
                            tv[a][2 * h + 0] *= qfac[0];
                            tv[a][2 * h + 1] *= qfac[1];
                        }
                    }
                if (!(key0 + DEC_BN - 1 <= all_hi && key0 >= all_lo)) {
                    // rare (the tiles at the ends of the live range): the limits of this lane's two
                    // columns are recomputed here rather than kept in registers
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const int r = 8 * nt_idx + 2 * t + c;
                        const int qi = r < p.rows ? r / p.g : 0;           // padding rows copy row 0's window
                        int hi = lloc_i - 1;
                        if (p.new_rows && pos_loc + qi < hi) hi = pos_loc + qi;
                        const int lo = p.window > 0 ? pos_loc + qi - p.window + 1 : 0;
#pragma unroll
                        for (int a = 0; a < GS; ++a)
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const int kv = key0 + gb + a * 16 + g + 8 * h;
                                if (!(kv <= hi && kv >= lo)) tv[a][2 * h + c] = -INFINITY;
                                if (kv >= lloc_i) vr[a][h] = 0.f;            // never-written rows: scale may be anything
                            }
                    }
                }
                // ---- online softmax over the keys (rows of S^T): reduce across the g lanes
                float alpha[2];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    float ml = fmaxf(tv[0][c], tv[0][2 + c]);
                    if (GS == 2) ml = fmaxf(ml, fmaxf(tv[GS - 1][c], tv[GS - 1][2 + c]));
                    ml = fmaxf(ml, __shfl_xor_sync(0xffffffffu, ml, 4));
                    ml = fmaxf(ml, __shfl_xor_sync(0xffffffffu, ml, 8));
                    ml = fmaxf(ml, __shfl_xor_sync(0xffffffffu, ml, 16));
                    const float mn = fmaxf(mx[c], ml);
                    const float msafe = mn == -INFINITY ? 0.f : mn;
                    alpha[c] = fast_exp2(mx[c] - msafe);
                    float lsum = 0.f;
#pragma unroll
                    for (int a = 0; a < GS; ++a)
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const float pv = fast_exp2(tv[a][2 * h + c] - msafe);
                            tv[a][2 * h + c] = pv;
                            lsum = fmaf(pv, vr[a][h], lsum);
                        }
                    ls[c] = fmaf(ls[c], alpha[c], lsum);
                    mx[c] = mn;
                }
                if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                    for (int a = 0; a < C::ACC; ++a) {
                        acc[a][0] *= alpha[0]; acc[a][1] *= alpha[1];
                        acc[a][2] *= alpha[0]; acc[a][3] *= alpha[1];
                    }
                }
                // ---- O^T[D dims, 8 columns] += V^T P^T per 16-key group; P^T as the B operand: pack the
                // two columns of a key, transpose the 8x8 blocks across the warp
#pragma unroll
                for (int a = 0; a < GS; ++a) {
                    const uint32_t pb0 = movmatrix_trans(FP8 ? pack_f16x2(tv[a][0], tv[a][1]) : pack_bf16x2(tv[a][0], tv[a][1]));
                    const uint32_t pb1 = movmatrix_trans(FP8 ? pack_f16x2(tv[a][2], tv[a][3]) : pack_bf16x2(tv[a][2], tv[a][3]));
#pragma unroll
                    for (int q = 0; q < NQ; ++q) {
                        const uint32_t va = vt + v_lane + (((2u * q + v_chunk) ^ urr) << 4) + (gb + a * 16) * 128;
#pragma unroll
                        for (int sg = 0; sg < NSEG; ++sg) {
                            const int cp = 4 * sg + q;
                            uint32_t w[4];
                            ldmatrix_x4_trans(w, va + sg * (DEC_BN * 128));
                            if (FP8) {
                                // a transposed register holds dims (2g, 2g+1) of keys (2t, 2t+1): regroup to
                                // (key 2t, key 2t+1) of dim 2g | of dim 2g+1, then e4m3 -> f16
                                uint32_t af[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) w[e] = prmt(w[e], 0u, 0x3120u);
#pragma unroll
                                for (int e = 0; e < 4; ++e) af[e] = e4m3x2_to_f16x2((uint16_t)(w[e] & 0xffffu));
                                mma_f16(acc[2 * cp], af, pb0, pb1);
#pragma unroll
                                for (int e = 0; e < 4; ++e) af[e] = e4m3x2_to_f16x2((uint16_t)(w[e] >> 16));
                                mma_f16(acc[2 * cp + 1], af, pb0, pb1);
                            } else {
                                mma_bf16(acc[cp], w, pb0, pb1);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_empty[s]);
            if (issuer) {                                      // refill the stage once every slice has left it
                issue_more(i + C::NSTAGE + 1);
                if (!pipe_ok) break;
            }
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            ls[c] += __shfl_xor_sync(0xffffffffu, ls[c], 4);
            ls[c] += __shfl_xor_sync(0xffffffffu, ls[c], 8);
            ls[c] += __shfl_xor_sync(0xffffffffu, ls[c], 16);
        }
    }

    // =============================== CTA epilogue =======================================
    // Everything from here on touches the workspace and the outputs: the launches before this one
    // must be complete.  One thread takes the kv head's ticket right away, so that its round trip
    // runs under the merge below.
    TRB_TL(sm_tl, 5);
    // (with a workspace that no launch in flight uses, the partial needs no wait: only the CTAs that
    // merge output rows wait, in the tail, before they write them)
    const bool ws_private = (flags & PDL_PRIVATE_WS) != 0;
    if (!ws_private) dep_wait();
    TRB_TL(sm_tl, 6);
    if (threadIdx.x == 0 && !ws_private) ticket = decode_ticket_take(p, j);
    // 1. merge the warps that share an 8-row slice (fixed order) through shared memory: every warp
    // stages its accumulators unscaled, together with its (max, sum); the reducing threads weigh them
    __syncthreads();                    // every stage has been consumed
    TRB_TL(sm_tl, 7);
    if (warp_on && g == 0) {
        sm_ml[(warp * 8 + 2 * t + 0) * 2 + 0] = mx[0]; sm_ml[(warp * 8 + 2 * t + 0) * 2 + 1] = ls[0];
        sm_ml[(warp * 8 + 2 * t + 1) * 2 + 0] = mx[1]; sm_ml[(warp * 8 + 2 * t + 1) * 2 + 1] = ls[1];
    }
    float *stage_acc = reinterpret_cast<float *>(smem);                // [warp][8][D + pad]
    constexpr int SROW = D + DEC_EPI_PAD;
    if (warp_on) {
        const bool live0 = 8 * nt_idx + 2 * t < p.rows, live1 = 8 * nt_idx + 2 * t + 1 < p.rows;
#pragma unroll
        for (int a = 0; a < C::ACC; ++a)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if ((i & 1) ? live1 : live0) stage_acc[(warp * 8 + 2 * t + (i & 1)) * SROW + acc_dim<FP8>(a, i, g)] = acc[a][i];
    }
    if (threadIdx.x == 0) decode_ticket(p, j, active, DEC_CTHREADS / (D / 4), sm_flag, ticket);
    __syncthreads();                    // also publishes the ticket's result (sm_flag)
    const int tid = threadIdx.x;                                       // 0..383 here
    const unsigned int tag = (unsigned int)sm_flag[2] + 1u;
    const long long part_base = ((long long)j * p.nsplit + split) * p.rows_pad;
    const int nw = p.kw * GPT;                                         // warps per slice
    for (int item = tid; item < p.nt * 8 * (D / 4); item += DEC_CTHREADS) {
        const int row = item / (D / 4), d4 = (item % (D / 4)) * 4;
        if (row >= p.rows) continue;
        const int nti = row >> 3, qc = row & 7;
        float mg = -INFINITY;
        for (int k = 0; k < nw; ++k) mg = fmaxf(mg, sm_ml[((k * p.nt + nti) * 8 + qc) * 2]);
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        float lg = 0.f;
        for (int k = 0; k < nw; ++k) {
            const float mk = sm_ml[((k * p.nt + nti) * 8 + qc) * 2];
            const float w = mk == -INFINITY ? 0.f : fast_exp2(mk - mg);
            const float4 v = *reinterpret_cast<const float4 *>(&stage_acc[((k * p.nt + nti) * 8 + qc) * SROW + d4]);
            sum.x = fmaf(w, v.x, sum.x); sum.y = fmaf(w, v.y, sum.y); sum.z = fmaf(w, v.z, sum.z); sum.w = fmaf(w, v.w, sum.w);
            lg = fmaf(w, sm_ml[((k * p.nt + nti) * 8 + qc) * 2 + 1], lg);
        }
        st_tagged4(p.part_acc + (part_base + row) * D + d4, sum, tag);
        if (d4 == 0) st_volatile_v4(p.part_ml + part_base + row, make_uint4(__float_as_uint(mg), tag, __float_as_uint(lg), tag));
    }

    TRB_TL(sm_tl, 8);
    TRB_TL_SET(sm_tl, 13, sm_flag[0]);
    TRB_TL_SET(sm_tl, 14, my_tiles);
    decode_tail<D, DEC_CTHREADS>(p, smem, C::SCALE_OFF, sm_flag, j, active, sm_tl);
    TRB_TL_FLUSH(sm_tl, (unsigned int)sm_flag[2], j * p.nsplit + split);
}

// ---------------------------------------------------------------------------------------------
// Softmax statistics of the b in-step block keys (all visible), one warp per (query, head).
template <int D>
__global__ void __launch_bounds__(32) block_partial_kernel(const __nv_bfloat16 *q, const __nv_bfloat16 *kb,
                                                           const __nv_bfloat16 *vb, int b, int hq, int hkv,
                                                           float scale_log2, float *ml, float *acc) {
    constexpr int EPT = D / 32;
    const int i = blockIdx.x / hq, h = blockIdx.x % hq, lane = threadIdx.x;
    const int j = h / (hq / hkv);
    float qv[EPT];
#pragma unroll
    for (int e = 0; e < EPT; ++e) qv[e] = __bfloat162float(q[((long long)i * hq + h) * D + lane * EPT + e]);
    float mrun = -INFINITY, lrun = 0.f, o[EPT];
#pragma unroll
    for (int e = 0; e < EPT; ++e) o[e] = 0.f;
    for (int k = 0; k < b; ++k) {
        const __nv_bfloat16 *kp = kb + ((long long)j * b + k) * D + lane * EPT;
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < EPT; ++e) dot = fmaf(qv[e], __bfloat162float(kp[e]), dot);
        dot = warp_sum(dot) * scale_log2;
        const float mn = fmaxf(mrun, dot);
        const float al = fast_exp2(mrun - mn), pk = fast_exp2(dot - mn);
        lrun = lrun * al + pk;
        const __nv_bfloat16 *vp = vb + ((long long)j * b + k) * D + lane * EPT;
#pragma unroll
        for (int e = 0; e < EPT; ++e) o[e] = fmaf(o[e], al, pk * __bfloat162float(vp[e]));
        mrun = mn;
    }
    const long long row = (long long)i * hq + h;
    if (lane == 0) { ml[row * 2] = mrun; ml[row * 2 + 1] = lrun; }
#pragma unroll
    for (int e = 0; e < EPT; ++e) acc[row * D + lane * EPT + e] = o[e];
}

// LSE merge of n_parts partials per row (one CTA per row), fixed order.
__global__ void __launch_bounds__(64) lse_merge_kernel(const float *ml, const float *acc, int n_parts, int rows, int d,
                                                       __nv_bfloat16 *out, const __nv_bfloat16 *gate, long long gate_rs,
                                                       long long gate_hs, int hq) {
    const int row = blockIdx.x;
    float mmax = -INFINITY;
    for (int s = 0; s < n_parts; ++s) mmax = fmaxf(mmax, ml[((long long)s * rows + row) * 2]);
    float lsum = 0.f;
    for (int s = 0; s < n_parts; ++s) {
        const float ms = ml[((long long)s * rows + row) * 2];
        lsum += ms == -INFINITY ? 0.f : fast_exp2(ms - mmax) * ml[((long long)s * rows + row) * 2 + 1];
    }
    const float inv = 1.f / lsum;
    for (int x = threadIdx.x * 4; x < d; x += blockDim.x * 4) {
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < n_parts; ++s) {
            const float ms = ml[((long long)s * rows + row) * 2];
            const float w = ms == -INFINITY ? 0.f : fast_exp2(ms - mmax);
            const float4 v = *reinterpret_cast<const float4 *>(&acc[((long long)s * rows + row) * d + x]);
            o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
        }
        float r[4] = {o.x * inv, o.y * inv, o.z * inv, o.w * inv};
        __nv_bfloat16 ob[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) ob[e] = __float2bfloat16_rn(r[e]);
        if (gate) {
            const int qi = row / hq, h = row % hq;
            const __nv_bfloat16 *gp = gate + (long long)qi * gate_rs + (long long)h * gate_hs + x;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float sg = __bfloat162float(__float2bfloat16_rn(1.f / (1.f + __expf(-__bfloat162float(gp[e])))));
                ob[e] = __float2bfloat16_rn(__bfloat162float(ob[e]) * sg);
            }
        }
        *reinterpret_cast<uint2 *>(&out[(long long)row * d + x]) = *reinterpret_cast<const uint2 *>(ob);
    }
}

static int g_sm_count = 0;
static int sm_count() {
    if (g_sm_count == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
            g_sm_count = n;
        else
            g_sm_count = 148;
    }
    return g_sm_count;
}

// Shared memory that the tail of the smallest kernel variant has for a row's partials, and the
// bytes of its bookkeeping before them (see decode_tail): upper bounds, used to size the splits.
constexpr int DEC_TAIL_SMEM_MIN = DEC_HALF_WARPS * DEC_STAGE_BYTES_PER_WARP;
static int tail_bookkeeping_bytes(int d, int m) { return 9216 + 2 * m * d * 4 + 256; }

// splits per kv head: one CTA per SM over all heads, and no more than a helper's shared memory
// can hold of one row's partials (which only matters with one or two kv heads)
static int decode_nsplit(int hq, int hkv, int d, int m) {
    int n = sm_count() / hkv;
    if (n > DEC_MAX_SPLITS) n = DEC_MAX_SPLITS;
    // (the half-size CTA only serves one 8-row slice; every other variant has twice its shared memory or more)
    const int tail_smem = (hq / hkv) * m <= 8 ? DEC_TAIL_SMEM_MIN : 2 * DEC_TAIL_SMEM_MIN;
    const int fit = (tail_smem - tail_bookkeeping_bytes(d, m)) / (d * 8 + 16);
    if (n > fit) n = fit;
    return n < 1 ? 1 : n;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct WorkspaceLayout {
    size_t counters, ml, acc, total;
};
static WorkspaceLayout workspace_layout(int hkv, int nsplit, int rows_pad, int d) {
    WorkspaceLayout w;
    w.counters = 0;
    w.ml = 1024;
    // every float of a partial travels with a tag: (max, tag, sum, tag) and (value, tag) pairs
    w.acc = align_up(w.ml + (size_t)hkv * nsplit * rows_pad * sizeof(uint4), 256);
    w.total = w.acc + (size_t)hkv * nsplit * rows_pad * d * sizeof(uint2);
    return w;
}

template <int D, bool FP8, int GS, int NW>
static int launch_decode_gs(const CUtensorMap &mk, const CUtensorMap &mv, const DecodeParams &p, cudaStream_t st) {
    using C = DecodeCfg<D, FP8, NW>;
    static bool attr_set[64] = {};
    int dev = 0;
    TRB_CUDA_CHECK(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        TRB_CUDA_CHECK(cudaFuncSetAttribute(decode_kernel<D, FP8, GS, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        TRB_CUDA_CHECK(cudaFuncSetAttribute(decode_kernel<D, FP8, GS, NW>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                            cudaSharedmemCarveoutMaxShared));
        attr_set[dev & 63] = true;
    }
    dim3 grid(p.nsplit, p.hkv);
    TRB_CUDA_CHECK(launch_kernel(decode_kernel<D, FP8, GS, NW>, grid, dim3(NW * 32), (size_t)C::SMEM, st, true, mk, mv, p));
    return TRB_OK;
}

// One slice (M = 1, the bandwidth-bound case): two warps share a tile, one 16-key group each, so
// that half of the stage ring is always in flight.  More slices are bound by instruction issue
// and the tensor pipe; there a warp takes whole 32-key tiles (one softmax step per 32 keys).
static int decode_groups_per_warp(int nt) { return nt == 1 ? 1 : 2; }

// A decode that runs inside a chain of library launches (it releases its dependents at its top)
// and has one slice takes half-size CTAs: 6 warps and 96 KB of stages, so that two CTAs fit one
// SM.  The grid stays one CTA per SM: the second slot of every SM is taken by the CTA of the next
// layer's launch, whose prologue (cursor, descriptors, first tiles, under load several
// microseconds) and epilogue then run beside this launch's streaming instead of leaving the SM
// idle.  A launch that runs alone keeps the full-size CTA (all 192 KB in flight are its own).
static int decode_warps(const DecodeParams &p) {
    return (p.nt == 1 && (p.pdl_flags & PDL_TRIGGER_TOP)) ? DEC_HALF_WARPS : DEC_CONSUMERS;
}

template <int D, bool FP8>
static int launch_decode(const CUtensorMap &mk, const CUtensorMap &mv, const DecodeParams &p, cudaStream_t st) {
    if (decode_groups_per_warp(p.nt) == 2) return launch_decode_gs<D, FP8, 2, DEC_CONSUMERS>(mk, mv, p, st);
    return decode_warps(p) == DEC_HALF_WARPS ? launch_decode_gs<D, FP8, 1, DEC_HALF_WARPS>(mk, mv, p, st)
                                              : launch_decode_gs<D, FP8, 1, DEC_CONSUMERS>(mk, mv, p, st);
}

// Query rows per kv head (heads per kv head x M) from which the tensor-core kernel takes FP8
// caches of head dim 256 without ring or window.
constexpr int DEC_TC_DEFAULT_MIN_ROWS = 12;
static int g_tc_min_rows = DEC_TC_DEFAULT_MIN_ROWS;

template <int NROW>
static int launch_decode_tc_n(const CUtensorMap &mk, const CUtensorMap &mv, const DecodeParams &p, cudaStream_t st) {
    static bool attr_set[64] = {};
    int dev = 0;
    TRB_CUDA_CHECK(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        TRB_CUDA_CHECK(cudaFuncSetAttribute(decode_tc_kernel<NROW>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
        attr_set[dev & 63] = true;
    }
    dim3 grid(p.nsplit, p.hkv);
    TRB_CUDA_CHECK(launch_kernel(decode_tc_kernel<NROW>, grid, dim3(8 * NROW + 64), (size_t)TC_SMEM, st, true, mk, mv, p));
    return TRB_OK;
}

static int launch_decode_tc(const CUtensorMap &mk, const CUtensorMap &mv, const DecodeParams &p, cudaStream_t st) {
    if (p.rows <= 16) return launch_decode_tc_n<16>(mk, mv, p, st);
    if (p.rows <= 32) return launch_decode_tc_n<32>(mk, mv, p, st);
    return launch_decode_tc_n<48>(mk, mv, p, st);
}

}  // namespace trb

using namespace trb;

extern "C" int trb_set_decode_tensor_rows(int32_t min_rows) {
    g_tc_min_rows = min_rows > 0 ? min_rows : DEC_TC_DEFAULT_MIN_ROWS;
    return TRB_OK;
}

extern "C" size_t trb_decode_workspace_bytes(int32_t hq, int32_t hkv, int32_t d, int32_t m) {
    if (hq < 1 || hkv < 1 || hq % hkv || m < 1) return 0;
    const int rows = (hq / hkv) * m;
    if (rows > DEC_MAX_ROWS) return 0;
    const int rows_pad = (rows + 7) / 8 * 8;
    return workspace_layout(hkv, decode_nsplit(hq, hkv, d, m), rows_pad, d).total;
}

extern "C" int trb_attn_decode(const trb_cache_t *cache, const trb_decode_args_t *a, trb_stream_t stream) {
    CacheView c;
    int rc = make_cache_view(cache, &c);
    if (rc) return rc;
    if (!a || !a->q || (!a->out && !a->partial_acc) || !a->workspace) return TRB_E_ARG;
    if (a->m < 1 || a->hq < 1 || a->hq % c.hkv) return TRB_E_ARG;
    const int g = a->hq / c.hkv, rows = g * a->m;
    if (rows > DEC_MAX_ROWS) return TRB_E_UNSUPPORTED;
    if (c.hkv > 65535) return TRB_E_UNSUPPORTED;
    if (a->n_extra < 0 || a->n_extra > 1 || (a->n_extra && (!a->extra_ml || !a->extra_acc))) return TRB_E_ARG;
    if ((a->partial_ml == nullptr) != (a->partial_acc == nullptr)) return TRB_E_ARG;
    if (a->window < 0) return TRB_E_ARG;
    if (c.ring > 0 && (c.ring % DEC_BN)) return TRB_E_UNSUPPORTED;
    if (c.ring > 0 && a->window + a->m > c.ring) return TRB_E_CAPACITY;
    if (c.max_len >= (1LL << 31) - 64 || c.shard_lo < 0 || c.shard_lo >= (1LL << 40)) return TRB_E_UNSUPPORTED;
    if ((rc = check_cursor(&a->pos))) return rc;
    if (((uintptr_t)a->q | (uintptr_t)a->out | (uintptr_t)a->workspace | (uintptr_t)a->partial_acc | (uintptr_t)a->extra_acc) & 15)
        return TRB_E_ALIGN;
    if (a->gate && (((uintptr_t)a->gate & 7) || (a->gate_row_stride % 4) || (a->gate_head_stride % 4))) return TRB_E_ALIGN;
    if (!a->pos.dev && c.ring == 0 && !c.sharded && a->pos.host + (a->new_rows ? a->m : 0) > c.max_len) return TRB_E_CAPACITY;

    DecodeParams p;
    p.q = (const __nv_bfloat16 *)a->q; p.out = (__nv_bfloat16 *)a->out; p.gate = (const __nv_bfloat16 *)a->gate;
    p.gate_rs = a->gate_row_stride; p.gate_hs = a->gate_head_stride;
    p.ks = c.k_scale; p.vs = c.v_scale;
    p.m = a->m; p.hq = a->hq; p.hkv = c.hkv; p.g = g; p.rows = rows;
    p.nt = (rows + 7) / 8; p.kw = 0;                              // kw: set once the launch plan is known
    p.nsplit = decode_nsplit(a->hq, c.hkv, c.d, a->m); p.rows_pad = p.nt * 8;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.new_rows = a->new_rows ? 1 : 0; p.window = a->window; p.n_extra = a->n_extra;
    p.extra_ml = a->extra_ml; p.extra_acc = a->extra_acc;
    p.pos = make_cursor(&a->pos);
    p.max_len = c.max_len; p.ring = c.ring; p.shard_lo = c.shard_lo; p.sharded = c.sharded;
    const WorkspaceLayout w = workspace_layout(c.hkv, p.nsplit, p.rows_pad, c.d);
    if (a->workspace_bytes < w.total) return TRB_E_CAPACITY;
    uint8_t *ws = (uint8_t *)a->workspace;
    p.word = (unsigned long long *)(ws + w.counters);
    p.part_ml = (uint4 *)(ws + w.ml); p.part_acc = (uint2 *)(ws + w.acc);
    p.shard_ml = a->partial_ml; p.shard_acc = a->partial_acc;
    p.p2p_world = 0; p.p2p_rank = 0;
    p.xtag_mul = a->ws_slots > 1 ? (unsigned int)a->ws_slots : 1u;
    p.xtag_add = a->ws_slots > 1 ? (unsigned int)a->ws_slot : 0u;
    if (a->ws_slots > 1 && (a->ws_slot < 0 || a->ws_slot >= a->ws_slots)) return TRB_E_ARG;
    for (int r = 0; r < 8; ++r) p.p2p_ptr[r] = nullptr;
    if (a->p2p_xchg) {
        if (a->p2p_world < 1 || a->p2p_world > P2P_MAX_WORLD || a->p2p_rank < 0 || a->p2p_rank >= a->p2p_world || a->partial_acc) return TRB_E_ARG;
        p.p2p_world = a->p2p_world; p.p2p_rank = a->p2p_rank;
        for (int r = 0; r < a->p2p_world; ++r) {
            if (!a->p2p_xchg[r]) return TRB_E_ARG;
            p.p2p_ptr[r] = a->p2p_xchg[r];
        }
    }

    const int row_bytes = c.d * (c.fp8 ? 1 : 2);
    CUtensorMap mk, mv;
    cudaStream_t st = (cudaStream_t)stream;
    const bool tensor_kernel = c.fp8 && c.d == TC_D && c.ring == 0 && a->window == 0 && rows >= g_tc_min_rows;
    if ((rc = get_row_tile_map(c.k, c.max_len, c.hkv, row_bytes, tensor_kernel ? TC_BN : DEC_BN, &mk))) return rc;
    if ((rc = get_row_tile_map(c.v, c.max_len, c.hkv, row_bytes, tensor_kernel ? TC_BN : DEC_BN, &mv))) return rc;
    // nothing fails after this point except the launch itself: record the launch for the next one
    const size_t out_rows = (size_t)a->m * a->hq;
    const WrittenRange outs[3] = {{a->out, a->out ? out_rows * c.d * sizeof(__nv_bfloat16) : 0},
                                  {a->partial_ml, a->partial_ml ? out_rows * 2 * sizeof(float) : 0},
                                  {a->partial_acc, a->partial_acc ? out_rows * c.d * sizeof(float) : 0}};
    AppendSource fresh;
    p.pdl_flags = pdl_plan_decode(st, c.k, &a->pos, p.new_rows, a->m, WrittenRange{a->q, out_rows * c.d * sizeof(__nv_bfloat16)}, outs,
                                  a->workspace, &fresh);
    // The tensor-core kernel fills an SM alone: CTAs that ran ahead of the launch before would start
    // and finish far apart, and its helpers would sit on their SMs waiting for the stragglers.  Its
    // CTAs (and the full-size CTAs of the several-slice kernel) therefore all wait before the
    // epilogue and finish together.
    if (tensor_kernel || p.nt != 1) p.pdl_flags &= ~PDL_PRIVATE_WS;
    // Only the launches that run ahead of the launch before them (one slice, half-size CTAs) take the
    // new rows from the append's source: the others wait for the append anyway before their epilogue.
    p.fresh_k = p.fresh_v = nullptr; p.fresh_hs = p.fresh_rs = 0;
    if (fresh.k && !tensor_kernel && p.nt == 1 && (p.pdl_flags & PDL_PRIVATE_WS)) {
        p.fresh_k = (const __nv_bfloat16 *)fresh.k; p.fresh_v = (const __nv_bfloat16 *)fresh.v;
        p.fresh_hs = fresh.head_stride; p.fresh_rs = fresh.row_stride;
        p.new_rows = 0;                                       // the scan covers the rows below the cursor, all visible to every row
        p.pdl_flags |= PDL_ALL_STABLE;                        // ... and all complete
    }
    // a ring cache maps several positions to one row: the rows below the cursor are not the rows
    // below the in-flight append
    if (c.ring > 0 && !(p.pdl_flags & PDL_ALL_STABLE)) p.pdl_flags &= (PDL_TRIGGER_TOP | PDL_PRIVATE_WS);
    p.tail_teams = tensor_kernel ? 1 : 0;
    p.kw = decode_warps(p) / (p.nt * (2 / decode_groups_per_warp(p.nt)));
    {   // a helper merges several rows when its tail can hold two rows' partials (the next row's copies fly during a merge)
        const int tail_smem = tensor_kernel ? TC_OFF_SC : decode_warps(p) * DEC_STAGE_BYTES_PER_WARP;
        const int row_bytes_tail = (p.nsplit * 16 + 127) / 128 * 128 + p.nsplit * c.d * 8;
        p.tail_rows_per_helper = (tail_smem - tail_bookkeeping_bytes(c.d, a->m) >= 2 * row_bytes_tail) ? 2 : 1;
    }
    if (tensor_kernel) return launch_decode_tc(mk, mv, p, st);
    if (c.d == 256) return c.fp8 ? launch_decode<256, true>(mk, mv, p, st) : launch_decode<256, false>(mk, mv, p, st);
    return c.fp8 ? launch_decode<128, true>(mk, mv, p, st) : launch_decode<128, false>(mk, mv, p, st);
}

extern "C" int trb_attn_block_partial(const void *q, const void *k_blk, const void *v_blk, int32_t b, int32_t hq, int32_t hkv,
                                      int32_t d, float scale, float *extra_ml, float *extra_acc, trb_stream_t stream) {
    if (!q || !k_blk || !v_blk || !extra_ml || !extra_acc || b < 1 || hq < 1 || hkv < 1 || hq % hkv) return TRB_E_ARG;
    if (d != 128 && d != 256) return TRB_E_UNSUPPORTED;
    const float sl2 = scale * 1.4426950408889634f;
    cudaStream_t st = (cudaStream_t)stream;
    pdl_note_fence((cudaStream_t)stream);
    if (d == 256)
        block_partial_kernel<256><<<b * hq, 32, 0, st>>>((const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k_blk,
                                                         (const __nv_bfloat16 *)v_blk, b, hq, hkv, sl2, extra_ml, extra_acc);
    else
        block_partial_kernel<128><<<b * hq, 32, 0, st>>>((const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k_blk,
                                                         (const __nv_bfloat16 *)v_blk, b, hq, hkv, sl2, extra_ml, extra_acc);
    TRB_CUDA_CHECK(cudaGetLastError());
    return TRB_OK;
}

extern "C" int trb_lse_merge(const float *ml, const float *acc, int32_t n_parts, int32_t rows, int32_t d, void *out,
                             const void *gate, int64_t gate_row_stride, int64_t gate_head_stride, int32_t hq,
                             trb_stream_t stream) {
    if (!ml || !acc || !out || n_parts < 1 || rows < 1 || d < 4 || (d % 4) || hq < 1) return TRB_E_ARG;
    if (((uintptr_t)acc & 15) || ((uintptr_t)out & 7)) return TRB_E_ALIGN;
    pdl_note_fence((cudaStream_t)stream);
    lse_merge_kernel<<<rows, 64, 0, (cudaStream_t)stream>>>(ml, acc, n_parts, rows, d, (__nv_bfloat16 *)out,
                                                             (const __nv_bfloat16 *)gate, gate_row_stride, gate_head_stride, hq);
    TRB_CUDA_CHECK(cudaGetLastError());
    return TRB_OK;
}

// ---------------------------------------------------------------------------------------------
// Decode without caller-provided scratch.
//
// Some callers cannot hand the library a scratch buffer because they cannot allocate device
// memory at the point of the call: a host runtime that owns all device memory through its own
// arena and exposes no allocation hook to plugins, or a thin FFI binding (cgo / JNI style) that
// only forwards the buffers it was given.  For them the split-partial scratch lives in the array below, which is part of the
// library image: every GPU that loads the library holds TRB_STATIC_SCRATCH_BYTES until the
// process exits.
//
// The array's name is only a handle on the host side; the device address is looked up once
// per device with cudaGetSymbolAddress (with that device current) and handed to the kernel.
static __device__ __align__(256) unsigned char g_static_scratch[TRB_STATIC_SCRATCH_BYTES];

namespace trb {
static std::mutex g_static_mu;
static void *g_static_ptr[64] = {};

static int static_scratch_ptr(void **out) {
    int dev = 0;
    TRB_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return TRB_E_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
        void *ptr = nullptr;
        TRB_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_static_scratch));
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return TRB_OK;
}
}  // namespace trb

namespace trb {
// count <- 0 and epoch <- epoch + 1 in every ticket word: a call that was cut short leaves
// neither a count nor tagged partials that a later call could take for its own
__global__ void static_scratch_reset_kernel(unsigned long long *word, int n) {
    const int i = threadIdx.x;
    if (i < n) word[i] = ((word[i] >> 16) + 1ull) << 16;
}
}  // namespace trb

extern "C" int trb_attn_decode_static(const trb_cache_t *cache, const trb_decode_args_t *args, trb_stream_t stream) {
    if (!cache || !args) return TRB_E_ARG;
    if (cache->hkv < 1 || cache->hkv > 64 || args->hq < 1 || args->m < 1 || args->hq % cache->hkv) return TRB_E_ARG;
    // The exchange between GPUs is tagged with the launch count of the workspace, which must be the
    // same on every GPU; the built-in array is shared by all callers of a process, so its count is not.
    if (args->p2p_xchg) return TRB_E_UNSUPPORTED;
    const size_t need = trb_decode_workspace_bytes(args->hq, cache->hkv, cache->d, args->m);
    if (need == 0) return TRB_E_UNSUPPORTED;
    if (need > TRB_STATIC_SCRATCH_BYTES) return TRB_E_SCRATCH_LIMIT;
    void *scratch = nullptr;
    int rc = static_scratch_ptr(&scratch);
    if (rc) return rc;
    // The array keeps whatever the previous call left.  Only the arrival counts in the header have
    // to start from zero; the partials are recognised by their tags, so nothing else is cleared.
    cudaStream_t st = (cudaStream_t)stream;
    pdl_note_fence(st);
    static_scratch_reset_kernel<<<1, 64, 0, st>>>((unsigned long long *)scratch, cache->hkv);
    TRB_CUDA_CHECK(cudaGetLastError());
    trb_decode_args_t a = *args;
    a.workspace = scratch;
    a.workspace_bytes = TRB_STATIC_SCRATCH_BYTES;
    return trb_attn_decode(cache, &a, stream);
}

#ifdef TRB_TIMELINE
// Diagnostic build only: copy the per-CTA timeline stamps of the last TL_LAUNCHES decode launches
// ([launch % 64][cta][16] nanosecond stamps of %globaltimer) to the host.  Synchronises the device.
extern "C" int trb_dbg_timeline(void *host_out, size_t bytes) {
    if (!host_out || bytes < sizeof(unsigned long long) * TL_LAUNCHES * TL_CTAS * TL_SLOTS) return TRB_E_ARG;
    TRB_CUDA_CHECK(cudaDeviceSynchronize());
    TRB_CUDA_CHECK(cudaMemcpyFromSymbol(host_out, trb::g_timeline, sizeof(unsigned long long) * TL_LAUNCHES * TL_CTAS * TL_SLOTS));
    return TRB_OK;
}
#endif
