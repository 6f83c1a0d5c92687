// Chunked prefill attention over the KV cache (e4m3 + scales, or bf16) on the 5th-generation
// tensor cores (tcgen05.mma, accumulators and the A operands in tensor memory).
//
// One CTA per (128-query block, query head).  Keys stream in tiles of 128 (e4m3) or 64 (bf16) through a
// TMA ring; per tile
//     S[128 x 128]  = (Qhi + Qlo) K^T         tcgen05.mma kind::f8f6f4, K straight from the TMA tile
//     P             = exp2(S * k_scale * c + log2 v_scale - m)     256 threads, (query row, key half) each
//     O[128 x 256] += (Phi + Plo) V           tcgen05.mma, V as an MN-major operand, same tile
// The e4m3 codes of the cache feed the tensor cores unconverted.  The bf16 queries and the fp32
// probabilities are each split into two e4m3 terms (x ~= hi + lo: 8 significant bits, what bf16
// carries), so every product is exact and accumulation is fp32 in tensor memory; at the FP8 rate
// the two terms cost what one bf16 pass would.  Per-key scales never touch the codes: the K scale
// multiplies the fp32 score, the V scale is moved into the exponent of the probability.
// Over a bf16 cache the same kernel issues kind::f16 MMAs on the bf16 rows as they are.
//
// The probabilities of a tile are written over the scores they came from, in tensor memory, and
// enter the PV product as a tensor-memory A operand (tcgen05.st by the thread that owns the row: no
// shared-memory staging, no proxy fence).  A tcgen05.mma with N = 64 takes about 65 cycles where
// its math needs 32 (measured: 16 of them per tile, 1040 cycles, with A in shared or in tensor
// memory alike), so the e4m3 kernel works on 128 keys per tile: S is two buffers of 128 columns, O
// 256 columns, which fills tensor memory, and the query block (hi + lo, 64 KB) stays in shared
// memory.  A bf16 tile of 128 keys would be 128 KB of K and V per stage; the bf16 kernel keeps 64 keys
// per tile and holds its query block in the 128 tensor-memory columns that leaves free.
//
// Warp roles: warps 0-7 softmax / correction / epilogue (two warpgroups; thread = one query row
// = one TMEM lane, and one half of the tile's keys / of the output columns), warp 8 TMA
// producer, warp 9 MMA issuer.  S is double-buffered in tensor memory, so QK of tile i+1 runs
// on the tensor pipe while tile i is in softmax.  Every wait is bounded.
#include "common.cuh"
#include "tc.cuh"
#include "tmap.h"

namespace trb {

constexpr int PF_BM = 128;              // queries per CTA
constexpr int PF_D = 256;               // head dim
constexpr int PF_MAXST = 3;             // pipeline stages of (32 KB K tile, 32 KB V tile): 2 for e4m3 (beside the query block), 3 for bf16
constexpr int PF_SOFTMAX_THREADS = 256;     // two warpgroups: thread = (query row, half of the tile's keys)
constexpr int PF_THREADS = PF_SOFTMAX_THREADS + 64;   // + TMA warp + MMA warp
constexpr int PF_TILE = 32 * 1024;      // 128 keys x 256 B (e4m3) or 64 keys x 512 B (bf16)
constexpr int PF_Q_BYTES = PF_BM * PF_D;               // one e4m3 copy of the query block
constexpr int PF_OFF_SC = 192 * 1024;                  // [3][2][keys per tile] floats (e4m3 only): the scales of tile i in slot i mod 3
constexpr int PF_OFF_FAC = PF_OFF_SC + 3 * 2 * 128 * 4;            // [3][3][128] floats: per-key factors of a tile, tiles i-1, i, i+1
constexpr int PF_OFF_MX = PF_OFF_FAC + 3 * 3 * 128 * 4;            // [2][2][128] floats: row maxima of the two key halves
constexpr int PF_OFF_BAR = PF_OFF_MX + 2 * 2 * PF_BM * 4;
constexpr int PF_SMEM = PF_OFF_BAR + 256 + 1024;
constexpr int PF_TMEM_COLS = 512;
constexpr int PF_TMEM_O = 256;          // O: columns [256, 512); S, P and (bf16) Q below it, see the kernel

struct PrefillParams {
    const __nv_bfloat16 *q;
    __nv_bfloat16 *out;
    const float *ks, *vs;
    int t, hq, hkv, g;
    long long pos, max_len;
    float scale_log2;
};

// FP8 = false: the same kernel over a bf16 cache (the reference's default mode, tokenrush/fused.py:523-533
// with FP8 = False): K, V and Q feed tcgen05.mma kind::f16 as bf16 as they are, the probabilities
// are written as bf16; no scales, no hi + lo terms.  Rows are 512 bytes (four 128-byte column
// blocks), tiles 32 KB, three stages; K and V tiles have barriers of their own, so that a K tile is
// refilled as soon as its QK^T has run.
__device__ __forceinline__ float pf_max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Diagnostic build only: the last query block of head 0 stamps clock64 at fixed points of 32 late tiles
// (slots 0-7: lane 0 of softmax warp 0, slots 8-15: lane 0 of the MMA warp) into timeline launch slot 63.
#ifdef TRB_TIMELINE
#define PF_TL(i, slot) do { if (lane == 0 && tl_on && (i) >= tl_base && (i) < tl_base + 32) g_timeline[63][(i) - tl_base][slot] = (unsigned long long)clock64(); } while (0)
#else
#define PF_TL(i, slot) do { } while (0)
#endif

template <bool FP8>
__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const PrefillParams p) {
    constexpr int PF_BN = FP8 ? 128 : 64;               // keys per tile
    constexpr int KPT = PF_BN / 2;                      // keys per softmax thread
    constexpr int ROWB = PF_D * (FP8 ? 1 : 2), SEGS = ROWB / 128, TILE = PF_BN * ROWB, STAGES = FP8 ? 2 : 3;
    constexpr int VB = PF_MAXST;                        // barrier index of a stage's V tile relative to its K tile
    constexpr int PF_OFF_Q = 0, PF_OFF_KV = FP8 ? 2 * PF_Q_BYTES : 0;   // e4m3: Qhi, Qlo in shared memory, then the stages
    // tensor memory below O: S in two buffers of PF_BN columns (P of a tile over the first columns of its S);
    // bf16: the query block in columns [128, 256), two dims per column
    constexpr int PF_TMEM_S = 0, PF_TMEM_Q = 128;
    static_assert(TILE == PF_TILE && PF_OFF_KV + STAGES * 2 * TILE == PF_OFF_SC, "shared-memory layout");
    extern __shared__ uint8_t pf_smem_raw[];
    uint8_t *smem = pf_smem_raw + ((1024u - (smem_u32(pf_smem_raw) & 1023u)) & 1023u);
    float *sm_sc = reinterpret_cast<float *>(smem + PF_OFF_SC);
    float *sm_fac = reinterpret_cast<float *>(smem + PF_OFF_FAC);
    float *sm_mx = reinterpret_cast<float *>(smem + PF_OFF_MX);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + PF_OFF_BAR);
    uint64_t *kv_full = bars, *kv_free = bars + 2 * PF_MAXST;   // [s]: K tile (+ scales) of stage s, [VB + s]: its V tile
    uint64_t *s_full = bars + 4 * PF_MAXST, *p_full = s_full + 2, *o_done = s_full + 3, *q_ready = s_full + 4;
    uint64_t *fac_full = s_full + 5;                            // [3]: the factor table of tile i (slot i mod 3) is written
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(s_full + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = blockIdx.x, h = blockIdx.y, j = h / p.g;
    const int q0 = qb * PF_BM;
    const int rows_here = p.t - q0 < PF_BM ? p.t - q0 : PF_BM;
    // keys below `hi` can be seen by some row of this block
    const long long hi = p.pos + q0 + rows_here;
    const int n_tiles = (int)((hi + PF_BN - 1) / PF_BN);
#ifdef TRB_TIMELINE
    const bool tl_on = blockIdx.x == gridDim.x - 1 && blockIdx.y == 0 && (warp == 0 || warp == 9);
    const int tl_base = n_tiles > 48 ? n_tiles - 48 : 0;      // late tiles: row maxima rarely move there
#endif

    if (threadIdx.x == 0) {
        // K and V tiles have barriers of their own, so that a K tile is refilled as soon as its QK^T has run;
        // the per-key scales of an e4m3 tile (cp.async by the 32 lanes of the producer) come with its K tile
        for (int s = 0; s < PF_MAXST; ++s) {
            mbar_init(&kv_full[s], FP8 ? 33u : 1u); mbar_init(&kv_full[VB + s], 1u);
            mbar_init(&kv_free[s], 1u); mbar_init(&kv_free[VB + s], 1u);
        }
        for (int b = 0; b < 2; ++b) mbar_init(&s_full[b], 1u);
        for (int b = 0; b < 3; ++b) mbar_init(&fac_full[b], 1u);
        mbar_init(p_full, 8u); mbar_init(o_done, 1u); mbar_init(q_ready, 8u);
        mbar_fence_init();
        tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
    }
    if (warp == 0) { tmem_alloc(tmem_slot, PF_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 8) {
        // ================================ TMA producer ================================
        // Between its loads this warp also turns the scales of a landed e4m3 tile into the per-key factors the
        // softmax threads use (score scale, log2 of the V scale, 1 / V scale), four keys per lane, a tile ahead
        // of the softmax pass that reads them.
        auto build_factors = [&](int t) -> bool {
            if (!mbar_wait(&kv_full[t % STAGES], (t / STAGES) & 1)) return false;   // the tile's scales have landed
            float *fn = sm_fac + (t % 3) * 3 * PF_BN;
#pragma unroll
            for (int hh = 0; hh < PF_BN / 32; ++hh) {
                const int k = lane + 32 * hh;
                const float kscv = sm_sc[((t % 3) * 2 + 0) * PF_BN + k], vscv = sm_sc[((t % 3) * 2 + 1) * PF_BN + k];
                fn[k] = kscv * p.scale_log2;
                fn[PF_BN + k] = vscv > 0.f ? __log2f(vscv) : -INFINITY;
                fn[2 * PF_BN + k] = vscv > 0.f ? __fdividef(1.f, vscv) : 0.f;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&fac_full[t % 3]);
            return true;
        };
        for (int i = 0; i < n_tiles; ++i) {
            const int s = i % STAGES;
            const int row0 = i * PF_BN;
            uint8_t *kt = smem + PF_OFF_KV + s * 2 * TILE, *vt = kt + TILE;
            const uint32_t par = ((i / STAGES) & 1) ^ 1;
            if (i >= STAGES && !mbar_wait(&kv_free[s], par)) break;                // QK^T of the stage's last tile has run
            if (lane == 0) {
                mbar_arrive_expect_tx(&kv_full[s], TILE);
#pragma unroll
                for (int sg = 0; sg < SEGS; ++sg) tma_load_4d(kt + sg * (PF_BN * 128), &tm_k, &kv_full[s], 0, sg, row0, j);
            }
            if constexpr (FP8) {
#pragma unroll
                for (int hh = 0; hh < PF_BN / 32; ++hh) {
                    const long long r = (long long)row0 + lane + 32 * hh;
                    const bool ok = r < p.max_len;
                    const long long off = (long long)j * p.max_len + (ok ? r : 0);
                    // slot i mod 3, not the stage: the slot is rewritten for tile i+3, whose K load waits for QK(i+1),
                    // which is issued after the softmax pass that read this slot has published its P
                    cp_async_4(&sm_sc[((i % 3) * 2 + 0) * PF_BN + lane + 32 * hh], p.ks + off, ok ? 4u : 0u);
                    cp_async_4(&sm_sc[((i % 3) * 2 + 1) * PF_BN + lane + 32 * hh], p.vs + off, ok ? 4u : 0u);
                }
                cp_async_mbar_arrive_noinc(&kv_full[s]);
            }
            // (before the wait for the V buffer, which ends a softmax pass later than the wait above: the table of
            // tile i-1 is then ready a whole pass before it is read)
            if constexpr (FP8) { if (i >= 1 && !build_factors(i - 1)) break; }
            if (i >= STAGES && !mbar_wait(&kv_free[VB + s], par)) break;           // PV of the stage's last tile has run
            if (lane == 0) {
                mbar_arrive_expect_tx(&kv_full[VB + s], TILE);
#pragma unroll
                for (int sg = 0; sg < SEGS; ++sg) tma_load_4d(vt + sg * (PF_BN * 128), &tm_v, &kv_full[VB + s], 0, sg, row0, j);
            }
            __syncwarp();
        }
        if constexpr (FP8) { if (n_tiles > 0) build_factors(n_tiles - 1); }
    } else if (warp == 9) {
        // ================================ MMA issuer ==================================
        // order on the tensor pipe: QK(0), QK(1), PV(0), QK(2), PV(1), ...  S is double-buffered so
        // that QK(i+1) runs while the softmax warps work on tile i.  The pipe runs in order of issue:
        // QK(i+2) overwrites the S buffer whose first columns hold P(i) only after PV(i) has read them.
        const uint32_t q_tm = tmem + PF_TMEM_Q;                                             // bf16 query block
        const uint32_t q_hi = smem_u32(smem + PF_OFF_Q), q_lo = q_hi + PF_Q_BYTES;          // e4m3 query block
        constexpr uint32_t IDESC_QK = FP8 ? umma_idesc_f8(PF_BM, PF_BN, false, false) : umma_idesc_bf16(PF_BM, PF_BN, false, false);
        constexpr uint32_t IDESC_PV = FP8 ? umma_idesc_f8(PF_BM, PF_D, false, true) : umma_idesc_bf16(PF_BM, PF_D, false, true);
        auto issue_qk = [&](int i) -> bool {
            const int s = i % STAGES, b = i & 1;
            const uint32_t kt = smem_u32(smem + PF_OFF_KV + s * 2 * TILE);
            PF_TL(i, 8);
            if (!mbar_wait(&kv_full[s], (i / STAGES) & 1)) return false;
            PF_TL(i, 9);
            PF_TL(i, 10);
            tc_fence_after();
            if (lane == 0) {
                if constexpr (FP8) {
                    // S = Qhi K^T + Qlo K^T : 2 column blocks x 4 k-steps of 32 dims, hi then lo; N = 128 keys
#pragma unroll
                    for (int term = 0; term < 2; ++term)
#pragma unroll
                        for (int sg = 0; sg < 2; ++sg)
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const uint64_t a = umma_desc((term ? q_lo : q_hi) + sg * (PF_BM * 128) + k * 32, 16, 1024);
                                const uint64_t bd = umma_desc(kt + sg * (PF_BN * 128) + k * 32, 16, 1024);
                                tc_mma_f8(tmem + PF_TMEM_S + b * PF_BN, a, bd, IDESC_QK, (term | sg | k) ? 1u : 0u);
                            }
                } else {
                    // S = Q K^T : 4 column blocks of 64 dims x 4 k-steps of 16 dims (8 TMEM columns of Q)
#pragma unroll
                    for (int sg = 0; sg < 4; ++sg)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t bd = umma_desc(kt + sg * (PF_BN * 128) + k * 32, 16, 1024);
                            tc_mma_bf16_ts(tmem + PF_TMEM_S + b * PF_BN, q_tm + (sg * 4 + k) * 8, bd, IDESC_QK, (sg | k) ? 1u : 0u);
                        }
                }
                tc_commit(&kv_free[s]);                                              // the K tile may be refilled
                tc_commit(&s_full[b]);
            }
            PF_TL(i, 11);
            __syncwarp();
            return true;
        };
        bool ok = mbar_wait(q_ready, 0);                                      // query block staged
        if (ok && n_tiles > 0) ok = issue_qk(0);
        for (int i = 0; i < n_tiles && ok; ++i) {
            const int s = i % STAGES;
            const uint32_t vt = smem_u32(smem + PF_OFF_KV + s * 2 * TILE) + TILE;
            const uint32_t p_tm = tmem + PF_TMEM_S + (i & 1) * PF_BN;                // P(i) lies over the first columns of S(i)
            if (i + 1 < n_tiles && !(ok = issue_qk(i + 1))) break;
            PF_TL(i, 12);
            if (!(ok = mbar_wait(&kv_full[VB + s], (i / STAGES) & 1))) break;      // V tile landed
            PF_TL(i, 13);
            if (!(ok = mbar_wait(p_full, i & 1))) break;                        // P of tile i staged (and O corrected)
            PF_TL(i, 14);
            tc_fence_after();
            if (lane == 0) {
                if constexpr (FP8) {
                    // O += Phi V + Plo V : P row = hi codes in columns [0, 32), lo in [32, 64); V tile MN-major, 32 keys per step
#pragma unroll
                    for (int term = 0; term < 2; ++term)
#pragma unroll
                        for (int k = 0; k < PF_BN / 32; ++k) {
                            const uint64_t bd = umma_desc(vt + k * (32 * 128), PF_BN * 128, 1024);
                            tc_mma_f8_ts(tmem + PF_TMEM_O, p_tm + term * (PF_BN / 4) + k * 8, bd, IDESC_PV, (i | term | k) ? 1u : 0u);
                        }
                } else {
                    // O += P V : P row = 64 keys in 32 columns; V tile MN-major (four 64-dim column blocks), 16 keys per step
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t bd = umma_desc(vt + k * (16 * 128), PF_BN * 128, 1024);
                        tc_mma_bf16_ts(tmem + PF_TMEM_O, p_tm + k * 8, bd, IDESC_PV, (i | k) ? 1u : 0u);
                    }
                }
                tc_commit(&kv_free[VB + s]);
                tc_commit(o_done);
            }
            PF_TL(i, 15);
            __syncwarp();
        }
    } else {
        // ============ softmax / correction / epilogue: warps 0-7, thread = (row, key half) ============
        const int row = (warp & 3) * 32 + lane;                               // query row = TMEM lane
        const int half = warp >> 2;                                           // keys [KPT half, KPT half + KPT) of a tile
        const bool row_ok = row < rows_here;
        const long long qpos = p.pos + q0 + row;
        const uint32_t lane_addr = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const int tid = threadIdx.x;                                          // 0..255
        // ---- stage the query block as two e4m3 copies (power-of-two row scale, hi + lo): both
        // threads of a row find the row maximum, each converts its 128 dims
        float qinv = 1.f;
        if constexpr (!FP8) {
            // bf16: the query rows as they are, two dims per TMEM column; this thread's 128 dims = 64 columns;
            // rows past t are zero
            const __nv_bfloat16 *qp = p.q + ((long long)(q0 + (row_ok ? row : 0)) * p.hq + h) * PF_D + half * (PF_D / 2);
#pragma unroll
            for (int blk = 0; blk < 2; ++blk) {
                uint32_t w[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 raw = row_ok ? *reinterpret_cast<const uint4 *>(qp + blk * 64 + c * 8) : make_uint4(0u, 0u, 0u, 0u);
                    w[c * 4 + 0] = raw.x; w[c * 4 + 1] = raw.y; w[c * 4 + 2] = raw.z; w[c * 4 + 3] = raw.w;
                }
                tmem_st32_raw(lane_addr + PF_TMEM_Q + half * 64 + blk * 32, w);
            }
            tmem_st_wait();
        } else {
            const __nv_bfloat16 *qp = p.q + ((long long)(q0 + (row_ok ? row : 0)) * p.hq + h) * PF_D;
            float amax = 0.f;
            for (int c = 0; c < PF_D / 8; ++c) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(qp + c * 8);
                const __nv_bfloat162 *b2 = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(b2[e]); amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y))); }
            }
            int e = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
            if (amax == 0.f || e < -90 || !row_ok) e = 7;
            if (e > 90) e = 90;
            const float sc = row_ok ? __uint_as_float((uint32_t)(127 + 7 - e) << 23) : 0.f;
            qinv = __uint_as_float((uint32_t)(127 - 7 + e) << 23);
            for (int cc = 0; cc < PF_D / 32; ++cc) {                           // this thread's 8 chunks of 16 dims
                const int c = half * (PF_D / 32) + cc;
                uint32_t hw[4], lw[4];
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const uint2 raw = *reinterpret_cast<const uint2 *>(qp + c * 16 + w * 4);
                    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
                    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
                    const float y[4] = {a.x * sc, a.y * sc, b.x * sc, b.y * sc};
                    pf_split4(y, hw[w], lw[w]);
                }
                const uint32_t off = (c >> 3) * (PF_BM * 128) + sw128(row, (c & 7) * 16);
                *reinterpret_cast<uint4 *>(smem + PF_OFF_Q + off) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
                *reinterpret_cast<uint4 *>(smem + PF_OFF_Q + PF_Q_BYTES + off) = make_uint4(lw[0], lw[1], lw[2], lw[3]);
            }
            fence_async_smem();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(q_ready);

        float m_run = -INFINITY, l_run = 0.f;                                  // l_run: this thread's half of the keys
        bool ok = true;
        const long long qpos_warp_min = p.pos + q0 + (warp & 3) * 32;            // lane 0's position
        const bool warp_has_padding = (warp & 3) * 32 + 31 >= rows_here;
        for (int i = 0; i < n_tiles && ok; ++i) {
            const int b = i & 1;
            float *fac = sm_fac + (i % 3) * 3 * PF_BN;            // per-key factors of this tile, written by the producer warp
            float *mxbuf = sm_mx + b * 2 * PF_BM;
            PF_TL(i, 0);
            if (!(ok = mbar_wait(&s_full[b], (i >> 1) & 1))) break;
            if constexpr (FP8) { if (!(ok = mbar_wait(&fac_full[i % 3], (i / 3) & 1))) break; }
            PF_TL(i, 1);
            tc_fence_after();
            float sv[KPT];
#pragma unroll
            for (int c = 0; c < KPT / 32; ++c)
                tmem_ld32(lane_addr + PF_TMEM_S + b * PF_BN + half * KPT + c * 32, *reinterpret_cast<float (*)[32]>(&sv[c * 32]));
            PF_TL(i, 2);
            // scores -> exponent domain (t = raw * k_scale * c * q_inv + log2 v_scale), row maximum
            const long long key0 = (long long)i * PF_BN + half * KPT;
            const float *fa_ = fac + half * KPT, *fb_ = fac + PF_BN + half * KPT, *fr_ = fac + 2 * PF_BN + half * KPT;
            if constexpr (!FP8) {
                const float2 sl2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
                for (int c = 0; c < KPT / 2; ++c) {
                    const float2 a = __fmul2_rn(make_float2(sv[2 * c], sv[2 * c + 1]), sl2);
                    sv[2 * c] = a.x; sv[2 * c + 1] = a.y;
                }
            } else {
                const float2 qinv2 = make_float2(qinv, qinv);
#pragma unroll
                for (int c4 = 0; c4 < KPT / 4; ++c4) {                             // two scores per FMA-pipe instruction
                    const float4 fa = *reinterpret_cast<const float4 *>(fa_ + c4 * 4);
                    const float4 fb = *reinterpret_cast<const float4 *>(fb_ + c4 * 4);
                    const float2 a = __ffma2_rn(__fmul2_rn(make_float2(sv[c4 * 4 + 0], sv[c4 * 4 + 1]), make_float2(fa.x, fa.y)), qinv2, make_float2(fb.x, fb.y));
                    const float2 c = __ffma2_rn(__fmul2_rn(make_float2(sv[c4 * 4 + 2], sv[c4 * 4 + 3]), make_float2(fa.z, fa.w)), qinv2, make_float2(fb.z, fb.w));
                    sv[c4 * 4 + 0] = a.x; sv[c4 * 4 + 1] = a.y; sv[c4 * 4 + 2] = c.x; sv[c4 * 4 + 3] = c.y;
                }
            }
            if (key0 + KPT - 1 > qpos_warp_min || warp_has_padding) {          // the tile crosses this warp's diagonal
#pragma unroll
                for (int c = 0; c < KPT; ++c)
                    if (!(key0 + c <= qpos && row_ok)) sv[c] = -INFINITY;
            }
            float mt4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < KPT / 2; ++c) mt4[c & 3] = pf_max3(mt4[c & 3], sv[2 * c], sv[2 * c + 1]);
            float mt = fmaxf(fmaxf(mt4[0], mt4[1]), fmaxf(mt4[2], mt4[3]));
            mxbuf[half * PF_BM + row] = mt;
            PF_TL(i, 3);
            named_barrier(1, PF_SOFTMAX_THREADS);
            PF_TL(i, 4);
            mt = fmaxf(mt, mxbuf[(half ^ 1) * PF_BM + row]);
            const float m_new = fmaxf(m_run, mt);
            const float m_safe = m_new == -INFINITY ? 0.f : m_new;
            const float m_off = FP8 ? m_safe - 8.f : m_safe;                    // e4m3 probabilities are staged x 256
            const float alpha = m_new == -INFINITY ? 1.f : fast_exp2(m_run - m_safe);   // rows with no visible key yet
            // O is corrected only where a row maximum of this warp moved, and only then the previous PV must
            // have landed (S of this tile exists, so PV(i-2) has completed: the parity cannot be mistaken)
            if (__any_sync(0xffffffffu, alpha != 1.f) && i > 0) {               // this thread corrects its 128 columns
                if (!(ok = mbar_wait(o_done, (i - 1) & 1))) break;
                tc_fence_after();
#pragma unroll 1
                for (int c = 0; c < PF_D / 64; ++c) {
                    float ov[32];
                    tmem_ld32(lane_addr + PF_TMEM_O + half * (PF_D / 2) + c * 32, ov);
#pragma unroll
                    for (int e = 0; e < 32; ++e) ov[e] *= alpha;
                    tmem_st32(lane_addr + PF_TMEM_O + half * (PF_D / 2) + c * 32, ov);
                }
            }
            PF_TL(i, 5);
            const uint32_t p_tm = lane_addr + PF_TMEM_S + b * PF_BN;            // P over the first columns of this tile's S (all of S was read before the barrier above)
            float lsum = 0.f;
            if constexpr (!FP8) {
                uint32_t w[16];                                                 // this thread's 32 keys, two per column
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float p0 = fast_exp2(sv[e * 2] - m_off), p1 = fast_exp2(sv[e * 2 + 1] - m_off);
                    lsum += p0 + p1;
                    w[e] = pack_bf16x2(p0, p1);
                }
                tmem_st16_raw(p_tm + half * 16, w);
            } else {
                // hi codes of the tile's keys in columns [0, PF_BN / 4), lo codes in the next PF_BN / 4; four keys per column
                const float2 nm2 = make_float2(-m_off, -m_off);
                float2 lsa = make_float2(0.f, 0.f), lsb = make_float2(0.f, 0.f);
#pragma unroll
                for (int g32 = 0; g32 < KPT / 32; ++g32) {                      // 32 keys -> 8 columns of hi and of lo codes
                    uint32_t hw8[8], lw8[8];
#pragma unroll
                    for (int w = 0; w < 8; ++w) {
                        const int k0 = g32 * 32 + w * 4;
                        const float4 fr = *reinterpret_cast<const float4 *>(fr_ + k0);
                        const float2 d01 = __fadd2_rn(make_float2(sv[k0 + 0], sv[k0 + 1]), nm2);
                        const float2 d23 = __fadd2_rn(make_float2(sv[k0 + 2], sv[k0 + 3]), nm2);
                        const float2 p01 = make_float2(fast_exp2(d01.x), fast_exp2(d01.y));
                        const float2 p23 = make_float2(fast_exp2(d23.x), fast_exp2(d23.y));
                        lsa = __ffma2_rn(p01, make_float2(fr.x, fr.y), lsa);
                        lsb = __ffma2_rn(p23, make_float2(fr.z, fr.w), lsb);
                        uint32_t h01, l01, h23, l23;
                        pf_split2_h(p01.x, p01.y, h01, l01);
                        pf_split2_h(p23.x, p23.y, h23, l23);
                        hw8[w] = h01 | (h23 << 16);
                        lw8[w] = l01 | (l23 << 16);
                    }
                    tmem_st8_raw(p_tm + half * (KPT / 4) + g32 * 8, hw8);
                    tmem_st8_raw(p_tm + PF_BN / 4 + half * (KPT / 4) + g32 * 8, lw8);
                }
                lsum = (lsa.x + lsa.y) + (lsb.x + lsb.y);
            }
            l_run = fmaf(l_run, alpha, lsum);
            m_run = m_new;
            PF_TL(i, 6);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            PF_TL(i, 7);
        }
        // ---- epilogue: O / l -> bf16 (with e4m3 both carry the factor 256); l = sum of the two halves' partial sums
        // (a warp that skipped corrections may be two PVs behind the barrier's phase: one step at a time,
        // so that a parity always names the phase it is meant for)
        if (ok && n_tiles > 1) ok = mbar_wait(o_done, (n_tiles - 2) & 1);
        if (ok && n_tiles > 0) ok = mbar_wait(o_done, (n_tiles - 1) & 1);
        tc_fence_after();
        sm_mx[half * PF_BM + row] = l_run;
        named_barrier(1, PF_SOFTMAX_THREADS);
        const float l_tot = l_run + sm_mx[(half ^ 1) * PF_BM + row];
        if (ok) {
            const float inv = 1.f / l_tot;
            __nv_bfloat16 *op = p.out + ((long long)(q0 + (row_ok ? row : 0)) * p.hq + h) * PF_D + half * (PF_D / 2);
#pragma unroll 1
            for (int c = 0; c < PF_D / 64; ++c) {
                float ov[32];
                tmem_ld32(lane_addr + PF_TMEM_O + half * (PF_D / 2) + c * 32, ov);
                if (row_ok) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        uint4 o4;
                        o4.x = pack_bf16x2(ov[e * 8 + 0] * inv, ov[e * 8 + 1] * inv);
                        o4.y = pack_bf16x2(ov[e * 8 + 2] * inv, ov[e * 8 + 3] * inv);
                        o4.z = pack_bf16x2(ov[e * 8 + 4] * inv, ov[e * 8 + 5] * inv);
                        o4.w = pack_bf16x2(ov[e * 8 + 6] * inv, ov[e * 8 + 7] * inv);
                        *reinterpret_cast<uint4 *>(op + c * 32 + e * 8) = o4;
                    }
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, PF_TMEM_COLS); }
}

}  // namespace trb

using namespace trb;

extern "C" int trb_attn_prefill(const trb_cache_t *cache, const void *q, void *out, int32_t t, int32_t hq, int64_t pos,
                                float scale, trb_stream_t stream) {
    CacheView c;
    int rc = make_cache_view(cache, &c);
    if (rc) return rc;
    if (!q || !out || t < 1 || hq < 1 || hq % c.hkv || pos < 0) return TRB_E_ARG;
    if (c.d != PF_D || c.ring > 0 || c.sharded) return TRB_E_UNSUPPORTED;
    if (pos + t > c.max_len) return TRB_E_CAPACITY;
    if (((uintptr_t)q | (uintptr_t)out) & 15) return TRB_E_ALIGN;
    if (c.max_len >= (1LL << 31) - 128) return TRB_E_UNSUPPORTED;
    PrefillParams p;
    p.q = (const __nv_bfloat16 *)q; p.out = (__nv_bfloat16 *)out; p.ks = c.k_scale; p.vs = c.v_scale;
    p.t = t; p.hq = hq; p.hkv = c.hkv; p.g = hq / c.hkv; p.pos = pos; p.max_len = c.max_len;
    p.scale_log2 = scale * 1.4426950408889634f;
    CUtensorMap mk, mv;
    const int row_bytes = PF_D * (c.fp8 ? 1 : 2);
    const int tile_rows = c.fp8 ? 128 : 64;
    if ((rc = get_row_tile_map(c.k, c.max_len, c.hkv, row_bytes, tile_rows, &mk))) return rc;
    if ((rc = get_row_tile_map(c.v, c.max_len, c.hkv, row_bytes, tile_rows, &mv))) return rc;
    static bool attr_set[64] = {};
    int dev = 0;
    TRB_CUDA_CHECK(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        TRB_CUDA_CHECK(cudaFuncSetAttribute(prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM));
        TRB_CUDA_CHECK(cudaFuncSetAttribute(prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM));
        attr_set[dev & 63] = true;
    }
    dim3 grid((t + PF_BM - 1) / PF_BM, hq);
    pdl_note_fence((cudaStream_t)stream);
    if (c.fp8) prefill_kernel<true><<<grid, PF_THREADS, PF_SMEM, (cudaStream_t)stream>>>(mk, mv, p);
    else prefill_kernel<false><<<grid, PF_THREADS, PF_SMEM, (cudaStream_t)stream>>>(mk, mv, p);
    TRB_CUDA_CHECK(cudaGetLastError());
    return TRB_OK;
}
