// Split-K flash-decoding over the live length of an FP8 (e4m3 + per-row scale) or bf16 KV
// cache, with the split partial-combine fused into the tail of the same launch.
//
// Shape of the kernel (one CTA per (split, kv head), 2 CTAs per SM):
//   * one producer warp streams 32-key tiles of K and V into a ring of shared-memory stages
//     with TMA (cp.async.bulk.tensor, 128-byte swizzle) and the two scale vectors with
//     cp.async; completion is tracked by one mbarrier per stage;
//   * six consumer warps each own an 8-row slice of the (query row x query head) rows of
//     this kv head and a subset of the 16-key groups.  Per group: S^T = K Q^T and
//     O^T += V^T P^T on mma.sync m16n8k16 with the KEYS (resp. dims) as the 16-row operand,
//     so the 6..48 query rows fill n = 8 columns instead of padding a 16-row tile;
//     e4m3 codes go to f16 in registers (exact) and the per-key scales are applied to the
//     fp32 scores / folded into the probabilities, never to the codes;
//   * online softmax in registers with warp shuffles; every warp keeps its own running
//     (max, sum, acc) and the warps of a CTA, the CTAs of a kv head and (for sequence
//     shards) the GPUs are all merged with the same log-sum-exp formula in a fixed order;
//   * the last CTA of a kv head to finish (an atomic ticket that resets itself, so the
//     launch replays inside a CUDA graph) merges the split partials and writes the output.
//
// The live length and all split ranges are derived on the device from the cursor, so the
// grid is static and one captured graph serves every length.
#include "common.cuh"
#include "tmap.h"

namespace trb {

constexpr int DEC_BN = 32;                       // keys per pipeline stage
constexpr int DEC_CONSUMERS = 6;                 // consumer warps per CTA
constexpr int DEC_CTHREADS = DEC_CONSUMERS * 32;
constexpr int DEC_THREADS = DEC_CTHREADS + 32;   // + one producer warp
constexpr int DEC_MAX_ROWS = 48;                 // (hq / hkv) * m
constexpr int DEC_MIN_TILES = 4;                 // a split is not made smaller than this
constexpr int DEC_STAGE_BYTES_TOTAL = 96 * 1024;
constexpr int DEC_MAX_SPLITS = 148;              // bounds the tail's weight table in shared memory
constexpr int DEC_EPI_PAD = 4;                   // floats of padding per staged output row

struct DecodeParams {
    const __nv_bfloat16 *q;
    __nv_bfloat16 *out;
    const __nv_bfloat16 *gate;
    long long gate_rs, gate_hs;
    const float *ks, *vs;
    int m, hq, hkv, g, rows;      // rows = g * m
    int nt, kw;                   // 8-row slices, key groups in flight (nt * kw <= 6)
    int nsplit, rows_pad;
    float scale_log2;             // softmax scale * log2(e)
    int new_rows, window, n_extra;
    const float *extra_ml, *extra_acc;
    Cursor pos;
    long long max_len, ring, shard_lo;
    int sharded;
    unsigned int *counters;
    float *part_ml, *part_acc;
    float *shard_ml, *shard_acc;
};

template <int D, bool FP8>
struct DecodeCfg {
    static constexpr int ROWB = D * (FP8 ? 1 : 2);
    static constexpr int SEGS = ROWB / 128;
    static constexpr int TILE = DEC_BN * ROWB;
    static constexpr int NSTAGE_RAW = DEC_STAGE_BYTES_TOTAL / (2 * TILE);
    static constexpr int NSTAGE = NSTAGE_RAW > 8 ? 8 : NSTAGE_RAW;
    static constexpr int NCP = ROWB / 32;                        // 32-byte chunk pairs per row
    static constexpr int ACC = FP8 ? NCP * 2 : NCP;              // m16n8 accumulator tiles
    static constexpr int SCALE_OFF = NSTAGE * 2 * TILE;          // [NSTAGE][2][BN] floats
    static constexpr int BAR_OFF = SCALE_OFF + NSTAGE * 2 * DEC_BN * 4;
    static constexpr int MISC_OFF = BAR_OFF + 2 * NSTAGE * 8;    // small epilogue scratch
    static constexpr int MISC_BYTES = DEC_CONSUMERS * 8 * 2 * 4 + 64;
    static constexpr int SMEM = MISC_OFF + MISC_BYTES + 1024;    // + slack to align the base
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

template <int D, bool FP8>
__global__ void __maxnreg__(144)
decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v, const DecodeParams p) {
    using C = DecodeCfg<D, FP8>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    float *sm_scale = reinterpret_cast<float *>(smem + C::SCALE_OFF);
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(smem + C::BAR_OFF);
    uint64_t *bar_empty = bar_full + C::NSTAGE;
    float *sm_ml = reinterpret_cast<float *>(smem + C::MISC_OFF);                 // [6][8][2]
    int *sm_flag = reinterpret_cast<int *>(smem + C::MISC_OFF + DEC_CONSUMERS * 64);

    const int split = blockIdx.x, j = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

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

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::NSTAGE; ++s) {
            mbar_init(&bar_full[s], FP8 ? 33u : 1u);
            mbar_init(&bar_empty[s], (uint32_t)((DEC_BN / 16) * p.nt));
        }
        mbar_fence_init();
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
    }
    __syncthreads();

    // =============================== producer warp =======================================
    if (warp == DEC_CONSUMERS) {
        for (int i = 0; i < my_tiles; ++i) {
            const int s = i % C::NSTAGE;
            if (i >= C::NSTAGE && !mbar_wait(&bar_empty[s], ((i / C::NSTAGE) & 1) ^ 1)) break;
            const long long vrow0 = (long long)(t0 + i) * DEC_BN;
            const int prow0 = (int)(p.ring > 0 ? vrow0 % p.ring : vrow0);
            if (lane == 0) {
                mbar_arrive_expect_tx(&bar_full[s], 2 * C::TILE);
#pragma unroll
                for (int sg = 0; sg < C::SEGS; ++sg) {          // one 128-byte column of the rows per copy
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
        }
        return;
    }

    // =============================== consumer warps ======================================
    const int g = lane >> 2, t = lane & 3;
    const bool warp_on = warp < p.nt * p.kw;
    const int nt_idx = warp_on ? warp % p.nt : 0;
    const int kw_idx = warp_on ? warp / p.nt : 0;

    // Query fragments (the B operand of S^T = K Q^T), column n = g of this warp's 8-row slice.
    uint32_t qf[C::NCP][FP8 ? 2 : 1][2];
    {
        const int r = 8 * nt_idx + g;
        const bool valid = warp_on && r < p.rows;
        const int qi = valid ? r / p.g : 0, hq = valid ? j * p.g + r % p.g : 0;
        const __nv_bfloat16 *qp = p.q + ((long long)qi * p.hq + hq) * D;
#pragma unroll
        for (int cp = 0; cp < C::NCP; ++cp) {
            if (FP8) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int w = 0; w < 2; ++w) {
                        const int d0 = 32 * cp + 16 * w + 4 * t + 2 * h;
                        float2 f = make_float2(0.f, 0.f);
                        if (valid) f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(qp + d0));
                        qf[cp][h][w] = pack_f16x2(f.x, f.y);
                    }
                }
            } else {
#pragma unroll
                for (int w = 0; w < 2; ++w) {
                    const int d0 = 16 * cp + 8 * w + 2 * t;
                    qf[cp][0][w] = valid ? *reinterpret_cast<const uint32_t *>(qp + d0) : 0u;
                }
            }
        }
    }

    // Visibility window of this lane's two query columns, in virtual rows of this cache.
    long long lim_hi[2], lim_lo[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int r = 8 * nt_idx + 2 * t + c;
        const int qi = r < p.rows ? r / p.g : 0;               // padding rows copy row 0's window
        long long hi = lloc - 1;
        if (p.new_rows && pos + qi - p.shard_lo < hi) hi = pos + qi - p.shard_lo;
        lim_hi[c] = hi;
        lim_lo[c] = p.window > 0 ? pos + qi - p.window + 1 - p.shard_lo : 0;
    }
    // bounds within which a whole 16-key group needs no masking for any column of the slice
    long long all_hi = lloc - 1, all_lo = 0;
    if (p.new_rows) {
        const long long h0 = pos + (8 * nt_idx < p.rows ? (8 * nt_idx) / p.g : 0) - p.shard_lo;
        if (h0 < all_hi) all_hi = h0;
    }
    if (p.window > 0) {
        int rmax = 8 * nt_idx + 7;
        if (rmax >= p.rows) rmax = p.rows - 1;
        all_lo = pos + (rmax >= 0 ? rmax / p.g : 0) - p.window + 1 - p.shard_lo;
    }

    float mx[2] = {-INFINITY, -INFINITY}, ls[2] = {0.f, 0.f};
    float acc[C::ACC][4];
#pragma unroll
    for (int a = 0; a < C::ACC; ++a)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[a][i] = 0.f;

    const int mi = lane >> 3, rr = lane & 7;
    const int k_key = rr + 8 * (mi & 1), k_chunk = mi >> 1;    // ldmatrix lane roles for K
    const int v_key = rr + 8 * (mi >> 1), v_chunk = mi & 1;    // ... and for V (transposed)
    bool dead = false;

    if (warp_on) {
        for (int i = 0; i < my_tiles && !dead; ++i) {
            const int s = i % C::NSTAGE;
            bool waited = false;
#pragma unroll 1
            for (int grp = 0; grp < DEC_BN / 16; ++grp) {
                const int gi = i * (DEC_BN / 16) + grp;
                if (gi % p.kw != kw_idx) continue;
                if (!waited) {
                    if (!mbar_wait(&bar_full[s], (i / C::NSTAGE) & 1)) { dead = true; break; }
                    waited = true;
                }
                const long long key0 = (long long)(t0 + i) * DEC_BN + grp * 16;       // virtual row of the group
                if (key0 < lloc && key0 + 15 >= row_lo) {
                    const uint32_t kt = smem_u32(smem + s * 2 * C::TILE);
                    const uint32_t vt = kt + C::TILE;
                    // ---- S^T[16 keys, 8 columns] = K Q^T, four independent accumulation chains
                    float s4[4][4];
#pragma unroll
                    for (int c = 0; c < 4; ++c)
#pragma unroll
                        for (int e = 0; e < 4; ++e) s4[c][e] = 0.f;
#pragma unroll
                    for (int cp = 0; cp < C::NCP; ++cp) {
                        uint32_t r[4];
                        ldmatrix_x4(r, kt + tile_off(grp * 16 + k_key, (2 * cp + k_chunk) * 16));
                        if (FP8) {
                            uint32_t a[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) a[e] = e4m3x2_to_f16x2((uint16_t)(r[e] & 0xffffu));
                            mma_f16(s4[(2 * cp) & 3], a, qf[cp][0][0], qf[cp][0][1]);
#pragma unroll
                            for (int e = 0; e < 4; ++e) a[e] = e4m3x2_to_f16x2((uint16_t)(r[e] >> 16));
                            mma_f16(s4[(2 * cp + 1) & 3], a, qf[cp][1][0], qf[cp][1][1]);
                        } else {
                            mma_bf16(s4[cp & 3], r, qf[cp][0][0], qf[cp][0][1]);
                        }
                    }
                    float tv[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) tv[e] = (s4[0][e] + s4[1][e]) + (s4[2][e] + s4[3][e]);

                    // ---- per-key factors: score scale, and the V scale moved into the exponent
                    float ka[2], vb[2], vr[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (FP8) {
                            const float ksc = sm_scale[(s * 2 + 0) * DEC_BN + grp * 16 + g + 8 * h];
                            const float vsc = sm_scale[(s * 2 + 1) * DEC_BN + grp * 16 + g + 8 * h];
                            ka[h] = ksc * p.scale_log2;
                            vb[h] = __log2f(vsc);
                            vr[h] = __frcp_rn(vsc);
                        } else {
                            ka[h] = p.scale_log2; vb[h] = 0.f; vr[h] = 1.f;
                        }
                    }
                    // tv[e]: e = 2*h + c  ->  key g + 8h, column 2t + c
#pragma unroll
                    for (int e = 0; e < 4; ++e) tv[e] = fmaf(tv[e], ka[e >> 1], vb[e >> 1]);
                    const bool full_vis = key0 + 15 <= all_hi && key0 >= all_lo;
                    if (!full_vis) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const long long kv = key0 + g + 8 * (e >> 1);
                            const bool vis = kv <= lim_hi[e & 1] && kv >= lim_lo[e & 1];
                            if (!vis) { tv[e] = -INFINITY; }
                        }
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const long long kv = key0 + g + 8 * h;
                            if (kv >= lloc) vr[h] = 0.f;                       // never-written rows: scale may be anything
                        }
                    }
                    // ---- online softmax over the keys (rows of S^T): reduce across the g lanes
                    float pr[4], alpha[2];
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        float ml = fmaxf(tv[c], tv[2 + c]);
                        ml = fmaxf(ml, __shfl_xor_sync(0xffffffffu, ml, 4));
                        ml = fmaxf(ml, __shfl_xor_sync(0xffffffffu, ml, 8));
                        ml = fmaxf(ml, __shfl_xor_sync(0xffffffffu, ml, 16));
                        const float mn = fmaxf(mx[c], ml);
                        const float msafe = mn == -INFINITY ? 0.f : mn;
                        alpha[c] = fast_exp2(mx[c] - msafe);
                        pr[c] = fast_exp2(tv[c] - msafe);
                        pr[2 + c] = fast_exp2(tv[2 + c] - msafe);
                        ls[c] = fmaf(ls[c], alpha[c], fmaf(pr[c], vr[0], pr[2 + c] * vr[1]));
                        mx[c] = mn;
                    }
                    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                        for (int a = 0; a < C::ACC; ++a) {
                            acc[a][0] *= alpha[0]; acc[a][1] *= alpha[1];
                            acc[a][2] *= alpha[0]; acc[a][3] *= alpha[1];
                        }
                    }
                    // ---- P^T as the B operand: transpose the 8x8 blocks across the warp
                    const uint32_t w0 = FP8 ? pack_f16x2(pr[0], pr[1]) : pack_bf16x2(pr[0], pr[1]);
                    const uint32_t w1 = FP8 ? pack_f16x2(pr[2], pr[3]) : pack_bf16x2(pr[2], pr[3]);
                    const uint32_t pb0 = movmatrix_trans(w0), pb1 = movmatrix_trans(w1);
                    // ---- O^T[D dims, 8 columns] += V^T P^T
#pragma unroll
                    for (int cp = 0; cp < C::NCP; ++cp) {
                        uint32_t w[4];
                        ldmatrix_x4_trans(w, vt + tile_off(grp * 16 + v_key, (2 * cp + v_chunk) * 16));
                        if (FP8) {
                            uint32_t a[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) w[e] = prmt(w[e], 0u, 0x3120u);
#pragma unroll
                            for (int e = 0; e < 4; ++e) a[e] = e4m3x2_to_f16x2((uint16_t)(w[e] & 0xffffu));
                            mma_f16(acc[2 * cp], a, pb0, pb1);
#pragma unroll
                            for (int e = 0; e < 4; ++e) a[e] = e4m3x2_to_f16x2((uint16_t)(w[e] >> 16));
                            mma_f16(acc[2 * cp + 1], a, pb0, pb1);
                        } else {
                            mma_bf16(acc[cp], w, pb0, pb1);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_empty[s]);
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
    // 1. merge the kw warps that share an 8-row slice (fixed order), through shared memory
    named_barrier(1, DEC_CTHREADS);                    // every stage has been consumed
    if (warp_on && g == 0) {
        sm_ml[(warp * 8 + 2 * t + 0) * 2 + 0] = mx[0]; sm_ml[(warp * 8 + 2 * t + 0) * 2 + 1] = ls[0];
        sm_ml[(warp * 8 + 2 * t + 1) * 2 + 0] = mx[1]; sm_ml[(warp * 8 + 2 * t + 1) * 2 + 1] = ls[1];
    }
    named_barrier(1, DEC_CTHREADS);
    float *stage_acc = reinterpret_cast<float *>(smem);                // [warp][8][D + pad]
    constexpr int SROW = D + DEC_EPI_PAD;
    if (warp_on) {
        float wgt[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            float mg = -INFINITY;
            for (int k = 0; k < p.kw; ++k) mg = fmaxf(mg, sm_ml[((k * p.nt + nt_idx) * 8 + 2 * t + c) * 2]);
            wgt[c] = mg == -INFINITY ? 0.f : fast_exp2(mx[c] - mg);
        }
#pragma unroll
        for (int a = 0; a < C::ACC; ++a)
#pragma unroll
            for (int i = 0; i < 4; ++i)
                stage_acc[(warp * 8 + 2 * t + (i & 1)) * SROW + acc_dim<FP8>(a, i, g)] = acc[a][i] * wgt[i & 1];
    }
    named_barrier(1, DEC_CTHREADS);
    const int tid = threadIdx.x;                                       // 0..191 here
    const long long part_base = ((long long)j * p.nsplit + split) * p.rows_pad;
    for (int item = tid; item < p.nt * 8 * (D / 4); item += DEC_CTHREADS) {
        const int row = item / (D / 4), d4 = (item % (D / 4)) * 4;
        if (row >= p.rows) continue;
        const int nti = row >> 3, qc = row & 7;
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < p.kw; ++k) {
            const float4 v = *reinterpret_cast<const float4 *>(&stage_acc[((k * p.nt + nti) * 8 + qc) * SROW + d4]);
            sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
        }
        *reinterpret_cast<float4 *>(&p.part_acc[(part_base + row) * D + d4]) = sum;
    }
    for (int row = tid; row < p.rows; row += DEC_CTHREADS) {
        const int nti = row >> 3, qc = row & 7;
        float mg = -INFINITY;
        for (int k = 0; k < p.kw; ++k) mg = fmaxf(mg, sm_ml[((k * p.nt + nti) * 8 + qc) * 2]);
        float lg = 0.f;
        for (int k = 0; k < p.kw; ++k) {
            const float mk = sm_ml[((k * p.nt + nti) * 8 + qc) * 2], lk = sm_ml[((k * p.nt + nti) * 8 + qc) * 2 + 1];
            lg += mk == -INFINITY ? 0.f : lk * fast_exp2(mk - mg);
        }
        p.part_ml[(part_base + row) * 2 + 0] = mg;
        p.part_ml[(part_base + row) * 2 + 1] = lg;
    }

    // 2. ticket: the last CTA of this kv head merges the splits
    __threadfence();
    named_barrier(1, DEC_CTHREADS);
    if (tid == 0) {
        const unsigned int old = atomicAdd(&p.counters[j], 1u);
        const int last = old == (unsigned int)(active - 1);
        if (last) p.counters[j] = 0u;                                  // ready for the next launch / replay
        *sm_flag = last;
    }
    named_barrier(1, DEC_CTHREADS);
    if (!*sm_flag) return;
    __threadfence();

    // 3. tail: LSE merge over the active splits (+ extra partials), fixed order
    const int n_parts = active + p.n_extra;
    float *sm_w = stage_acc + DEC_CONSUMERS * 8 * SROW;               // [rows][n_parts] weights, then [rows] 1/l
    float *sm_inv = sm_w + DEC_MAX_ROWS * (p.nsplit + 1);
    for (int row = warp; row < p.rows; row += DEC_CONSUMERS) {
        const int qi = row / p.g, hq = j * p.g + row % p.g;
        const long long grow = (long long)qi * p.hq + hq;
        float mmax = -INFINITY;
        for (int s = lane; s < n_parts; s += 32) {
            const float ms = s < active ? __ldcg(&p.part_ml[(((long long)j * p.nsplit + s) * p.rows_pad + row) * 2])
                                        : p.extra_ml[(grow * p.n_extra + (s - active)) * 2];
            mmax = fmaxf(mmax, ms);
        }
        mmax = warp_max(mmax);
        float lsum = 0.f;
        for (int s = lane; s < n_parts; s += 32) {
            float ms, lsv;
            if (s < active) {
                const float2 v = __ldcg(reinterpret_cast<const float2 *>(&p.part_ml[(((long long)j * p.nsplit + s) * p.rows_pad + row) * 2]));
                ms = v.x; lsv = v.y;
            } else {
                ms = p.extra_ml[(grow * p.n_extra + (s - active)) * 2];
                lsv = p.extra_ml[(grow * p.n_extra + (s - active)) * 2 + 1];
            }
            const float w = ms == -INFINITY ? 0.f : fast_exp2(ms - mmax);
            sm_w[row * n_parts + s] = w;
            lsum += w * lsv;
        }
        lsum = warp_sum(lsum);
        if (lane == 0) {
            sm_inv[row] = 1.f / lsum;
            if (p.shard_ml) { p.shard_ml[grow * 2] = mmax; p.shard_ml[grow * 2 + 1] = lsum; }
        }
    }
    named_barrier(1, DEC_CTHREADS);
    for (int item = tid; item < p.rows * (D / 4); item += DEC_CTHREADS) {
        const int row = item / (D / 4), d4 = (item % (D / 4)) * 4;
        const int qi = row / p.g, hq = j * p.g + row % p.g;
        const long long grow = (long long)qi * p.hq + hq;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        const float *wr = sm_w + row * n_parts;
#pragma unroll 4
        for (int s = 0; s < active; ++s) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(&p.part_acc[(((long long)j * p.nsplit + s) * p.rows_pad + row) * D + d4]));
            const float w = wr[s];
            o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
        }
        for (int e = 0; e < p.n_extra; ++e) {
            const float4 v = *reinterpret_cast<const float4 *>(&p.extra_acc[(grow * p.n_extra + e) * D + d4]);
            const float w = wr[active + e];
            o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
        }
        if (p.shard_acc) {
            *reinterpret_cast<float4 *>(&p.shard_acc[grow * D + d4]) = o;
            continue;
        }
        const float inv = sm_inv[row];
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

// splits per kv head: two CTAs per SM over all heads
static int decode_nsplit(int hkv) {
    int n = (2 * sm_count()) / hkv;
    if (n > DEC_MAX_SPLITS) n = DEC_MAX_SPLITS;
    return n < 1 ? 1 : n;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

struct WorkspaceLayout {
    size_t counters, ml, acc, total;
};
static WorkspaceLayout workspace_layout(int hkv, int nsplit, int rows_pad, int d) {
    WorkspaceLayout w;
    w.counters = 0;
    w.ml = 256;
    w.acc = align_up(w.ml + (size_t)hkv * nsplit * rows_pad * 2 * sizeof(float), 256);
    w.total = w.acc + (size_t)hkv * nsplit * rows_pad * d * sizeof(float);
    return w;
}

template <int D, bool FP8>
static int launch_decode(const CUtensorMap &mk, const CUtensorMap &mv, const DecodeParams &p, cudaStream_t st) {
    using C = DecodeCfg<D, FP8>;
    static bool attr_set[64] = {};
    int dev = 0;
    TRB_CUDA_CHECK(cudaGetDevice(&dev));
    if (!attr_set[dev & 63]) {
        TRB_CUDA_CHECK(cudaFuncSetAttribute(decode_kernel<D, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        attr_set[dev & 63] = true;
    }
    dim3 grid(p.nsplit, p.hkv);
    decode_kernel<D, FP8><<<grid, DEC_THREADS, C::SMEM, st>>>(mk, mv, p);
    TRB_CUDA_CHECK(cudaGetLastError());
    return TRB_OK;
}

}  // namespace trb

using namespace trb;

extern "C" size_t trb_decode_workspace_bytes(int32_t hq, int32_t hkv, int32_t d, int32_t m) {
    if (hq < 1 || hkv < 1 || hq % hkv || m < 1) return 0;
    const int rows = (hq / hkv) * m;
    if (rows > DEC_MAX_ROWS) return 0;
    const int rows_pad = (rows + 7) / 8 * 8;
    return workspace_layout(hkv, decode_nsplit(hkv), rows_pad, d).total;
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
    if (c.max_len >= (1LL << 31)) return TRB_E_UNSUPPORTED;
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
    p.nt = (rows + 7) / 8; p.kw = DEC_CONSUMERS / p.nt;
    p.nsplit = decode_nsplit(c.hkv); p.rows_pad = p.nt * 8;
    p.scale_log2 = a->scale * 1.4426950408889634f;
    p.new_rows = a->new_rows ? 1 : 0; p.window = a->window; p.n_extra = a->n_extra;
    p.extra_ml = a->extra_ml; p.extra_acc = a->extra_acc;
    p.pos = make_cursor(&a->pos);
    p.max_len = c.max_len; p.ring = c.ring; p.shard_lo = c.shard_lo; p.sharded = c.sharded;
    const WorkspaceLayout w = workspace_layout(c.hkv, p.nsplit, p.rows_pad, c.d);
    if (a->workspace_bytes < w.total) return TRB_E_CAPACITY;
    uint8_t *ws = (uint8_t *)a->workspace;
    p.counters = (unsigned int *)(ws + w.counters);
    p.part_ml = (float *)(ws + w.ml); p.part_acc = (float *)(ws + w.acc);
    p.shard_ml = a->partial_ml; p.shard_acc = a->partial_acc;

    const int row_bytes = c.d * (c.fp8 ? 1 : 2);
    CUtensorMap mk, mv;
    if ((rc = get_row_tile_map(c.k, c.max_len, c.hkv, row_bytes, DEC_BN, &mk))) return rc;
    if ((rc = get_row_tile_map(c.v, c.max_len, c.hkv, row_bytes, DEC_BN, &mv))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (c.d == 256) return c.fp8 ? launch_decode<256, true>(mk, mv, p, st) : launch_decode<256, false>(mk, mv, p, st);
    return c.fp8 ? launch_decode<128, true>(mk, mv, p, st) : launch_decode<128, false>(mk, mv, p, st);
}

extern "C" int trb_attn_block_partial(const void *q, const void *k_blk, const void *v_blk, int32_t b, int32_t hq, int32_t hkv,
                                      int32_t d, float scale, float *extra_ml, float *extra_acc, trb_stream_t stream) {
    if (!q || !k_blk || !v_blk || !extra_ml || !extra_acc || b < 1 || hq < 1 || hkv < 1 || hq % hkv) return TRB_E_ARG;
    if (d != 128 && d != 256) return TRB_E_UNSUPPORTED;
    const float sl2 = scale * 1.4426950408889634f;
    cudaStream_t st = (cudaStream_t)stream;
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
    lse_merge_kernel<<<rows, 64, 0, (cudaStream_t)stream>>>(ml, acc, n_parts, rows, d, (__nv_bfloat16 *)out,
                                                             (const __nv_bfloat16 *)gate, gate_row_stride, gate_head_stride, hq);
    TRB_CUDA_CHECK(cudaGetLastError());
    return TRB_OK;
}
