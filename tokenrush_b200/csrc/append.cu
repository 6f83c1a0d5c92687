// KV append-on-write (FP8 e4m3 + per-row scale, or bf16), the decode-side prep
// (q/k RMSNorm + partial rope + append) and the device-side cursor arithmetic
// (speculative commit, advance).
//
// One warp owns one (head, row): 16-byte coalesced loads of the bf16 source row, a
// warp-shuffle amax, IEEE divisions, and one 8-byte store of codes per lane.
#include "common.cuh"

namespace trb {

struct CacheView {
    uint8_t *k, *v;        // codes or bf16
    float *k_scale, *v_scale;
    int hkv, d, fp8, sharded;
    long long max_len, ring, shard_lo;
};

__host__ inline int make_cache_view(const trb_cache_t *c, CacheView *o) {
    if (!c || !c->k || !c->v) return TRB_E_ARG;
    if (c->d != 128 && c->d != 256) return TRB_E_UNSUPPORTED;
    if (c->hkv < 1 || c->max_len < 1) return TRB_E_ARG;
    if (c->kv_dtype != TRB_KV_BF16 && c->kv_dtype != TRB_KV_FP8) return TRB_E_ARG;
    if (c->kv_dtype == TRB_KV_FP8 && (!c->k_scale || !c->v_scale)) return TRB_E_ARG;
    if (c->ring < 0 || c->ring > c->max_len) return TRB_E_ARG;
    if (c->ring > 0 && (c->shard_lo != 0 || c->sharded)) return TRB_E_ARG;
    if (!c->sharded && c->shard_lo != 0) return TRB_E_ARG;
    if (c->hkv > 64) return TRB_E_UNSUPPORTED;
    if (((uintptr_t)c->k | (uintptr_t)c->v) & 15) return TRB_E_ALIGN;
    o->k = (uint8_t *)c->k; o->v = (uint8_t *)c->v;
    o->k_scale = c->k_scale; o->v_scale = c->v_scale;
    o->hkv = c->hkv; o->d = c->d; o->fp8 = c->kv_dtype == TRB_KV_FP8; o->sharded = c->sharded != 0;
    o->max_len = c->max_len; o->ring = c->ring; o->shard_lo = c->shard_lo;
    return TRB_OK;
}

// Row index inside this cache for position p, or -1 when the position is not held here.
__device__ __forceinline__ long long row_of_position(const CacheView &c, long long p) {
    if (p < 0) return -1;
    long long r = c.ring > 0 ? p % c.ring : p - c.shard_lo;
    return (r < 0 || r >= c.max_len) ? -1 : r;
}

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// Quantise one row held as EPT fp32 values per lane and store it: the arithmetic of
// tokenrush/fused.py:336-340 (amax -> clamp -> / 448 -> x / scale -> e4m3 RNE).
template <int EPT>
__device__ __forceinline__ void store_row(const CacheView &c, uint8_t *cache, float *scale, int head, long long row,
                                          const float (&f)[EPT], const __nv_bfloat16 (&raw)[EPT], int lane) {
    const long long off = ((long long)head * c.max_len + row) * c.d + lane * EPT;
    if (c.fp8) {
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < EPT; ++i) amax = fmaxf(amax, fabsf(f[i]));
        amax = warp_max(amax);
        const float sc = __fdiv_rn(fmaxf(amax, 1e-6f), 448.0f);
        uint32_t w[EPT / 4];
#pragma unroll
        for (int i = 0; i < EPT / 4; ++i) {
            uint32_t acc = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const float q = __fdiv_rn(f[i * 4 + b], sc);
                acc |= (uint32_t)__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3) << (8 * b);
            }
            w[i] = acc;
        }
        if (EPT == 8) *reinterpret_cast<uint2 *>(cache + off) = make_uint2(w[0], w[1]);
        else *reinterpret_cast<uint32_t *>(cache + off) = w[0];
        if (lane == 0) scale[(long long)head * c.max_len + row] = sc;
    } else {
        __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(cache) + off;
        if (EPT == 8) *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(raw);
        else *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(raw);
    }
}

template <int EPT>
__device__ __forceinline__ void load_row(const __nv_bfloat16 *src, int lane, float (&f)[EPT], __nv_bfloat16 (&raw)[EPT]) {
    if (EPT == 8) *reinterpret_cast<uint4 *>(raw) = *reinterpret_cast<const uint4 *>(src + lane * EPT);
    else *reinterpret_cast<uint2 *>(raw) = *reinterpret_cast<const uint2 *>(src + lane * EPT);
#pragma unroll
    for (int i = 0; i < EPT; ++i) f[i] = __bfloat162float(raw[i]);
}

// grid (n_rows, hkv, 2 [K|V]), one warp each.
template <int D>
__global__ void __launch_bounds__(32) kv_append_kernel(CacheView c, const __nv_bfloat16 *k_src, const __nv_bfloat16 *v_src,
                                                       long long head_stride, long long row_stride, Cursor pos, Cursor n_valid,
                                                       int has_valid, int trigger_top) {
    constexpr int EPT = D / 32;
    const int i = blockIdx.x, head = blockIdx.y, which = blockIdx.z, lane = threadIdx.x;
    // Inside a chain of library launches the decode that follows may start streaming the rows
    // below the cursor at once; otherwise it starts once everything before this launch is complete.
    if (trigger_top) pdl_launch_dependents();
    pdl_wait();                       // whatever produced the inputs, and every earlier launch, is complete
    if (!trigger_top) pdl_launch_dependents();
    if (has_valid && i >= load_cursor(n_valid)) return;
    const long long p = load_cursor(pos) + i;
    const long long row = row_of_position(c, p);
    if (row < 0) {
        if (!c.sharded && c.ring == 0 && lane == 0) raise_status(TRB_ST_CURSOR_RANGE);
        return;
    }
    const __nv_bfloat16 *src = (which ? v_src : k_src) + head * head_stride + i * row_stride;
    float f[EPT];
    __nv_bfloat16 raw[EPT];
    load_row<EPT>(src, lane, f, raw);
    store_row<EPT>(c, which ? c.v : c.k, which ? c.v_scale : c.k_scale, head, row, f, raw, lane);
}

// Decode-side prep, one warp per (head, row): heads 0..hq-1 are queries, hq..hq+hkv-1 keys
// (+ the value row of the same kv head).  Arithmetic order follows the torch form of the
// reference (tokenrush/ops.py:16-20,46-56): fp32 mean of squares, 1/sqrt, two fp32 products,
// round to bf16; rope products and their sum each rounded to bf16.
template <int D>
__global__ void __launch_bounds__(32) attn_prep_kernel(CacheView c, const __nv_bfloat16 *qkv, const __nv_bfloat16 *qw,
                                                       const __nv_bfloat16 *kw, const __nv_bfloat16 *cos_t,
                                                       const __nv_bfloat16 *sin_t, long long table_rows, int rd, float eps,
                                                       int hq, Cursor pos, __nv_bfloat16 *q_out, int trigger_top) {
    constexpr int EPT = D / 32;
    const int head = blockIdx.x, i = blockIdx.y, lane = threadIdx.x;
    const long long qkv_w = (long long)hq * 2 * D + 2LL * c.hkv * D;
    const bool is_q = head < hq;
    const int j = head - hq;
    const __nv_bfloat16 *src = qkv + i * qkv_w + (is_q ? (long long)head * 2 * D : (long long)hq * 2 * D + (long long)j * D);
    const __nv_bfloat16 *w = is_q ? qw : kw;
    if (trigger_top) pdl_launch_dependents();
    pdl_wait();
    if (!trigger_top) pdl_launch_dependents();
    const long long p = load_cursor(pos) + i;

    float x[EPT];
    __nv_bfloat16 raw[EPT];
    load_row<EPT>(src, lane, x, raw);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < EPT; ++e) ss = __fadd_rn(ss, __fmul_rn(x[e], x[e]));
    ss = warp_sum(ss);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)D), eps)));
    float wf[EPT];
    __nv_bfloat16 wraw[EPT];
    load_row<EPT>(w, lane, wf, wraw);
    __nv_bfloat16 nb[EPT];
#pragma unroll
    for (int e = 0; e < EPT; ++e) nb[e] = __float2bfloat16_rn(__fmul_rn(__fmul_rn(x[e], inv), __fadd_rn(1.0f, wf[e])));

    // rope on dims [0, rd): partner of dim x is x + rd/2 (first half) or x - rd/2 (second half)
    const int half = rd / 2;
    const long long tp = p < 0 ? 0 : (p >= table_rows ? table_rows - 1 : p);
    if (p < 0 || p >= table_rows) { if (lane == 0) raise_status(TRB_ST_CURSOR_RANGE); }
    __nv_bfloat16 ob[EPT];
    // half is a multiple of EPT, so the partner of (lane, e) is (lane +- half / EPT, e)
    const int hl = half / EPT;
    const int plane = (lane < hl ? lane + hl : lane - hl) & 31;
#pragma unroll
    for (int e = 0; e < EPT; ++e) {
        const int dim = lane * EPT + e;
        const float other = __shfl_sync(0xffffffffu, __bfloat162float(nb[e]), plane);
        if (dim < rd) {
            const float cs = __bfloat162float(cos_t[tp * rd + dim]);
            const float sn = __bfloat162float(sin_t[tp * rd + dim]);
            const float a = __bfloat162float(__float2bfloat16_rn(__fmul_rn(__bfloat162float(nb[e]), cs)));
            const float rot = dim < half ? -other : other;
            const float b = __bfloat162float(__float2bfloat16_rn(__fmul_rn(rot, sn)));
            ob[e] = __float2bfloat16_rn(__fadd_rn(a, b));
        } else {
            ob[e] = nb[e];
        }
    }
    if (is_q) {
        __nv_bfloat16 *dst = q_out + ((long long)i * hq + head) * D + lane * EPT;
        if (EPT == 8) *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(ob);
        else *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(ob);
        return;
    }
    const long long row = row_of_position(c, p);
    if (row < 0) {
        if (!c.sharded && c.ring == 0 && lane == 0) raise_status(TRB_ST_CURSOR_RANGE);
        return;
    }
    float kf[EPT];
#pragma unroll
    for (int e = 0; e < EPT; ++e) kf[e] = __bfloat162float(ob[e]);
    store_row<EPT>(c, c.k, c.k_scale, j, row, kf, ob, lane);
    const __nv_bfloat16 *vsrc = qkv + i * qkv_w + (long long)hq * 2 * D + (long long)c.hkv * D + (long long)j * D;
    float vf[EPT];
    __nv_bfloat16 vraw[EPT];
    load_row<EPT>(vsrc, lane, vf, vraw);
    store_row<EPT>(c, c.v, c.v_scale, j, row, vf, vraw, lane);
}

__global__ void spec_commit_kernel(const long long *pred, const long long *drafts, int k, long long *n_accepted,
                                   long long *tok, void *pos, int pos_width) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int n = 0;
    while (n < k && pred[n] == drafts[n]) ++n;
    if (n_accepted) *n_accepted = n;
    if (tok) *tok = pred[n];
    if (pos) {
        if (pos_width == 4) *(int *)pos += n + 1;
        else *(long long *)pos += n + 1;
    }
}

__global__ void cursor_advance_kernel(void *pos, int pos_width, long long delta) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    if (pos_width == 4) *(int *)pos += (int)delta;
    else *(long long *)pos += delta;
}

}  // namespace trb

using namespace trb;

static int check_cursor(const trb_cursor_t *c) {
    if (!c) return TRB_E_ARG;
    if (c->dev && c->width != 4 && c->width != 8) return TRB_E_ARG;
    if (c->dev && ((uintptr_t)c->dev & (c->width - 1))) return TRB_E_ALIGN;
    return TRB_OK;
}

extern "C" int trb_kv_append(const trb_cache_t *cache, const void *k_src, const void *v_src, int64_t src_head_stride,
                             int64_t src_row_stride, int32_t n_rows, const trb_cursor_t *pos, const trb_cursor_t *n_valid,
                             trb_stream_t stream) {
    CacheView c;
    int rc = make_cache_view(cache, &c);
    if (rc) return rc;
    if (n_rows < 0) return TRB_E_ARG;
    if ((rc = check_cursor(pos))) return rc;
    if (n_valid && (rc = check_cursor(n_valid))) return rc;
    if (n_rows == 0) return TRB_OK;
    if (!k_src || !v_src) return TRB_E_ARG;
    if ((((uintptr_t)k_src | (uintptr_t)v_src) & 15) || (src_head_stride % 8) || (src_row_stride % 8)) return TRB_E_ALIGN;
    if (!pos->dev && c.ring == 0) {          // host position: capacity can be checked here
        const long long lo = pos->host - c.shard_lo;
        if (!c.sharded && (lo < 0 || lo + n_rows > c.max_len)) return TRB_E_CAPACITY;
    }
    if (c.ring > 0 && n_rows > c.ring) return TRB_E_CAPACITY;
    dim3 grid(n_rows, c.hkv, 2);
    Cursor pc = make_cursor(pos), nv = make_cursor(n_valid);
    cudaStream_t st = (cudaStream_t)stream;
    const int hv = n_valid != nullptr;
    const AppendSource src = {k_src, v_src, (long long)src_head_stride, (long long)src_row_stride, (int)n_rows};
    const int plan = pdl_plan_writer(st, c.k, pos, WrittenRange{nullptr, 0}, (n_valid || c.ring > 0) ? nullptr : &src);
    TRB_CUDA_CHECK(launch_kernel(c.d == 256 ? kv_append_kernel<256> : kv_append_kernel<128>, grid, dim3(32), 0, st, true, c,
                                 (const __nv_bfloat16 *)k_src, (const __nv_bfloat16 *)v_src, (long long)src_head_stride,
                                 (long long)src_row_stride, pc, nv, hv, (plan & PDL_TRIGGER_TOP) ? 1 : 0));
    return TRB_OK;
}

extern "C" int trb_attn_prep(const trb_cache_t *cache, const void *qkv, const void *q_norm_w, const void *k_norm_w,
                             const void *cos, const void *sin, int64_t table_rows, int32_t rotary_dim, float eps, int32_t m,
                             int32_t hq, const trb_cursor_t *pos, void *q_out, trb_stream_t stream) {
    CacheView c;
    int rc = make_cache_view(cache, &c);
    if (rc) return rc;
    if (!qkv || !q_norm_w || !k_norm_w || !cos || !sin || !q_out || m < 1 || hq < 1 || table_rows < 1) return TRB_E_ARG;
    if (rotary_dim < 0 || rotary_dim > c.d || rotary_dim % (2 * (c.d / 32)) != 0) return TRB_E_UNSUPPORTED;
    if ((rc = check_cursor(pos))) return rc;
    if (((uintptr_t)qkv | (uintptr_t)q_norm_w | (uintptr_t)k_norm_w | (uintptr_t)q_out) & 15) return TRB_E_ALIGN;
    if (!pos->dev && c.ring == 0 && !c.sharded && (pos->host < 0 || pos->host + m > c.max_len)) return TRB_E_CAPACITY;
    dim3 grid(hq + c.hkv, m);
    Cursor pc = make_cursor(pos);
    cudaStream_t st = (cudaStream_t)stream;
    const int plan = pdl_plan_writer(st, c.k, pos, WrittenRange{q_out, (size_t)m * hq * c.d * sizeof(__nv_bfloat16)}, nullptr);
    TRB_CUDA_CHECK(launch_kernel(c.d == 256 ? attn_prep_kernel<256> : attn_prep_kernel<128>, grid, dim3(32), 0, st, true, c,
                                 (const __nv_bfloat16 *)qkv, (const __nv_bfloat16 *)q_norm_w, (const __nv_bfloat16 *)k_norm_w,
                                 (const __nv_bfloat16 *)cos, (const __nv_bfloat16 *)sin, (long long)table_rows, (int)rotary_dim, eps,
                                 (int)hq, pc, (__nv_bfloat16 *)q_out, (plan & PDL_TRIGGER_TOP) ? 1 : 0));
    return TRB_OK;
}

extern "C" int trb_spec_commit(const int64_t *pred, const int64_t *drafts, int32_t k, int64_t *n_accepted, int64_t *tok,
                               void *pos, int32_t pos_width, trb_stream_t stream) {
    if (!pred || !drafts || k < 0 || k > 64) return TRB_E_ARG;
    if (pos && pos_width != 4 && pos_width != 8) return TRB_E_ARG;
    pdl_note_fence((cudaStream_t)stream);
    spec_commit_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((const long long *)pred, (const long long *)drafts, k,
                                                           (long long *)n_accepted, (long long *)tok, pos, pos_width);
    TRB_CUDA_CHECK(cudaGetLastError());
    return TRB_OK;
}

extern "C" int trb_cursor_advance(void *pos, int32_t pos_width, int64_t delta, trb_stream_t stream) {
    if (!pos || (pos_width != 4 && pos_width != 8)) return TRB_E_ARG;
    pdl_note_fence((cudaStream_t)stream);
    cursor_advance_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(pos, pos_width, delta);
    TRB_CUDA_CHECK(cudaGetLastError());
    return TRB_OK;
}
