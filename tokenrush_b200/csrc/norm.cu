// Residual add + RMSNorm, the step after the attention output projection
// (tokenrush/fused.py:22-60; callers tokenrush/model.py:119-120).  h may be the fp32 partial
// rows of a split-K projection ([S, T, N]): they are summed in split order and rounded to bf16
// first - the value a plain projection would have produced - then added to the bf16 residual
// stream, which is rounded to bf16 again before the norm.
//
// One CTA per row, 16-byte loads, fp32 statistics: a few tens of KB per call, launch-latency-bound.
#include "common.cuh"

namespace trb {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_EPT = 32;          // elements per thread: rows up to 8192

__global__ void __launch_bounds__(NORM_THREADS) add_rmsnorm_kernel(const __nv_bfloat16 *x, const void *h, int h_splits, int t_rows, int n,
                                                                   const __nv_bfloat16 *w, float eps, int plain, __nv_bfloat16 *xo,
                                                                   __nv_bfloat16 *y) {
    const int row = blockIdx.x, tid = threadIdx.x;
    __shared__ float red[NORM_THREADS / 32];
    float v[NORM_MAX_EPT];
    float ss = 0.f;
    int cnt = 0;
    for (int c = tid * 8; c < n; c += NORM_THREADS * 8, ++cnt) {
        __nv_bfloat16 xb[8];
        *reinterpret_cast<uint4 *>(xb) = *reinterpret_cast<const uint4 *>(x + (long long)row * n + c);
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __bfloat162float(xb[e]);
        if (h_splits != 0) {
            float hs[8];
            if (h_splits < 0) {                                   // h [T, N] bf16
                __nv_bfloat16 hb[8];
                *reinterpret_cast<uint4 *>(hb) = *reinterpret_cast<const uint4 *>((const __nv_bfloat16 *)h + (long long)row * n + c);
#pragma unroll
                for (int e = 0; e < 8; ++e) hs[e] = __bfloat162float(hb[e]);
            } else {                                              // h [S, T, N] fp32 partial rows, summed in split order
#pragma unroll
                for (int e = 0; e < 8; ++e) hs[e] = 0.f;
                for (int s = 0; s < h_splits; ++s) {
                    const float *hp = (const float *)h + ((long long)s * t_rows + row) * n + c;
                    const float4 a = *reinterpret_cast<const float4 *>(hp), b = *reinterpret_cast<const float4 *>(hp + 4);
                    if (s == 0) { hs[0] = a.x; hs[1] = a.y; hs[2] = a.z; hs[3] = a.w; hs[4] = b.x; hs[5] = b.y; hs[6] = b.z; hs[7] = b.w; }
                    else {
                        hs[0] = __fadd_rn(hs[0], a.x); hs[1] = __fadd_rn(hs[1], a.y); hs[2] = __fadd_rn(hs[2], a.z); hs[3] = __fadd_rn(hs[3], a.w);
                        hs[4] = __fadd_rn(hs[4], b.x); hs[5] = __fadd_rn(hs[5], b.y); hs[6] = __fadd_rn(hs[6], b.z); hs[7] = __fadd_rn(hs[7], b.w);
                    }
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) hs[e] = __bfloat162float(__float2bfloat16_rn(hs[e]));
            }
            __nv_bfloat16 ob[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                ob[e] = __float2bfloat16_rn(__fadd_rn(f[e], hs[e]));   // the residual stream is bf16
                f[e] = __bfloat162float(ob[e]);
            }
            *reinterpret_cast<uint4 *>(xo + (long long)row * n + c) = *reinterpret_cast<const uint4 *>(ob);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            v[cnt * 8 + e] = f[e];
            ss = fmaf(f[e], f[e], ss);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) red[tid >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_THREADS / 32; ++i) tot += red[i];
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(tot, (float)n), eps)));
    cnt = 0;
    for (int c = tid * 8; c < n; c += NORM_THREADS * 8, ++cnt) {
        __nv_bfloat16 wb[8], ob[8];
        *reinterpret_cast<uint4 *>(wb) = *reinterpret_cast<const uint4 *>(w + c);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float nrm = __fmul_rn(v[cnt * 8 + e], inv);
            // plain: Qwen3's norm (cast, then weight * x); else the (1 + weight) gain (tokenrush/ops.py:16-20)
            ob[e] = plain ? __float2bfloat16_rn(__fmul_rn(__bfloat162float(wb[e]), __bfloat162float(__float2bfloat16_rn(nrm))))
                          : __float2bfloat16_rn(__fmul_rn(nrm, __fadd_rn(1.0f, __bfloat162float(wb[e]))));
        }
        *reinterpret_cast<uint4 *>(y + (long long)row * n + c) = *reinterpret_cast<const uint4 *>(ob);
    }
}

}  // namespace trb

using namespace trb;

extern "C" int trb_add_rmsnorm(const void *x, const void *h, int32_t h_splits, const void *weight, float eps, int32_t plain,
                               int32_t t_rows, int32_t n, void *x_out, void *y, trb_stream_t stream) {
    if (!x || !weight || !y || t_rows < 1 || n < 8) return TRB_E_ARG;
    if ((n % 8) || n > NORM_THREADS * NORM_MAX_EPT) return TRB_E_UNSUPPORTED;
    if (h_splits != 0 && (!h || !x_out)) return TRB_E_ARG;
    if (((uintptr_t)x | (uintptr_t)h | (uintptr_t)weight | (uintptr_t)x_out | (uintptr_t)y) & 15) return TRB_E_ALIGN;
    pdl_note_fence((cudaStream_t)stream);
    add_rmsnorm_kernel<<<t_rows, NORM_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16 *)x, h, h_splits, t_rows, n,
                                                                          (const __nv_bfloat16 *)weight, eps, plain ? 1 : 0,
                                                                          (__nv_bfloat16 *)x_out, (__nv_bfloat16 *)y);
    TRB_CUDA_CHECK(cudaGetLastError());
    return TRB_OK;
}
