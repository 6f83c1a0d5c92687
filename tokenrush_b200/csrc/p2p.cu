// Sequence-sharded decode over several GPUs of one box: every GPU scans its own shard of the
// KV cache and ends with one partial (max, sum, unnormalised acc) per (query row, head).
// The partials are exchanged by plain peer stores over NVLink into exchange buffers that
// were shared with cudaIpc handles at set-up, and merged on every GPU in rank order with
// the same log-sum-exp formula that merges the splits of one GPU.
//
// Two forms.  Fused into the decode kernel's tail (the default): every 8 bytes sent are a
// (value, tag) pair, the receiver polls the data itself.  As a separate kernel
// (p2p_merge_kernel below), one CTA per row: push the row to every peer, publish a per-row flag
// (release, system scope), wait for every peer's flag of the same call with an iteration limit, merge.
// Flags carry the call's sequence number, so nothing is ever reset; buffers are used
// round-robin over P2P_SLOTS calls, which is safe because a GPU can be at most one call
// ahead of the slowest peer (it cannot pass its own wait).
#include "common.cuh"

namespace trb {

constexpr int P2P_SLOTS = 4;
constexpr int P2P_MAX_WORLD = 8;
constexpr unsigned int P2P_SPIN_LIMIT = 1u << 22;     // about a second with the back-off below

struct P2PLayout {
    size_t flags, data, ll, total;
    int row_floats;
};
__host__ __device__ inline P2PLayout p2p_layout(int world, int rows, int d) {
    P2PLayout l;
    l.row_floats = d + 4;                                    // acc[d], max, sum, 2 pad floats (16-byte rows)
    l.flags = 256;                                           // header: ticket counter
    l.data = l.flags + (((size_t)P2P_SLOTS * world * rows * sizeof(unsigned int) + 255) / 256) * 256;
    // region of the exchange fused into the decode kernel's tail: per (slot, source rank, row) d / 4
    // threads x 3 packets of 16 bytes, each 8 bytes a (value, tag) pair
    l.ll = ((l.data + (size_t)P2P_SLOTS * world * rows * l.row_floats * sizeof(float) + 255) / 256) * 256;
    l.total = l.ll + (size_t)P2P_SLOTS * world * rows * (d / 4) * 3 * 16;
    return l;
}

struct P2PParams {
    void *const *xchg;
    int world, rank, rows, d, hq;
    unsigned int *seq;
    const float *ml, *acc;
    __nv_bfloat16 *out;
    const __nv_bfloat16 *gate;
    long long gate_rs, gate_hs;
};

__device__ __forceinline__ void st_volatile_v4(uint4 *p, const uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4 *p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// blockDim.x * 4 == d
__global__ void p2p_merge_kernel(const P2PParams p) {
    const int row = blockIdx.x, tid = threadIdx.x;
    const P2PLayout l = p2p_layout(p.world, p.rows, p.d);
    const unsigned int seq = *(volatile unsigned int *)p.seq + 1u;
    const int slot = (int)(seq % P2P_SLOTS);
    __shared__ float sm_ml[P2P_MAX_WORLD][2];
    __shared__ int sm_ok;
    if (tid == 0) sm_ok = 1;

    // 1. push this GPU's row into every GPU's buffer (its own included)
    const float4 mine = *reinterpret_cast<const float4 *>(&p.acc[(long long)row * p.d + tid * 4]);
    const float2 mlv = *reinterpret_cast<const float2 *>(&p.ml[(long long)row * 2]);
    for (int r = 0; r < p.world; ++r) {
        uint8_t *base = (uint8_t *)p.xchg[r];
        float *dst = (float *)(base + l.data) + (((size_t)slot * p.world + p.rank) * p.rows + row) * l.row_floats;
        *reinterpret_cast<float4 *>(dst + tid * 4) = mine;
        if (tid == 0) *reinterpret_cast<float2 *>(dst + p.d) = mlv;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.world) {
        uint8_t *base = (uint8_t *)p.xchg[tid];
        unsigned int *flag = (unsigned int *)(base + l.flags) + ((size_t)slot * p.world + p.rank) * p.rows + row;
        st_release_sys(flag, seq);
    }
    // 2. wait (bounded) for every GPU's row of this call
    uint8_t *local = (uint8_t *)p.xchg[p.rank];
    if (tid < p.world) {
        const unsigned int *flag = (const unsigned int *)(local + l.flags) + ((size_t)slot * p.world + tid) * p.rows + row;
        bool ok = false;
        for (unsigned int it = 0; it < P2P_SPIN_LIMIT; ++it) {
            if (ld_acquire_sys(flag) == seq) { ok = true; break; }
            if (it > 32) __nanosleep(200);
        }
        if (!ok) { raise_status(TRB_ST_PEER_TIMEOUT); sm_ok = 0; }
    }
    __syncthreads();
    // 3. merge in rank order
    if (sm_ok) {
        const float *data = (const float *)(local + l.data);
        if (tid < p.world) {
            const float *src = data + (((size_t)slot * p.world + tid) * p.rows + row) * l.row_floats + p.d;
            sm_ml[tid][0] = __ldcg(src);
            sm_ml[tid][1] = __ldcg(src + 1);
        }
        __syncthreads();
        float mmax = -INFINITY;
        for (int r = 0; r < p.world; ++r) mmax = fmaxf(mmax, sm_ml[r][0]);
        float lsum = 0.f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < p.world; ++r) {
            const float w = sm_ml[r][0] == -INFINITY ? 0.f : fast_exp2(sm_ml[r][0] - mmax);
            lsum = fmaf(w, sm_ml[r][1], lsum);
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(data + (((size_t)slot * p.world + r) * p.rows + row) * l.row_floats + tid * 4));
            o.x = fmaf(w, v.x, o.x); o.y = fmaf(w, v.y, o.y); o.z = fmaf(w, v.z, o.z); o.w = fmaf(w, v.w, o.w);
        }
        const float inv = 1.f / lsum;
        float rr[4] = {o.x * inv, o.y * inv, o.z * inv, o.w * inv};
        __nv_bfloat16 ob[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) ob[e] = __float2bfloat16_rn(rr[e]);
        if (p.gate) {
            const int qi = row / p.hq, h = row % p.hq;
            const __nv_bfloat16 *gp = p.gate + (long long)qi * p.gate_rs + (long long)h * p.gate_hs + tid * 4;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float sg = __bfloat162float(__float2bfloat16_rn(1.f / (1.f + __expf(-__bfloat162float(gp[e])))));
                ob[e] = __float2bfloat16_rn(__bfloat162float(ob[e]) * sg);
            }
        }
        *reinterpret_cast<uint2 *>(&p.out[(long long)row * p.d + tid * 4]) = *reinterpret_cast<const uint2 *>(ob);
    }
    // 4. the last CTA of the launch advances the call counter
    __syncthreads();
    if (tid == 0) {
        unsigned int *ticket = (unsigned int *)local;
        __threadfence();
        if (atomicAdd(ticket, 1u) == (unsigned int)(gridDim.x - 1)) {
            *ticket = 0u;
            *(volatile unsigned int *)p.seq = seq;
        }
    }
}

}  // namespace trb

using namespace trb;

extern "C" size_t trb_p2p_exchange_bytes(int32_t world, int32_t rows, int32_t d) {
    if (world < 1 || world > P2P_MAX_WORLD || rows < 1 || d < 4) return 0;
    return p2p_layout(world, rows, d).total;
}

extern "C" int trb_p2p_create(size_t bytes, void **local_ptr, void *handle_out) {
    if (!bytes || !local_ptr || !handle_out) return TRB_E_ARG;
    static_assert(sizeof(cudaIpcMemHandle_t) == TRB_IPC_HANDLE_BYTES, "handle size");
    void *p = nullptr;
    TRB_CUDA_CHECK(cudaMalloc(&p, bytes));
    TRB_CUDA_CHECK(cudaMemset(p, 0, bytes));
    TRB_CUDA_CHECK(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    TRB_CUDA_CHECK(cudaIpcGetMemHandle(&h, p));
    memcpy(handle_out, &h, sizeof(h));
    *local_ptr = p;
    return TRB_OK;
}

extern "C" int trb_p2p_open(const void *handle, void **peer_ptr) {
    if (!handle || !peer_ptr) return TRB_E_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    TRB_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *peer_ptr = p;
    return TRB_OK;
}

extern "C" int trb_p2p_close(void *peer_ptr) {
    if (!peer_ptr) return TRB_E_ARG;
    TRB_CUDA_CHECK(cudaIpcCloseMemHandle(peer_ptr));
    return TRB_OK;
}

extern "C" int trb_p2p_destroy(void *local_ptr) {
    if (!local_ptr) return TRB_E_ARG;
    TRB_CUDA_CHECK(cudaDeviceSynchronize());
    TRB_CUDA_CHECK(cudaFree(local_ptr));
    return TRB_OK;
}

extern "C" int trb_p2p_merge(const trb_p2p_merge_args_t *a, trb_stream_t stream) {
    if (!a || !a->xchg || !a->seq || !a->partial_ml || !a->partial_acc || !a->out) return TRB_E_ARG;
    if (a->world < 1 || a->world > P2P_MAX_WORLD || a->rank < 0 || a->rank >= a->world) return TRB_E_ARG;
    if (a->rows < 1 || (a->d != 128 && a->d != 256) || a->hq < 1) return TRB_E_ARG;
    if (((uintptr_t)a->partial_acc & 15) || ((uintptr_t)a->partial_ml & 7) || ((uintptr_t)a->out & 7)) return TRB_E_ALIGN;
    P2PParams p;
    p.xchg = a->xchg; p.world = a->world; p.rank = a->rank; p.rows = a->rows; p.d = a->d; p.hq = a->hq;
    p.seq = a->seq; p.ml = a->partial_ml; p.acc = a->partial_acc;
    p.out = (__nv_bfloat16 *)a->out; p.gate = (const __nv_bfloat16 *)a->gate;
    p.gate_rs = a->gate_row_stride; p.gate_hs = a->gate_head_stride;
    pdl_note_fence((cudaStream_t)stream);
    p2p_merge_kernel<<<a->rows, a->d / 4, 0, (cudaStream_t)stream>>>(p);
    TRB_CUDA_CHECK(cudaGetLastError());
    return TRB_OK;
}
