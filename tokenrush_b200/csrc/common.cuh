// Shared device helpers for the sm_100a attention / KV kernels: PTX wrappers for mbarrier,
// TMA (cp.async.bulk.tensor), ldmatrix / movmatrix / mma.sync, e4m3 conversion, and the
// device status word.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/trb_kv.h"

#define TRB_CUDA_CHECK(expr)                                   \
    do {                                                       \
        cudaError_t _e = (expr);                               \
        if (_e != cudaSuccess) { trb_set_last_cuda_error(_e, __FILE__, __LINE__); return TRB_E_CUDA; } \
    } while (0)

void trb_set_last_cuda_error(cudaError_t e, const char *file, int line);

namespace trb {

// Device status word: bits TRB_ST_*.  Sticky until read by trb_device_status().  The library is
// one translation unit, so one copy exists.
static __device__ unsigned int g_status = 0;

__device__ __forceinline__ void raise_status(unsigned int bits) { atomicOr(&g_status, bits); }

// Optional per-CTA timeline of the decode kernels (a diagnostic build: -DTRB_TIMELINE).  Thread 0
// of a CTA stamps %globaltimer at fixed points into shared memory and copies the stamps out when
// the CTA leaves; the host reads them with trb_dbg_timeline().  The normal build compiles none of it.
#ifdef TRB_TIMELINE
constexpr int TL_SLOTS = 16, TL_CTAS = 256, TL_LAUNCHES = 64;
static __device__ unsigned long long g_timeline[TL_LAUNCHES][TL_CTAS][TL_SLOTS];
__device__ __forceinline__ unsigned long long tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define TRB_TL(buf, slot) do { if (threadIdx.x == 0) (buf)[slot] = tl_now(); } while (0)
#define TRB_TL_IF(cond, buf, slot) do { if (cond) (buf)[slot] = tl_now(); } while (0)
#define TRB_TL_SET(buf, slot, v) do { if (threadIdx.x == 0) (buf)[slot] = (unsigned long long)(v); } while (0)
#define TRB_TL_FLUSH(buf, launch, cta)                                                                   \
    do {                                                                                                  \
        if (threadIdx.x == 0) {                                                                           \
            (buf)[12] = tl_now();                                                                         \
            for (int _i = 0; _i < TL_SLOTS; ++_i) g_timeline[(launch) % TL_LAUNCHES][(cta) % TL_CTAS][_i] = (buf)[_i]; \
        }                                                                                                 \
    } while (0)
#else
#define TRB_TL(buf, slot) do { } while (0)
#define TRB_TL_IF(cond, buf, slot) do { } while (0)
#define TRB_TL_SET(buf, slot, v) do { } while (0)
#define TRB_TL_FLUSH(buf, launch, cta) do { } while (0)
#endif

// Cursor value = (dev ? *dev : 0) + host; the integer at dev is 4 or 8 bytes wide.
struct Cursor {
    const void *dev;
    int width;
    long long host;
};

__host__ inline Cursor make_cursor(const trb_cursor_t *c) {
    Cursor r;
    r.dev = c ? c->dev : nullptr;
    r.width = c ? c->width : 8;
    r.host = c ? c->host : 0;
    return r;
}

__device__ __forceinline__ long long load_cursor(const Cursor &c) {
    long long v = c.host;
    if (c.dev) v += (c.width == 4) ? (long long)(*(const volatile int *)c.dev) : *(const volatile long long *)c.dev;
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Poll limits of the bounded waits, per device, set by trb_set_wait_limits():
//   [0] pipeline barriers (mbarrier polls, about a second by default),
//   [1] split partials in the decode tail,  [2] packets of another GPU.
__constant__ unsigned int c_wait_limit[3] = {1u << 20, 1u << 17, 1u << 22};

// Bounded wait: gives up after c_wait_limit[0] polls, records TRB_ST_WAIT_TIMEOUT and returns
// false so that the caller can leave its loop instead of hanging the GPU.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    const uint32_t limit = c_wait_limit[0];
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 64) __nanosleep(64);
    }
    raise_status(TRB_ST_WAIT_TIMEOUT);
    return false;
}

// ------------------------------------------------------------------------------ TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 4-D tiled load, coordinates innermost first; completes on the mbarrier with its byte count.
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *m, uint64_t *bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
// 4-byte cp.async with zero fill when src_bytes == 0, and its arrival on an mbarrier.
__device__ __forceinline__ void cp_async_4(void *dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint64_t *bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Byte offset inside a TMA tile written with CU_TENSOR_MAP_SWIZZLE_128B whose rows are
// `SEGS` 128-byte lines: logical (row, byte) -> physical offset.  The tile base must be
// 1024-byte aligned.
template <int SEGS>
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t byte_in_row) {
    uint32_t line = row * SEGS + (byte_in_row >> 7);
    uint32_t chunk = (byte_in_row >> 4) & 7u;
    return line * 128u + (((chunk ^ (line & 7u)) << 4) | (byte_in_row & 15u));
}

// ----------------------------------------------------------- ldmatrix / movmatrix / mma
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}
// D = A(16x16, row) * B(16x8, col) + C, fp32 accumulate.
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Two e4m3 bytes (a 16-bit value) -> f16x2, exact.
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
    uint32_t d;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(d) : "h"(v));
    return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor in the stream is still running.  It must execute pdl_wait() before it reads
// anything that a launch still in flight may have written; pdl_launch_dependents() lets its own
// successor start.  Both are no-ops for a kernel launched the ordinary way.  Which launches can
// still be in flight when a kernel starts is worked out on the host (PdlPlan below).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}


// ---- host-side plan of a launch under programmatic dependent launch ----------------------------
// A kernel that triggers its dependents before its own wait lets them run beside everything that
// is still in flight before it, so what a kernel may touch before its wait depends on the
// launches that precede it in the stream.  The library keeps, per stream, the list of its own
// launches since the last point at which everything earlier was known to be complete, and
// derives the flags below from it.  Modes (trb_set_programmatic_launch):
//   0  ordinary launches;
//   1  every kernel waits before it triggers, so only the direct predecessor can be in flight;
//   2  "chained": appends and decodes trigger at their top; the caller promises that between
//      two library launches on a stream nothing else writes the caches, cursors or queries.
enum PdlFlags : int {
    PDL_PRE_CURSOR = 1,    // decode: the cursor and the rows below the in-flight append are complete
    PDL_ALL_STABLE = 2,    // decode: no launch in flight writes this cache: every live row is complete
    PDL_PRE_Q = 4,         // decode: the query rows are complete
    PDL_TRIGGER_TOP = 8,   // trigger the dependents before the first wait
    PDL_WAIT_FIRST = 16,   // append / prep: wait, then trigger
    PDL_PRIVATE_WS = 32,   // decode: no launch in flight uses this workspace: partials and ticket need no wait,
                           // and a CTA that merges no output row leaves without waiting
};
struct WrittenRange { const void *lo; size_t bytes; };
// bf16 source rows of an append: element (head j, row i, dim x) at j * head_stride + i * row_stride + x
struct AppendSource { const void *k, *v; long long head_stride, row_stride; int n_rows; };
int pdl_mode();
// a launch that writes rows of `cache_k` at `pos`.. (and `extra`, the q_out of attn_prep); `src`: the
// rows of a plain append (nullptr for attn_prep, whose K rows are not its input rows)
int pdl_plan_writer(cudaStream_t st, const void *cache_k, const trb_cursor_t *pos, WrittenRange extra, const AppendSource *src);
// a decode of `cache_k` at `pos` reading `q`, writing `out[0..2]`
// `fresh` <- the source rows of the one append in flight on this cache, when the decode may take its
// m new rows from there instead of waiting for them in the cache (fresh->k == nullptr otherwise)
int pdl_plan_decode(cudaStream_t st, const void *cache_k, const trb_cursor_t *pos, int new_rows, int m, WrittenRange q,
                    const WrittenRange (&out)[3], const void *workspace, AppendSource *fresh);
// an ordinary launch of the library on `st`: everything before it completes before anything after it starts
void pdl_note_fence(cudaStream_t st);

// Host: launch with (or without) the programmatic-stream-serialization attribute.
inline bool pdl_enabled() { return pdl_mode() != 0; }
void note_launch();                               // counts the kernels this library launches (trb_launch_count)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
    note_launch();
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

}  // namespace trb
