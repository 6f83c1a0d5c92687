// Library-wide host state: error strings, the device status word, and the cache of TMA
// tensor maps (one per distinct cache view) used by the decode and prefill kernels.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "tmap.h"

static thread_local char g_last_cuda[256] = "";

void trb_set_last_cuda_error(cudaError_t e, const char *file, int line) {
    snprintf(g_last_cuda, sizeof(g_last_cuda), "%s (%s:%d)", cudaGetErrorString(e), file, line);
}

// ------------------------------------------------------------------ programmatic launch plans
static int g_pdl = -1;

namespace trb {

int pdl_mode() {
    if (g_pdl < 0) {
        const char *e = getenv("TRB_PDL");
        g_pdl = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
    }
    return g_pdl;
}

namespace {
struct InFlight {
    const void *cache_k;          // cache whose rows this launch writes (nullptr: none)
    const void *cur_dev;          // ... at this cursor
    long long cur_host;
    WrittenRange w[3];            // other memory it writes (q_out of attn_prep, outputs of a decode)
    const void *ws;               // decode workspace it uses (nullptr: none)
    AppendSource src;             // source rows of a plain append (k == nullptr: none)
};
struct StreamTrack {
    std::vector<InFlight> s;      // library launches that may still be running when the next one starts
    unsigned long long capture_id = 0;
    int capture_status = 0;
};
std::mutex g_track_mu;
std::unordered_map<cudaStream_t, StreamTrack> g_track;
constexpr size_t MAX_IN_FLIGHT = 64;

// The list belongs to one stretch of stream order: a stream that enters or leaves graph capture
// (or starts another capture) starts an empty list, because what precedes a captured node at
// replay time is not what preceded the call at capture time.
StreamTrack &track_of(cudaStream_t st) {
    StreamTrack &t = g_track[st];
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    unsigned long long id = 0;
    if (cudaStreamGetCaptureInfo(st, &status, &id) != cudaSuccess) {
        (void)cudaGetLastError();
        status = cudaStreamCaptureStatusNone;
        id = 0;
        t.s.clear();
    }
    if ((int)status != t.capture_status || id != t.capture_id) {
        t.s.clear();
        t.capture_status = (int)status;
        t.capture_id = id;
    }
    return t;
}
bool overlaps(const WrittenRange &a, const WrittenRange &b) {
    if (!a.lo || !b.lo || !a.bytes || !b.bytes) return false;
    const uintptr_t a0 = (uintptr_t)a.lo, b0 = (uintptr_t)b.lo;
    return a0 < b0 + b.bytes && b0 < a0 + a.bytes;
}
}  // namespace

int pdl_plan_writer(cudaStream_t st, const void *cache_k, const trb_cursor_t *pos, WrittenRange extra, const AppendSource *src) {
    const int mode = pdl_mode();
    if (mode == 0) return PDL_WAIT_FIRST;
    std::lock_guard<std::mutex> lock(g_track_mu);
    StreamTrack &t = track_of(st);
    InFlight me = {cache_k, pos ? pos->dev : nullptr, pos ? pos->host : 0, {extra, {nullptr, 0}, {nullptr, 0}}, nullptr,
                   src ? *src : AppendSource{nullptr, nullptr, 0, 0, 0}};
    // Triggering before the wait is harmless for this kernel (it reads its inputs after its wait);
    // whoever starts because of it decides from the list what it may touch.  The first launch
    // of a chain waits first, so that everything before the chain is complete for all of it.
    const bool chained = mode == 2 && !t.s.empty() && t.s.size() < MAX_IN_FLIGHT;
    if (!chained) t.s.clear();
    t.s.push_back(me);
    return chained ? PDL_TRIGGER_TOP : PDL_WAIT_FIRST;
}

int pdl_plan_decode(cudaStream_t st, const void *cache_k, const trb_cursor_t *pos, int new_rows, int m, WrittenRange q,
                    const WrittenRange (&out)[3], const void *workspace, AppendSource *fresh) {
    const int mode = pdl_mode();
    *fresh = AppendSource{nullptr, nullptr, 0, 0, 0};
    if (mode == 0) return 0;
    std::lock_guard<std::mutex> lock(g_track_mu);
    StreamTrack &t = track_of(st);
    int flags = 0;
    // With an empty list nothing is known about what precedes this launch: it waits at its top
    // and becomes the point before which everything is complete.
    if (!t.s.empty() && t.s.size() < MAX_IN_FLIGHT) {
        int writers = 0;
        bool same_rows = true, q_clean = true, ws_free = true;
        const InFlight *writer = nullptr;
        for (const InFlight &e : t.s) {
            if (e.cache_k && e.cache_k == cache_k) writer = &e;
            if (e.ws && e.ws == workspace) ws_free = false;
            for (const WrittenRange &w : e.w)                  // an output of this launch that an earlier one still writes
                for (const WrittenRange &o : out)
                    if (overlaps(w, o)) ws_free = false;
            if (e.cache_k && e.cache_k == cache_k) {
                ++writers;
                // the rows in flight must be the ones this decode expects at its cursor
                if (!new_rows || e.cur_dev != pos->dev || e.cur_host != pos->host) same_rows = false;
            }
            for (const WrittenRange &w : e.w)
                if (overlaps(w, q)) q_clean = false;
        }
        if (writers == 0 || same_rows) {
            flags |= PDL_PRE_CURSOR;
            if (writers == 0) flags |= PDL_ALL_STABLE;
            if (q_clean) flags |= PDL_PRE_Q;
            if (mode == 2) flags |= PDL_TRIGGER_TOP;
            static const bool run_ahead = !(getenv("TRB_RUNAHEAD") && getenv("TRB_RUNAHEAD")[0] == '0');   // (for measurements)
            if (mode == 2 && ws_free && run_ahead) flags |= PDL_PRIVATE_WS;
            // In a chain, the m rows of the one append in flight need not be awaited in the cache: the
            // decode quantises them from the append's own source rows (same arithmetic, same values)
            // and merges them as one more partial, while the scan covers the rows below the cursor.
            if (mode == 2 && writers == 1 && writer->src.k && writer->src.n_rows == m) {
                bool src_clean = true;                           // nobody in flight writes the source rows
                const WrittenRange sk = {writer->src.k, (size_t)1}, sv = {writer->src.v, (size_t)1};
                for (const InFlight &e : t.s)
                    for (const WrittenRange &w : e.w)
                        if (overlaps(w, sk) || overlaps(w, sv)) src_clean = false;
                if (src_clean) *fresh = writer->src;             // (a caller that takes them may treat every scanned row as complete)
            }
        }
    }
    InFlight me = {nullptr, nullptr, 0, {out[0], out[1], out[2]}, workspace, AppendSource{nullptr, nullptr, 0, 0, 0}};
    if (!(flags & PDL_TRIGGER_TOP)) t.s.clear();      // it triggers after its wait: only it is in flight afterwards
    t.s.push_back(me);
    return flags;
}

static std::atomic<unsigned long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// A kernel launched without the programmatic attribute: everything before it on the stream is
// complete when it runs (every such launch site calls this right before its one launch).
void pdl_note_fence(cudaStream_t st) {
    note_launch();
    std::lock_guard<std::mutex> lock(g_track_mu);
    auto it = g_track.find(st);
    if (it != g_track.end()) it->second.s.clear();
}

}  // namespace trb

extern "C" unsigned long long trb_launch_count(void) { return trb::g_launches.load(std::memory_order_relaxed); }

extern "C" int trb_set_programmatic_launch(int mode) {
    if (mode < 0 || mode > 2) return TRB_E_ARG;
    std::lock_guard<std::mutex> lock(trb::g_track_mu);
    g_pdl = mode;
    trb::g_track.clear();
    return TRB_OK;
}

extern "C" int trb_set_wait_limits(uint32_t pipeline_polls, uint32_t tail_polls, uint32_t peer_polls) {
    const unsigned int v[3] = {pipeline_polls ? pipeline_polls : 1u << 20, tail_polls ? tail_polls : 1u << 17,
                               peer_polls ? peer_polls : 1u << 22};
    TRB_CUDA_CHECK(cudaDeviceSynchronize());
    TRB_CUDA_CHECK(cudaMemcpyToSymbol(trb::c_wait_limit, v, sizeof(v)));
    return TRB_OK;
}

extern "C" int trb_version(void) { return 100; }

extern "C" const char *trb_strerror(int code) {
    switch (code) {
        case TRB_OK: return "ok";
        case TRB_E_ARG: return "bad argument (shape, null pointer or inconsistent sizes)";
        case TRB_E_ALIGN: return "pointer or stride misses its alignment";
        case TRB_E_CAPACITY: return "rows do not fit the cache, or the workspace is too small";
        case TRB_E_CUDA: return g_last_cuda[0] ? g_last_cuda : "CUDA call failed";
        case TRB_E_UNSUPPORTED: return "geometry outside what the kernels are built for";
        case TRB_E_DEVICE: return "device status word is non-zero";
        case TRB_E_SCRATCH_LIMIT:
            return "trb_attn_decode_static: this geometry needs more split scratch than the built-in "
                   "TRB_STATIC_SCRATCH_BYTES (8 MiB); call trb_attn_decode with a caller-provided workspace";
        default: return "unknown error";
    }
}

extern "C" int trb_device_status(uint32_t *status_out) {
    if (!status_out) return TRB_E_ARG;
    unsigned int v = 0, zero = 0;
    TRB_CUDA_CHECK(cudaDeviceSynchronize());
    TRB_CUDA_CHECK(cudaMemcpyFromSymbol(&v, trb::g_status, sizeof(v)));
    if (v) TRB_CUDA_CHECK(cudaMemcpyToSymbol(trb::g_status, &zero, sizeof(zero)));
    *status_out = v;
    return TRB_OK;
}

// ------------------------------------------------------------------ tensor-map cache
namespace trb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

struct Key {
    const void *base;
    long long max_len;
    int hkv, row_bytes, box_rows;
    bool operator==(const Key &o) const {
        return base == o.base && max_len == o.max_len && hkv == o.hkv && row_bytes == o.row_bytes && box_rows == o.box_rows;
    }
};
struct KeyHash {
    size_t operator()(const Key &k) const {
        size_t h = reinterpret_cast<size_t>(k.base);
        h ^= (size_t)k.max_len * 0x9E3779B97F4A7C15ull;
        h ^= ((size_t)k.hkv << 40) ^ ((size_t)k.row_bytes << 20) ^ (size_t)k.box_rows;
        return h;
    }
};

static std::mutex g_mu;
static std::unordered_map<Key, CUtensorMap, KeyHash> g_maps;

// A [hkv, max_len, row_bytes] byte tensor seen as 4-D {128 B, row_bytes/128, max_len, hkv}
// with a {128, 1, box_rows, 1} box (one 128-byte column of box_rows rows) and the 128-byte
// swizzle.  Rows past max_len read as zero.
int get_row_tile_map(const void *base, long long max_len, int hkv, int row_bytes, int box_rows, CUtensorMap *out) {
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return TRB_E_ALIGN;
    if (row_bytes % 128 != 0 || box_rows < 1 || box_rows > 256) return TRB_E_UNSUPPORTED;
    Key key{base, max_len, hkv, row_bytes, box_rows};
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
        *out = it->second;
        return TRB_OK;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return TRB_E_CUDA;
    const cuuint32_t segs = row_bytes / 128;
    cuuint64_t dims[4] = {128, segs, (cuuint64_t)max_len, (cuuint64_t)hkv};
    cuuint64_t strides[3] = {128, (cuuint64_t)row_bytes, (cuuint64_t)row_bytes * (cuuint64_t)max_len};
    cuuint32_t box[4] = {128, 1, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_last_cuda, sizeof(g_last_cuda), "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
        return TRB_E_CUDA;
    }
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, m);
    *out = m;
    return TRB_OK;
}

}  // namespace trb
