/*
 * trb_kv.h - C ABI of the B200 (sm_100a) attention / KV-cache library.
 *
 * Drop-in boundary for the attention + KV entry points of Token Rush
 * (tokenrush/fused.py, tokenrush/ops.py, tokenrush/state.py, and the commit lines of
 * tokenrush/model.py).  The reference has no FFI on this path: its boundary is a set of
 * Python callables that launch Triton kernels.  Each entry point below names the
 * reference callable (file:line, relative to the reference tree) whose GPU work it does.
 *
 * Conventions
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless it says host;
 *   - no entry point allocates or frees device memory unless its comment says so, and none
 *     synchronises the device (so all of them can be captured into a CUDA graph) unless
 *     its comment says so;
 *   - `stream` is a cudaStream_t passed as void*;
 *   - return value: TRB_OK (0) or a negative TRB_E_* code; nothing was launched when a
 *     call fails with TRB_E_ARG / TRB_E_ALIGN / TRB_E_CAPACITY / TRB_E_UNSUPPORTED;
 *   - problems that only the device can see (a cursor that runs past the cache, a wait
 *     on a peer that ran out) are recorded in a device status word, read with
 *     trb_device_status() outside of any graph.
 */
#ifndef TRB_KV_H
#define TRB_KV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRB_OK              0
#define TRB_E_ARG          (-1)  /* bad shape / null pointer / inconsistent sizes      */
#define TRB_E_ALIGN        (-2)  /* a pointer or stride misses its alignment           */
#define TRB_E_CAPACITY     (-3)  /* rows do not fit the cache / workspace too small    */
#define TRB_E_CUDA         (-4)  /* a CUDA runtime / driver call failed                */
#define TRB_E_UNSUPPORTED  (-5)  /* geometry outside what the kernels are built for    */
#define TRB_E_DEVICE       (-6)  /* the device status word is non-zero                 */

/* bits of the device status word */
#define TRB_ST_CURSOR_RANGE   1u   /* an append / scan saw a position outside the cache   */
#define TRB_ST_WAIT_TIMEOUT   2u   /* a bounded wait (pipeline barrier) gave up            */
#define TRB_ST_PEER_TIMEOUT   4u   /* a bounded wait on another GPU's packets gave up      */
#define TRB_ST_WORKSPACE      8u   /* a decode workspace was not zeroed before its first use,
                                      or two launches that share it overlapped              */

#define TRB_KV_BF16 0
#define TRB_KV_FP8  1              /* e4m3fn codes + one fp32 scale per (head, row)       */

typedef void *trb_stream_t;

/* One layer's KV cache, the per-layer slices of State.k/.v/.k_scale/.v_scale
 * (tokenrush/state.py:19-29): k, v [hkv, max_len, d] contiguous; scales [hkv, max_len]. */
typedef struct trb_cache {
    void   *k, *v;
    float  *k_scale, *v_scale;   /* NULL for a bf16 cache                                   */
    int32_t hkv, d;              /* d in {128, 256}                                         */
    int32_t kv_dtype;            /* TRB_KV_BF16 or TRB_KV_FP8                               */
    int32_t sharded;             /* non-zero: this cache is one shard of a longer sequence;
                                    positions outside it are skipped, not reported          */
    int64_t max_len;             /* rows per head                                           */
    int64_t ring;                /* > 0: row = position mod ring (DFlash draft cache,
                                    tokenrush/dflash.py:139-146); multiple of 32, <= max_len */
    int64_t shard_lo;            /* first position held by this cache when sharded           */
} trb_cache_t;

/* A position / count that may live on the device (State.pos_t, tokenrush/state.py:40-43,
 * is int64[1]; int32 is accepted too).  value = (dev ? *dev : 0) + host. */
typedef struct trb_cursor {
    const void *dev;
    int32_t     width;           /* 4 or 8: bytes of the integer at dev                     */
    int32_t     reserved;
    int64_t     host;
} trb_cursor_t;

int         trb_version(void);
const char *trb_strerror(int code);

/* Programmatic dependent launch.  The append / prep / decode kernels are launched with
 * programmatic stream serialization, so that a kernel may start while the launch before it
 * drains.  What a kernel may touch before its dependency wait (griddepcontrol.wait) depends on
 * which launches can still be running when it starts; the library works that out on the host
 * from its own launches on the stream.  mode:
 *   0  ordinary launches (also: environment variable TRB_PDL=0);
 *   1  (default) every kernel waits before it releases its dependents, so only the launch
 *      directly before a kernel can still be running.  A decode that directly follows the
 *      append / prep of its own rows (same cache, same cursor) reads the cursor and streams the
 *      rows below it while that append runs; every other decode waits first.  Safe with any
 *      other work in the stream;
 *   2  chained: appends release their dependents at once and a decode runs beside the tail of
 *      the decode before it (its cache rows and, unless attn_prep made them, its query rows are
 *      read before its wait; workspace, new rows and outputs after it).  The caller promises
 *      that, between two library launches on one stream, no other work writes the caches, the
 *      cursors or the query rows; the first library launch after any ordinary library launch
 *      (trb_cursor_advance, trb_spec_commit, ...) or at the start of a graph capture waits
 *      first.  Meant for a decode step captured as one graph of library calls.
 * Results are the same in all modes.  Returns TRB_E_ARG for another value. */
int trb_set_programmatic_launch(int mode);

/* Kernels launched by this library in this process so far (every entry point counts its own launches,
 * also while a stream is being captured: a captured launch counts once, not once per replay). */
unsigned long long trb_launch_count(void);

/* Poll limits of the bounded device-side waits on the current device (0 restores a default):
 * pipeline_polls - shared-memory pipeline barriers (default 2^20, about a second);
 * tail_polls     - split partials in the decode tail (default 2^17);
 * peer_polls     - packets of another GPU in the fused exchange (default 2^22).
 * A wait that runs out sets TRB_ST_WAIT_TIMEOUT or TRB_ST_PEER_TIMEOUT, the kernel returns and
 * the call's output is undefined; nothing hangs.  Synchronises the device: set-up time only. */
int trb_set_wait_limits(uint32_t pipeline_polls, uint32_t tail_polls, uint32_t peer_polls);

/* trb_attn_decode has two kernels for FP8 caches of head dim 256 without ring or window: a
 * mma.sync kernel (any M; the bandwidth kernel for M = 1) and a tcgen05 kernel that keeps the
 * tensor work off the issue slots when several query rows share a kv head (speculative verify).
 * The second one runs when (hq / hkv) * m >= min_rows.  min_rows <= 0 restores the default (12,
 * i.e. M >= 2 at 24/4 heads); a value above 48 keeps every call on the first kernel.  Both give
 * results within the same tolerance; the switch exists for testing and measurement. */
int trb_set_decode_tensor_rows(int32_t min_rows);

/* Read and clear the device status word of the current device.  Synchronises the device:
 * call it outside graph capture. */
int trb_device_status(uint32_t *status_out);

/* ------------------------------------------------------------------ FP8 / bf16 append
 * Replaces fused.kv_write_prefill (tokenrush/fused.py:327-340) and the cache-write half of
 * fused.attn_prep (tokenrush/fused.py:288-311).  Rows i = 0..n_rows-1 of k_src / v_src
 * (bf16; element (head j, row i, dim x) at j*src_head_stride + i*src_row_stride + x) are
 * written at positions pos+i.  FP8: scale = max(amax, 1e-6) / 448 and code = e4m3_rne(x / scale)
 * with IEEE fp32 divisions, bit-identical to the reference's torch code on CPU.
 * n_valid (optional): device count; rows i >= *n_valid are not written.
 * Positions that fall outside this cache (shards) are skipped. */
int trb_kv_append(const trb_cache_t *cache, const void *k_src, const void *v_src,
                  int64_t src_head_stride, int64_t src_row_stride, int32_t n_rows,
                  const trb_cursor_t *pos, const trb_cursor_t *n_valid, trb_stream_t stream);

/* ------------------------------------------------------------------ decode-side prep
 * Replaces fused.attn_prep (tokenrush/fused.py:246-324): for the m rows of
 * qkv [m, hq*2*d + 2*hkv*d] bf16 ([q|gate per head][k heads][v heads]) at positions pos+i:
 * q/k RMSNorm with (1+w) gain, rope on the first rotary_dim dims with bf16 rounding of
 * every product, q_out [m, hq*d] bf16, K and V rows appended to the cache.
 * cos, sin [table_rows, rotary_dim] bf16 (tokenrush/ops.py:37-43). */
int trb_attn_prep(const trb_cache_t *cache, const void *qkv, const void *q_norm_w, const void *k_norm_w,
                  const void *cos, const void *sin, int64_t table_rows, int32_t rotary_dim, float eps,
                  int32_t m, int32_t hq, const trb_cursor_t *pos, void *q_out, trb_stream_t stream);

/* ------------------------------------------------------------------ split-K decode
 * Replaces fused.attn_decode_fused (tokenrush/fused.py:346-470: split kernel + reduce
 * kernel) and, with window / ring / extra partials, the cache part of
 * fused.attn_window_block (tokenrush/fused.py:600-622). */
typedef struct trb_decode_args {
    const void *q;               /* [m, hq*d] bf16                                          */
    void       *out;             /* [m, hq*d] bf16                                          */
    const void *gate;            /* optional bf16: gate of (row i, head h, dim x) at
                                    i*gate_row_stride + h*gate_head_stride + x; out is
                                    bf16(o) * bf16(sigmoid(gate)) (tokenrush/fused.py:439-445) */
    int64_t     gate_row_stride, gate_head_stride;
    int32_t     m, hq;           /* (hq / hkv) * m <= 48                                    */
    float       scale;           /* softmax scale, d^-0.5 in the reference                  */
    int32_t     new_rows;        /* 1: the m rows are already appended, live = pos + m, row i
                                    sees keys <= pos+i (tokenrush/fused.py:364-366,382);
                                    0: live = pos, every row sees all live keys             */
    int32_t     window;          /* > 0: row i ignores keys < pos+i-window+1 (:383,402-403) */
    int32_t     n_extra;         /* extra partials merged in the tail (the block keys of
                                    attn_window_block); 0 or 1                              */
    const float *extra_ml;       /* [m*hq, n_extra, 2] (max in log2 units, sum)             */
    const float *extra_acc;      /* [m*hq, n_extra, d]                                      */
    trb_cursor_t pos;
    void       *workspace;       /* trb_decode_workspace_bytes() bytes, zeroed once before
                                    the first use (and again after a call that reported
                                    TRB_ST_WAIT_TIMEOUT / TRB_ST_WORKSPACE); calls that share
                                    it must be ordered on one stream                         */
    size_t      workspace_bytes;
    /* sequence shards over several GPUs: when partial_out is set the tail writes this
     * GPU's merged partial (max, sum, unnormalised acc) instead of out               */
    float      *partial_ml;      /* [m*hq, 2]                                               */
    float      *partial_acc;     /* [m*hq, d]                                               */
    /* ... or, fused: when p2p_xchg is set (and p2p_world > 1) the tail exchanges the partials
     * with the other GPUs itself (tagged peer stores, bounded wait, rank-order merge) and
     * writes the final out on every GPU.  p2p_xchg: HOST array of p2p_world device pointers to the
     * GPUs' exchange buffers (trb_p2p_exchange_bytes(world, m*hq, d) bytes each, from
     * trb_p2p_create / trb_p2p_open).  All GPUs must make the same sequence of decode calls on
     * their workspaces: the launch count of the workspace tags the exchange.               */
    void *const *p2p_xchg;
    int32_t     p2p_world, p2p_rank;
    /* A caller that rotates over several workspaces (so that consecutive calls never share one) says
     * which one this is: workspace number ws_slot of ws_slots, used strictly in turn.  The exchange
     * between GPUs is then tagged with launch count of this workspace * ws_slots + ws_slot, i.e. with
     * the call count of the whole rotation.  0 / 0 (or ws_slots = 1): a single workspace.            */
    int32_t     ws_slot, ws_slots;
} trb_decode_args_t;

/* Precondition on the cache: the kernels load whole tiles (32 or 128 rows), so rows beyond the
 * live length inside the allocation take part in the products with weight zero.  They must
 * hold finite codes: a cache that starts zero-filled and is only written by trb_kv_append /
 * trb_attn_prep (which never produce a NaN code) satisfies this, as the reference's State does
 * (tokenrush/state.py:19-29); a cache made with an uninitialised allocator does not. */
size_t trb_decode_workspace_bytes(int32_t hq, int32_t hkv, int32_t d, int32_t m);
int    trb_attn_decode(const trb_cache_t *cache, const trb_decode_args_t *args, trb_stream_t stream);

/* ------------------------------------------------------------------ decode without a workspace
 * No counterpart in the reference (its wrappers allocate the split partials with torch.empty on
 * every call).
 *
 * For callers that cannot give the library device memory at the point of the call: a host
 * runtime whose device memory belongs to its own arena and has no allocation hook for plugins,
 * or a thin FFI binding that only forwards the buffers it received and has no way to create
 * one more.  Same arguments and result as trb_attn_decode, except that args->workspace /
 * workspace_bytes are ignored: the split partials and ticket words live in a file-scope device
 * array of TRB_STATIC_SCRATCH_BYTES that is part of the library image (every GPU that loads the
 * library holds it until the process exits).  The call itself allocates and frees nothing.
 *
 *   - Limit: the scratch need of the geometry, trb_decode_workspace_bytes(hq, hkv, d, m), must
 *     not exceed TRB_STATIC_SCRATCH_BYTES (8 MiB: up to m = 4 rows for 24 query / 4 KV heads
 *     x 256); larger calls return TRB_E_SCRATCH_LIMIT and launch nothing.
 *   - args->p2p_xchg must be NULL (TRB_E_UNSUPPORTED otherwise): the exchange between GPUs is
 *     tagged with the launch count of the workspace, which all GPUs must agree on, and this
 *     array is shared by every caller in the process.
 *   - The first call on each device looks up the array's device address (with that device
 *     current) and keeps it; make that first call before any stream capture begins.
 *   - All calls share the one array, which keeps the previous call's contents.  Before its
 *     kernel, each call zeroes the arrival counts in the array's header and advances the tag
 *     that marks this call's partials (one tiny launch, stream-ordered); partials are
 *     recognised by that tag, so nothing else needs clearing.  Two calls whose kernels overlap
 *     on the GPU (different streams, or several host threads) race on the array: order them on
 *     one stream. */
#define TRB_STATIC_SCRATCH_BYTES (8u << 20)
#define TRB_E_SCRATCH_LIMIT (-7)
int trb_attn_decode_static(const trb_cache_t *cache, const trb_decode_args_t *args, trb_stream_t stream);

/* Softmax statistics of the b in-step block keys, all visible to all b queries, written as
 * one extra partial for trb_attn_decode.  Replaces _attn_block_kernel
 * (tokenrush/fused.py:575-597).  q [b, hq*d], k_blk / v_blk [hkv, b, d] bf16. */
int trb_attn_block_partial(const void *q, const void *k_blk, const void *v_blk, int32_t b, int32_t hq,
                           int32_t hkv, int32_t d, float scale, float *extra_ml, float *extra_acc,
                           trb_stream_t stream);

/* LSE merge of n_parts partials per row in fixed order (tokenrush/fused.py:423-446; also the
 * merge of per-GPU partials of a sequence-sharded cache).  ml [n_parts, rows, 2],
 * acc [n_parts, rows, d] -> out [rows, d] bf16; optional gate as in trb_decode_args. */
int trb_lse_merge(const float *ml, const float *acc, int32_t n_parts, int32_t rows, int32_t d,
                  void *out, const void *gate, int64_t gate_row_stride, int64_t gate_head_stride,
                  int32_t hq, trb_stream_t stream);

/* ------------------------------------------------------------------ speculative commit
 * Replaces the commit lines of Engine._verify_step (tokenrush/model.py:306-312): n = number of
 * leading drafts equal to the prediction of the row before; n_accepted <- n; tok <- pred[n];
 * pos <- pos + n + 1.  Rejected rows are not erased: they lie beyond the live length and the
 * next append overwrites them (tokenrush/mtp.py:84-85).  pred [k+1], drafts [k] int64;
 * n_accepted, tok int64[1]; pos int32 or int64 (pos_width). */
int trb_spec_commit(const int64_t *pred, const int64_t *drafts, int32_t k, int64_t *n_accepted,
                    int64_t *tok, void *pos, int32_t pos_width, trb_stream_t stream);

/* pos <- pos + delta (State.advance, tokenrush/state.py:60-62), on the device. */
int trb_cursor_advance(void *pos, int32_t pos_width, int64_t delta, trb_stream_t stream);

/* ------------------------------------------------------------------ the step after attention
 * Replaces fused.add_rmsnorm (tokenrush/fused.py:22-60), the consumer of the attention output once
 * it has gone through the output projection (tokenrush/model.py:119-120).  The decode entry
 * points write `out` as [m, hq*d] bf16 with the sigmoid gate applied, which is the row layout the
 * projection's split-K GEMV reads; its result comes back as h:
 *   h_splits  = 0: no h (x_out is not written: the residual is x itself);
 *   h_splits  < 0: h [t_rows, n] bf16;
 *   h_splits  > 0: h [h_splits, t_rows, n] fp32 partial rows, summed in split order and rounded to
 *                  bf16 first (what a plain projection would have produced).
 * x_out = bf16(x + h); y = RMSNorm(x_out) with the (1 + weight) gain, or, plain != 0, Qwen3's
 * weight * bf16(normalised) form (the DFlash draft).  x, weight bf16; n a multiple of 8, <= 8192. */
int trb_add_rmsnorm(const void *x, const void *h, int32_t h_splits, const void *weight, float eps, int32_t plain,
                    int32_t t_rows, int32_t n, void *x_out, void *y, trb_stream_t stream);

/* ------------------------------------------------------------------ chunked prefill
 * Replaces fused.attn_prefill_fused (tokenrush/fused.py:476-533): t queries q [t, hq, d] bf16 at
 * host position pos over cache rows 0..pos+t-1 (the chunk's own rows already appended, e4m3 +
 * scales or bf16 as the cache is), query i sees keys <= pos+i; out [t, hq, d] bf16, ungated.
 * Head dim 256, no ring, no shard (TRB_E_UNSUPPORTED otherwise). */
int trb_attn_prefill(const trb_cache_t *cache, const void *q, void *out, int32_t t, int32_t hq,
                     int64_t pos, float scale, trb_stream_t stream);

/* ------------------------------------------------------------------ sequence shards over NVLink
 * No counterpart in the reference (it is single-GPU); the math is its split merge
 * (tokenrush/fused.py:432-438) applied to one partial per GPU.
 *
 * Exchange buffers are plain cudaMalloc memory shared with cudaIpc handles.  create/open/close
 * allocate, map and free device memory and synchronise: set-up time only. */
#define TRB_IPC_HANDLE_BYTES 64
int trb_p2p_create(size_t bytes, void **local_ptr, void *handle_out /* host, 64 bytes */);
int trb_p2p_open(const void *handle /* host, 64 bytes */, void **peer_ptr);
int trb_p2p_close(void *peer_ptr);
int trb_p2p_destroy(void *local_ptr);
size_t trb_p2p_exchange_bytes(int32_t world, int32_t rows, int32_t d);

/* Push this GPU's partial (partial_ml / partial_acc from trb_attn_decode) into every peer's
 * exchange buffer, wait (bounded) until all peers' partials of the same call arrived here,
 * merge them in rank order and write out [rows, d] bf16.  xchg[r] is rank r's exchange
 * buffer as mapped on this GPU (xchg[rank] is the local one); `seq` is a device counter
 * incremented by every call, identical on all ranks.  A wait that runs out sets
 * TRB_ST_PEER_TIMEOUT and the call's output is undefined; nothing hangs. */
typedef struct trb_p2p_merge_args {
    void *const *xchg;           /* DEVICE array of `world` pointers                        */
    int32_t      world, rank;
    uint32_t    *seq;            /* device counter, zeroed at set-up                        */
    const float *partial_ml;     /* [rows, 2]                                               */
    const float *partial_acc;    /* [rows, d]                                               */
    int32_t      rows, d, hq;
    int32_t      reserved;
    void        *out;
    const void  *gate;
    int64_t      gate_row_stride, gate_head_stride;
} trb_p2p_merge_args_t;
int trb_p2p_merge(const trb_p2p_merge_args_t *args, trb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TRB_KV_H */
