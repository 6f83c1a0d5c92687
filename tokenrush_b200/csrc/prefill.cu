// Chunked prefill attention over the FP8 cache (placeholder until the tcgen05 kernel lands).
#include "common.cuh"

extern "C" int trb_attn_prefill(const trb_cache_t *cache, const void *q, void *out, int32_t t, int32_t hq, int64_t pos,
                                float scale, trb_stream_t stream) {
    (void)cache; (void)q; (void)out; (void)t; (void)hq; (void)pos; (void)scale; (void)stream;
    return TRB_E_UNSUPPORTED;
}
