// Single translation unit of libtrb_kv.so: the kernels share the device status word and a
// few inline helpers, so they are compiled together.
#include <cstring>

#include "runtime.cu"
#include "append.cu"
#include "p2p.cu"
#include "decode.cu"
#include "prefill.cu"
#include "norm.cu"
