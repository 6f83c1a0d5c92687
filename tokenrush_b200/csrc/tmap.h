// Host-side cache of TMA tensor maps for [hkv, max_len, row_bytes] cache views.
#pragma once
#include <cuda.h>

namespace trb {
int get_row_tile_map(const void *base, long long max_len, int hkv, int row_bytes, int box_rows, CUtensorMap *out);
}
