// Host helper: encodes a TMA descriptor for a contiguous (BH, N, D) 16-bit tensor, 128-byte swizzle.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace moddit {

// Box = (64 elements of D) x (box_rows rows of N) x (1 head).  Rows beyond N read as zeros and never
// touch the next head.  Returns MODDIT_OK or a failure code (message set).
int make_tmap_rows(CUtensorMap* map, const void* base, int dtype, int BH, int N, int D, int box_rows);

}  // namespace moddit
