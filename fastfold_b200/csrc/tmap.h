// Host-side construction of TMA tensor maps (bf16, rank 3) through the driver entry point.
#pragma once
#include <cuda.h>

namespace ffb {

// bf16 tensor [d2][d1][d0] (d0 contiguous) with element strides s1 (dim 1) and s2 (dim 2); box b0 x b1 x 1;
// swizzle_bytes in {0, 32, 64, 128}.  Returns 0 or the CUresult of the failing driver call (-1: no driver entry).
int encode_tmap3_bf16(CUtensorMap* map, const void* ptr, long long d0, long long d1, long long d2, long long s1, long long s2,
                      int b0, int b1, int swizzle_bytes);

}  // namespace ffb
