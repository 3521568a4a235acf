// Host-side construction of TMA tensor maps through the driver entry point (no link-time
// dependency on libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace agb {

// Encodes a bf16 tensor of up to 5 dimensions for tiled loads with 128-byte swizzle.
//   dims[0] is the contiguous dimension; strides_bytes[i] is the byte stride of dims[i+1]
//   (multiples of 16); box[0] * 2 bytes must be 128 (one swizzle span).
// Out-of-range parts of a box read as zero.  Returns false when the driver refuses.
bool make_tensor_map_bf16(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box);

}  // namespace agb
