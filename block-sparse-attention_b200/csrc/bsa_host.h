// Host-side helpers shared by the entry points: thread-local error text, TMA tensor-map encoding
// through the driver entry point (no link-time dependency on libcuda), device queries.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bsa {

// Stores a printf-style message for bsa_last_error() and returns `code`.
int set_error(int code, const char* fmt, ...);

// Encodes a tiled tensor map with 128-byte swizzle and zero fill for out-of-range elements.
//   dims[rank]            extents, innermost first
//   strides_bytes[rank-1] byte strides of dimensions 1..rank-1 (multiples of 16)
//   box[rank]             box extents; box[0] * element size must be 128 bytes
// Returns 0 or a negative bsa_error (message set).
int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    const char* what);

}  // namespace bsa
