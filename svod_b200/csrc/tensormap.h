// Host-side construction of TMA tensor maps. The driver entry point is resolved
// at run time through the CUDA runtime, so the library links no libcuda stub.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace svodb {

// A tiled map over a dense tensor of 16-bit (or 32-bit) elements with the
// 128-byte shared-memory swizzle. `dims` are innermost first; `strides` are the
// element strides of dims 1..rank-1 (dim 0 is contiguous); out-of-bounds
// elements read as zero. Returns false (with `svodb_last_error` set by the
// caller) when the driver rejects the map: bases must be 16-byte aligned and
// byte strides multiples of 16.
bool make_tmap(CUtensorMap* map, const void* base, int dtype, int rank, const uint64_t* dims,
               const uint64_t* strides_elems, const uint32_t* box);

// [rows, inner] row-major with `row_stride` elements between rows; box = box_rows x box_inner.
bool make_tmap_2d(CUtensorMap* map, const void* base, int dtype, uint64_t inner, uint64_t rows, uint64_t row_stride,
                  uint32_t box_inner, uint32_t box_rows);

}  // namespace svodb
