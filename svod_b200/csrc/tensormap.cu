#include "tensormap.h"

#include <cuda_runtime.h>

#include "svodb.h"

namespace svodb {

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

}  // namespace

bool make_tmap(CUtensorMap* map, const void* base, int dtype, int rank, const uint64_t* dims,
               const uint64_t* strides_elems, const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  CUtensorMapDataType dt;
  uint64_t esize;
  switch (dtype) {
    case SVODB_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, esize = 2; break;
    case SVODB_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16, esize = 2; break;
    case SVODB_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32, esize = 4; break;
    default: return false;
  }
  cuuint64_t gdim[5], gstride[4];
  cuuint32_t bdim[5], estride[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estride[i] = 1;
    if (i > 0) gstride[i - 1] = strides_elems[i - 1] * esize;
  }
  CUresult r = fn(map, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, bdim, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool make_tmap_2d(CUtensorMap* map, const void* base, int dtype, uint64_t inner, uint64_t rows, uint64_t row_stride,
                  uint32_t box_inner, uint32_t box_rows) {
  const uint64_t dims[2] = {inner, rows};
  const uint64_t strides[1] = {row_stride};
  const uint32_t box[2] = {box_inner, box_rows};
  return make_tmap(map, base, dtype, 2, dims, strides, box);
}

}  // namespace svodb
