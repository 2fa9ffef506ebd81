// Tensor maps (TMA descriptors) built on the host. The encoder lives in the driver library; it is looked up
// through the runtime so that the shared object does not link against the driver and loads on machines
// without one.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include "common.cuh"

namespace bt {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline int encode_fn(EncodeTiledFn *out) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    BT_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (!p || q != cudaDriverEntryPointSuccess) return fail(BT_DEVICE, "the driver does not provide cuTensorMapEncodeTiled");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  *out = fn;
  return BT_OK;
}

// A tiled tensor map over `rank` dimensions of `dtype` elements. dims[0] is the contiguous dimension; strides[i] is
// the byte stride of dimension i + 1 (a multiple of 16); box[] is the tile a copy moves.
inline int make_tmap(CUtensorMap *map, CUtensorMapDataType dtype, int rank, const void *base, const uint64_t *dims,
                     const uint64_t *strides, const uint32_t *box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn encode;
  if (int s = encode_fn(&encode)) return s;
  cuuint64_t d[5], st[4];
  cuuint32_t b[5], es[5];
  for (int i = 0; i < rank; i++) d[i] = dims[i], b[i] = box[i], es[i] = 1;
  for (int i = 0; i + 1 < rank; i++) st[i] = strides[i];
  CUresult r = encode(map, dtype, (cuuint32_t)rank, const_cast<void *>(base), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(BT_BAD_ARGUMENT, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return BT_OK;
}

}  // namespace bt
