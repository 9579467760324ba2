// Host-side calls into the CUDA driver: encoding of 2-D TMA tensor maps and the address range of
// an allocation.  The driver functions are resolved through the CUDA runtime at first use, so the
// library has no link-time dependency on libcuda and still loads on a machine without a driver.
#include <cuda.h>

#include "kernels.h"

namespace tb200 {

namespace {
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}
}  // namespace

bool make_tensor_map_2d(void* map_out, TmaType type, const void* base, unsigned long long inner,
                        unsigned long long outer, unsigned long long row_stride_bytes, unsigned box_inner,
                        unsigned box_outer, bool swizzle_128b) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return false;
  const CUtensorMapDataType dt = type == TmaType::kBF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                        : CU_TENSOR_MAP_DATA_TYPE_UINT64;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode(static_cast<CUtensorMap*>(map_out), dt, 2, const_cast<void*>(base), dims, strides, box,
                            elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle_128b ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

bool allocation_range(const void* ptr, void** base, size_t* size) {
  using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<RangeFn>(p);
  }();
  if (!fn) return false;
  CUdeviceptr b = 0;
  size_t n = 0;
  if (fn(&b, &n, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return false;
  *base = reinterpret_cast<void*>(b);
  *size = n;
  return true;
}

}  // namespace tb200
