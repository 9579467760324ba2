// Standalone fp32 dequantisation: out[n, k] = dequant(w).  This kernel carries the bit-exact
// gate against the reference's decode (benchmarks/kernels/showcase/triton_kernels.py:133-181).
// It is bound by the fp32 store traffic (4 B per weight out, <= 1.06 B in).
#include "common.cuh"
#include "kernels.h"

namespace tb200 {

template <int FMT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ w,
                                                      float* __restrict__ out, long long n,
                                                      long long k) {
  const long long rb = row_bytes(FMT, k);
  const long long quads_per_row = k >> 2;
  const long long total = n * quads_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r = i / quads_per_row;
    int c = (int)(i - r * quads_per_row) << 2;
    const uint8_t* row = w + r * rb;
    float4 v;
    v.x = decode_one<FMT>(row, c);
    v.y = decode_one<FMT>(row, c + 1);
    v.z = decode_one<FMT>(row, c + 2);
    v.w = decode_one<FMT>(row, c + 3);
    *reinterpret_cast<float4*>(out + r * k + c) = v;
  }
}

cudaError_t launch_dequant(int fmt, const uint8_t* w, float* out, long long n, long long k,
                           cudaStream_t stream) {
  if (n == 0 || k == 0) return cudaSuccess;
  cudaError_t err;
  const DeviceInfo* dev = device_info(&err);
  if (!dev) return err;
  long long total = n * (k >> 2);
  long long want = (total + 255) / 256;
  int grid = (int)(want < (long long)dev->sm_count * 16 ? want : (long long)dev->sm_count * 16);
  switch (fmt) {
    case kQ4_0: dequant_kernel<kQ4_0><<<grid, 256, 0, stream>>>(w, out, n, k); break;
    case kQ8_0: dequant_kernel<kQ8_0><<<grid, 256, 0, stream>>>(w, out, n, k); break;
    case kQ4_K: dequant_kernel<kQ4_K><<<grid, 256, 0, stream>>>(w, out, n, k); break;
    case kQ6_K: dequant_kernel<kQ6_K><<<grid, 256, 0, stream>>>(w, out, n, k); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace tb200
