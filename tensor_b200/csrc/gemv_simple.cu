// SIMT fallback GEMV/GEMM: out[m, n] = x[m, k] . dequant(w[n, k])^T, one warp per weight row,
// fp32 decode and fp32 FMA.  It accepts every shape the formats allow and is the kernel the
// library falls back to when the pipelined kernels' layout requirements do not hold (row stride
// not a multiple of 16 bytes, K not a multiple of 256, m > 16 for the GEMV).  Contract:
// benchmarks/kernels/showcase/triton_kernels.py:213-222 (fp32 weight x fp32 activation); with
// weights_bf16 the decoded weight is rounded to bf16 first (the GEMM contract, :201-207).
#include "common.cuh"
#include "kernels.h"

namespace tb200 {

template <int FMT, typename XT, int NB>
__global__ void __launch_bounds__(256) gemv_simple_kernel(const XT* __restrict__ x,
                                                          const uint8_t* __restrict__ w,
                                                          const OutSpec out, int m,
                                                          long long n, int k, int weights_bf16) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int b0 = blockIdx.y * NB;
  if (row >= n) return;
  const uint8_t* wrow = w + row * row_bytes(FMT, k);
  float acc[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) acc[b] = 0.f;
  const int groups = k >> 5;
  for (int g = lane; g < groups; g += 32) {
#pragma unroll 4
    for (int i = 0; i < 32; ++i) {
      int c = (g << 5) + i;
      float wv = decode_one<FMT>(wrow, c);
      if (weights_bf16) wv = __bfloat162float(__float2bfloat16_rn(wv));
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        int bb = b0 + b < m ? b0 + b : m - 1;
        acc[b] = fmaf(to_f32<XT>(x[(long long)bb * k + c]), wv, acc[b]);
      }
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    float v = acc[b];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0 && b0 + b < m)
      for (int d = 0; d < out.count; ++d) out.ptr[d][(long long)(b0 + b) * out.ld + row] = v;
  }
}

template <int FMT, typename XT>
static cudaError_t launch_typed(const void* x, const uint8_t* w, const OutSpec& out, long long m,
                                long long n, long long k, bool weights_bf16, cudaStream_t stream) {
  const int warps = 8;
  dim3 block(warps * 32);
  const XT* xp = static_cast<const XT*>(x);
  long long gx = (n + warps - 1) / warps;
  if (m == 1) {
    gemv_simple_kernel<FMT, XT, 1><<<dim3((unsigned)gx, 1), block, 0, stream>>>(
        xp, w, out, (int)m, n, (int)k, weights_bf16);
  } else if (m <= 4) {
    gemv_simple_kernel<FMT, XT, 4><<<dim3((unsigned)gx, 1), block, 0, stream>>>(
        xp, w, out, (int)m, n, (int)k, weights_bf16);
  } else {
    long long gy = (m + 7) / 8;
    if (gy > 65535) return cudaErrorInvalidValue;
    gemv_simple_kernel<FMT, XT, 8><<<dim3((unsigned)gx, (unsigned)gy), block, 0, stream>>>(
        xp, w, out, (int)m, n, (int)k, weights_bf16);
  }
  return cudaGetLastError();
}

template <int FMT>
static cudaError_t launch_fmt(int xt, const void* x, const uint8_t* w, const OutSpec& out, long long m,
                              long long n, long long k, bool wb, cudaStream_t s) {
  switch (xt) {
    case kF16: return launch_typed<FMT, __half>(x, w, out, m, n, k, wb, s);
    case kBF16: return launch_typed<FMT, __nv_bfloat16>(x, w, out, m, n, k, wb, s);
    case kF32: return launch_typed<FMT, float>(x, w, out, m, n, k, wb, s);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_gemv_simple(int fmt, int xt, const void* x, const uint8_t* w, const OutSpec& out,
                               long long m, long long n, long long k, bool weights_bf16,
                               cudaStream_t stream) {
  if (m == 0 || n == 0) return cudaSuccess;
  if (k > 0x7fffffffLL || m > 0x7fffffffLL || (n + 7) / 8 > 0x7fffffffLL) return cudaErrorInvalidValue;
  switch (fmt) {
    case kQ4_0: return launch_fmt<kQ4_0>(xt, x, w, out, m, n, k, weights_bf16, stream);
    case kQ8_0: return launch_fmt<kQ8_0>(xt, x, w, out, m, n, k, weights_bf16, stream);
    case kQ4_K: return launch_fmt<kQ4_K>(xt, x, w, out, m, n, k, weights_bf16, stream);
    case kQ6_K: return launch_fmt<kQ6_K>(xt, x, w, out, m, n, k, weights_bf16, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace tb200
