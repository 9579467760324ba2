// The steps either side of a decode projection, as kernels that chain with the GEMVs through
// programmatic dependent launch: RMS normalisation (fp32 residual stream -> bf16 activations of the next
// projection), SwiGLU (the fp32 [m, 2I] output of a grouped gate + up GEMV -> the bf16 activations of the
// down projection) and the residual add behind a projection.  The reference fuses such steps into its
// generated matmul epilogues (packages/tensor-nn/src/tensor_nn/kernels/linear.py:6-100: gemm_gelu,
// gemm_residual) and states normalisation as its own kernel (tensor_nn/kernels/normalization.py); for
// batch 1..16 they are a few KB of HBM traffic each, so what matters is that they add no launch gap.
#include <cuda_bf16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace tb200 {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// out[r, :] = bf16(x[r, :] * rsqrt(mean(x[r, :]^2) + eps) * weight[:]); one CTA per row.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                                      __nv_bfloat16* __restrict__ out, int k, float eps) {
  __shared__ float s_part[8];
  if (threadIdx.x == 0) ptx::grid_launch_dependents();  // the GEMV behind starts streaming its weights now
  ptx::grid_dependency_wait();                           // x comes from the kernel before
  const float* xr = x + (size_t)blockIdx.x * k;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < k; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + i);
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) total += s_part[i];
  const float scale = rsqrtf(total / (float)k + eps);
  __nv_bfloat16* o = out + (size_t)blockIdx.x * k;
  for (int i = threadIdx.x * 4; i < k; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(xr + i);
    const float4 w = *reinterpret_cast<const float4*>(weight + i);
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x * scale * w.x, v.y * scale * w.y);
    const __nv_bfloat162 b = __floats2bfloat162_rn(v.z * scale * w.z, v.w * scale * w.w);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&a);
    packed.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(o + i) = packed;
  }
}

// out[r, c] = bf16(silu(gate_up[r, c]) * gate_up[r, width + c]) for the [m, 2 * width] output of a grouped
// gate + up launch.
__global__ void __launch_bounds__(256) swiglu_kernel(const float* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                                     int m, int width) {
  if (threadIdx.x == 0) ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();
  const long long quads = (long long)m * width / 4;
  for (long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x; q < quads; q += (long long)gridDim.x * blockDim.x) {
    const long long e = q * 4;
    const int r = (int)(e / width), c = (int)(e - (long long)r * width);
    const float4 g = *reinterpret_cast<const float4*>(gate_up + (size_t)r * 2 * width + c);
    const float4 u = *reinterpret_cast<const float4*>(gate_up + (size_t)r * 2 * width + width + c);
    auto act = [](float a, float b) { return a / (1.f + __expf(-a)) * b; };
    const __nv_bfloat162 a = __floats2bfloat162_rn(act(g.x, u.x), act(g.y, u.y));
    const __nv_bfloat162 b = __floats2bfloat162_rn(act(g.z, u.z), act(g.w, u.w));
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&a);
    packed.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(out + e) = packed;
  }
}

// stream[i] += delta[i]
__global__ void __launch_bounds__(256) residual_add_kernel(float* __restrict__ stream_, const float* __restrict__ delta,
                                                           long long quads) {
  if (threadIdx.x == 0) ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();
  for (long long q = blockIdx.x * (long long)blockDim.x + threadIdx.x; q < quads; q += (long long)gridDim.x * blockDim.x) {
    float4 a = reinterpret_cast<float4*>(stream_)[q];
    const float4 b = reinterpret_cast<const float4*>(delta)[q];
    a.x += b.x;
    a.y += b.y;
    a.z += b.z;
    a.w += b.w;
    reinterpret_cast<float4*>(stream_)[q] = a;
  }
}

template <typename... Args>
cudaError_t launch_chained(void (*kernel)(Args...), unsigned grid, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace

cudaError_t launch_rmsnorm(const float* x, const float* weight, void* out_bf16, long long m, long long k, float eps,
                           cudaStream_t stream) {
  if (m < 1 || k < 4 || k % 4 || k > 0x7fffffffLL || m > 0x7fffffffLL) return cudaErrorInvalidValue;
  return launch_chained(rmsnorm_kernel, (unsigned)m, stream, x, weight, static_cast<__nv_bfloat16*>(out_bf16), (int)k, eps);
}

cudaError_t launch_swiglu(const float* gate_up, void* out_bf16, long long m, long long width, cudaStream_t stream) {
  if (m < 1 || width < 4 || width % 4 || m > 0x7fffffffLL || width > 0x3fffffffLL) return cudaErrorInvalidValue;
  const long long quads = m * width / 4;
  const unsigned grid = (unsigned)(quads / 256 + 1 < 592 ? quads / 256 + 1 : 592);
  return launch_chained(swiglu_kernel, grid, stream, gate_up, static_cast<__nv_bfloat16*>(out_bf16), (int)m, (int)width);
}

cudaError_t launch_residual_add(float* stream_buffer, const float* delta, long long count, cudaStream_t stream) {
  if (count < 4 || count % 4) return cudaErrorInvalidValue;
  const long long quads = count / 4;
  const unsigned grid = (unsigned)(quads / 256 + 1 < 592 ? quads / 256 + 1 : 592);
  return launch_chained(residual_add_kernel, grid, stream, stream_buffer, delta, quads);
}

}  // namespace tb200
