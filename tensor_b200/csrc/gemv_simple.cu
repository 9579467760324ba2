// SIMT fallback GEMV/GEMM: out[m, n] = x[m, k] . dequant(w[n, k])^T, one warp per weight row,
// fp32 decode and fp32 FMA.  It accepts every shape the formats allow and is the kernel the
// library falls back to when the pipelined kernels' layout requirements do not hold (row stride
// not a multiple of 16 bytes, K not a multiple of 256, m > 16 for the GEMV).  Contract:
// benchmarks/kernels/showcase/triton_kernels.py:213-222 (fp32 weight x fp32 activation); with
// weights_bf16 the decoded weight is rounded to bf16 first (the GEMM contract, :201-207).
#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace tb200 {

template <int FMT, typename XT, int NB>
__device__ __forceinline__ void gemv_simple_body(const XT* __restrict__ x, const uint8_t* __restrict__ w,
                                                 const OutSpec& out, int m, long long n, int k, int weights_bf16) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int b0 = blockIdx.y * NB;
  if (row >= n) return;
  const uint8_t* wrow = w + row * row_bytes(FMT, k);
  float acc[NB];
#pragma unroll
  for (int b = 0; b < NB; ++b) acc[b] = 0.f;
  // Lane l takes weights l, l + 32, ... of the row: the 32 lanes of a step read neighbouring bytes
  // of one block (coalesced), its scale is a broadcast load, and the activations are contiguous.
  // (One lane per 32-weight block, the obvious alternative, strides the lanes by the block size:
  // every load instruction then touches 32 different sectors.)
#pragma unroll 8
  for (int c = lane; c < k; c += 32) {
    float wv = decode_one<FMT>(wrow, c);
    if (weights_bf16) wv = __bfloat162float(__float2bfloat16_rn(wv));
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      int bb = b0 + b < m ? b0 + b : m - 1;
      acc[b] = fmaf(to_f32<XT>(x[(long long)bb * k + c]), wv, acc[b]);
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

// Static-shape entry used by generated .tbin wrappers: the reference's own kernels for this path take
// fp32 activations and present `kernel(const float* x, const uint8_t* w, float* out)` over flat buffers.
template <int FMT, typename XT, int NB>
__device__ __forceinline__ void gemv_simple_static_entry(const XT* x, const uint8_t* w, float* out, int m, long long n,
                                                         int k) {
  OutSpec spec{};
  spec.ptr[0] = out;
  spec.count = 1;
  spec.ld = n;
  gemv_simple_body<FMT, XT, NB>(x, w, spec, m, n, k, 0);
}

#ifndef TB200_TBIN_WRAPPER
template <int FMT, typename XT, int NB>
__global__ void __launch_bounds__(256) gemv_simple_kernel(const XT* __restrict__ x,
                                                          const uint8_t* __restrict__ w,
                                                          const OutSpec out, int m,
                                                          long long n, int k, int weights_bf16) {
  gemv_simple_body<FMT, XT, NB>(x, w, out, m, n, k, weights_bf16);
}

// The same arithmetic with everything staged in shared memory first: the CTA converts the
// activations to fp32 once, and every warp copies its weight row with coalesced 16-byte loads before
// it decodes it (lane l takes weights l, l + 32, ...: consecutive bytes of a block, no bank
// conflicts, the block scale a broadcast).  Decode GEMVs of the formats the pipelined kernel does not
// cover spend their time here at batches up to 4; it needs rows that are a multiple of 16 bytes and
// activations plus sixteen rows that fit in shared memory.
constexpr int kRowWarps = 8;
template <int FMT, typename XT, int MB>
__global__ void __launch_bounds__(kRowWarps * 32) gemv_rows_kernel(const XT* __restrict__ x,
                                                                  const uint8_t* __restrict__ w, const OutSpec out,
                                                                  int m, long long n, int k, int row_bytes_) {
  extern __shared__ __align__(16) uint8_t smem_rows[];
  float* xs = reinterpret_cast<float*>(smem_rows);                       // [MB][k]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // two row buffers per warp: the next row is copied (cp.async) while this one is decoded
  uint8_t* bufs = smem_rows + (size_t)MB * k * 4 + (size_t)warp * 2 * row_bytes_;
  const int b0 = blockIdx.y * MB;
  // activations -> fp32, 16 bytes per load and several loads in flight per thread (a scalar loop
  // here pays one L2 round trip per element and dominates the kernel)
  constexpr int kPer = 16 / (int)sizeof(XT);
  const int vecs = (MB * k) / kPer;  // K is a multiple of 32
#pragma unroll 4
  for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
    const int i = v * kPer, b = i / k, c = i - b * k;
    XT tmp[kPer];
    if (b0 + b < m) {
      *reinterpret_cast<uint4*>(tmp) = __ldg(reinterpret_cast<const uint4*>(x + (long long)(b0 + b) * k + c));
#pragma unroll
      for (int j = 0; j < kPer; ++j) xs[i + j] = to_f32<XT>(tmp[j]);
    } else {
#pragma unroll
      for (int j = 0; j < kPer; ++j) xs[i + j] = 0.f;
    }
  }
  __syncthreads();
  const int chunks = row_bytes_ >> 4;
  const long long row_step = (long long)gridDim.x * kRowWarps;
  auto copy_row = [&](long long row, uint8_t* dst) {
    if (row < n) {
      const uint8_t* src = w + row * row_bytes_;
      const uint32_t d0 = (uint32_t)__cvta_generic_to_shared(dst);
      for (int i = lane; i < chunks; i += 32)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d0 + 16u * i), "l"(src + 16 * i) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  int cur = 0;
  copy_row((long long)blockIdx.x * kRowWarps + warp, bufs);
  for (long long row = (long long)blockIdx.x * kRowWarps + warp; row < n; row += row_step, cur ^= 1) {
    const uint8_t* mine = bufs + (size_t)cur * row_bytes_;
    copy_row(row + row_step, bufs + (size_t)(cur ^ 1) * row_bytes_);
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the copy just issued has landed
    __syncwarp();
    float acc[MB];
#pragma unroll
    for (int b = 0; b < MB; ++b) acc[b] = 0.f;
    if constexpr (FMT == kQ8_0) {
      // Lane l takes 8 consecutive weights of block l / 4 (+ 8 per step): four 2-byte loads (blocks
      // are 34 bytes, so nothing wider is aligned), one scale conversion per 8 weights, activations
      // as two 16-byte loads.  A byte b becomes the float 2^23 + (b ^ 0x80) = 2^23 + 128 + q with one
      // logic op (after a byte permute for the odd bytes); subtracting 2^23 + 128 gives q exactly.
      const int blocks = k >> 5;
      for (int blk = lane >> 2; blk < blocks; blk += 8) {
        const uint8_t* bp = mine + blk * 34;
        const float d = f16_at(bp);
        const unsigned short* q = reinterpret_cast<const unsigned short*>(bp + 2 + 8 * (lane & 3));
        const int c0 = blk * 32 + 8 * (lane & 3);
        float part[MB];
#pragma unroll
        for (int b = 0; b < MB; ++b) part[b] = 0.f;
        float wq[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t h = q[j];
          const uint32_t lo = (h & 0xFFu) ^ 0x4B000080u;
          const uint32_t hi = __byte_perm(h, 0x4B000000u, 0x7541u) ^ 0x80u;
          wq[2 * j] = __uint_as_float(lo) - 8388736.f;
          wq[2 * j + 1] = __uint_as_float(hi) - 8388736.f;
        }
#pragma unroll
        for (int b = 0; b < MB; ++b) {
          const float4 x0 = *reinterpret_cast<const float4*>(xs + b * k + c0);
          const float4 x1 = *reinterpret_cast<const float4*>(xs + b * k + c0 + 4);
          // the reference contract multiplies d * q first (exact), then by x: keep that rounding
          part[b] = fmaf(__fmul_rn(d, wq[0]), x0.x, part[b]);
          part[b] = fmaf(__fmul_rn(d, wq[1]), x0.y, part[b]);
          part[b] = fmaf(__fmul_rn(d, wq[2]), x0.z, part[b]);
          part[b] = fmaf(__fmul_rn(d, wq[3]), x0.w, part[b]);
          part[b] = fmaf(__fmul_rn(d, wq[4]), x1.x, part[b]);
          part[b] = fmaf(__fmul_rn(d, wq[5]), x1.y, part[b]);
          part[b] = fmaf(__fmul_rn(d, wq[6]), x1.z, part[b]);
          part[b] = fmaf(__fmul_rn(d, wq[7]), x1.w, part[b]);
          acc[b] += part[b];
        }
      }
    } else if constexpr (FMT == kQ6_K) {
      // Lane l takes the 16 weights of scale group l % 16 of super-block l / 16 (+ 2 per step): their
      // low nibbles are 16 consecutive bytes of ql (one nibble of each), their high bit pairs 16
      // consecutive bytes of qh (one bit pair of each), read as eight 2-byte loads each (blocks are
      // 210 bytes, so nothing wider is aligned).  (q - 32) * sc * d is exact in fp32 in any order
      // (6 + 7 + 11 bits), so d * sc is formed once per group.
      const int sbs = k >> 8;
      const int g = lane & 15, half = g >> 3, quarter = (g & 7) >> 1, odd = g & 1;
      const int nsh = (quarter >> 1) * 4, hsh = quarter * 2;
      for (int sb = lane >> 4; sb < sbs; sb += 2) {
        const uint8_t* bp = mine + sb * 210;
        const unsigned short* lo = reinterpret_cast<const unsigned short*>(bp + half * 64 + (quarter & 1) * 32 + odd * 16);
        const unsigned short* hi = reinterpret_cast<const unsigned short*>(bp + 128 + half * 32 + odd * 16);
        const float dsc = __fmul_rn(f16_at(bp + 208), (float)(int)(int8_t)bp[192 + g]);
        float wv[16];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t l16 = lo[j], h16 = hi[j];
          const uint32_t t = ((l16 >> nsh) & 0x0F0Fu) | (((h16 >> hsh) & 0x0303u) << 4);
          wv[2 * j] = __fmul_rn(__uint_as_float((t & 0xFFu) | 0x4B000000u) - 8388640.f, dsc);      // 2^23 + 32
          wv[2 * j + 1] = __fmul_rn(__uint_as_float((t >> 8) | 0x4B000000u) - 8388640.f, dsc);
        }
#pragma unroll
        for (int b = 0; b < MB; ++b) {
          const float4* xp = reinterpret_cast<const float4*>(xs + b * k + sb * 256 + 16 * g);
          float part = 0.f;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 xv = xp[j];
            part = fmaf(wv[4 * j], xv.x, part);
            part = fmaf(wv[4 * j + 1], xv.y, part);
            part = fmaf(wv[4 * j + 2], xv.z, part);
            part = fmaf(wv[4 * j + 3], xv.w, part);
          }
          acc[b] += part;
        }
      }
    } else if constexpr (FMT == kQ4_0) {
      // Lane l takes bytes 4 (l % 4) .. + 3 of block l / 4 (+ 8 per step): their low nibbles are
      // weights 4 (l % 4) .. + 3 of the block, their high nibbles the same positions + 16.
      const int blocks = k >> 5, qtr = lane & 3;
      for (int blk = lane >> 2; blk < blocks; blk += 8) {
        const uint8_t* bp = mine + blk * 18;
        const float d = f16_at(bp);
        const unsigned short* q16 = reinterpret_cast<const unsigned short*>(bp + 2 + 4 * qtr);
        const uint32_t w32 = (uint32_t)q16[0] | ((uint32_t)q16[1] << 16);
        const uint32_t lo = w32 & 0x0F0F0F0Fu, hi = (w32 >> 4) & 0x0F0F0F0Fu;
        float wl[4], wh[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          wl[j] = __fmul_rn(__uint_as_float(((lo >> (8 * j)) & 0xFFu) | 0x4B000000u) - 8388616.f, d);  // 2^23 + 8
          wh[j] = __fmul_rn(__uint_as_float(((hi >> (8 * j)) & 0xFFu) | 0x4B000000u) - 8388616.f, d);
        }
#pragma unroll
        for (int b = 0; b < MB; ++b) {
          const float4 x0 = *reinterpret_cast<const float4*>(xs + b * k + blk * 32 + 4 * qtr);
          const float4 x1 = *reinterpret_cast<const float4*>(xs + b * k + blk * 32 + 16 + 4 * qtr);
          float part = fmaf(wl[0], x0.x, 0.f);
          part = fmaf(wl[1], x0.y, part);
          part = fmaf(wl[2], x0.z, part);
          part = fmaf(wl[3], x0.w, part);
          part = fmaf(wh[0], x1.x, part);
          part = fmaf(wh[1], x1.y, part);
          part = fmaf(wh[2], x1.z, part);
          part = fmaf(wh[3], x1.w, part);
          acc[b] += part;
        }
      }
    } else {
#pragma unroll 4
      for (int c = lane; c < k; c += 32) {
        const float wv = decode_one<FMT>(mine, c);
#pragma unroll
        for (int b = 0; b < MB; ++b) acc[b] = fmaf(xs[b * k + c], wv, acc[b]);
      }
    }
#pragma unroll
    for (int b = 0; b < MB; ++b) {
      float v = acc[b];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0 && b0 + b < m)
        for (int d = 0; d < out.count; ++d) out.ptr[d][(long long)(b0 + b) * out.ld + row] = v;
    }
    __syncwarp();  // this buffer is the target of the copy the next iteration issues
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int FMT, typename XT, int MB>
static cudaError_t launch_rows(const XT* x, const uint8_t* w, const OutSpec& out, long long m, long long n, long long k,
                               int smem, cudaStream_t stream) {
  auto kernel = gemv_rows_kernel<FMT, XT, MB>;
  cudaError_t e = allow_full_shared_memory(kernel);
  if (e != cudaSuccess) return e;
  const DeviceInfo* dev = device_info(&e);
  if (!dev) return e;
  // persistent-ish: a few CTAs per SM, every warp walking its rows with the next one in flight
  const long long row_ctas = (n + kRowWarps - 1) / kRowWarps;
  const int per_sm = dev->max_smem_optin / (smem + 1024) < 1 ? 1 : dev->max_smem_optin / (smem + 1024);  // what shared memory allows
  const long long resident = (long long)dev->sm_count * (per_sm > 4 ? 4 : per_sm);
  const unsigned gx = (unsigned)(row_ctas < resident ? row_ctas : resident);
  const unsigned gy = (unsigned)((m + MB - 1) / MB);
  kernel<<<dim3(gx, gy), kRowWarps * 32, smem, stream>>>(x, w, out, (int)m, n, (int)k, (int)row_bytes(FMT, k));
  return cudaGetLastError();
}

template <int FMT, typename XT>
static cudaError_t launch_typed(const void* x, const uint8_t* w, const OutSpec& out, long long m,
                                long long n, long long k, bool weights_bf16, cudaStream_t stream) {
  const XT* xp = static_cast<const XT*>(x);
  // decode GEMVs (fp32 weights) whose rows and activations fit: the shared-memory staged kernel
  const long long rb = row_bytes(FMT, k);
  // (measured against the kernel below at 4096 x 4096: Q8_0 4x faster at batch 1, 2.5x at batch 2,
  // 1.4x at batch 3-4; from batch 5 on, where the weights are decoded once per four rows, it loses)
  constexpr int rows_max_m = 4;
  if (!weights_bf16 && m <= rows_max_m && m <= 16 && rb % 16 == 0) {
    const int mb = m == 1 ? 1 : (m == 2 ? 2 : 4);
    const long long smem = (long long)mb * k * 4 + 2 * kRowWarps * rb;  // activations + two row buffers per warp
    if (smem <= (m == 1 ? 110 : 200) * 1024) {
      if (mb == 1) return launch_rows<FMT, XT, 1>(xp, w, out, m, n, k, (int)smem, stream);
      if (mb == 2) return launch_rows<FMT, XT, 2>(xp, w, out, m, n, k, (int)smem, stream);
      return launch_rows<FMT, XT, 4>(xp, w, out, m, n, k, (int)smem, stream);
    }
  }
  const int warps = 8;
  dim3 block(warps * 32);
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

#endif  // TB200_TBIN_WRAPPER

}  // namespace tb200
