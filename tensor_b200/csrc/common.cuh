// Shared definitions for the GGUF quantised-matmul kernels (sm_100a).
//
// Block layouts follow the reference's statement of them in
// benchmarks/kernels/showcase/triton_kernels.py:133-181 (Q4_0 / Q4_K / Q6_K, GGML type ids
// 2 / 12 / 14); Q8_0 (type id 8) follows the GGML format definition (fp16 d + 32 int8).
// Weights are [N, K] row-major, each row K/block consecutive blocks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb200 {

enum Format : int { kQ4_0 = 2, kQ8_0 = 8, kQ4_K = 12, kQ6_K = 14 };
// Activation dtypes use the runtime ABI's dtype ids (TENSOR_FLOAT16 / FLOAT32 / BFLOAT16).
enum XType : int { kF16 = 10, kF32 = 11, kBF16 = 13 };

template <int FMT> struct Fmt;
template <> struct Fmt<kQ4_0> { static constexpr int kWeights = 32, kBytes = 18; };
template <> struct Fmt<kQ8_0> { static constexpr int kWeights = 32, kBytes = 34; };
template <> struct Fmt<kQ4_K> { static constexpr int kWeights = 256, kBytes = 144; };
template <> struct Fmt<kQ6_K> { static constexpr int kWeights = 256, kBytes = 210; };

__host__ __device__ inline int block_weights(int fmt) { return (fmt == kQ4_0 || fmt == kQ8_0) ? 32 : 256; }
__host__ __device__ inline int block_bytes(int fmt) {
  return fmt == kQ4_0 ? 18 : fmt == kQ8_0 ? 34 : fmt == kQ4_K ? 144 : fmt == kQ6_K ? 210 : 0;
}
__host__ __device__ inline bool valid_format(int fmt) { return block_bytes(fmt) != 0; }
__host__ __device__ inline long long row_bytes(int fmt, long long k) {
  return k / block_weights(fmt) * block_bytes(fmt);
}

// ---- little helpers -------------------------------------------------------------------------

__device__ __forceinline__ float f16_at(const uint8_t* p) {  // 2-byte aligned fp16 field
  return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(p)));
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// ---- exact fp32 decode of one weight, from global or shared bytes -----------------------------
// Every product below is exactly representable in fp32 (fp16 scale 11 bits x small integers);
// Q4_K rounds once, at the subtraction.  The intrinsics forbid contraction so the statement of
// the arithmetic is literal, although a fused multiply-add would round identically here.

// Q4_K: 6-bit scale / min of group g (0..7) from the 12 packed bytes at s.
__device__ __forceinline__ void q4k_scale_min(const uint8_t* s, int g, int& sc, int& mn) {
  int j = g & 3;
  if (g < 4) {
    sc = s[j] & 63;
    mn = s[4 + j] & 63;
  } else {
    sc = (s[8 + j] & 15) | ((s[j] >> 6) << 4);
    mn = (s[8 + j] >> 4) | ((s[4 + j] >> 6) << 4);
  }
}

template <int FMT>
__device__ __forceinline__ float decode_one(const uint8_t* row, int c) {
  if constexpr (FMT == kQ4_0) {
    const uint8_t* b = row + (c >> 5) * 18;
    int byte = b[2 + (c & 15)];
    int nib = (byte >> (((c & 31) >> 4) * 4)) & 15;
    return __fmul_rn((float)(nib - 8), f16_at(b));
  } else if constexpr (FMT == kQ8_0) {
    const uint8_t* b = row + (c >> 5) * 34;
    return __fmul_rn(f16_at(b), (float)(int)(int8_t)b[2 + (c & 31)]);
  } else if constexpr (FMT == kQ4_K) {
    const uint8_t* b = row + (c >> 8) * 144;
    int l = c & 255, g = l >> 5, sc, mn;
    q4k_scale_min(b + 4, g, sc, mn);
    int byte = b[16 + (l >> 6) * 32 + (l & 31)];
    int nib = (byte >> (((l & 63) >> 5) * 4)) & 15;
    float scale = __fmul_rn(f16_at(b), (float)sc);
    float minimum = __fmul_rn(f16_at(b + 2), (float)mn);
    return __fsub_rn(__fmul_rn(scale, (float)nib), minimum);
  } else {
    const uint8_t* b = row + (c >> 8) * 210;
    int l = c & 255, half = l >> 7, lane = l & 31, quarter = (l & 127) >> 5;
    int lo = b[half * 64 + lane + (quarter & 1) * 32];
    int hi = b[128 + half * 32 + lane];
    int q = ((lo >> ((quarter >> 1) * 4)) & 15) | (((hi >> (quarter * 2)) & 3) << 4);
    float sc = (float)(int)(int8_t)b[192 + (l >> 4)];
    return __fmul_rn(__fmul_rn((float)(q - 32), sc), f16_at(b + 208));
  }
}

// ---- error reporting from host code ------------------------------------------------------------

struct Status {
  int code = 0;  // 0 ok, 1 ABI, 2 argument, 3 provider
  char message[480] = {0};
};

}  // namespace tb200
