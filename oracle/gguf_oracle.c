/* CPU restatement of the GGUF dequant / GEMV / GEMM arithmetic in plain C.
 *
 * TEST INFRASTRUCTURE: this file is the checker and the timed CPU baseline.
 * Nothing in the CUDA product path calls it.
 *
 * Block arithmetic follows the reference's own statement of it,
 * benchmarks/kernels/showcase/triton_kernels.py:133-181 (decode_ggml, GGML type
 * ids 2 / 12 / 14 = Q4_0 / Q4_K / Q6_K); the GEMV contract (fp32 weight x fp32
 * activation, fp32 sum) follows triton_kernels.py:213-222 and the GEMM contract
 * (operands rounded to the MMA type, fp32 accumulate) triton_kernels.py:184-210
 * and benchmarks/kernels/showcase/benchmark.py:466-477.  Q8_0 (type id 8) is
 * not in the reference; it follows the GGML format definition (fp16 d, 32 int8).
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp -shared).
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <stdlib.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { FMT_Q4_0 = 2, FMT_Q8_0 = 8, FMT_Q4_K = 12, FMT_Q6_K = 14 };

static float half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else { /* subnormal: renormalise */
      int shift = 0;
      while (!(man & 0x400u)) { man <<= 1; ++shift; }
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

static float load_f16(const uint8_t *p) {
  return half_to_float((uint16_t)(p[0] | (p[1] << 8)));
}

/* Round fp32 to bfloat16 (nearest even), returned widened to fp32. */
static float round_bf16(float v) {
  uint32_t bits;
  memcpy(&bits, &v, 4);
  if ((bits & 0x7F800000u) == 0x7F800000u) return v;
  bits += 0x7FFFu + ((bits >> 16) & 1u);
  bits &= 0xFFFF0000u;
  memcpy(&v, &bits, 4);
  return v;
}

static int block_weights(int fmt) { return (fmt == FMT_Q4_0 || fmt == FMT_Q8_0) ? 32 : 256; }
static int block_bytes(int fmt) {
  switch (fmt) {
    case FMT_Q4_0: return 18;
    case FMT_Q8_0: return 34;
    case FMT_Q4_K: return 144;
    case FMT_Q6_K: return 210;
  }
  return 0;
}

int64_t gguf_oracle_row_bytes(int fmt, int64_t k) {
  int bw = block_weights(fmt), bb = block_bytes(fmt);
  if (!bb || k % bw) return -1;
  return k / bw * bb;
}

/* triton_kernels.py:135-142 */
static void decode_block_q4_0(const uint8_t *b, float *out) {
  float d = load_f16(b);
  for (int i = 0; i < 16; ++i) {
    out[i] = (float)((int)(b[2 + i] & 15) - 8) * d;
    out[16 + i] = (float)((int)(b[2 + i] >> 4) - 8) * d;
  }
}

/* GGML format definition */
static void decode_block_q8_0(const uint8_t *b, float *out) {
  float d = load_f16(b);
  for (int i = 0; i < 32; ++i) out[i] = d * (float)(int8_t)b[2 + i];
}

/* triton_kernels.py:143-162 */
static void decode_block_q4_k(const uint8_t *b, float *out) {
  float d = load_f16(b), dmin = load_f16(b + 2);
  const uint8_t *s = b + 4;
  for (int g = 0; g < 8; ++g) {
    int j = g % 4, sc, mn;
    if (g < 4) {
      sc = s[j] & 63;
      mn = s[4 + j] & 63;
    } else {
      sc = (s[8 + j] & 15) | ((s[j] >> 6) << 4);
      mn = (s[8 + j] >> 4) | ((s[4 + j] >> 6) << 4);
    }
    float scale = d * (float)sc, minimum = dmin * (float)mn;
    const uint8_t *q = b + 16 + (g / 2) * 32;
    int shift = (g % 2) * 4;
    for (int i = 0; i < 32; ++i) {
      /* both products are exact in fp32; one rounding at the subtraction */
      float prod = scale * (float)((q[i] >> shift) & 15);
      out[g * 32 + i] = prod - minimum;
    }
  }
}

/* triton_kernels.py:163-180 */
static void decode_block_q6_k(const uint8_t *b, float *out) {
  float d = load_f16(b + 208);
  for (int l = 0; l < 256; ++l) {
    int half = l / 128, lane = l % 32, quarter = (l % 128) / 32;
    int lo = b[half * 64 + lane + (quarter % 2) * 32];
    int hi = b[128 + half * 32 + lane];
    int q = ((lo >> (quarter / 2 * 4)) & 15) | (((hi >> (quarter * 2)) & 3) << 4);
    float sc = (float)(int8_t)b[192 + l / 16];
    out[l] = (float)(q - 32) * sc * d;
  }
}

static void decode_row(int fmt, const uint8_t *row, int64_t k, float *out) {
  int bw = block_weights(fmt), bb = block_bytes(fmt);
  for (int64_t i = 0; i < k / bw; ++i) {
    const uint8_t *b = row + i * bb;
    float *o = out + i * bw;
    switch (fmt) {
      case FMT_Q4_0: decode_block_q4_0(b, o); break;
      case FMT_Q8_0: decode_block_q8_0(b, o); break;
      case FMT_Q4_K: decode_block_q4_k(b, o); break;
      default: decode_block_q6_k(b, o); break;
    }
  }
}

int gguf_oracle_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Launchers such as torch.distributed.run export OMP_NUM_THREADS=1 to their children; a timed CPU
 * baseline sets the thread count it wants explicitly (the cores the process may run on). */
void gguf_oracle_set_threads(int count) {
#ifdef _OPENMP
  if (count > 0) omp_set_num_threads(count);
#else
  (void)count;
#endif
}

/* raw [n, row_bytes] -> out fp32 [n, k] */
int gguf_oracle_dequant(int fmt, const uint8_t *raw, int64_t n, int64_t k, float *out) {
  int64_t rb = gguf_oracle_row_bytes(fmt, k);
  if (rb < 0) return 2;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r) decode_row(fmt, raw + r * rb, k, out + r * k);
  return 0;
}

/* out[b, n] = sum_k x[b, k] * dequant(W)[n, k]; x fp32 [batch, k]; fp32 accumulate in
 * ascending k with 8 interleaved partial sums (any fp32 order is inside the 1e-3 gate). */
int gguf_oracle_gemv(int fmt, const uint8_t *raw, int64_t n, int64_t k, const float *x,
                     int64_t batch, float *out) {
  int64_t rb = gguf_oracle_row_bytes(fmt, k);
  if (rb < 0) return 2;
#pragma omp parallel
  {
    float *w = (float *)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
      decode_row(fmt, raw + r * rb, k, w);
      for (int64_t b = 0; b < batch; ++b) {
        const float *xb = x + b * k;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int64_t i = 0; i < k; i += 8)
          for (int j = 0; j < 8; ++j) acc[j] += xb[i + j] * w[i + j];
        out[b * n + r] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
      }
    }
    free(w);
  }
  return 0;
}

/* out[m, n] = sum_k round(x[m,k]) * round(dequant(W)[n,k]); operand = 0 keeps fp32 weights,
 * operand = 1 rounds decoded weights to bf16.  x must already hold values representable in
 * the operand type.  Blocked over rows of W so each decoded row is reused for all m. */
int gguf_oracle_gemm(int fmt, const uint8_t *raw, int64_t n, int64_t k, const float *x,
                     int64_t m, int operand, float *out) {
  int64_t rb = gguf_oracle_row_bytes(fmt, k);
  if (rb < 0) return 2;
#pragma omp parallel
  {
    float *w = (float *)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t r = 0; r < n; ++r) {
      decode_row(fmt, raw + r * rb, k, w);
      if (operand == 1)
        for (int64_t i = 0; i < k; ++i) w[i] = round_bf16(w[i]);
      for (int64_t t = 0; t < m; ++t) {
        const float *xt = x + t * k;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int64_t i = 0; i < k; i += 8)
          for (int j = 0; j < 8; ++j) acc[j] += xt[i + j] * w[i + j];
        out[t * n + r] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
      }
    }
    free(w);
  }
  return 0;
}
