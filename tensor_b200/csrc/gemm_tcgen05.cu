// Prefill GEMM on sm_100a: out[m, n] (fp32) = x[m, k] (bf16) . dequant(w[n, k])^T, weights rounded
// to bf16 (round-to-nearest-even of the exact fp32 decode), fp32 accumulation in tensor memory.
//
// Replaces the reference's `_packed` kernel (benchmarks/kernels/showcase/kernels.py:116-119),
// which decodes GGML blocks to 16-bit operands in shared memory and runs `mma.sync`
// (benchmarks/kernels/showcase/benchmark.py:471-477, showcase/README.md:105-108).
//
// Orientation: the 128 weight rows of a tile sit on the MMA M axis (TMEM lanes), up to 256 tokens
// on the MMA N axis (TMEM columns), so one decoded weight tile is reused by 256 tokens.
//
// One CTA = one 128 x 256 output tile, 10 warps:
//   warp 0      TMA producer: activation tiles [256 tokens x 64 k] bf16, 128-byte swizzle
//   warp 1      allocates TMEM, issues tcgen05.mma (one elected lane), commits to mbarriers
//   warps 2..9  decode raw GGUF blocks -> bf16, store the weight tile [128 x 64] into shared
//               memory in the same swizzled K-major layout TMA would produce, then drain the
//               accumulator (tcgen05.ld) and store fp32 results
// Two CTAs are resident per SM (256 TMEM columns and ~97 KB shared memory each), so one CTA's
// decode / epilogue overlaps the other's MMAs.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tb200 {
namespace {

constexpr int kTileN = 128;    // weight rows per tile (MMA M)
constexpr int kMmaTok = 256;   // tokens per MMA (MMA N)
constexpr int kBlockK = 64;    // K per pipeline stage: 64 bf16 = one 128-byte swizzle row
constexpr int kDecodeThreads = 256;              // threads that decode one [128 x 64] weight tile
constexpr int kABytes = kTileN * kBlockK * 2;    // 16 KB
constexpr int kHalfBBytes = kMmaTok * kBlockK * 2;  // 32 KB: the activation tile of one MMA

// Shapes of CTA.  TT = 1: 256 tokens per tile.  TT = 2 (M above 256): 512 tokens per
// tile, i.e. every decoded weight tile feeds two MMAs (decoding is what bounds this kernel, and
// it is paid per weight tile, not per token), all 512 TMEM columns, one CTA per SM, and two groups
// of decode warps that work on alternate k-blocks so that the SM keeps as many decode warps busy
// as two narrow CTAs would.
// G = decode warp groups (8 warps each, on alternate k-blocks).  <1, 1> is the two-CTAs-per-SM shape;
// <1, 2> serves small M, where there are fewer CTAs than SMs anyway and a lone CTA needs all the
// decode warps the SM can hold; <2, 2> is the 512-token shape.
template <int TT, int G> struct Cfg {
  static constexpr int kTileTok = kMmaTok * TT;
  static constexpr int kGroups = G;
  static constexpr int kAStages = 2 * G;
  static constexpr int kBStages = 2;
  static constexpr int kDecodeWarps = 8 * kGroups;
  static constexpr int kThreads = (2 + kDecodeWarps) * 32;
  static constexpr int kBBytes = kHalfBBytes * TT;
  static constexpr int kTmemCols = kMmaTok * TT;
  static constexpr int kCtasPerSm = (TT == 1 && G == 1) ? 2 : 1;
  static constexpr int kEpilogueCols = kTileTok / (kDecodeWarps / 4);  // token columns per four decode warps
  static constexpr int kSmemBytes = kAStages * kABytes + kBStages * kBBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
};
constexpr int kTileTok = Cfg<1, 1>::kTileTok;
constexpr int kThreads = Cfg<1, 1>::kThreads;
constexpr int kSmemBytes = Cfg<1, 1>::kSmemBytes;

// tcgen05 shared-memory matrix descriptor, K-major, 128-byte swizzle: rows are 128 bytes, eight
// rows form a 1024-byte swizzle atom (stride byte offset), version 1 (sm_100), layout type 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                    // descriptor version
  d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return d;
}

// kind::f16 instruction descriptor: fp32 accumulate, bf16 x bf16, both K-major, M = 128, N = 256.
constexpr uint32_t kInstrDesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kMmaTok >> 3) << 17) |
                                ((uint32_t)(kTileN >> 4) << 24);

// 2^23 + v for byte j of `bytes`
__device__ __forceinline__ float byte_magic(uint32_t bytes, int j) {
  return __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7540u | (uint32_t)j));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// ---- per-format decode of the [128 rows x 64 k] weight tile of one k-block by 256 threads --------
// Split into `fetch` (global loads into registers, issued one k-block ahead), `decode` (exact fp32
// arithmetic, rounded to bf16) and `store` (swizzled K-major tile: 16-byte chunk c of row r lives
// at r*128 + ((c ^ (r & 7)) * 16), exactly what a 128-byte-swizzle TMA load would produce).

template <int FMT> struct Decoder;

template <> struct Decoder<kQ4_K> {
  static constexpr int kShare = 1;  // k-blocks served by one fetch
  static constexpr int kAhead = 1;  // fetches in flight ahead of the decode (deeper was measured no faster)
  // thread t -> row t/2, half h = t%2: 32 weights of group 2p+h (p = kb%4), i.e. the low / high
  // nibbles of quant bytes 32p .. 32p+31 of super-block kb/4.
  struct Ctx {
    const uint8_t* wrow;
    int r, h;
  };
  struct Raw {
    uint4 hdr, q0, q1;
  };
  struct Out {
    uint32_t v[16];
  };
  __device__ static __forceinline__ Ctx context(const uint8_t* w, long long row_bytes_, int n0, int N, int t) {
    Ctx c;
    c.r = t >> 1;
    c.h = t & 1;
    c.wrow = w + (long long)min(n0 + c.r, N - 1) * row_bytes_;  // rows past N: decoded and dropped
    return c;
  }
  __device__ static __forceinline__ Raw fetch(const Ctx& c, int kb) {
    const uint8_t* blk = c.wrow + (kb >> 2) * 144;
    const int p = kb & 3;
    Raw r;
    r.hdr = __ldg(reinterpret_cast<const uint4*>(blk));
    r.q0 = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 32 * p));
    r.q1 = __ldg(reinterpret_cast<const uint4*>(blk + 32 + 32 * p));
    return r;
  }
  __device__ static __forceinline__ void decode(const Ctx& c, const Raw& r, int kb, Out& o) {
    const int h = c.h;
    const int p = kb & 3, g = 2 * p + h;
    const uint4 hdr = r.hdr;
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    const int j = g & 3, sh = 8 * j;
    uint32_t sc, mn;
    if (g < 4) {
      sc = (hdr.y >> sh) & 63u;
      mn = (hdr.z >> sh) & 63u;
    } else {
      sc = ((hdr.w >> sh) & 15u) | (((hdr.y >> (sh + 6)) & 3u) << 4);
      mn = ((hdr.w >> (sh + 4)) & 15u) | (((hdr.z >> (sh + 6)) & 3u) << 4);
    }
    const float dsc = d * (float)sc;
    const float dm = dmin * (float)mn;
    const uint32_t words[8] = {r.q0.x, r.q0.y, r.q0.z, r.q0.w, r.q1.x, r.q1.y, r.q1.z, r.q1.w};
    // A nibble that sits at bit s < 20 of a word becomes the float 2^23 + q * 2^s with one logic op
    // ((w & mask) | 0x4B000000), q * 2^s after subtracting 2^23, and d*sc*q - dmin*mn with one FMA
    // against d*sc*2^-s (a power-of-two rescale: exact).  The nibbles of bytes 2 and 3 that sit at
    // bit 20 or above are reached through w >> 12.  Masks and shifts depend on the thread's half.
    const uint32_t m0 = h ? 0x000000F0u : 0x0000000Fu, m1 = h ? 0x0000F000u : 0x00000F00u;
    const uint32_t m2 = h ? 0x00000F00u : 0x000000F0u, m3 = h ? 0x000F0000u : 0x0000F000u;
    const float s0 = dsc * (h ? 0.0625f : 1.f), s1 = dsc * (h ? 0x1p-12f : 0x1p-8f);
    const float s2 = dsc * (h ? 0x1p-8f : 0x1p-4f), s3 = dsc * (h ? 0x1p-16f : 0x1p-12f);
    const uint32_t magic = 0x4B000000u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t w = words[i], ws = w >> 12;
      uint32_t t0, t1, t2, t3;
      asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t0) : "r"(w), "r"(m0), "r"(magic));
      asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t1) : "r"(w), "r"(m1), "r"(magic));
      asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t2) : "r"(ws), "r"(m2), "r"(magic));
      asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(t3) : "r"(ws), "r"(m3), "r"(magic));
      const float f0 = fmaf(s0, __uint_as_float(t0) - 8388608.f, -dm);
      const float f1 = fmaf(s1, __uint_as_float(t1) - 8388608.f, -dm);
      const float f2 = fmaf(s2, __uint_as_float(t2) - 8388608.f, -dm);
      const float f3 = fmaf(s3, __uint_as_float(t3) - 8388608.f, -dm);
      o.v[2 * i] = pack_bf16(f0, f1);
      o.v[2 * i + 1] = pack_bf16(f2, f3);
    }
  }
  __device__ static __forceinline__ void store(const Ctx& c, uint8_t* a_tile, const Out& o) {
    uint8_t* row = a_tile + c.r * 128;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int chunk = (4 * c.h + q) ^ (c.r & 7);
      *reinterpret_cast<uint4*>(row + chunk * 16) = make_uint4(o.v[4 * q], o.v[4 * q + 1], o.v[4 * q + 2], o.v[4 * q + 3]);
    }
  }
};

template <> struct Decoder<kQ6_K> {
  // Blocks are 210 bytes: a row's blocks are only 2-byte aligned, and one thread per (row, half)
  // would issue 4-byte loads that touch 32 different cache lines per warp instruction (measured:
  // the L1 data pipe becomes the bound).  Instead eight lanes share a row: lane i of the group
  // owns 4-byte word i of each 32-byte span, so a warp instruction covers four rows x 32
  // contiguous bytes.  Four passes of 32 rows cover the tile.  Per pass a thread decodes 8 weights:
  // 4 of quarter 2*(kb%2) from its low-span word and 4 of quarter 2*(kb%2)+1 from its high-span
  // word, both with the same qh word.  Misaligned words are rebuilt from two aligned ones, the
  // second taken from the neighbouring lane (lane 7 loads its own).
  static constexpr int kPasses = 4;
  // Two consecutive k-blocks read the same words (the even one their low nibbles / low qh bit pairs,
  // the odd one the high ones), so the words are fetched once per pair.
  static constexpr int kShare = 2;
  static constexpr int kAhead = 2;  // fetches in flight ahead of the decode
  struct Ctx {
    const uint8_t* wrow[kPasses];
    int row0, i;  // first row of the thread (pass p adds 32 p), word index 0..7
  };
  struct Raw {
    uint32_t lo[kPasses], hi[kPasses], qh[kPasses];
    // int8 scales: low quarter | high quarter << 8 of the even k-block, the same << 16 of the odd one
    uint32_t meta[kPasses];
    uint32_t dbits[kPasses];  // fp16 d
  };
  struct Out {
    uint2 a[kPasses], b[kPasses];  // bf16 x 4 of the low / high quarter
  };
  __device__ static __forceinline__ Ctx context(const uint8_t* w, long long row_bytes_, int n0, int N, int t) {
    Ctx c;
    c.i = t & 7;
    c.row0 = t >> 3;
#pragma unroll
    for (int p = 0; p < kPasses; ++p) c.wrow[p] = w + (long long)min(n0 + c.row0 + 32 * p, N - 1) * row_bytes_;
    return c;
  }
  __device__ static __forceinline__ Raw fetch(const Ctx& c, int kb) {
    const int half = (kb & 3) >> 1;  // kb and kb ^ 1 share everything fetched here
    Raw r;
#pragma unroll
    for (int p = 0; p < kPasses; ++p) {
      const uint8_t* blk = c.wrow[p] + (kb >> 2) * 210;
      // the three words sit at multiples of 4 bytes from one another: one aligned base, one
      // misalignment, constant word offsets
      const uintptr_t first = reinterpret_cast<uintptr_t>(blk) + 64 * half + 4 * c.i;
      const uint32_t* base = reinterpret_cast<const uint32_t*>(first & ~uintptr_t(3));
      const uint32_t sh = (uint32_t)(first & 2) * 8;
      const int qh_words = 32 - 8 * half;  // (128 + 32 half) - 64 half bytes further
      const uint32_t l0 = __ldg(base), h0 = __ldg(base + 8), q0 = __ldg(base + qh_words);
      uint32_t l1 = __shfl_down_sync(0xffffffffu, l0, 1, 8);
      uint32_t h1 = __shfl_down_sync(0xffffffffu, h0, 1, 8);
      uint32_t q1 = __shfl_down_sync(0xffffffffu, q0, 1, 8);
      if (c.i == 7) {  // the last lane of a row group has no neighbour to take the next word from
        l1 = __ldg(base + 1);
        h1 = __ldg(base + 9);
        q1 = __ldg(base + qh_words + 1);
      }
      r.lo[p] = __funnelshift_r(l0, l1, sh);
      r.hi[p] = __funnelshift_r(h0, h1, sh);
      r.qh[p] = __funnelshift_r(q0, q1, sh);
      const uint8_t* sc = blk + 192 + 8 * half + (c.i >> 2);
      r.meta[p] = (uint32_t)__ldg(sc) | ((uint32_t)__ldg(sc + 2) << 8) | ((uint32_t)__ldg(sc + 4) << 16) |
                  ((uint32_t)__ldg(sc + 6) << 24);
      r.dbits[p] = (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(blk + 208));
    }
    return r;
  }
  __device__ static __forceinline__ void decode(const Ctx&, const Raw& r, int kb, Out& o) {
    const int nib = kb & 1;
    const int lsh = 4 * nib;
#pragma unroll
    for (int p = 0; p < kPasses; ++p) {
      const float d = __half2float(__ushort_as_half((unsigned short)r.dbits[p]));
      const uint32_t scales = r.meta[p] >> (16 * nib);
      const float dsa = d * (float)(int)(int8_t)(scales & 0xFF);
      const float dsb = d * (float)(int)(int8_t)((scales >> 8) & 0xFF);
      const uint32_t qa = ((r.lo[p] >> lsh) & 0x0F0F0F0Fu) | (((r.qh[p] >> lsh) & 0x03030303u) << 4);
      const uint32_t qb = ((r.hi[p] >> lsh) & 0x0F0F0F0Fu) | (((r.qh[p] >> (lsh + 2)) & 0x03030303u) << 4);
      float fa[4], fb[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        fa[b] = (byte_magic(qa, b) - 8388640.f) * dsa;  // 2^23 + 32
        fb[b] = (byte_magic(qb, b) - 8388640.f) * dsb;
      }
      o.a[p] = make_uint2(pack_bf16(fa[0], fa[1]), pack_bf16(fa[2], fa[3]));
      o.b[p] = make_uint2(pack_bf16(fb[0], fb[1]), pack_bf16(fb[2], fb[3]));
    }
  }
  __device__ static __forceinline__ void store(const Ctx& c, uint8_t* a_tile, const Out& o) {
#pragma unroll
    for (int p = 0; p < kPasses; ++p) {
      const int r = c.row0 + 32 * p;
      uint8_t* row = a_tile + r * 128 + (c.i & 1) * 8;
      // k = 4 i .. 4 i + 3 of the low quarter: chunk i / 2; the high quarter is 32 k (4 chunks) further
      *reinterpret_cast<uint2*>(row + ((((c.i >> 1)) ^ (r & 7)) << 4)) = o.a[p];
      *reinterpret_cast<uint2*>(row + (((4 + (c.i >> 1)) ^ (r & 7)) << 4)) = o.b[p];
    }
  }
};

template <int FMT, int TT, int G>
__device__ __forceinline__ void gemm_tcgen05_body(const CUtensorMap& tmap_x, const uint8_t* __restrict__ w,
                                                  float* __restrict__ out, int M, int N, int K,
                                                  long long row_bytes_) {
  using C = Cfg<TT, G>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle needs 1024-byte aligned tiles
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_tiles = smem;
  uint8_t* b_tiles = smem + C::kAStages * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kAStages * kABytes + C::kBStages * C::kBBytes);
  uint64_t* full_a = bars;                               // decode warps -> MMA
  uint64_t* empty_a = full_a + C::kAStages;              // MMA -> decode warps
  uint64_t* full_b = empty_a + C::kAStages;              // TMA -> MMA
  uint64_t* empty_b = full_b + C::kBStages;              // MMA -> TMA
  uint64_t* acc_full = empty_b + C::kBStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * C::kTileTok;
  const int n0 = blockIdx.y * kTileN;
  const int k_blocks = K / kBlockK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kAStages; ++s) {
      ptx::mbar_init(&full_a[s], kDecodeThreads);
      ptx::mbar_init(&empty_a[s], 1);
    }
    for (int s = 0; s < C::kBStages; ++s) {
      ptx::mbar_init(&full_b[s], 1);
      ptx::mbar_init(&empty_b[s], 1);
    }
    ptx::mbar_init(acc_full, 1);
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_x);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer: activations (one 256-token box per MMA) ----------------
    if (lane == 0) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % C::kBStages;
        if (kb >= C::kBStages && !ptx::mbar_wait(&empty_b[s], ((kb / C::kBStages) - 1) & 1)) {
          report_timeout(0x10000u | (unsigned)kb);
          break;
        }
        ptx::mbar_arrive_expect_tx(&full_b[s], C::kBBytes);
#pragma unroll
        for (int h = 0; h < TT; ++h)
          ptx::tma_load_2d(b_tiles + s * C::kBBytes + h * kHalfBBytes, &tmap_x, kb * kBlockK, m0 + h * kMmaTok,
                           &full_b[s]);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; ++kb) {
        const int sa = kb % C::kAStages, sb = kb % C::kBStages;
        if (!ptx::mbar_wait(&full_a[sa], (kb / C::kAStages) & 1) || !ptx::mbar_wait(&full_b[sb], (kb / C::kBStages) & 1)) {
          report_timeout(0x20000u | (unsigned)kb);
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint64_t a_desc = smem_desc_sw128(ptx::smem_addr(a_tiles + sa * kABytes));
#pragma unroll
        for (int h = 0; h < TT; ++h) {
          const uint64_t b_desc = smem_desc_sw128(ptx::smem_addr(b_tiles + sb * C::kBBytes + h * kHalfBBytes));
#pragma unroll
          for (int i = 0; i < kBlockK / 16; ++i)  // advance 16 bf16 = 32 bytes = 2 descriptor units
            ptx::umma_f16(tmem_base + (uint32_t)(h * kMmaTok), a_desc + 2 * i, b_desc + 2 * i, kInstrDesc,
                          (kb | i) ? 1u : 0u);
        }
        ptx::umma_commit(&empty_a[sa]);
        ptx::umma_commit(&empty_b[sb]);
      }
      ptx::umma_commit(acc_full);
    }
  } else {
    // ---------------- decode warps, then epilogue ----------------
    using D = Decoder<FMT>;
    const int group = (warp - 2) >> 3;  // which decode group; groups take alternate fetch units
    const typename D::Ctx ctx = D::context(w, row_bytes_, n0, N, (int)threadIdx.x - 64 - group * kDecodeThreads);
    bool ok = true;
    constexpr int kStep = C::kGroups * D::kShare;
    // K is a multiple of 256, so the k-blocks come in whole units of kShare that share one fetch,
    // and in whole rounds of one unit per group
    // The loads of a unit are issued kAhead units before it is decoded (clamped on the last ones): one
    // unit ahead left the decode warps waiting on memory for most of their stall cycles.
    constexpr int kAhead = D::kAhead;
    typename D::Raw raw[kAhead];
#pragma unroll
    for (int a = 0; a < kAhead; ++a) raw[a] = D::fetch(ctx, min(group * D::kShare + a * kStep, k_blocks - 1));
    for (int kb0 = group * D::kShare; kb0 < k_blocks && ok; kb0 += kStep) {
      const typename D::Raw next = D::fetch(ctx, min(kb0 + kAhead * kStep, k_blocks - 1));
#pragma unroll
      for (int j = 0; j < D::kShare; ++j) {
        const int kb = kb0 + j;
        const int s = kb % C::kAStages;
        typename D::Out decoded;
        D::decode(ctx, raw[0], kb, decoded);
        if (kb >= C::kAStages && !ptx::mbar_wait(&empty_a[s], ((kb / C::kAStages) - 1) & 1)) {
          report_timeout(0x30000u | (unsigned)kb);
          ok = false;
          break;
        }
        D::store(ctx, a_tiles + s * kABytes, decoded);
        ptx::fence_proxy_async_smem();  // make the generic-proxy stores visible to the tensor core
        ptx::mbar_arrive(&full_a[s]);
      }
#pragma unroll
      for (int a = 0; a + 1 < kAhead; ++a) raw[a] = raw[a + 1];
      raw[kAhead - 1] = next;
    }
    if (ok) {
      if (!ptx::mbar_wait(acc_full, 0)) {
        report_timeout(0x40000u);
        ok = false;
      }
    }
    if (ok) {
      ptx::tc_fence_after();
      const int quarter = warp & 3;            // TMEM lanes this warp may read
      const int col_group = (warp - 2) >> 2;   // every four decode warps take a band of token columns
      const int n = n0 + quarter * 32 + lane;  // output column (weight row) of this thread
#pragma unroll 1
      for (int c = 0; c < C::kEpilogueCols / 32; ++c) {
        const int col0 = col_group * C::kEpilogueCols + c * 32;
        if (m0 + col0 >= M) break;
        uint32_t acc[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)col0, acc);
        ptx::tmem_ld_wait();
        if (n < N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int tok = m0 + col0 + j;
            if (tok < M) out[(long long)tok * N + n] = __uint_as_float(acc[j]);
          }
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int FMT, int TT, int G>
__global__ void __launch_bounds__(Cfg<TT, G>::kThreads, Cfg<TT, G>::kCtasPerSm)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const uint8_t* __restrict__ w,
                        float* __restrict__ out, int M, int N, int K, long long row_bytes_) {
  gemm_tcgen05_body<FMT, TT, G>(tmap_x, w, out, M, N, K, row_bytes_);
}

// ---- host side -------------------------------------------------------------------------------------
#ifndef TB200_TBIN_WRAPPER

template <int FMT, int TT, int G>
cudaError_t launch_shape(const CUtensorMap& tmap, const uint8_t* w, float* out, long long m, long long n,
                         long long k, cudaStream_t stream) {
  using C = Cfg<TT, G>;
  auto kernel = gemm_tcgen05_kernel<FMT, TT, G>;
  cudaError_t e = allow_full_shared_memory(kernel);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)((m + C::kTileTok - 1) / C::kTileTok), (unsigned)((n + kTileN - 1) / kTileN));
  kernel<<<grid, C::kThreads, C::kSmemBytes, stream>>>(tmap, w, out, (int)m, (int)n, (int)k, row_bytes(FMT, k));
  return cudaGetLastError();
}

// <token tiles, decode groups>: 512 tokens per tile above M = 256 and one 256-token CTA with two
// decode groups up to there, unless a schedule pins the shape (11, 12 or 22).
template <int FMT>
cudaError_t launch_fmt(const CUtensorMap& tmap, const uint8_t* w, float* out, long long m, long long n,
                       long long k, cudaStream_t stream, bool big_ok, int pinned) {
  int shape = !big_ok ? 11 : (m > 256 ? 22 : 12);
  if (pinned == 11 || (big_ok && (pinned == 12 || pinned == 22))) shape = pinned;
  if (shape == 22) return launch_shape<FMT, 2, 2>(tmap, w, out, m, n, k, stream);
  if (shape == 12) return launch_shape<FMT, 1, 2>(tmap, w, out, m, n, k, stream);
  return launch_shape<FMT, 1, 1>(tmap, w, out, m, n, k, stream);
}

#endif  // TB200_TBIN_WRAPPER
}  // namespace

// static-shape entry used by generated .tbin wrappers
constexpr int kGemmThreads = kThreads;
template <int FMT>
__device__ __forceinline__ void gemm_static_entry(const CUtensorMap& x, const uint8_t* w, float* out, int m, int n,
                                                  int k) {
  gemm_tcgen05_body<FMT, 1, 1>(x, w, out, m, n, k, row_bytes(FMT, k));
}

#ifndef TB200_TBIN_WRAPPER
TB200_DEFINE_STATUS_READER(read_gemm_status)

void gemm_launch_config(long long m, long long n, int* out8) {
  const int vals[8] = {(int)((m + kTileTok - 1) / kTileTok), (int)((n + kTileN - 1) / kTileN), kThreads, kSmemBytes,
                       kTileTok, kBlockK, 0, 0};
  for (int i = 0; i < 8; ++i) out8[i] = vals[i];
}


bool gemm_fast_supported(int fmt, long long m, long long n, long long k, const DeviceInfo& dev) {
  if (fmt != kQ4_K && fmt != kQ6_K) return false;
  if (m < 1 || n < 1 || k < 256 || k % 256) return false;
  if (m > (1 << 24) || n > (1 << 24) || k > (1 << 24)) return false;
  if ((n + kTileN - 1) / kTileN > 65535) return false;
  // Q4_K rows are always multiples of 16 bytes (16-byte vector loads); Q6_K rows are only
  // 2-byte aligned in general and are read with 4-byte loads realigned in registers.
  return dev.max_smem_optin >= kSmemBytes;
}

bool gemm_shape_legal(int shape, long long, const DeviceInfo& dev) {
  if (shape == 0 || shape == 11) return true;
  return (shape == 12 || shape == 22) && dev.max_smem_optin >= Cfg<2, 2>::kSmemBytes;
}

cudaError_t launch_gemm_fast(int fmt, const void* x, const uint8_t* w, float* out, long long m, long long n,
                             long long k, cudaStream_t stream, const char** detail, const Schedule* sched) {
  if (!sched) sched = lookup_schedule(kOpGemm, fmt, m, n, k);
  const int pinned = sched ? sched->gemm_shape : 0;
  // x as a 2-D tensor [m rows, k columns] of bf16; box = 64 columns (128 bytes) x 256 rows,
  // 128-byte swizzle, rows past m read as zero.
  alignas(64) CUtensorMap tmap;
  if (!make_tensor_map_2d(&tmap, TmaType::kBF16, x, (unsigned long long)k, (unsigned long long)m,
                          (unsigned long long)k * 2, kBlockK, kTileTok, true)) {
    if (detail) *detail = "cuTensorMapEncodeTiled is unavailable or rejected the activation layout";
    return cudaErrorNotSupported;
  }
  int dev = 0, optin = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  const bool wide_ok = optin >= Cfg<2, 2>::kSmemBytes;
  switch (fmt) {
    case kQ4_K: return launch_fmt<kQ4_K>(tmap, w, out, m, n, k, stream, wide_ok, pinned);
    case kQ6_K: return launch_fmt<kQ6_K>(tmap, w, out, m, n, k, stream, wide_ok, pinned);
  }
  return cudaErrorInvalidValue;
}
#endif  // TB200_TBIN_WRAPPER

}  // namespace tb200
