// Decode GEMV for batch 1..16 on the 5th-generation tensor cores of sm_100a, as ONE persistent launch
// over a list of projections: out_i[m_i, n_i] = x_i[m_i, k_i] . dequant(w_i[n_i, k_i])^T.
//
// Replaces the reference's `gemv_packed` (benchmarks/kernels/showcase/kernels.py:116-119) with its
// fp32-weight x fp32-activation contract (benchmarks/kernels/showcase/benchmark.py:468-470); a list
// is what a decoder layer launches back to back (q/k/v, gate/up, ...): the reference launches them
// one kernel each.
//
// Regime: HBM-bound, so the whole design serves one goal: keep weight bytes streaming.
//
//  * Work unit = 128 weight rows x one 256-weight column of blocks.  The units of all projections
//    of the list form one sequence that is cut into equal contiguous ranges, one per CTA (one CTA
//    per SM).  A CTA streams its units through a shared-memory ring (one 2-D TMA copy of the raw
//    blocks + one bulk copy of the matching activation tile per unit), so ring fill, barrier set-up
//    and tail are paid once per list, not once per projection.  Where a range ends inside a row
//    tile the partial sums go to scratch and the last CTA to arrive adds them in K order
//    (deterministic).
//  * 16 decode warps: thread (row r, quarter p) reads its 64 weights of the unit from the ring,
//    turns nibble pairs into the fp16 numbers 1024 + q (or 1024 + 16 q for a high nibble) with one
//    logic op per pair -- exact -- and stores them straight into tensor memory as the A operand
//    (tcgen05.st).  No decoded weight ever touches shared memory.
//  * One thread issues tcgen05.mma (M = 128 rows, N = 16 activation rows, K = 16) with A from tensor
//    memory and the fp16 activations from the ring.  Each 32-weight scale group accumulates into
//    its own block of accumulator columns; the block scales are applied to those 32-weight sums in
//    fp32 by 8 drain warps of their own (tcgen05.ld), so that the decode warps never wait for the
//    tensor core:
//        sum_k (d*sc*q - dmin*mn) x = d*sc*(S - 1024*Sx) - dmin*mn*Sx,   S = sum (1024 + q) x.
//    The Sx terms use the fp32 sums of each scale group that travel with the activation tile.
//  * Activations are converted once per list by a small kernel ahead of this one: fp16 after one
//    power-of-two scale per activation row (largest magnitude -> [2^9, 2^10), so bf16 -> fp16 is exact
//    for every value within 2^-26 of the row's largest), laid out as the K-major core matrices the
//    MMA reads, k permuted the way the decode threads emit weights.
//  * Every wait is bounded and sets a status word; tensor memory is released on every path.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tb200 {
namespace {

constexpr int kRows = 128;                    // weight rows per tile = TMEM lanes
constexpr int kParts = 4;                     // decode threads per row; each owns a quarter of a unit
constexpr int kDecodeWarps = 4 * kParts;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kHalves = 2;                    // drain threads per row; each owns the scale groups of two quarters
constexpr int kDrainWarps = 4 * kHalves;
constexpr int kDrainThreads = kDrainWarps * 32;
constexpr int kProducerWarp = kDecodeWarps + kDrainWarps, kMmaWarp = kProducerWarp + 1;
constexpr int kMmaWarps = 2;                  // two issuers take alternate sub-units
constexpr int kThreads = (kMmaWarp + kMmaWarps) * 32;
constexpr int kUnitK = 256;                   // weights per row and unit
constexpr int kXMainBytes = 16 * kUnitK * 2;  // activation tile: 16 rows x 256 k, fp16; the sums of its scale groups follow
constexpr int kMaxStagesTc = 8;
constexpr int kSlotFloats = 16 * kRows;       // one partial-sum slot
constexpr int kSmemHeader = 1024;
// tensor memory columns: two A buffers (256 fp16 weights per lane each) and two accumulator sets
// (8 scale groups x 16 activation rows each)
constexpr uint32_t kColA = 0, kColD = 256, kBufCols = 128, kTmemCols = 512;
// kind::f16 instruction descriptor: fp32 accumulate, fp16 x fp16, both K-major, M = 128, N = 16
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);

struct TcItem {
  const uint8_t* xprep;      // converted activations: one kXTileBytes tile per 256-weight column
  const float* unscale;      // [16] factor that undoes the activation scaling of each row
  float* outs[kMaxOutputs];  // destinations (own output first, then peer-mapped ones)
  long long n, out_ld;
  int n_out, m, nb;          // nb: m rounded up to 1, 2, 4, 8 or 16
  int nsb, row_tiles;
  int unit_base, tile_base;  // first unit / first row tile of this projection in the list
};

struct alignas(64) TcParams {
  CUtensorMap wmap[kTcMaxItems];  // weights as [n rows] x [row bytes / 8] 8-byte words, box = one unit
  TcItem item[kTcMaxItems];
  int n_items, total_units, stages, stage_bytes, red_floats;
  float* partials;
  unsigned int* counters;
  unsigned int* pads[kMaxOutputs];
  int rank, world, sync;
  unsigned long long wait_limit_ns;
#ifdef TB200_TC_TRACE
  long long* trace;  // diagnostic timeline of CTA 0 (trace builds only)
#endif
};
#ifdef TB200_TC_TRACE
#define TC_STAMP(cond, idx, slot) do { if (p.trace && blockIdx.x == 0 && (cond) && (idx) < 64) p.trace[(idx) * 16 + (slot)] = clock64(); } while (0)
#else
#define TC_STAMP(cond, idx, slot) do { } while (0)
#endif
#ifdef TB200_TC_TRACE
#define TC_WALL(cond, slot) do { if (p.trace && blockIdx.x == 0 && (cond)) p.trace[63 * 16 + (slot)] = (long long)ptx::global_timer_ns(); } while (0)
#else
#define TC_WALL(cond, slot) do { } while (0)
#endif

struct Cursor {
  int item, tile, sb;
};
__device__ __forceinline__ Cursor locate(const TcParams& p, int unit) {
  Cursor c;
  c.item = 0;
  while (c.item + 1 < p.n_items && unit >= p.item[c.item + 1].unit_base) ++c.item;
  const int rem = unit - p.item[c.item].unit_base;
  c.tile = rem / p.item[c.item].nsb;
  c.sb = rem - c.tile * p.item[c.item].nsb;
  return c;
}
__device__ __forceinline__ void advance(const TcParams& p, Cursor& c) {
  if (++c.sb == p.item[c.item].nsb) {
    c.sb = 0;
    if (++c.tile == p.item[c.item].row_tiles) {
      c.tile = 0;
      ++c.item;
    }
  }
}

// One probe of an mbarrier phase without a suspend-time hint (the waits of this kernel sit on its
// critical path: a waiting warp should see the completing arrival at once).
__device__ __forceinline__ bool try_wait_now(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(ptx::smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait that also gives up when another warp of the CTA has given up.  The clock is only
// consulted after a few thousand failed probes: a wait of this kernel normally ends within a
// microsecond, and reading the global timer costs about as much as such a wait.
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort, unsigned code) {
#pragma unroll 1
  for (int i = 0; i < 4096; ++i)
    if (try_wait_now(bar, parity)) return true;
  const uint64_t start = ptx::global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (try_wait_now(bar, parity)) return true;
    if (*abort) return false;
    if (ptx::global_timer_ns() - start > ptx::kWaitLimitNs) {
      *abort = 1;
      report_timeout(code);
      return false;
    }
  }
}

__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  // no swizzle, K-major: core matrices of 8 rows x 16 bytes; the two core matrices of a k-step are
  // 256 bytes apart (16 rows x 16 bytes), 8-row groups 128 bytes apart
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(256 >> 4) << 16;
  d |= (uint64_t)(128 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// D[tmem] (+)= A[tmem] * B[smem descriptor], issued by the lanes whose `leader` is set.  The whole warp
// runs the issue loop with uniform control flow, so the addresses and descriptors stay in uniform
// registers: with a divergent `if (lane == 0)` around the loop every operand of every MMA is moved
// there one by one, and the issue rate of these small MMAs (about 60 cycles each) suffers.
template <bool ACCUMULATE>
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t leader) {
  if constexpr (ACCUMULATE) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.eq.u32 p, 1, 1;\n\tsetp.ne.u32 q, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc),
        "r"(leader)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.eq.u32 p, 1, 0;\n\tsetp.ne.u32 q, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc),
        "r"(leader)
        : "memory");
  }
}
// tcgen05.commit by the lanes whose `leader` is set
__device__ __forceinline__ void umma_commit_if(uint64_t* bar, uint32_t leader) {
  asm volatile(
      "{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(ptx::smem_addr(bar)),
      "r"(leader)
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
      "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[N]) {
  if constexpr (N == 1) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v[0]) : "r"(taddr) : "memory");
  } else if constexpr (N == 2) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=r"(v[0]), "=r"(v[1]) : "r"(taddr) : "memory");
  } else if constexpr (N == 4) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3])
                 : "r"(taddr)
                 : "memory");
  } else if constexpr (N == 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
  } else {
    static_assert(N == 16, "accumulator blocks are 1, 2, 4, 8 or 16 columns");
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
  }
}

// N consecutive floats of shared memory that every lane of the warp reads alike (a broadcast)
template <int N>
__device__ __forceinline__ void lds_floats(uint32_t addr, float (&v)[N]) {
  if constexpr (N == 1) {
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v[0]) : "r"(addr));
  } else if constexpr (N == 2) {
    const float2 t = ptx::lds64f(addr);
    v[0] = t.x;
    v[1] = t.y;
  } else {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const uint4 t = ptx::lds128(addr + 16 * i);
      v[4 * i] = __uint_as_float(t.x);
      v[4 * i + 1] = __uint_as_float(t.y);
      v[4 * i + 2] = __uint_as_float(t.z);
      v[4 * i + 3] = __uint_as_float(t.w);
    }
  }
}

// (a & mask) | bits in one logic op, constants in registers (with immediates the compiler emits two)
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t bits) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(bits));
  return d;
}

// What a decode thread keeps of a unit: the scales of its two groups.  With S_g = sum (1024 + f q) x
// (f = 1 for the even group, 16 for the odd one) and Sx_g = sum x over the group,
//   sum_k (d sc q - dmin mn) x = s_g S_g - e_g Sx_g,   s_g = d sc_g / f,   e_g = 1024 s_g + dmin mn_g.
struct UnitScales {
  float s_lo, s_hi, e_lo, e_hi;
};

// ---- Q4_K: 144-byte blocks; quarter p = quant bytes 32p .. 32p+31 = groups 2p (low nibbles) and
// 2p+1 (high nibbles).  Word w of the quarter gives cells 2w = bytes (4w, 4w+2) and 2w+1 = bytes
// (4w+1, 4w+3): position 4w + 2e + h of a group holds byte 4w + e + 2h, and the activation tiles
// are written in the same order. ------------------------------------------------------------------
template <int FMT> struct TcFormat;
template <> struct TcFormat<kQ4_K> {
  static constexpr int kBoxBytes = 144;    // bytes of a row inside a unit's ring stage
  static constexpr int kSub = 1;           // sub-units a staged block is decoded in
  static constexpr int kSumGroups = 8;     // scale groups per block whose activation sums travel with the tile
  static constexpr int kXTileBytes = kXMainBytes + kSumGroups * 64;
  __host__ __device__ static __forceinline__ int box_x(int sb) { return sb * 18; }  // 8-byte units
  __host__ __device__ static __forceinline__ int box_offset(int) { return 0; }
  // two k-steps of 16 per 32-weight group; a k-step's activations are 512 bytes (32 descriptor units)
  __device__ static __forceinline__ void issue(uint32_t d, uint32_t a, uint64_t xdesc, int, uint32_t idesc, uint32_t leader) {
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      umma_ts<false>(d + 16 * g, a + 16 * g, xdesc + 64 * g, idesc, leader);
      umma_ts<true>(d + 16 * g, a + 16 * g + 8, xdesc + 64 * g + 32, idesc, leader);
    }
  }
  __device__ static __forceinline__ void decode(uint32_t wrow, int part, int, int, uint32_t tmem_a) {
    const uint4 q0 = ptx::lds128(wrow + 16 + 32 * part), q1 = ptx::lds128(wrow + 32 + 32 * part);
    const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    uint32_t mlo, mhi, bits;
    asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(mlo));
    asm volatile("mov.b32 %0, 0x00F000F0;" : "=r"(mhi));
    asm volatile("mov.b32 %0, 0x64006400;" : "=r"(bits));
    uint32_t lo[16], hi[16];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const uint32_t v = words[w], v8 = v >> 8;
      lo[2 * w] = and_or(v, mlo, bits);
      hi[2 * w] = and_or(v, mhi, bits);
      lo[2 * w + 1] = and_or(v8, mlo, bits);
      hi[2 * w + 1] = and_or(v8, mhi, bits);
    }
    tmem_st16(tmem_a + 32 * part, lo);
    tmem_st16(tmem_a + 32 * part + 16, hi);
  }
  // scales of the four groups 4 half .. 4 half + 3 of a row's block (quarters 2 half and 2 half + 1):
  // 6-bit scales / mins in bytes 4..15 of the block (hdr.y, hdr.z, hdr.w), fp16 d and dmin in hdr.x
  __device__ static __forceinline__ void scales2(uint32_t wrow, int half, int, int, UnitScales (&out)[2]) {
    const uint4 hdr = ptx::lds128(wrow);
    uint32_t sc[4], mn[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (half == 0) {
        sc[j] = (hdr.y >> (8 * j)) & 63u;
        mn[j] = (hdr.z >> (8 * j)) & 63u;
      } else {
        sc[j] = ((hdr.w >> (8 * j)) & 15u) | (((hdr.y >> (8 * j + 6)) & 3u) << 4);
        mn[j] = ((hdr.w >> (8 * j + 4)) & 15u) | (((hdr.z >> (8 * j + 6)) & 3u) << 4);
      }
    }
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));  // d, dmin
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      out[q].s_lo = dd.x * (float)sc[2 * q];
      out[q].s_hi = dd.x * (float)sc[2 * q + 1] * 0.0625f;  // the odd group's MMAs sum 1024 + 16 q
      out[q].e_lo = fmaf(1024.f, out[q].s_lo, dd.y * (float)mn[2 * q]);
      out[q].e_hi = fmaf(1024.f, out[q].s_hi, dd.y * (float)mn[2 * q + 1]);
    }
  }
};

// ---- Q6_K: 210-byte blocks (ql[128] low nibbles, qh[64] high bit pairs, 16 int8 scales, fp16 d), 16
// scale groups of 16 weights, w = d * sc * (q - 32).  A staged block is decoded as two sub-units of 128
// weights (the two halves of the block layout): quarter p of half h = bytes ql[64h + 32(p%2) ..+32]
// (low nibbles for p < 2, high ones else) joined with bit pair p of qh[32h ..+32]; its 32 weights are
// the scale groups 2p and 2p + 1 of the half.  Every k-step of 16 is one scale group with its own
// accumulator block, so no MMA accumulates.  Blocks are only 2-byte aligned: the ring holds, per row, the
// 240 bytes from the 16-byte boundary below the block, and `O` says where the block starts in there.
template <> struct TcFormat<kQ6_K> {
  static constexpr int kBoxBytes = 240;
  static constexpr int kSub = 2;
  static constexpr int kSumGroups = 16;
  static constexpr int kXTileBytes = kXMainBytes + kSumGroups * 64;
  __host__ __device__ static __forceinline__ int box_x(int sb) { return (210 * sb / 16) * 2; }  // 8-byte units
  __host__ __device__ static __forceinline__ int box_offset(int sb) { return (210 * sb) & 15; }

  // 32 bytes that start O bytes into the three aligned 16-byte words at `addr`
  template <int O>
  __device__ static __forceinline__ void load32(uint32_t addr, uint32_t (&out)[8]) {
    const uint4 a = ptx::lds128(addr), b = ptx::lds128(addr + 16), c = ptx::lds128(addr + 32);
    const uint32_t w[12] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w, c.x, c.y, c.z, c.w};
    constexpr int kWord = O >> 2, kHalf = (O >> 1) & 1;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      out[i] = kHalf ? __funnelshift_r(w[i + kWord], w[i + kWord + 1], 16) : w[i + kWord];
  }

  template <int O>
  __device__ static __forceinline__ void decode_at(uint32_t wrow, int part, int sub, uint32_t tmem_a) {
    uint32_t ql[8], qh[8];
    load32<O>(wrow + sub * 64 + (part & 1) * 32, ql);
    load32<O>(wrow + 128 + sub * 32, qh);
    const int lsh = (part >> 1) * 4, hsh = 2 * part;
    uint32_t cells[16];
    uint32_t magic;
    asm volatile("mov.b32 %0, 0x64646464;" : "=r"(magic));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t q = ((ql[i] >> lsh) & 0x0F0F0F0Fu) | (((qh[i] >> hsh) & 0x03030303u) << 4);  // four 6-bit values
      cells[2 * i] = __byte_perm(q, magic, 0x4140);      // fp16 pair 1024 + q of bytes 0, 1
      cells[2 * i + 1] = __byte_perm(q, magic, 0x4342);  // bytes 2, 3
    }
    tmem_st16(tmem_a + 16 * part, cells);
  }
  __device__ static __forceinline__ void decode(uint32_t wrow, int part, int sub, int offset, uint32_t tmem_a) {
    switch (offset >> 1) {  // the same for every thread of the CTA
      case 0: decode_at<0>(wrow, part, sub, tmem_a); break;
      case 1: decode_at<2>(wrow, part, sub, tmem_a); break;
      case 2: decode_at<4>(wrow, part, sub, tmem_a); break;
      case 3: decode_at<6>(wrow, part, sub, tmem_a); break;
      case 4: decode_at<8>(wrow, part, sub, tmem_a); break;
      case 5: decode_at<10>(wrow, part, sub, tmem_a); break;
      case 6: decode_at<12>(wrow, part, sub, tmem_a); break;
      default: decode_at<14>(wrow, part, sub, tmem_a); break;
    }
  }
  // int8 scales of the four groups 4 half .. 4 half + 3 of this half of the block; fp16 d
  __device__ static __forceinline__ void scales2(uint32_t wrow, int half, int sub, int offset, UnitScales (&out)[2]) {
    unsigned short dbits;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(dbits) : "r"(wrow + offset + 208));
    const float d = __half2float(__ushort_as_half(dbits));
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      unsigned short sc2;
      asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sc2) : "r"(wrow + offset + 192 + 8 * sub + 4 * half + 2 * q));
      out[q].s_lo = d * (float)(int)(signed char)(sc2 & 0xFF);
      out[q].s_hi = d * (float)(int)(signed char)(sc2 >> 8);
      out[q].e_lo = 1056.f * out[q].s_lo;  // (1024 + q) - 1056 = q - 32
      out[q].e_hi = 1056.f * out[q].s_hi;
    }
  }
  // one accumulator block per 16-weight group: 8 MMAs per sub-unit, none accumulating
  __device__ static __forceinline__ void issue(uint32_t d, uint32_t a, uint64_t xdesc, int sub, uint32_t idesc, uint32_t leader) {
#pragma unroll
    for (int g = 0; g < 8; ++g) umma_ts<false>(d + 16 * g, a + 8 * g, xdesc + 32 * (8 * sub + g), idesc, leader);
  }
};

// accumulators of one unit -> this thread's running sums (its two groups, NB activation rows)
template <int NB>
__device__ __forceinline__ void drain(uint32_t tmem_d, int part, const UnitScales& sc, float (&acc)[16]) {
  uint32_t lo[NB], hi[NB];
  tmem_ld<NB>(tmem_d + 32 * part, lo);
  tmem_ld<NB>(tmem_d + 32 * part + 16, hi);
  ptx::tmem_ld_wait();
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    acc[b] = fmaf(sc.s_lo, __uint_as_float(lo[b]), acc[b]);
    acc[b] = fmaf(sc.s_hi, __uint_as_float(hi[b]), acc[b]);
  }
}
// the e_g Sx_g terms of a unit, from the group sums that travel with its activation tile
template <int NB>
__device__ __forceinline__ void correct(uint32_t sums, int group, const UnitScales& sc, float (&acc)[16]) {
  float sx_lo[NB], sx_hi[NB];
  lds_floats<NB>(sums + group * 64, sx_lo);
  lds_floats<NB>(sums + (group + 1) * 64, sx_hi);
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    acc[b] = fmaf(-sc.e_lo, sx_lo[b], acc[b]);
    acc[b] = fmaf(-sc.e_hi, sx_hi[b], acc[b]);
  }
}

// State the drain warps share when they meet among themselves.
struct DecodeSync {
  uint64_t* cbar;
  volatile int* abort;
  volatile int* s_last;
  uint32_t phase;
  __device__ __forceinline__ bool sync() {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) ptx::mbar_arrive(cbar);
    const bool ok = wait_bar(cbar, phase & 1, abort, 0x50000u);
    ++phase;
    return ok;
  }
};

// A segment = the units of one row tile that this CTA owns (columns sb0 .. at.sb).  The drain
// threads have put their sums into `red` ([half][activation row][weight row]).  All of K: add the
// two halves and store.  Part of K: the sum goes to this CTA's scratch slot and the last CTA of the
// tile to arrive adds the slots in K order (deterministic).
__device__ __noinline__ bool finish_segment(const TcParams& p, const Cursor at, int sb0, int u0, const float* red,
                                            DecodeSync& ds) {
  const TcItem& it = p.item[at.item];
  const int nb = it.nb, tid = threadIdx.x - kDecodeThreads;
  if (!ds.sync()) return false;
  const bool whole = sb0 == 0 && at.sb == it.nsb - 1;
  const long long tile_unit0 = (long long)it.unit_base + (long long)at.tile * it.nsb;
  const bool from_range_start = tile_unit0 + sb0 == u0;
  float* slot = p.partials + ((size_t)2 * blockIdx.x + (from_range_start ? 0 : 1)) * kSlotFloats;
  for (int i = tid; i < nb * kRows; i += kDrainThreads) {
    const int b = i >> 7, r = i & (kRows - 1);
    float v = red[b * kRows + r];
#pragma unroll
    for (int q = 1; q < kHalves; ++q) v += red[(q * nb + b) * kRows + r];
    if (whole) {
      const long long grow = (long long)at.tile * kRows + r;
      if (b < it.m && grow < it.n) {
        v *= __ldg(it.unscale + b);
        for (int d = 0; d < it.n_out; ++d) it.outs[d][(long long)b * it.out_ld + grow] = v;
      }
    } else {
      slot[i] = v;
    }
  }
  if (!whole) {
    __threadfence();
    if (!ds.sync()) return false;
    // CTAs that own a part of this tile: those whose ranges meet [tile_unit0, tile_unit0 + nsb)
    const long long G = gridDim.x, U = p.total_units;
    const int c_first = (int)(((tile_unit0 + 1) * G - 1) / U);
    const int c_last = (int)(((tile_unit0 + it.nsb) * G - 1) / U);
    if (tid == 0) {
      unsigned int* counter = p.counters + it.tile_base + at.tile;
      const unsigned int old = atomicAdd(counter, 1u);
      const bool last = old == (unsigned)(c_last - c_first);
      if (last) *counter = 0u;  // everybody else has arrived: ready for the next launch
      *ds.s_last = last ? 1 : 0;
    }
    if (!ds.sync()) return false;
    if (*ds.s_last) {
      __threadfence();
      // Every element this thread owns (up to 8: one per 256 of the nb x 128 sums) is the sum over the
      // CTAs of the tile in K order.  All loads of a batch of four CTAs are issued before any of them
      // is used: as a chain of dependent round trips to L2 this sum took tens of microseconds.
      constexpr int kOwn = 16 * kRows / kDrainThreads;
      const int own = (nb * kRows + kDrainThreads - 1) / kDrainThreads;
      float v[kOwn];
#pragma unroll
      for (int j = 0; j < kOwn; ++j) v[j] = 0.f;
      for (int c0 = c_first; c0 <= c_last; c0 += 4) {
        float part[4][kOwn];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u;
          const long long range0 = (long long)c * U / G;
          const float* theirs = p.partials + ((size_t)2 * c + (range0 < tile_unit0 ? 1 : 0)) * kSlotFloats;
#pragma unroll
          for (int j = 0; j < kOwn; ++j) {
            const int i = tid + j * kDrainThreads;
            part[u][j] = (c <= c_last && j < own && i < nb * kRows) ? __ldcg(theirs + i) : 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int j = 0; j < kOwn; ++j) v[j] += part[u][j];
      }
#pragma unroll
      for (int j = 0; j < kOwn; ++j) {
        const int i = tid + j * kDrainThreads;
        if (j >= own || i >= nb * kRows) continue;
        const int b = i >> 7, r = i & (kRows - 1);
        const long long grow = (long long)at.tile * kRows + r;
        if (b >= it.m || grow >= it.n) continue;
        const float out = v[j] * __ldg(it.unscale + b);
        for (int d = 0; d < it.n_out; ++d) it.outs[d][(long long)b * it.out_ld + grow] = out;
      }
    }
  }
  return ds.sync();  // the staging buffer may be overwritten by the next segment
}

// What the producer tells the other warps about the unit in a ring stage.
struct StageMeta {
  int item, tile, sb;
  int seg_end;  // the unit is the last one of its row tile that this CTA owns
};

template <int FMT>
__global__ void __launch_bounds__(kThreads, 1) gemv_tc_kernel(const __grid_constant__ TcParams p) {
  using F = TcFormat<FMT>;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kMaxStagesTc;     // the MMAs of a unit have completed and every reader is done with its stage
  uint64_t* a_ready = empty + kMaxStagesTc;  // [2] decode warps -> MMA: an A buffer is complete
  uint64_t* d_ready = a_ready + 2;           // [2] MMA -> drain and decode warps: the accumulators are final, the A buffer is free
  uint64_t* d_free = d_ready + 2;            // [2] drain warps -> MMA: the accumulators have been read
  uint64_t* cbar = d_free + 2;               // drain warps among themselves
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 512);
  volatile int* abort = reinterpret_cast<volatile int*>(smem + 516);
  volatile int* s_last = reinterpret_cast<volatile int*>(smem + 520);
  StageMeta* meta = reinterpret_cast<StageMeta*>(smem + 640);  // [kMaxStagesTc]
  const uint32_t stage0 = ptx::smem_addr(smem) + kSmemHeader;
  const uint32_t meta0 = ptx::smem_addr(smem) + 640;
  float* red = reinterpret_cast<float*>(smem + kSmemHeader + p.stages * p.stage_bytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  TC_WALL(threadIdx.x == 0, 0);
  const int S = p.stages;
  const int u0 = (int)((long long)blockIdx.x * p.total_units / gridDim.x);
  const int u1 = (int)((long long)(blockIdx.x + 1) * p.total_units / gridDim.x);
  const int count = u1 - u0;
  constexpr int kWTileBytes = kRows * F::kBoxBytes;
  constexpr int kXTileBytes = F::kXTileBytes;
  constexpr int kSub = F::kSub;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], kSub + kDecodeWarps + kDrainWarps);  // one commit per sub-unit
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&a_ready[b], kDecodeWarps);
      ptx::mbar_init(&d_ready[b], 1);
      ptx::mbar_init(&d_free[b], kDrainWarps);
    }
    ptx::mbar_init(cbar, kDrainWarps);
    *abort = 0;
    *s_last = 0;
    ptx::fence_mbar_init();
    // the next kernel on the stream (the conversion of the next list's activations) may start early
    ptx::grid_launch_dependents();
  }
  if (warp == kMmaWarp) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == kProducerWarp) {
    // ---------------- producer: one TMA box of raw blocks + one activation tile per unit ----------------
    if (lane == 0 && count > 0) {
      for (int i = 0; i < p.n_items; ++i) ptx::prefetch_tensormap(&p.wmap[i]);
      const Cursor first = locate(p, u0);
      // what the readers of a stage need to know about its unit; published by the arrive that follows
      auto describe = [&](int s, const Cursor& c, int idx) {
        StageMeta m;
        m.item = c.item;
        m.tile = c.tile;
        m.sb = c.sb;
        m.seg_end = (idx == count - 1 || c.sb == p.item[c.item].nsb - 1) ? 1 : 0;
        meta[s] = m;
      };
      // Weights never depend on the kernel before this one, activations do: fill the ring with
      // weights, then wait for that kernel, then fetch the activation tiles of those stages.
      const int pre = count < S ? count : S;
      Cursor c = first;
      for (int i = 0; i < pre; ++i) {
        describe(i, c, i);
        ptx::mbar_arrive_expect_tx(&full[i], (uint32_t)(kWTileBytes + kXTileBytes));
        ptx::tma_load_2d(smem + kSmemHeader + i * p.stage_bytes, &p.wmap[c.item], F::box_x(c.sb), c.tile * kRows,
                         &full[i]);
        advance(p, c);
      }
      ptx::grid_dependency_wait();
      TC_WALL(true, 1);
      if (p.sync & kPeerWait) {
        // until every peer has signalled as often as this rank has (their stores into buffers this
        // list reads have landed); bounded
        const unsigned int* mine = p.pads[p.rank];
        const unsigned int expected = *reinterpret_cast<const volatile unsigned int*>(mine + 32);
        const unsigned long long t0 = ptx::global_timer_ns();
        for (int peer = 0; peer < p.world; ++peer) {
          if (peer == p.rank) continue;
          for (;;) {
            unsigned int seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + peer) : "memory");
            if ((int)(seen - expected) >= 0) break;
            if (ptx::global_timer_ns() - t0 > p.wait_limit_ns) {
              report_timeout(0x80000u | (unsigned)peer);
              break;
            }
            __nanosleep(100);
          }
        }
        asm volatile("fence.proxy.async.global;" ::: "memory");
      }
      Cursor c2 = first;
      for (int i = 0; i < pre; ++i) {
        ptx::bulk_g2s(smem + kSmemHeader + i * p.stage_bytes + kWTileBytes,
                      p.item[c2.item].xprep + (size_t)c2.sb * kXTileBytes, kXTileBytes, &full[i]);
        advance(p, c2);
      }
      for (int idx = pre; idx < count; ++idx) {
        const int s = idx % S;
        if (!wait_bar(&empty[s], ((idx / S) - 1) & 1, abort, 0x10000u | (unsigned)s)) break;
        TC_STAMP(true, idx, 0);
        uint8_t* dst = smem + kSmemHeader + s * p.stage_bytes;
        describe(s, c, idx);
        ptx::mbar_arrive_expect_tx(&full[s], (uint32_t)(kWTileBytes + kXTileBytes));
        ptx::tma_load_2d(dst, &p.wmap[c.item], F::box_x(c.sb), c.tile * kRows, &full[s]);
        ptx::bulk_g2s(dst + kWTileBytes, p.item[c.item].xprep + (size_t)c.sb * kXTileBytes, kXTileBytes, &full[s]);
        advance(p, c);
      }
    }
  } else if (warp >= kMmaWarp) {
    // ---------------- MMA issuers ----------------
    // Two threads (in warps of different schedulers) take alternate sub-units, i.e. one accumulator
    // set and one A buffer each: the waits and commits one of them executes around its batch of MMAs
    // (several hundred cycles, during which its own MMAs have long drained from the pipe) overlap
    // the other one's MMAs.
    {
      uint32_t idesc;
      asm volatile("mov.b32 %0, %1;" : "=r"(idesc) : "n"(kIdesc));
      const uint32_t leader = lane == 0 ? 1u : 0u;  // the one lane that issues and commits
      const int which = warp - kMmaWarp;
      constexpr int kAdvance = 2 / kSub;  // stages between two sub-units of one issuer
      static_assert(kSub == 1 || kSub == 2, "a staged block is one or two sub-units");
      int s = (which / kSub) % S, full_phase = 0;
      for (int step = which; step < count * kSub; step += 2) {
        const int idx = step / kSub, sub = step % kSub;
        TC_STAMP(which == 0 && leader, idx, 8);
        if (!wait_bar(&full[s], full_phase, abort, 0x20000u | (unsigned)s)) break;
        TC_STAMP(which == 0 && leader, idx, 9);
        const uint64_t xdesc = desc_kmajor(stage0 + s * p.stage_bytes + kWTileBytes);
        const int buf = step & 1, use = step >> 1;
        if (!wait_bar(&a_ready[buf], use & 1, abort, 0x30000u)) break;
        TC_STAMP(which == 0 && leader, idx, 10);
        if (use > 0 && !wait_bar(&d_free[buf], (use - 1) & 1, abort, 0x40000u)) break;
        TC_STAMP(leader, idx, 1);
        ptx::tc_fence_after();
        F::issue(tmem + kColD + buf * kBufCols, tmem + kColA + buf * kBufCols, xdesc, sub, idesc, leader);
        umma_commit_if(&empty[s], leader);
        umma_commit_if(&d_ready[buf], leader);
        TC_STAMP(leader, idx, 2);
        __syncwarp();
        s += kAdvance;
        if (s >= S) {
          s -= S;
          full_phase ^= 1;
        }
      }
    }
  } else if (warp < kDecodeWarps) {
    // ---------------- decode warps: raw blocks -> fp16 A operand in tensor memory ----------------
    const int part = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int tid = threadIdx.x;
    int s = 0, full_phase = 0, step = 0;  // step counts sub-units
    bool ok = true;
    for (int idx = 0; idx < count && ok; ++idx) {
      if (!wait_bar(&full[s], full_phase, abort, 0x70000u | (unsigned)s)) break;
      TC_STAMP(tid == 0, idx, 3);
      TC_STAMP(tid == 15 * 32, idx, 13);
      TC_WALL(tid == 0 && idx == 0, 2);
      const uint32_t stage = stage0 + s * p.stage_bytes;
      int offset = 0;
      if constexpr (FMT == kQ6_K) {
        int sb;
        asm volatile("ld.shared.s32 %0, [%1];" : "=r"(sb) : "r"(meta0 + 16 * s + 8));
        offset = F::box_offset(sb);
      }
#pragma unroll
      for (int sub = 0; sub < kSub; ++sub, ++step) {
        const int buf = step & 1, use = step >> 1;
        // the MMAs that read this A buffer two sub-units ago have completed
        if (use > 0 && !wait_bar(&d_ready[buf], (use - 1) & 1, abort, 0x60000u)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        F::decode(stage + row * F::kBoxBytes, part, sub, offset, tmem + lane_base + kColA + buf * kBufCols);
        tmem_st_wait();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&a_ready[buf]);
        TC_STAMP(tid == 0, idx, 4);
        TC_STAMP(tid == 15 * 32, idx, 12);
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&empty[s]);  // this warp is done with the stage
      if (++s == S) {
        s = 0;
        full_phase ^= 1;
      }
    }
  } else {
    // ---------------- drain warps: accumulators -> scaled running sums -> outputs ----------------
    const int dw = warp - kDecodeWarps;
    const int half = dw >> 2, quarter = dw & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int tid = threadIdx.x - kDecodeThreads;  // 0 .. 255
    ptx::grid_dependency_wait();  // outputs and scratch may still be in use by the kernel before
    DecodeSync ds{cbar, abort, s_last, 0u};
    float acc[16];
#pragma unroll
    for (int b = 0; b < 16; ++b) acc[b] = 0.f;
    int seg_sb0 = -1;
    bool ok = true;
    int s = 0, full_phase = 0, step = 0;
    for (int idx = 0; idx < count && ok; ++idx) {
      if (!wait_bar(&full[s], full_phase, abort, 0x70000u | (unsigned)s)) break;
      const uint32_t stage = stage0 + s * p.stage_bytes;
      const uint4 mraw = ptx::lds128(meta0 + 16 * s);
      const Cursor at{(int)mraw.x, (int)mraw.y, (int)mraw.z};
      const bool seg_end = mraw.w != 0;
      if (seg_sb0 < 0) seg_sb0 = at.sb;
      const int nb = p.item[at.item].nb;
      const int offset = F::box_offset(at.sb);
      const uint32_t sums = stage + kWTileBytes + kXMainBytes;
#pragma unroll
      for (int sub = 0; sub < kSub; ++sub, ++step) {
        const int buf = step & 1, use = step >> 1;
        UnitScales sc[2];
        F::scales2(stage + row * F::kBoxBytes, half, sub, offset, sc);
        const int group = (F::kSumGroups / kSub) * sub + 4 * half;
        if (!wait_bar(&d_ready[buf], use & 1, abort, 0x60000u)) {
          ok = false;
          break;
        }
        TC_STAMP(tid == 0, idx, 5);
        ptx::tc_fence_after();
        const uint32_t d = tmem + lane_base + kColD + buf * kBufCols;
        switch (nb) {
          case 1: drain<1>(d, 2 * half, sc[0], acc); drain<1>(d, 2 * half + 1, sc[1], acc); break;
          case 2: drain<2>(d, 2 * half, sc[0], acc); drain<2>(d, 2 * half + 1, sc[1], acc); break;
          case 4: drain<4>(d, 2 * half, sc[0], acc); drain<4>(d, 2 * half + 1, sc[1], acc); break;
          case 8: drain<8>(d, 2 * half, sc[0], acc); drain<8>(d, 2 * half + 1, sc[1], acc); break;
          default: drain<16>(d, 2 * half, sc[0], acc); drain<16>(d, 2 * half + 1, sc[1], acc); break;
        }
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&d_free[buf]);  // the tensor core may overwrite this accumulator set
        // the Sx terms need nothing from the tensor core: they come after it has been released
        switch (nb) {
          case 1: correct<1>(sums, group, sc[0], acc); correct<1>(sums, group + 2, sc[1], acc); break;
          case 2: correct<2>(sums, group, sc[0], acc); correct<2>(sums, group + 2, sc[1], acc); break;
          case 4: correct<4>(sums, group, sc[0], acc); correct<4>(sums, group + 2, sc[1], acc); break;
          case 8: correct<8>(sums, group, sc[0], acc); correct<8>(sums, group + 2, sc[1], acc); break;
          default: correct<16>(sums, group, sc[0], acc); correct<16>(sums, group + 2, sc[1], acc); break;
        }
        TC_STAMP(tid == 0, idx, 6);
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&empty[s]);  // this warp is done with the stage
      if (seg_end) {
        // this thread's sums of the segment -> staging buffer, then the CTA-wide part
#pragma unroll
        for (int b = 0; b < 16; ++b) {
          if (b < nb) red[(half * nb + b) * kRows + row] = acc[b];
          acc[b] = 0.f;
        }
        ok = finish_segment(p, at, seg_sb0, u0, red, ds);
        seg_sb0 = -1;
      }
      if (++s == S) {
        s = 0;
        full_phase ^= 1;
      }
    }
    TC_WALL(tid == 0, 3);
#ifdef TB200_TC_TRACE
    if (p.trace && tid == 0) atomicMax(reinterpret_cast<unsigned long long*>(p.trace + 63 * 16 + 7), (unsigned long long)ptx::global_timer_ns());
#endif
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    if (*abort && lane == 0) {
      // a wait gave up: let copies that may still be in flight land before the CTA's memory is reused
      const unsigned long long t = ptx::global_timer_ns();
      while (ptx::global_timer_ns() - t < 50000ull) {
      }
    }
    __syncwarp();
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
  TC_WALL(threadIdx.x == 0, 4);
#ifdef TB200_TC_TRACE
  if (p.trace && threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned long long*>(p.trace + 63 * 16 + 6), (unsigned long long)ptx::global_timer_ns());
#endif
  if (threadIdx.x == 0 && (p.sync & kPeerSignal)) {
    // every warp of this CTA has stored what it will store; the last CTA of the grid tells the peers
    unsigned int* mine = p.pads[p.rank];
    __threadfence();
    if (atomicAdd(mine + 34, 1u) == gridDim.x - 1) {
      __threadfence_system();
      mine[34] = 0u;
      const unsigned int epoch = mine[32] + 1u;
      mine[32] = epoch;
      for (int peer = 0; peer < p.world; ++peer)
        if (peer != p.rank)
          asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p.pads[peer] + p.rank), "r"(epoch) : "memory");
    }
  }
}

// ---- activation conversion ----------------------------------------------------------------------
// One CTA per (activation matrix, row b of 16).  Rows below m: find the row's largest magnitude,
// scale by the power of two that puts it in [2^9, 2^10), convert to fp16 and scatter into the tiles
// the GEMV copies; rows from m on are written as zeros.  A tile: [32 core columns of 8 k][16 rows][8 k]
// fp16, then the sums of the converted values over each 32-value scale group as fp32 [8 groups][16 rows].
struct PrepX {
  const uint16_t* x;
  uint8_t* xprep;
  float* unscale;
  int m, k;
};
struct PrepArgs {
  PrepX x[kTcMaxItems];
#ifdef TB200_TC_TRACE
  long long* trace;
#endif
};
#ifdef TB200_TC_TRACE
#define PREP_WALL(slot) do { if (a.trace && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) a.trace[63 * 16 + (slot)] = (long long)ptx::global_timer_ns(); } while (0)
#else
#define PREP_WALL(slot) do { } while (0)
#endif

constexpr int kPrepThreads = 1024;
constexpr int kPrepHeld = 3;  // 16-byte chunks a thread keeps in registers between the two passes over a row

template <int FMT, bool F16>
__global__ void __launch_bounds__(kPrepThreads) gemv_tc_prepare_kernel(const PrepArgs a) {
  constexpr int kXTileBytes = TcFormat<FMT>::kXTileBytes;
  constexpr int kSumGroups = TcFormat<FMT>::kSumGroups;
  __shared__ uint32_t s_max[kPrepThreads / 32];
  const PrepX px = a.x[blockIdx.y];
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
  PREP_WALL(8);
  if (tid == 0) ptx::grid_launch_dependents();  // the GEMV behind fills its weight ring meanwhile
  ptx::grid_dependency_wait();                   // the GEMV before may still read these tiles
  PREP_WALL(9);
  const int chunks = px.k >> 3;                  // 8 values = 16 bytes; a multiple of 32
  if (b >= px.m) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int c = tid; c < chunks; c += kPrepThreads) {
      const int j = c >> 5, k8 = c & 31;
      *reinterpret_cast<uint4*>(px.xprep + (size_t)j * kXTileBytes + k8 * 256 + b * 16) = zero;
      if (k8 < kSumGroups) *reinterpret_cast<float*>(px.xprep + (size_t)j * kXTileBytes + kXMainBytes + k8 * 64 + b * 4) = 0.f;
    }
    if (tid == 0) px.unscale[b] = 1.f;
    return;
  }
  // First pass: the row's largest magnitude.  Rows of up to kPrepHeld * kPrepThreads chunks (24576
  // values) are read once, all loads in flight together, and stay in registers for the second pass:
  // a loop of dependent round trips to memory was most of this kernel's time on long rows.
  const uint16_t* xr = px.x + (size_t)b * px.k;
  const bool held = chunks <= kPrepHeld * kPrepThreads;
  uint4 keep[kPrepHeld];
  uint32_t mx = 0;
  auto magnitude = [&](const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) mx = max(mx, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
  };
  if (held) {
#pragma unroll
    for (int i = 0; i < kPrepHeld; ++i) {
      const int c = tid + i * kPrepThreads;
      keep[i] = c < chunks ? *reinterpret_cast<const uint4*>(xr + (c << 3)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < kPrepHeld; ++i) magnitude(keep[i]);
  } else {
    for (int c = tid; c < chunks; c += kPrepThreads) magnitude(*reinterpret_cast<const uint4*>(xr + (c << 3)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) s_max[tid >> 5] = mx;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kPrepThreads / 32; ++i) mx = max(mx, s_max[i]);
  // biased exponent of the largest magnitude -> shift that lands it in [2^9, 2^10)
  const int e = F16 ? (int)(mx >> 10) : (int)(mx >> 7);
  const int bias = F16 ? 15 : 127, emax = F16 ? 31 : 255;
  int sh = 0;
  if (e > 0 && e < emax) sh = bias + 9 - e;
  sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
  const float scale = __uint_as_float((uint32_t)(sh + 127) << 23);
  if (tid == 0) px.unscale[b] = __uint_as_float((uint32_t)(127 - sh) << 23);

  // Second pass: chunk c of the row (a whole warp at a time: c < chunks is warp-uniform) -> its tile
  auto emit = [&](int c, const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float f[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (F16) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        f[2 * i] = t.x * scale;
        f[2 * i + 1] = t.y * scale;
      } else {
        f[2 * i] = __uint_as_float(w[i] << 16) * scale;
        f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u) * scale;
      }
    }
    __half h[8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      h[i] = __float2half_rn(f[i]);
      sum += __half2float(h[i]);
    }
    const int j = c >> 5, cc = c & 31;  // unit, chunk inside the unit: values 8 cc .. 8 cc + 7
    uint8_t* tile = px.xprep + (size_t)j * kXTileBytes;
    auto pack = [&](int lo, int hi) { return (uint32_t)__half_as_ushort(h[lo]) | ((uint32_t)__half_as_ushort(h[hi]) << 16); };
    if constexpr (FMT == kQ4_K) {
      // the four chunks of a 32-value scale group sit in four neighbouring lanes
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      // scale group g (low / high nibbles of a 32-byte quarter), core column k8; order inside each
      // 4-value word [x0, x2, x1, x3] (see TcFormat<kQ4_K>)
      const int quarter = cc >> 3, nib = (cc >> 2) & 1, i8 = cc & 3;
      const int g = 2 * quarter + nib;
      *reinterpret_cast<uint4*>(tile + (4 * g + i8) * 256 + b * 16) = make_uint4(pack(0, 2), pack(1, 3), pack(4, 6), pack(5, 7));
      if (i8 == 0) *reinterpret_cast<float*>(tile + kXMainBytes + g * 64 + b * 4) = sum;
    } else {
      // Q6_K: natural order; a 16-value scale group is two neighbouring chunks
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      *reinterpret_cast<uint4*>(tile + cc * 256 + b * 16) = make_uint4(pack(0, 1), pack(2, 3), pack(4, 5), pack(6, 7));
      if ((cc & 1) == 0) *reinterpret_cast<float*>(tile + kXMainBytes + (cc >> 1) * 64 + b * 4) = sum;
    }
  };
  if (held) {
#pragma unroll
    for (int i = 0; i < kPrepHeld; ++i) {
      const int c = tid + i * kPrepThreads;
      if (c < chunks) emit(c, keep[i]);
    }
  } else {
    for (int c = tid; c < chunks; c += kPrepThreads) emit(c, *reinterpret_cast<const uint4*>(xr + (c << 3)));
  }
  PREP_WALL(10);
}

inline long long round_up_ll(long long v, long long to) { return (v + to - 1) / to * to; }
inline int batch_columns(long long m) { return m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : m <= 8 ? 8 : 16; }

unsigned long long g_peer_wait_limit_ns = 2000000000ull;

}  // namespace

TB200_DEFINE_STATUS_READER(read_gemv_tc_status)

void set_peer_wait_limit_ns(unsigned long long ns) { g_peer_wait_limit_ns = ns ? ns : 2000000000ull; }
unsigned long long peer_wait_limit_ns() { return g_peer_wait_limit_ns; }

static int x_tile_bytes(int fmt) { return fmt == kQ6_K ? TcFormat<kQ6_K>::kXTileBytes : TcFormat<kQ4_K>::kXTileBytes; }
static int box_bytes(int fmt) { return fmt == kQ6_K ? TcFormat<kQ6_K>::kBoxBytes : TcFormat<kQ4_K>::kBoxBytes; }

#ifdef TB200_TC_TRACE
static long long* trace_buffer() {
    static long long* buffer = nullptr;  // device memory: stamps must not wait on a host-memory store
    if (!buffer) {
      cudaMalloc((void**)&buffer, 64 * 16 * 8);
      cudaMemset(buffer, 0, 64 * 16 * 8);
      atexit([] {
        static long long host[64 * 16];
        cudaMemcpy(host, buffer, sizeof(host), cudaMemcpyDeviceToHost);
        printf("unit: stage free | mma start, issued | warp0 data ready, A stored | acc ready, drained | mma thread: loop top, data seen, A seen | warp15 data ready, A stored\n");
        const long long t0 = host[3];
        const long long* w = host + 63 * 16;
        printf("wall clock (ns after prepare entry): prepare past wait %lld, prepare end %lld | gemv entry %lld, past wait %lld, first data %lld, loop end %lld, last loop end of any CTA %lld, exit %lld\n",
               w[9] - w[8], w[10] - w[8], w[0] - w[8], w[1] - w[8], w[2] - w[8], w[3] - w[8], w[7] - w[8], w[4] - w[8]);
        printf("last CTA to leave: %lld\n", w[6] - w[8]);
        for (int i = 0; i < 63 && host[i * 16 + 3]; ++i) {
          const long long* h = host + i * 16;
          printf("%3d: %7lld | %7lld %7lld | %7lld %7lld | %7lld %7lld | %7lld %7lld %7lld | %7lld %7lld\n", i, h[0] ? h[0] - t0 : 0,
                 h[1] - t0, h[2] - t0, h[3] - t0, h[4] - t0, h[5] - t0, h[6] - t0, h[8] - t0, h[9] - t0, h[10] - t0, h[13] - t0, h[12] - t0);
        }
      });
    }
    return buffer;
}
#endif

bool gemv_tc_supported(int fmt, int xt, long long m, long long n, long long k) {
  if (fmt != kQ4_K && fmt != kQ6_K) return false;
  if (xt != kBF16 && xt != kF16) return false;
  if (m < 1 || m > 16 || n < 1 || k < kUnitK || k % kUnitK) return false;
  if (row_bytes(fmt, k) % 16) return false;
  if (n > (1ll << 30) || k > (1ll << 24)) return false;
  return true;
}

// Scratch layout of a list: arrival counters (one per row tile), partial-sum slots (two per CTA),
// then per distinct activation matrix its tiles and its 16 unscale factors.
struct TcLayout {
  long long counters = 0, partials = 0, x_base = 0, total = 0;
  long long x_offset[kTcMaxItems], unscale_offset[kTcMaxItems];
  int grid = 0, total_units = 0, total_tiles = 0;
};
static bool tc_layout(const TcLaunchItem* items, int count, const DeviceInfo& dev, TcLayout& L) {
  if (count < 1 || count > kTcMaxItems) return false;
  long long units = 0, tiles = 0;
  for (int i = 0; i < count; ++i) {
    const TcLaunchItem& it = items[i];
    if (!gemv_tc_supported(it.fmt, it.xt, it.m, it.n, it.k) || it.fmt != items[0].fmt) return false;
    if (it.x_share >= i) return false;
    if (it.x_share >= 0 && (items[it.x_share].k != it.k || items[it.x_share].m != it.m || items[it.x_share].xt != it.xt))
      return false;
    const long long rt = (it.n + kRows - 1) / kRows;
    units += rt * (it.k / kUnitK);
    tiles += rt;
  }
  if (units > 0x7fffffffLL) return false;
  L.total_units = (int)units;
  L.total_tiles = (int)tiles;
  L.grid = (int)(units < dev.sm_count ? units : dev.sm_count);
  L.counters = 0;
  L.partials = round_up_ll(tiles * 4, 256);
  long long off = L.partials + (long long)L.grid * 2 * kSlotFloats * 4;
  for (int i = 0; i < count; ++i) {
    if (items[i].x_share >= 0) {
      L.x_offset[i] = L.x_offset[items[i].x_share];
      L.unscale_offset[i] = L.unscale_offset[items[i].x_share];
      continue;
    }
    L.x_offset[i] = off;
    off += round_up_ll(items[i].k / kUnitK * (long long)x_tile_bytes(items[i].fmt), 256);
    L.unscale_offset[i] = off;
    off += 256;
  }
  L.total = off;
  return true;
}

long long gemv_tc_scratch_bytes(const TcLaunchItem* items, int count, const DeviceInfo& dev) {
  TcLayout L;
  return tc_layout(items, count, dev, L) ? L.total : 0;
}

cudaError_t launch_gemv_tc(const TcLaunchItem* items, int count, void* scratch, long long scratch_bytes,
                           cudaStream_t stream, const PeerSync* peers) {
  cudaError_t e;
  const DeviceInfo* dev = device_info(&e);
  if (!dev) return e;
  TcLayout L;
  if (!tc_layout(items, count, *dev, L)) return cudaErrorInvalidValue;
  if (!scratch || scratch_bytes < L.total || (reinterpret_cast<uintptr_t>(scratch) & 255)) return cudaErrorInvalidValue;
  uint8_t* base = static_cast<uint8_t*>(scratch);

  // ---- activations -> fp16 tiles (one small kernel for the whole list) ----
  PrepArgs prep{};
#ifdef TB200_TC_TRACE
  prep.trace = trace_buffer();
#endif
  int n_x = 0;
  for (int i = 0; i < count; ++i) {
    if (items[i].x_share >= 0) continue;
    PrepX& px = prep.x[n_x++];
    px.x = static_cast<const uint16_t*>(items[i].x);
    px.xprep = base + L.x_offset[i];
    px.unscale = reinterpret_cast<float*>(base + L.unscale_offset[i]);
    px.m = (int)items[i].m;
    px.k = (int)items[i].k;
    if (items[i].xt != items[0].xt) return cudaErrorInvalidValue;
  }
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(16, (unsigned)n_x);
    cfg.blockDim = dim3(kPrepThreads);
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const bool f16 = items[0].xt == kF16;
    if (items[0].fmt == kQ6_K)
      e = f16 ? cudaLaunchKernelEx(&cfg, gemv_tc_prepare_kernel<kQ6_K, true>, prep)
              : cudaLaunchKernelEx(&cfg, gemv_tc_prepare_kernel<kQ6_K, false>, prep);
    else
      e = f16 ? cudaLaunchKernelEx(&cfg, gemv_tc_prepare_kernel<kQ4_K, true>, prep)
              : cudaLaunchKernelEx(&cfg, gemv_tc_prepare_kernel<kQ4_K, false>, prep);
    if (e != cudaSuccess) return e;
  }

  // ---- the list ----
  TcParams p;
  memset(&p, 0, sizeof(p));
  int unit_base = 0, tile_base = 0, max_nb = 1;
  for (int i = 0; i < count; ++i) {
    const TcLaunchItem& src = items[i];
    TcItem& it = p.item[i];
    it.xprep = base + L.x_offset[i];
    it.unscale = reinterpret_cast<const float*>(base + L.unscale_offset[i]);
    if (src.out.count < 1 || src.out.count > kMaxOutputs || src.out.ld < src.n) return cudaErrorInvalidValue;
    for (int d = 0; d < src.out.count; ++d) it.outs[d] = src.out.ptr[d];
    it.n_out = src.out.count;
    it.out_ld = src.out.ld;
    it.n = src.n;
    it.m = (int)src.m;
    it.nb = batch_columns(src.m);
    max_nb = it.nb > max_nb ? it.nb : max_nb;
    it.nsb = (int)(src.k / kUnitK);
    it.row_tiles = (int)((src.n + kRows - 1) / kRows);
    it.unit_base = unit_base;
    it.tile_base = tile_base;
    unit_base += it.row_tiles * it.nsb;
    tile_base += it.row_tiles;
    const long long rb = row_bytes(src.fmt, src.k);
    if (!make_tensor_map_2d(&p.wmap[i], TmaType::kU64, src.w, (unsigned long long)rb / 8, (unsigned long long)src.n,
                            (unsigned long long)rb, box_bytes(src.fmt) / 8, kRows, false))
      return cudaErrorNotSupported;
  }
  p.n_items = count;
  p.total_units = L.total_units;
  p.stage_bytes = kRows * box_bytes(items[0].fmt) + x_tile_bytes(items[0].fmt);
  p.red_floats = kHalves * max_nb * kRows;
  const int spare = dev->max_smem_optin - kSmemHeader - p.red_floats * 4;
  p.stages = spare / p.stage_bytes;
  if (p.stages > kMaxStagesTc) p.stages = kMaxStagesTc;
  if (p.stages < 2) return cudaErrorInvalidValue;
  p.counters = reinterpret_cast<unsigned int*>(base + L.counters);
  p.partials = reinterpret_cast<float*>(base + L.partials);
  p.wait_limit_ns = g_peer_wait_limit_ns;
  if (peers && peers->flags) {
    if (peers->world < 1 || peers->world > kMaxOutputs || peers->rank < 0 || peers->rank >= peers->world)
      return cudaErrorInvalidValue;
    for (int i = 0; i < peers->world; ++i) p.pads[i] = peers->pads[i];
    p.rank = peers->rank;
    p.world = peers->world;
    p.sync = peers->flags;
  }
#ifdef TB200_TC_TRACE
  p.trace = trace_buffer();
#endif
  auto kernel = items[0].fmt == kQ6_K ? gemv_tc_kernel<kQ6_K> : gemv_tc_kernel<kQ4_K>;
  e = allow_full_shared_memory(kernel);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)L.grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = (size_t)(kSmemHeader + p.stages * p.stage_bytes + p.red_floats * 4);
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

}  // namespace tb200
