// Batch-1 decode GEMV for Q6_K, Q8_0, Q4_0 and Q4_K on the integer dot-product units:
// out[n] = sum_k dequant(w[n, k]) * x[k].
//
// Replaces the reference's `gemv_packed` (benchmarks/kernels/showcase/kernels.py:116-119) at batch 1, where no
// tensor-core form pays for these formats: at one activation row an MMA wastes all but one of its columns, the
// 6-bit decode of Q6_K costs more than the dot product itself, and Q8_0 weights are 8-bit integers already.
//
// Regime: HBM-bound, so everything serves streaming the raw blocks (Q6_K below; the other formats differ in
// the unpacking only) with as few instructions per weight as possible, all of them exact.
//
//  * Activations as 8-bit integers, without rounding: the CTA converts all K activations once.  Every
//    run of 32 values is scaled by the power of two that puts its largest magnitude in [32, 64); 2^14 times
//    the scaled value, rounded to an integer q of at most 21 bits, is split into three signed limbs of 7 + 7
//    + 7 bits, q = l0 2^14 + l1 2^7 + l2 (exact for every value within 2^-12 of the run's largest, within
//    2^-21 of it in absolute terms otherwise).
//  * Weights as unsigned bytes, nibble | bit pair << 4 four at a time; the offset of 32 (8 for Q4_0) is taken
//    out in integers against the limb sums of the activations: sum (q - 32) x = sum q x - 32 sum x.
//  * `dp4a` (four 8-bit products per lane and instruction) against each limb, int32 sums per
//    16-weight scale group; the limbs are joined with two shifts, and d * scale is applied in fp32.
//  * A warp owns eight consecutive blocks of every row it takes (1680 bytes, a multiple of 16): it copies
//    them into shared memory with 16-byte asynchronous copies, three rows ahead, perfectly coalesced
//    whatever the 2-byte alignment of the blocks; four lanes share a block (64 weights each: both
//    nibbles of 32 `ql` bytes) and read it back through aligned words and a funnel shift of 0 or 16 bits.
//    The lanes keep their 64 activations (48 registers of limbs) for the whole launch.
//  * The warps that share a row meet every eight rows (hardware named barrier) and add their sums in
//    warp order: deterministic, no scratch, no atomics.
//  * N-sharded launches: the sums go to the same columns of every rank's output (peer stores), one thread
//    per CTA waits (bounded) for the peers' signal before the activations are read, the last CTA signals.
#include <cuda_fp16.h>

#include <cstdint>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tb200 {
namespace {

constexpr int kMaxWarps = 16;               // warps per CTA at most
constexpr int kSegBlocks = 8;               // 256-weight blocks of a row one warp takes: 8 x 210 = 1680, 8 x 144 = 1152 or 8 x 272 = 2176 bytes, multiples of 16
constexpr int kStages = 3;                  // row segments in flight per warp
// bytes of 256 weights: one Q6_K or Q4_K block, eight Q8_0 or Q4_0 blocks
__host__ __device__ constexpr int dp_block_bytes(int fmt) { return fmt == kQ6_K ? 210 : fmt == kQ8_0 ? 272 : 144; }
constexpr int kBatch = 8;                   // rows between two meetings of the warps that share a row

struct DpArgs {
  const uint16_t* x;   // [k] bf16 or fp16
  const uint8_t* w;    // [n, k] raw Q6_K blocks
  float* outs[kMaxOutputs];
  int n_out;
  long long row_bytes;
  int n, k, nsb, warps_per_row, streams, rows_per_cta;
  // N-sharded launches: signal pads of all ranks (this rank's own is waited on), what to do, and for how long
  unsigned int* pads[kMaxOutputs];
  int rank, world, sync;
  unsigned long long wait_limit_ns;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void stream_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// 32 bytes of shared memory from a 2-byte aligned address: nine aligned words, re-joined by a funnel shift of
// 0 or 16 bits (the same code for every lane; only the shift differs)
__device__ __forceinline__ void lds32_unaligned(uint32_t addr, uint32_t shift, uint32_t (&out)[8]) {
  const uint32_t base = addr & ~3u;
  uint32_t w[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[i]) : "r"(base + 4 * i));
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = __funnelshift_r(w[i], w[i + 1], shift);
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}

// four unsigned bytes against four signed bytes
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int join_limbs(const int (&s)[3]) { return (s[0] << 14) + (s[1] << 7) + s[2]; }

// This lane's 64 weights of one staged block against its activations.  `blk`: the block in shared memory; h, jj:
// which 32 `ql` bytes (64 h + 32 jj) the lane owns.  xa / xb: limbs of the activations that meet the low / high
// nibbles; ua / ub: the factors that undo their scales; ca / cb: 32 x the joined limb sums of the four 16-value
// groups (the weights stay unsigned, q = nibble | bit pair << 4, and sum (q - 32) x = sum q x - 32 sum x, all in
// integers).  The bit pairs reach bits 4-5 of their bytes by one rotation of the `qh` word.
__device__ __forceinline__ float block_part(uint32_t blk, uint32_t shift, int h, int jj, const uint32_t (&xa)[3][8],
                                            const uint32_t (&xb)[3][8], float ua, float ub, const int (&ca)[2],
                                            const int (&cb)[2]) {
  uint32_t ql[8], qh[8];
  lds32_unaligned(blk + 64 * h + 32 * jj, shift, ql);
  lds32_unaligned(blk + 128 + 32 * h, shift, qh);
  const uint32_t sca = lds_u16(blk + 192 + 8 * h + 2 * jj);      // scales of the two groups of the low nibbles
  const uint32_t scb = lds_u16(blk + 192 + 8 * h + 2 * jj + 4);  // ... of the high nibbles
  const float d = __half2float(__ushort_as_half((unsigned short)lds_u16(blk + 208)));
  int sa[2][3] = {{0, 0, 0}, {0, 0, 0}}, sb[2][3] = {{0, 0, 0}, {0, 0, 0}};
  const uint32_t rot_a = (uint32_t)(2 * jj + 28) & 31u, rot_b = (uint32_t)(2 * jj);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t qa = (ql[i] & 0x0F0F0F0Fu) | (__funnelshift_r(qh[i], qh[i], rot_a) & 0x30303030u);
    const uint32_t qb = ((ql[i] >> 4) & 0x0F0F0F0Fu) | (__funnelshift_r(qh[i], qh[i], rot_b) & 0x30303030u);
    const int g = i >> 2;  // words 0..3: the first 16 weights of the run, one scale group
#pragma unroll
    for (int l = 0; l < 3; ++l) {
      sa[g][l] = dp4a_us(qa, xa[l][i], sa[g][l]);
      sb[g][l] = dp4a_us(qb, xb[l][i], sb[g][l]);
    }
  }
  float ta = 0.f, tb = 0.f;
#pragma unroll
  for (int g = 0; g < 2; ++g) {
    const int ja = join_limbs(sa[g]) - ca[g];
    const int jb = join_limbs(sb[g]) - cb[g];
    ta = fmaf((float)(int)(signed char)((sca >> (8 * g)) & 0xFF), (float)ja, ta);
    tb = fmaf((float)(int)(signed char)((scb >> (8 * g)) & 0xFF), (float)jb, tb);
  }
  return d * (ta * ua + tb * ub);
}

// Q8_0: the lane owns two 34-byte blocks (fp16 d, 32 signed bytes) at `part` = block + 68 * (lane % 4), a 4-byte
// aligned address: the first block's quants sit 2 bytes off the word grid, the second block's on it.
__device__ __forceinline__ float block_part_q80(uint32_t part, const uint32_t (&xa)[3][8], const uint32_t (&xb)[3][8],
                                                float ua, float ub) {
  uint32_t w[17];
#pragma unroll
  for (int i = 0; i < 17; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[i]) : "r"(part + 4 * i));
  int sa[3] = {0, 0, 0}, sb[3] = {0, 0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t qa = __funnelshift_r(w[i], w[i + 1], 16), qb = w[9 + i];
#pragma unroll
    for (int l = 0; l < 3; ++l) {
      sa[l] = __dp4a((int)qa, (int)xa[l][i], sa[l]);
      sb[l] = __dp4a((int)qb, (int)xb[l][i], sb[l]);
    }
  }
  const float d0 = __half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu)));
  const float d1 = __half2float(__ushort_as_half((unsigned short)(w[8] >> 16)));
  return d0 * ((float)join_limbs(sa) * ua) + d1 * ((float)join_limbs(sb) * ub);
}

// Q4_0: two 18-byte blocks (fp16 d, 16 bytes: low nibbles = weights 0..15, high nibbles = weights 16..31, each
// minus 8) at `part` = block + 36 * (lane % 4); ca / cb: 8 x the joined limb sums of the two runs.
__device__ __forceinline__ float block_part_q40(uint32_t part, const uint32_t (&xa)[3][8], const uint32_t (&xb)[3][8],
                                                float ua, float ub, int ca, int cb) {
  uint32_t w[9];
#pragma unroll
  for (int i = 0; i < 9; ++i) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[i]) : "r"(part + 4 * i));
  int sa[3] = {0, 0, 0}, sb[3] = {0, 0, 0};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t qa = __funnelshift_r(w[i], w[i + 1], 16), qb = w[5 + i];
    const uint32_t qa_lo = qa & 0x0F0F0F0Fu, qa_hi = (qa >> 4) & 0x0F0F0F0Fu;
    const uint32_t qb_lo = qb & 0x0F0F0F0Fu, qb_hi = (qb >> 4) & 0x0F0F0F0Fu;
#pragma unroll
    for (int l = 0; l < 3; ++l) {
      sa[l] = dp4a_us(qa_lo, xa[l][i], sa[l]);
      sa[l] = dp4a_us(qa_hi, xa[l][4 + i], sa[l]);
      sb[l] = dp4a_us(qb_lo, xb[l][i], sb[l]);
      sb[l] = dp4a_us(qb_hi, xb[l][4 + i], sb[l]);
    }
  }
  const float d0 = __half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu)));
  const float d1 = __half2float(__ushort_as_half((unsigned short)(w[4] >> 16)));
  return d0 * ((float)(join_limbs(sa) - ca) * ua) + d1 * ((float)(join_limbs(sb) - cb) * ub);
}

// The same for a Q4_K block: the lane owns quant bytes 32 p .. 32 p + 31, whose low nibbles are scale group 2 p
// and whose high nibbles are group 2 p + 1; sxa / sxb: the sums of the activations that meet them (for the
// dmin * min terms).  The 6-bit scales and mins come out of the 12 packed bytes with per-lane sources, shifts
// and masks, so that lanes of the lower and the upper half of a block run the same code.
struct Q4Lane {
  int p;
  bool upper;          // groups 4..7: low four bits in bytes 8..11, high two bits on top of bytes 0..7
  uint32_t sh, m_lo, m_hi;
};
__device__ __forceinline__ float block_part_q4k(uint32_t blk, const Q4Lane& ln, const uint32_t (&xa)[3][8],
                                                const uint32_t (&xb)[3][8], float ua, float ub, float sxa, float sxb) {
  const uint4 hdr = ptx::lds128(blk);
  const uint4 q0 = ptx::lds128(blk + 16 + 32 * ln.p), q1 = ptx::lds128(blk + 32 + 32 * ln.p);
  const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
  int sa[3] = {0, 0, 0}, sb[3] = {0, 0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t lo = words[i] & 0x0F0F0F0Fu, hi = (words[i] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
    for (int l = 0; l < 3; ++l) {
      sa[l] = __dp4a((int)lo, (int)xa[l][i], sa[l]);
      sb[l] = __dp4a((int)hi, (int)xb[l][i], sb[l]);
    }
  }
  // scales / mins of groups 2p (low nibbles) and 2p + 1 (high nibbles)
  const uint32_t sc_src = ln.upper ? hdr.w : hdr.y, mn_src = ln.upper ? (hdr.w >> 4) : hdr.z;
  const uint32_t sc_lo = ((sc_src >> ln.sh) & ln.m_lo) | (((hdr.y >> (ln.sh + 6)) & ln.m_hi) << 4);
  const uint32_t sc_hi = ((sc_src >> (ln.sh + 8)) & ln.m_lo) | (((hdr.y >> (ln.sh + 14)) & ln.m_hi) << 4);
  const uint32_t mn_lo = ((mn_src >> ln.sh) & ln.m_lo) | (((hdr.z >> (ln.sh + 6)) & ln.m_hi) << 4);
  const uint32_t mn_hi = ((mn_src >> (ln.sh + 8)) & ln.m_lo) | (((hdr.z >> (ln.sh + 14)) & ln.m_hi) << 4);
  const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));  // d, dmin
  const int ja = (sa[0] << 14) + (sa[1] << 7) + sa[2];
  const int jb = (sb[0] << 14) + (sb[1] << 7) + sb[2];
  const float dots = (float)sc_lo * ((float)ja * ua) + (float)sc_hi * ((float)jb * ub);
  const float mins = (float)mn_lo * sxa + (float)mn_hi * sxb;
  return dd.x * dots - dd.y * mins;
}

// Shared memory: limbs of all K activations [3][k], the factors of their runs of 32 [k / 32], the sums of the
// runs and the integer limb sums of the groups of 16 (for mins and offsets), the sums the warps of a row
// exchange, then per warp kStages row segments.
template <int FMT, bool F16>
__global__ void __launch_bounds__(kMaxWarps * 32, 1) gemv_dp4a_kernel(const DpArgs a) {
  constexpr int kBlockBytes = dp_block_bytes(FMT);
  constexpr int kSegBytes = kSegBlocks * kBlockBytes;
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* xl = smem;                                                      // [3][k]
  float* unscale = reinterpret_cast<float*>(smem + 3 * (size_t)a.k);       // [k / 32]
  float* xsum = unscale + a.k / 32;                                        // [k / 32]: sums of the runs (Q4_K's min terms)
  int* jsum = reinterpret_cast<int*>(xsum + a.k / 32);                     // [k / 16]: joined limb sums of the groups of 16
  float* red = reinterpret_cast<float*>(jsum + a.k / 16);                  // [2][kMaxWarps][kBatch]
  uint8_t* stages = reinterpret_cast<uint8_t*>(red + 2 * kMaxWarps * kBatch);  // 16-byte aligned: k is a multiple of 2048
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int threads = blockDim.x;

  ptx::grid_launch_dependents();

  // ---- which rows and which eight blocks of them this warp streams ----
  const int stream = warp / a.warps_per_row, seg = warp % a.warps_per_row;
  const int row0 = blockIdx.x * a.rows_per_cta;
  const int row_end = min(a.n, row0 + a.rows_per_cta);
  const int my_rows = row0 + stream < row_end ? (row_end - row0 - stream + a.streams - 1) / a.streams : 0;
  const uint8_t* src0 = a.w + (size_t)(row0 + stream) * a.row_bytes + (size_t)seg * kSegBytes;
  const size_t row_step = (size_t)a.streams * a.row_bytes;
  const uint32_t stage0 = ptx::smem_addr(stages) + (uint32_t)warp * (kStages * kSegBytes);
  const int seg_blocks = min(kSegBlocks, a.nsb - kSegBlocks * seg);  // the last warp of a row may have fewer
  const int seg_chunks = seg_blocks * kBlockBytes / 16;               // a whole number: 8 x 210 or any number of 144
  auto fetch = [&](int i) {  // row i of this warp's sequence -> stage i % kStages (weights never depend on the kernel before)
    if (i < my_rows) {
      const uint8_t* src = src0 + (size_t)i * row_step;
      const uint32_t dst = stage0 + (uint32_t)(i % kStages) * kSegBytes;
#pragma unroll
      for (int c = 0; c < (kSegBytes / 16 + 31) / 32; ++c) {
        const int chunk = lane + 32 * c;
        if (chunk < seg_chunks) cp_async16(dst + 16 * chunk, src + 16 * chunk);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < kStages - 1; ++i) fetch(i);

  // ---- all K activations -> three 8-bit limbs per value (they may come from the kernel before) ----
  ptx::grid_dependency_wait();
  if (a.sync & kPeerWait) {
    // until every peer has signalled as often as this rank has: their stores into the activations this launch
    // reads have landed (bounded; gives up with status 0x80000 | peer)
    if (tid == 0) {
      const unsigned int* mine = a.pads[a.rank];
      const unsigned int expected = *reinterpret_cast<const volatile unsigned int*>(mine + 32);
      const unsigned long long t0 = ptx::global_timer_ns();
      for (int peer = 0; peer < a.world; ++peer) {
        if (peer == a.rank) continue;
        for (;;) {
          unsigned int seen;
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + peer) : "memory");
          if ((int)(seen - expected) >= 0) break;
          if (ptx::global_timer_ns() - t0 > a.wait_limit_ns) {
            report_timeout(0x80000u | (unsigned)peer);
            break;
          }
          __nanosleep(100);
        }
      }
    }
    __syncthreads();
  }
  for (int v0 = 8 * tid; v0 < a.k; v0 += 8 * threads) {
    const uint4 raw = *reinterpret_cast<const uint4*>(a.x + v0);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t mx = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) mx = max(mx, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));  // a run of 32 values is four neighbouring threads
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const int e = F16 ? (int)(mx >> 10) : (int)(mx >> 7);
    const int bias = F16 ? 15 : 127, emax = F16 ? 31 : 255;
    int sh = 0;
    if (e > 0 && e < emax) sh = bias + 5 - e;
    sh = sh > 112 ? 112 : (sh < -125 ? -125 : sh);  // both factors stay normal numbers; every finite bf16 run fits
    // value * 2^(sh + 14), rounded to an integer q of at most 21 bits: l2 and l1 are its two low groups of
    // seven bits read as signed numbers, l0 what is left, so q = l0 2^14 + l1 2^7 + l2 exactly
    const float scale14 = __uint_as_float((uint32_t)(sh + 14 + 127) << 23);
    // a run that holds a NaN or an infinity has no limbs: its factor makes every output NaN
    if ((tid & 3) == 0)
      unscale[v0 >> 5] = e >= emax ? __uint_as_float(0x7FC00000u) : __uint_as_float((uint32_t)(127 - sh - 14) << 23);
    uint32_t limb[3][2] = {{0u, 0u}, {0u, 0u}, {0u, 0u}};
    int joined = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float f;
      if constexpr (F16) {
        f = __half2float(__ushort_as_half((unsigned short)((w[i >> 1] >> (16 * (i & 1))) & 0xFFFFu)));
      } else {
        f = __uint_as_float((i & 1) ? (w[i >> 1] & 0xFFFF0000u) : (w[i >> 1] << 16));
      }
      const int q = __float2int_rn(f * scale14);
      const int l2 = (int)((uint32_t)q << 25) >> 25;
      const int q1 = (q - l2) >> 7;
      const int l1 = (int)((uint32_t)q1 << 25) >> 25;
      const int l0 = (q1 - l1) >> 7;
      joined = (int)((uint32_t)joined + (uint32_t)q);  // (a non-finite value saturates q; its run's factor is NaN)
      constexpr uint32_t kInsert[4] = {0x3214u, 0x3240u, 0x3410u, 0x4210u};  // byte 0 of the limb into byte i % 4
      limb[0][i >> 2] = __byte_perm(limb[0][i >> 2], (uint32_t)l0, kInsert[i & 3]);
      limb[1][i >> 2] = __byte_perm(limb[1][i >> 2], (uint32_t)l1, kInsert[i & 3]);
      limb[2][i >> 2] = __byte_perm(limb[2][i >> 2], (uint32_t)l2, kInsert[i & 3]);
    }
    float sum = (float)joined * (1.f / 16384.f);
#pragma unroll
    for (int l = 0; l < 3; ++l) *reinterpret_cast<uint2*>(xl + (size_t)l * a.k + v0) = make_uint2(limb[l][0], limb[l][1]);
    if constexpr (FMT == kQ6_K || FMT == kQ4_0) {
      joined += __shfl_xor_sync(0xffffffffu, joined, 1);  // a group of 16 values is two neighbouring threads
      if ((tid & 1) == 0) jsum[v0 >> 4] = joined;
    }
    if constexpr (FMT == kQ4_K) {
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if ((tid & 3) == 0) xsum[v0 >> 5] = e >= emax ? __uint_as_float(0x7FC00000u) : sum * __uint_as_float((uint32_t)(127 - sh) << 23);
    }
  }
  __syncthreads();

  // ---- this lane's 64 activations: a quarter (u4) of block 8 seg + lane / 4 of a row ----
  // Q6_K: `ql` bytes 64 h + 32 jj, whose low nibbles are elements 128 h + 32 jj .. and whose high nibbles are
  // the elements 64 further on.  Q4_K: quant bytes 32 u4 .., low nibbles = elements 64 u4 .., high = 32 further on.
  // Q8_0 / Q4_0: two blocks of 32, elements 64 u4 .. and 64 u4 + 32 ...
  const int bi = lane >> 2, u4 = lane & 3;
  const bool has_block = bi < seg_blocks;
  const int h = u4 >> 1, jj = u4 & 1;
  const int block0 = 256 * (kSegBlocks * seg + (has_block ? bi : 0));
  const int run_a = FMT == kQ6_K ? block0 + 128 * h + 32 * jj : block0 + 64 * u4;
  const int run_b = FMT == kQ6_K ? run_a + 64 : run_a + 32;
  uint32_t xa[3][8], xb[3][8];
#pragma unroll
  for (int l = 0; l < 3; ++l) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 va = *reinterpret_cast<const uint4*>(xl + (size_t)l * a.k + run_a + 16 * i);
      const uint4 vb = *reinterpret_cast<const uint4*>(xl + (size_t)l * a.k + run_b + 16 * i);
      xa[l][4 * i] = va.x, xa[l][4 * i + 1] = va.y, xa[l][4 * i + 2] = va.z, xa[l][4 * i + 3] = va.w;
      xb[l][4 * i] = vb.x, xb[l][4 * i + 1] = vb.y, xb[l][4 * i + 2] = vb.z, xb[l][4 * i + 3] = vb.w;
    }
  }
  const float ua = unscale[run_a >> 5], ub = unscale[run_b >> 5];
  const float sxa = xsum[run_a >> 5], sxb = xsum[run_b >> 5];  // read for Q4_K only
  int ca[2] = {0, 0}, cb[2] = {0, 0};                          // offsets: 32 sum x per group of 16 (Q6_K), 8 sum x per run (Q4_0)
  if constexpr (FMT == kQ6_K) {
    ca[0] = 32 * jsum[run_a >> 4], ca[1] = 32 * jsum[(run_a >> 4) + 1];
    cb[0] = 32 * jsum[run_b >> 4], cb[1] = 32 * jsum[(run_b >> 4) + 1];
  } else if constexpr (FMT == kQ4_0) {
    ca[0] = 8 * (jsum[run_a >> 4] + jsum[(run_a >> 4) + 1]);
    cb[0] = 8 * (jsum[run_b >> 4] + jsum[(run_b >> 4) + 1]);
  }
  const uint32_t blk_off = (uint32_t)kBlockBytes * (uint32_t)bi;  // this lane's block inside a staged segment
  const uint32_t shift = (blk_off & 2u) * 8u;                     // Q6_K: segments start on 16-byte boundaries
  Q4Lane q4;
  q4.p = u4;
  q4.upper = u4 >= 2;
  q4.sh = 16u * (uint32_t)(u4 & 1);
  q4.m_lo = q4.upper ? 15u : 63u;
  q4.m_hi = q4.upper ? 3u : 0u;

  // ---- rows: kBatch at a time, then the warps of a row add their sums in warp order ----
  const int batches = ((a.rows_per_cta + a.streams - 1) / a.streams + kBatch - 1) / kBatch;  // the same for every warp of the CTA
  int buf = 0;
  for (int b = 0; b < batches; ++b, buf ^= 1) {
    float part[kBatch];
#pragma unroll
    for (int r = 0; r < kBatch; ++r) {
      const int i = b * kBatch + r;
      fetch(i + kStages - 1);
      cp_async_wait<kStages - 1>();
      __syncwarp();
      const uint32_t blk = stage0 + (uint32_t)(i % kStages) * kSegBytes + blk_off;
      float v = 0.f;
      if (i < my_rows && has_block) {
        if constexpr (FMT == kQ6_K) v = block_part(blk, shift, h, jj, xa, xb, ua, ub, ca, cb);
        else if constexpr (FMT == kQ4_K) v = block_part_q4k(blk, q4, xa, xb, ua, ub, sxa, sxb);
        else if constexpr (FMT == kQ8_0) v = block_part_q80(blk + 68u * (uint32_t)u4, xa, xb, ua, ub);
        else v = block_part_q40(blk + 36u * (uint32_t)u4, xa, xb, ua, ub, ca[0], cb[0]);
      }
      part[r] = v;
      __syncwarp();  // every lane is done with the stage before the next fetch overwrites it
    }
    // sum over the 32 lanes, for the eight rows at once: lane r ends up with row r's sum
#pragma unroll
    for (int r = 0; r < 4; ++r) {  // fold 8 -> 4: the upper half-warp keeps rows 4..7
      const float send = (lane & 16) ? part[r] : part[r + 4];
      const float keep = (lane & 16) ? part[r + 4] : part[r];
      part[r] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {  // 4 -> 2
      const float send = (lane & 8) ? part[r] : part[r + 2];
      const float keep = (lane & 8) ? part[r + 2] : part[r];
      part[r] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    {  // 2 -> 1
      const float send = (lane & 4) ? part[0] : part[1];
      const float keep = (lane & 4) ? part[1] : part[0];
      part[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    part[0] += __shfl_xor_sync(0xffffffffu, part[0], 2);
    part[0] += __shfl_xor_sync(0xffffffffu, part[0], 1);
    // lanes with the same bits 4, 3, 2 hold the same row: row index = 4 * bit4 + 2 * bit3 + bit2
    if ((lane & 3) == 0) red[(buf * kMaxWarps + warp) * kBatch + ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1)] = part[0];
    if (a.warps_per_row > 1) stream_sync(1 + stream, a.warps_per_row * 32);
    else __syncwarp();
    if (seg == 0 && lane < kBatch) {
      const int i = b * kBatch + lane;
      if (i < my_rows) {
        float total = 0.f;
        for (int wi = 0; wi < a.warps_per_row; ++wi) total += red[(buf * kMaxWarps + warp + wi) * kBatch + lane];
        const long long row = row0 + stream + (long long)i * a.streams;
        for (int d = 0; d < a.n_out; ++d) a.outs[d][row] = total;
      }
    }
  }
  cp_async_wait<0>();
  if (a.sync & kPeerSignal) {
    // every warp of this CTA has stored what it will store; the last CTA of the grid tells the peers
    __syncthreads();
    if (tid == 0) {
      unsigned int* mine = a.pads[a.rank];
      __threadfence();
      if (atomicAdd(mine + 34, 1u) == gridDim.x - 1) {
        __threadfence_system();
        mine[34] = 0u;
        const unsigned int epoch = mine[32] + 1u;
        mine[32] = epoch;
        for (int peer = 0; peer < a.world; ++peer)
          if (peer != a.rank)
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(a.pads[peer] + a.rank), "r"(epoch) : "memory");
      }
    }
  }
}

struct DpPlan {
  int warps_per_row, streams, rows_per_cta, grid;
  size_t smem;
};
bool dp_plan(int fmt, long long n, long long k, const DeviceInfo& dev, DpPlan& plan) {
  const int nsb = (int)(k / 256);
  plan.warps_per_row = (nsb + kSegBlocks - 1) / kSegBlocks;
  if (plan.warps_per_row > kMaxWarps) return false;
  plan.streams = kMaxWarps / plan.warps_per_row;
  // one CTA per SM (the register file holds no second one): the rows in as many chunks as there are SMs
  long long rows = (n + dev.sm_count - 1) / dev.sm_count;
  if (rows < plan.streams) rows = plan.streams;
  plan.rows_per_cta = (int)rows;
  plan.grid = (int)((n + rows - 1) / rows);
  plan.smem = 3 * (size_t)k + 2 * (size_t)(k / 32) * 4 + (size_t)(k / 16) * 4 + 2 * kMaxWarps * kBatch * 4 +
              (size_t)plan.streams * plan.warps_per_row * kStages * kSegBlocks * dp_block_bytes(fmt);
  return plan.smem <= (size_t)dev.max_smem_optin;
}

}  // namespace

bool gemv_dp4a_supported(int fmt, int xt, long long m, long long n, long long k) {
  if ((fmt != kQ6_K && fmt != kQ4_K && fmt != kQ8_0 && fmt != kQ4_0) || m != 1) return false;
  if (xt != kBF16 && xt != kF16) return false;
  if (n < 1 || n > (1LL << 30) || k < 256 || k % 256 || k > 32768) return false;
  if (fmt == kQ6_K && k % 2048) return false;  // rows of whole 8-block segments: every segment starts on a 16-byte boundary
  return true;
}

long long gemv_dp4a_scratch_bytes(long long, long long, const DeviceInfo&) { return 0; }

cudaError_t launch_gemv_dp4a(int fmt, int xt, const void* x, const uint8_t* w, const OutSpec& out, long long n,
                             long long k, cudaStream_t stream, const PeerSync* peers) {
  cudaError_t e;
  const DeviceInfo* dev = device_info(&e);
  if (!dev) return e;
  DpPlan plan;
  if (!dp_plan(fmt, n, k, *dev, plan)) return cudaErrorInvalidValue;
  if (out.count < 1 || out.count > kMaxOutputs) return cudaErrorInvalidValue;
  DpArgs a{};
  a.x = static_cast<const uint16_t*>(x);
  a.w = w;
  for (int d = 0; d < out.count; ++d) a.outs[d] = out.ptr[d];
  a.n_out = out.count;
  a.row_bytes = row_bytes(fmt, k);
  a.n = (int)n;
  a.k = (int)k;
  a.nsb = (int)(k / 256);
  a.warps_per_row = plan.warps_per_row;
  a.streams = plan.streams;
  a.rows_per_cta = plan.rows_per_cta;
  a.wait_limit_ns = peer_wait_limit_ns();
  if (peers && peers->flags) {
    if (peers->world < 1 || peers->world > kMaxOutputs || peers->rank < 0 || peers->rank >= peers->world)
      return cudaErrorInvalidValue;
    for (int i = 0; i < peers->world; ++i) a.pads[i] = peers->pads[i];
    a.rank = peers->rank;
    a.world = peers->world;
    a.sync = peers->flags;
  }
  const bool f16 = xt == kF16;
  void (*kernel)(const DpArgs) =
      fmt == kQ6_K   ? (f16 ? gemv_dp4a_kernel<kQ6_K, true> : gemv_dp4a_kernel<kQ6_K, false>)
      : fmt == kQ4_K ? (f16 ? gemv_dp4a_kernel<kQ4_K, true> : gemv_dp4a_kernel<kQ4_K, false>)
      : fmt == kQ8_0 ? (f16 ? gemv_dp4a_kernel<kQ8_0, true> : gemv_dp4a_kernel<kQ8_0, false>)
                     : (f16 ? gemv_dp4a_kernel<kQ4_0, true> : gemv_dp4a_kernel<kQ4_0, false>);
  e = allow_full_shared_memory(kernel);
  if (e != cudaSuccess) return e;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)plan.grid);
  cfg.blockDim = dim3((unsigned)(plan.streams * plan.warps_per_row * 32));
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, a);
}

}  // namespace tb200
