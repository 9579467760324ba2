// Decode GEMV for batch 1..16 on sm_100a: out[m, n] = x[m, k] . dequant(w[n, k])^T.
//
// Replaces the reference's `gemv_packed` (benchmarks/kernels/showcase/kernels.py:116-119) with
// its fp32-weight x fp32-activation contract (benchmarks/kernels/showcase/benchmark.py:468-470).
//
// Regime: HBM-bound.  B200 streams about 43 GB/s per SM, i.e. ~23 raw bytes per SM clock, which
// leaves ~3 issue slots per 4-bit weight.  A SIMT decode + FMA does not fit in that budget, so:
//
//  * a producer warp streams raw super-blocks into a shared-memory ring with 1-D bulk async
//    copies (cp.async.bulk + mbarrier), one copy per weight row of a 16-row tile, so tens of KB
//    per SM are in flight without holding registers;
//  * consumer warps never form fp32 weights.  The 4-bit (or 6-bit) integers are turned into
//    bf16/fp16 values `offset + q` by one logic op per pair (0x4300|q = 128+q in bf16), which is
//    exact, and fed to warp-level tensor-core MMAs (m16n8k16, fp32 accumulate) against the staged
//    activations.  The block scales are applied to the 32-weight partial sums in fp32:
//        sum_k (d*sc*q - dmin*mn) x = d*sc*(S - offset*Sx) - dmin*mn*Sx,   S = sum (offset+q) x
//    with Sx = sum of x over the group (computed once per CTA).  Operands are exact, so the result
//    differs from the fp32 oracle only by summation order.
//  * m == 1 puts the 8 scale groups of a super-block on the 8 MMA columns (x masked per group),
//    so scales are applied once per super-block and every lane owns distinct (row, group) pairs;
//    1 < m <= 16 puts the batch on the columns and applies scales per 32-weight group.
//  * the K range of a CTA is fixed for its lifetime (x is staged once); row tiles are strided
//    over CTAs; if K is split across CTAs, partial sums go to caller-provided scratch and the
//    last CTA to arrive for a row tile adds them in a fixed order (deterministic).
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tb200 {
namespace {

// Warp roles: warps 0 .. W-1 decode (W = consumer_warps, chosen per plan), warp W streams weights
// into the ring, warp W+1 adds the decode warps' partial sums and writes out.  Plans with two CTAs
// per SM use up to 8 decode warps, plans with one CTA per SM up to 16.
constexpr int kMaxConsumerWarps = 16;
constexpr int kNarrowWarps = 8;
constexpr int kThreadsNarrow = (kNarrowWarps + 2) * 32;
constexpr int kThreadsWide = (kMaxConsumerWarps + 2) * 32;
// Weight tiles a CTA requests before it waits for the kernel before it (programmatic dependent
// launch).  Whatever is requested earlier arrives earlier, but the activations, which can only be
// requested after that wait, come back behind every weight byte this SM has asked for by then, and
// nothing is decoded before they are staged.  One tile measured best at every batch (two: +4 % at
// batch 1; the whole ring: +4..8 %).
constexpr int kTilesBeforeWait = 1;
constexpr int kTileRows = 16;
constexpr int kMaxStages = 8;
constexpr int kCounterBytes = kGemvCounterBytes;  // one arrival counter per group of CTAs that share row tiles (<= 1024)
constexpr int kSclRowFloats = 18;  // 8 x (scale, offset) pairs + 2 floats of padding (bank spread)

struct GemvArgs {
  const void* x;
  const uint8_t* w;
  // Grouped launch: rows [n1, n) come from a second weight of the same K and format that shares
  // the activations (gate and up of an MLP); the output is the [m, n] concatenation.  n1 is a
  // multiple of the tile height; null = a single weight.
  const uint8_t* w2;
  long long n1;
  float* outs[kMaxOutputs];  // destinations of the result (own buffer first, then peer-mapped ones)
  float* outs2[kMaxOutputs]; // grouped launch: destinations of the second weight's columns
  int n_out;
  int out_vec;               // every destination takes 16-byte stores
  long long out_ld;          // elements between the batch rows of a destination
  // N-sharded runs: signal pads of every rank (as mapped here), see peer_barrier.cu for the layout.
  // sync bit 0: wait, before activations are read, until every peer has signalled as often as this
  // rank has; bit 1: signal every peer once all CTAs of this launch have stored their outputs.
  unsigned int* pads[kMaxOutputs];
  int rank, world, sync;
  unsigned long long wait_limit_ns;
  // batch plans: activations converted ahead of this launch (see gemv_prepare_kernel); null = convert here
  const uint16_t* x16;
  const float* x_table;    // [K / 32][NTB] group sums
  const float* x_unscale;  // [K / 256][NTB] one factor per super-block and activation row
  float* partials;
  unsigned int* counters;
  int m;
  long long n;
  int k;
  long long row_bytes;
  int nsb;           // 256-weight super-blocks per row
  int sb_per_split;  // super-blocks per K range
  int k_splits;
  int row_groups;
  int row_tiles;
  int stages;
  int stride_s;   // shared-memory bytes between the rows of a stage
  int xs_stride;  // shared-memory bytes between staged activation rows
  int off_stage, off_xs, off_sx, off_red, off_scl, off_zero, off_misc;
  int consumer_warps;  // warps that decode, chosen to divide the super-blocks of a K range evenly
#ifdef TB200_GEMV_TRACE
  unsigned long long* trace;  // diagnostic timeline (only in trace builds)
#endif
  int red_bufs;        // 2: partial-sum buffers alternate between tiles; 1: a single buffer (shared memory is tight)
  int contiguous;  // one bulk copy per tile (K not split): stage rows are packed like global rows
  int use_tma;     // K split: one 2-D tiled TMA copy per tile (16 rows x the K range)
};

// All MMAs run in fp16: q | 0x6400 is the fp16 number 1024 + q for q < 1024, and a nibble that
// sits in bits 4..7 gives 1024 + 16 q without a shift (the factor 16 is folded into the scale).
constexpr uint32_t kOr = 0x64006400u;
constexpr float kOffset = 1024.f;

// byte j of v as an exact float: 0x4B0000vv is 2^23 + vv.
__device__ __forceinline__ float byte_to_float(uint32_t v, int j) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7540u | (uint32_t)j)) - 8388608.f;
}

__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// 8 activations (16 bytes) -> 4 fp16x2 words, multiplied by `scale` (a power of two) when the
// source is bf16; fp16 sources pass through.
template <bool F16>
__device__ __forceinline__ uint4 to_f16x8(uint4 v, float scale) {
  if constexpr (F16) {
    return v;
  } else {
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
      w[i] = pack_f16(__uint_as_float(w[i] << 16) * scale, __uint_as_float(w[i] & 0xFFFF0000u) * scale);
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
}

__device__ __forceinline__ float sum_f16x8(uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  float part[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    part[i] = f.x + f.y;
  }
  return (part[0] + part[1]) + (part[2] + part[3]);
}

// Batch staging (1 < m <= 16): the activation rows of this CTA's K range are fetched with bulk
// async copies (one per row, a single round trip to L2 / HBM), then converted in place to fp16 in
// one pass: each aligned group of four values is stored as [x0, x2, x1, x3] so that an MMA B
// fragment is one contiguous load.  Every 32-value scale group of every row gets its own power of
// two (largest magnitude -> [2^14, 2^15)), so bf16 -> fp16 is exact for every value within 2^-32 of
// the group's largest; sxu[g][b] = {sum of the staged fp16 values, factor that undoes the scaling}.
template <bool F16, int NTB>
__device__ __forceinline__ bool stage_activations(const GemvArgs& a, uint8_t* smem, int ctid, int k0, int klen,
                                                  uint64_t* xbar) {
  const int threads = a.consumer_warps * 32;
  const int chunks = klen >> 3;  // 8 values (16 bytes) each; a multiple of 32
  const int total = NTB * chunks;
  uint8_t* xs = smem + a.off_xs;
  float2* sxu = reinterpret_cast<float2*>(smem + a.off_sx);
  // columns beyond m have no activation rows in shared memory (their B fragments are loaded from a
  // block of zeros); their group sums are zero (done while the copies are in flight)
  for (int idx = a.m * chunks + ctid; idx < total; idx += threads) {
    const int b = idx / chunks, c = idx - b * chunks;
    if ((c & 3) == 0) sxu[(c >> 2) * NTB + b] = make_float2(0.f, 1.f);
  }
  if (!ptx::mbar_wait(xbar, 0)) {  // the producer warp issued the row copies before any weight copy
    report_timeout(0x60000u);
    return false;
  }
#ifdef TB200_GEMV_TRACE
  if (a.trace && blockIdx.x == 0 && ctid == 0) a.trace[2] = ptx::global_timer_ns();
#endif
  // rows < m: convert in place.  Thread t walks chunks t, t + threads, ... of the flattened
  // (row, chunk) space, four at a time so that four independent dependency chains (load, quad
  // shuffles, convert, sum, store) overlap; trip counts are uniform, so the shuffles are warp-wide.
  const int live = a.m * chunks;
  const uint32_t xs_s = ptx::smem_addr(xs), sxu_s = ptx::smem_addr(sxu);
  constexpr int U = 4;
  int b = ctid / chunks, c = ctid - b * chunks;
  for (int base = 0; base < live; base += U * threads) {
#ifdef TB200_GEMV_TRACE
    if (a.trace && blockIdx.x == 0 && ctid == 0 && base / (U * threads) < 4) a.trace[3 + base / (U * threads)] = ptx::global_timer_ns();
#endif
    uint32_t slot[U];
    int cc[U], bb[U];
    bool valid[U];
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      valid[u] = base + u * threads + ctid < live;
      cc[u] = c;
      bb[u] = b;
      slot[u] = xs_s + (uint32_t)b * a.xs_stride + (c << 4);
      v[u] = valid[u] ? ptx::lds128(slot[u]) : make_uint4(0, 0, 0, 0);
      c += threads;
      while (c >= chunks) {
        c -= chunks;
        ++b;
      }
    }
    float unscale[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float scale = 1.f;
      unscale[u] = 1.f;
      if constexpr (!F16) {
        const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
        uint32_t mx = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) mx = max(mx, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const int e = (int)(mx >> 7);  // biased bf16 exponent of the group's largest magnitude
        if (e > 0 && e < 255) {
          int sh = 141 - e;
          sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
          scale = __uint_as_float((uint32_t)(sh + 127) << 23);
          unscale[u] = __uint_as_float((uint32_t)(127 - sh) << 23);
        }
      }
      v[u] = to_f16x8<F16>(v[u], scale);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float sum = sum_f16x8(v[u]);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (valid[u]) {
        uint4 p;
        p.x = __byte_perm(v[u].x, v[u].y, 0x5410);
        p.y = __byte_perm(v[u].x, v[u].y, 0x7632);
        p.z = __byte_perm(v[u].z, v[u].w, 0x5410);
        p.w = __byte_perm(v[u].z, v[u].w, 0x7632);
        ptx::sts128(slot[u], p);
        if ((cc[u] & 3) == 0) ptx::sts64f(sxu_s + (((cc[u] >> 2) * NTB + bb[u]) << 3), sum, unscale[u]);
      }
    }
  }
  return true;
}

// The conversion done ONCE per GEMV by a small kernel of its own, into global scratch, in the
// layout the CTAs keep in shared memory: x16[b][k] (fp16, each aligned group of four stored as
// [x0, x2, x1, x3]), table[k / 32][NTB] = sum of the staged values of a 32-value group and
// unscale[k / 256][NTB] (zero sums / unit factors for the columns past m).  One thread per 8 values,
// so a warp holds exactly one 256-value super-block of one row (K / 8 is a multiple of 32): the
// power-of-two scale is one per (row, super-block) (largest magnitude -> [2^14, 2^15); bf16 -> fp16
// is exact for every value within 2^-29 of it), found with warp shuffles alone, and the GEMV undoes
// it once per item instead of once per group.
#ifndef TB200_TBIN_WRAPPER
// N-sharded launches whose activations may come from the peers: the conversion reads them ahead of the GEMV's own
// wait, so it waits itself (`pad` = this rank's signal pad; bounded, status 0x80000 | peer).
__device__ __forceinline__ void prepare_wait_peers(const unsigned int* pad, int rank, int world,
                                                   unsigned long long wait_limit_ns) {
  if (!pad) return;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    const unsigned int expected = *reinterpret_cast<const volatile unsigned int*>(pad + 32);
    if (lane < world && lane != rank) {
      const unsigned long long t0 = ptx::global_timer_ns();
      for (;;) {
        unsigned int seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(pad + lane) : "memory");
        if ((int)(seen - expected) >= 0) break;
        if (ptx::global_timer_ns() - t0 > wait_limit_ns) {
          report_timeout(0x80000u | (unsigned)lane);
          break;
        }
        __nanosleep(200);
      }
    }
  }
  __syncthreads();
}

// Block `block` of the `nblocks` that convert one [m, k] activation tensor.
template <bool F16>
__device__ __forceinline__ void prepare_body(const uint16_t* __restrict__ x, uint16_t* __restrict__ x16,
                                             float* __restrict__ table, float* __restrict__ unscale_out, int m, int k,
                                             int ntb, int block, int nblocks) {
  const int chunks = k >> 3;
  const int live = m * chunks;
  const int tid = block * blockDim.x + threadIdx.x;
  if (tid < live) {
    const int b = tid / chunks, c = tid - b * chunks;
    uint4 v = *reinterpret_cast<const uint4*>(x + (long long)b * k + (c << 3));
    float scale = 1.f, unscale = 1.f;
    if constexpr (!F16) {
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      uint32_t mx = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) mx = max(mx, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const int e = (int)(mx >> 7);  // biased bf16 exponent of the super-block's largest magnitude
      if (e > 0 && e < 255) {
        int sh = 141 - e;
        sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
        scale = __uint_as_float((uint32_t)(sh + 127) << 23);
        unscale = __uint_as_float((uint32_t)(127 - sh) << 23);
      }
    }
    v = to_f16x8<F16>(v, scale);
    float sum = sum_f16x8(v);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    uint4 p;
    p.x = __byte_perm(v.x, v.y, 0x5410);
    p.y = __byte_perm(v.x, v.y, 0x7632);
    p.z = __byte_perm(v.z, v.w, 0x5410);
    p.w = __byte_perm(v.z, v.w, 0x7632);
    *reinterpret_cast<uint4*>(x16 + (long long)b * k + (c << 3)) = p;
    if ((c & 3) == 0) table[(long long)(c >> 2) * ntb + b] = sum;
    if ((c & 31) == 0) unscale_out[(long long)(c >> 5) * ntb + b] = unscale;
  }
  // columns past m: zero sums, unit factors
  const int groups = k >> 5, spare = ntb - m;
  for (int i = tid; i < groups * spare; i += nblocks * blockDim.x) {
    const int g = i / spare, b = m + (i - g * spare);
    table[(long long)g * ntb + b] = 0.f;
    if ((g & 7) == 0) unscale_out[(long long)(g >> 3) * ntb + b] = 1.f;
  }
}

template <bool F16>
__global__ void __launch_bounds__(256) gemv_prepare_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ x16,
                                                           float* __restrict__ table, float* __restrict__ unscale_out,
                                                           int m, int k, int ntb, const unsigned int* pad, int rank,
                                                           int world, unsigned long long wait_limit_ns) {
  // Let the GEMV behind this kernel start at once (it fills its weight ring, then waits for this
  // kernel to complete, which in turn has waited for the kernel before): the trigger must come
  // before the wait, or the GEMV could not be scheduled until the previous kernel has drained.
  if (threadIdx.x == 0) ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();  // x may come from the kernel before; the GEMV before may still read x16
  prepare_wait_peers(pad, rank, world, wait_limit_ns);
  prepare_body<F16>(x, x16, table, unscale_out, m, k, ntb, (int)blockIdx.x, (int)gridDim.x);
}

// The conversions of all batched projections of a list as ONE launch ahead of its GEMVs: block ranges per job.
struct PrepJobsArg {
  PrepJobs jobs;
  const unsigned int* pad;
  int rank, world;
  unsigned long long wait_limit_ns;
};
__global__ void __launch_bounds__(256) gemv_prepare_multi_kernel(const PrepJobsArg a) {
  if (threadIdx.x == 0) ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();
  prepare_wait_peers(a.pad, a.rank, a.world, a.wait_limit_ns);
  int block = (int)blockIdx.x, j = 0;
  while (j + 1 < a.jobs.count && block >= a.jobs.job[j].blocks) block -= a.jobs.job[j++].blocks;
  const PrepJob& p = a.jobs.job[j];
  const uint16_t* x = static_cast<const uint16_t*>(p.x);
  uint16_t* x16 = static_cast<uint16_t*>(p.x16);
  if (p.f16) prepare_body<true>(x, x16, p.table, p.unscale, p.m, p.k, p.ntb, block, p.blocks);
  else prepare_body<false>(x, x16, p.table, p.unscale, p.m, p.k, p.ntb, block, p.blocks);
}
#endif  // TB200_TBIN_WRAPPER

// Batch staging when the activations were converted ahead of the launch: the producer warp copies
// this CTA's K range of x16 and of the table into place; the decode warps only clear the rows past m.
template <int NTB>
__device__ __forceinline__ bool stage_prepared(const GemvArgs& a, uint8_t* smem, int ctid, int klen, uint64_t* xbar) {
  if (!ptx::mbar_wait(xbar, 0)) {
    report_timeout(0x60000u);
    return false;
  }
#ifdef TB200_GEMV_TRACE
  if (a.trace && blockIdx.x == 0 && ctid == 0) a.trace[2] = ptx::global_timer_ns();
#endif
  return true;
}

// m == 1 staging: one pass, no CTA-wide reduction.  Each 32-value scale group gets its own power of
// two (its largest magnitude lands in [2^14, 2^15)), so bf16 -> fp16 is exact for every value within
// 2^-32 of the group's largest; the factor that undoes it rides along with the group sum:
// sxu[g] = {sum of the staged fp16 values of group g, unscale of group g}.
template <bool F16>
__device__ __forceinline__ void stage_activations_groups(const GemvArgs& a, uint8_t* smem, int ctid, int k0,
                                                         int klen) {
  const int chunks = klen >> 3;  // 8 values each; four consecutive chunks (lanes) form a group
  const int threads = a.consumer_warps * 32;
  uint8_t* xs = smem + a.off_xs;
  float2* sxu = reinterpret_cast<float2*>(smem + a.off_sx);
  const uint16_t* xg = static_cast<const uint16_t*>(a.x);
  // the first two rounds' loads go out together (one round trip instead of two)
  uint4 ahead[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
#pragma unroll
  for (int r = 0; r < 2; ++r)
    if (r * threads + ctid < chunks) ahead[r] = *reinterpret_cast<const uint4*>(xg + k0 + ((r * threads + ctid) << 3));
  int round = 0;
  for (int base = 0; base < chunks; base += threads, ++round) {
    const int c = base + ctid;  // chunks is a multiple of 32: a warp is all-valid or all-invalid
    uint4 v = make_uint4(0, 0, 0, 0);
    if (round < 2) v = round ? ahead[1] : ahead[0];
    else if (c < chunks) v = *reinterpret_cast<const uint4*>(xg + k0 + (c << 3));
    float scale = 1.f, unscale = 1.f;
    if constexpr (!F16) {
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      uint32_t mx = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) mx = max(mx, max(w[i] & 0x7FFFu, (w[i] >> 16) & 0x7FFFu));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const int e = (int)(mx >> 7);  // biased bf16 exponent of the group's largest magnitude
      if (e > 0 && e < 255) {
        int sh = 141 - e;
        sh = sh > 126 ? 126 : (sh < -126 ? -126 : sh);
        scale = __uint_as_float((uint32_t)(sh + 127) << 23);
        unscale = __uint_as_float((uint32_t)(127 - sh) << 23);
      }
    }
    v = to_f16x8<F16>(v, scale);
    float sum = sum_f16x8(v);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (c < chunks) {
      uint4 p;
      p.x = __byte_perm(v.x, v.y, 0x5410);
      p.y = __byte_perm(v.x, v.y, 0x7632);
      p.z = __byte_perm(v.z, v.w, 0x5410);
      p.w = __byte_perm(v.z, v.w, 0x7632);
      *reinterpret_cast<uint4*>(xs + (c << 4)) = p;
      if ((c & 3) == 0) sxu[c >> 2] = make_float2(sum, unscale);
    }
  }
}

// Pin a value in a register.  Kernel parameters live in the constant bank and the compiler likes
// to re-load them inside hot loops instead of spending a register; those loads sit on the long
// scoreboard and stall an otherwise short dependency chain.
__device__ __forceinline__ uint32_t pin(uint32_t v) {
  uint32_t r;
  asm volatile("mov.b32 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ int pin(int v) { return (int)pin((uint32_t)v); }

// (a & mask) | bits in ONE logic op.  The constants are handed over in registers: with two
// immediates the compiler splits the expression into two LOP3s, and logic ops (half-rate ALU pipe)
// are what bounds this kernel.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t bits) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(bits));
  return d;
}
struct NibbleConsts {
  uint32_t lo, hi, bits;  // 0x000F000F, 0x00F000F0, 0x64006400, kept in registers
};
__device__ __forceinline__ NibbleConsts nibble_consts() {
  NibbleConsts c;
  asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(c.lo));
  asm volatile("mov.b32 %0, 0x00F000F0;" : "=r"(c.hi));
  asm volatile("mov.b32 %0, 0x64006400;" : "=r"(c.bits));
  return c;
}

// One 32-bit word of Q4_K quants (4 bytes = 4 low + 4 high nibbles) -> four fp16x2 registers:
// lo02 / lo13 hold 1024 + low nibble of bytes (0,2) / (1,3); hi02 / hi13 hold 1024 + 16 * high
// nibble.  Five logic ops for eight weights.
struct Nibbles {
  uint32_t lo02, hi02, lo13, hi13;
};
__device__ __forceinline__ Nibbles split_nibbles(uint32_t w, const NibbleConsts& k) {
  Nibbles r;
  const uint32_t w8 = w >> 8;  // (w * 2^24 >> 32 on the multiplier pipe was measured slower)
  r.lo02 = and_or(w, k.lo, k.bits);
  r.hi02 = and_or(w, k.hi, k.bits);
  r.lo13 = and_or(w8, k.lo, k.bits);
  r.hi13 = and_or(w8, k.hi, k.bits);
  return r;
}

// Shared-memory addresses (32-bit, shared window) a consumer warp needs; computed once per CTA.
struct SmemMap {
  uint32_t xs, sx, scl;  // staged activations, group sums, this warp's scale scratch
  uint32_t zero;         // zero bytes (B fragments of batch columns past m)
  uint32_t su;           // prepared activations: unscale factors [super-block][column]
  int m;
  int stride_s, xs_stride;
  NibbleConsts nc;
};

// ---- Q4_K, batch on the MMA columns (1 < m <= 16) ------------------------------------------------
// Shared memory holds only the m live activation rows.  PARTIAL (m below the columns of the MMA
// tiles): a lane whose batch column is past m loads its B fragments from a block of zeros instead
// (address and stride picked per lane), so no zero rows are stored.
// UNIFORM (activations prepared ahead of the launch): one unscale factor per (super-block, activation
// row), applied once per item, so the table holds the group sums alone and a value costs two FMAs
// per group.
template <int NT, bool PARTIAL, bool UNIFORM>
__device__ __forceinline__ void q4k_item_batch(const SmemMap& sm, uint32_t stage, int sbl, int lane,
                                               float (&acc)[NT][4]) {
  constexpr int NTB = NT * 8;
  const int gid = lane >> 2, tig = lane & 3;
  __syncwarp();
  {  // scale preparation: lane -> (row, half of the groups)
    const int r = lane >> 1, hf = lane & 1;
    const uint4 hdr = ptx::lds128(stage + r * sm.stride_s + sbl * 144);
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
    const uint32_t scv = hf ? ((hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u)) : (hdr.y & 0x3F3F3F3Fu);
    const uint32_t mnv =
        hf ? (((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u)) : (hdr.z & 0x3F3F3F3Fu);
    const uint32_t dst = sm.scl + (r * kSclRowFloats + hf * 8) * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // odd groups are the high nibbles, which enter the MMA as 16 * q
      const float dsc = d * byte_to_float(scv, j) * ((j & 1) ? 0.0625f : 1.f);
      const float e = fmaf(kOffset, dsc, dmin * byte_to_float(mnv, j));
      ptx::sts64f(dst + 8 * j, dsc, e);
    }
  }
  __syncwarp();
  const uint32_t rowA = stage + gid * sm.stride_s + sbl * 144 + 16 + tig * 8;
  const uint32_t rowB = rowA + 8 * sm.stride_s;
  const uint32_t sclA = sm.scl + gid * (kSclRowFloats * 4), sclB = sclA + 8 * (kSclRowFloats * 4);
  const uint32_t xrow = sm.xs + gid * sm.xs_stride + ((sbl * 256 + 8 * tig) << 1);
  uint32_t xlive[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const bool live = !PARTIAL || 8 * t + gid < sm.m;
    xlive[t] = live ? xrow + 8 * t * sm.xs_stride : sm.zero;  // the zero block spans all eight group offsets
  }
  const uint32_t sxp = sm.sx + ((sbl * 8) * NTB + 2 * tig) * (UNIFORM ? 4 : 8);
  const float zero[4] = {0.f, 0.f, 0.f, 0.f};
  float item[NT][4];  // UNIFORM: this item's sums before the super-block's unscale factor
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) item[t][j] = 0.f;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint2 wa = ptx::lds64(rowA + p * 32);
    const uint2 wb = ptx::lds64(rowB + p * 32);
    const Nibbles ax = split_nibbles(wa.x, sm.nc), ay = split_nibbles(wa.y, sm.nc);
    const Nibbles bx = split_nibbles(wb.x, sm.nc), by = split_nibbles(wb.y, sm.nc);
#pragma unroll
    for (int nib = 0; nib < 2; ++nib) {
      const int g = 2 * p + nib;
      const float2 sA = ptx::lds64f(sclA + g * 8);
      const float2 sB = ptx::lds64f(sclB + g * 8);
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const uint4 xb = ptx::lds128(xlive[t] + g * 64);
        float c[4];
        if (nib == 0) {
          ptx::mma16816<true>(c, ax.lo02, bx.lo02, ax.lo13, bx.lo13, xb.x, xb.y, zero);
          ptx::mma16816<true>(c, ay.lo02, by.lo02, ay.lo13, by.lo13, xb.z, xb.w, c);
        } else {
          ptx::mma16816<true>(c, ax.hi02, bx.hi02, ax.hi13, bx.hi13, xb.x, xb.y, zero);
          ptx::mma16816<true>(c, ay.hi02, by.hi02, ay.hi13, by.hi13, xb.z, xb.w, c);
        }
        if constexpr (UNIFORM) {
          const float2 sx = ptx::lds64f(sxp + (g * NTB + 8 * t) * 4);  // group sums of columns 2*tig, 2*tig+1
          item[t][0] = fmaf(sA.x, c[0], fmaf(-sA.y, sx.x, item[t][0]));
          item[t][1] = fmaf(sA.x, c[1], fmaf(-sA.y, sx.y, item[t][1]));
          item[t][2] = fmaf(sB.x, c[2], fmaf(-sB.y, sx.x, item[t][2]));
          item[t][3] = fmaf(sB.x, c[3], fmaf(-sB.y, sx.y, item[t][3]));
        } else {
          const uint4 su = ptx::lds128(sxp + (g * NTB + 8 * t) * 8);  // {Sx, u} of columns 2*tig, 2*tig+1
          const float sx0 = __uint_as_float(su.x), u0 = __uint_as_float(su.y);
          const float sx1 = __uint_as_float(su.z), u1 = __uint_as_float(su.w);
          acc[t][0] = fmaf(u0, fmaf(sA.x, c[0], -sA.y * sx0), acc[t][0]);
          acc[t][1] = fmaf(u1, fmaf(sA.x, c[1], -sA.y * sx1), acc[t][1]);
          acc[t][2] = fmaf(u0, fmaf(sB.x, c[2], -sB.y * sx0), acc[t][2]);
          acc[t][3] = fmaf(u1, fmaf(sB.x, c[3], -sB.y * sx1), acc[t][3]);
        }
      }
    }
  }
  if constexpr (UNIFORM) {
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const float2 u = ptx::lds64f(sm.su + (sbl * NTB + 8 * t + 2 * tig) * 4);  // columns 2*tig, 2*tig+1
      acc[t][0] = fmaf(u.x, item[t][0], acc[t][0]);
      acc[t][1] = fmaf(u.y, item[t][1], acc[t][1]);
      acc[t][2] = fmaf(u.x, item[t][2], acc[t][2]);
      acc[t][3] = fmaf(u.y, item[t][3], acc[t][3]);
    }
  }
}

// ---- Q4_K, scale groups on the MMA columns (m == 1) ----------------------------------------------
// Lane (gid, tig) holds the weights of rows gid and gid+8 that sit in 16-byte chunks tig and tig+4
// of the 128 quant bytes; chunk c belongs to group pair c/2, so in one MMA different lanes may feed
// different groups.  Column j of the MMA collects group j: the B fragment of lane (gid, tig) is its
// slice of x when the lane's weights are in group gid, else zero.  For a lane that is true for one
// of the four (chunk, nibble) combinations at most, so the four B fragments are loaded through
// per-combination addresses that point at x for that one and at a block of zeros otherwise (loads
// are cheap here; logic ops are the scarce resource).
struct GroupLane {
  uint32_t xbase[4];  // combination = 2 * chunk_index + nibble
  int xstep[4];       // bytes per super-block: 512 for the live combination, 0 otherwise
  uint32_t row_off;   // gid * stride: this lane's first weight row inside a stage
  uint32_t row8;      // 8 * stride: distance to its second row
  uint32_t quant_off; // 16 + 16 * tig: first quant chunk of the lane inside a super-block
  uint32_t sxu;       // shared address of {group sum, unscale} for group 2 * tig of super-block 0
  // scale extraction, fixed per lane: groups 2*tig, 2*tig+1 sit in bytes 2*(tig&1), +1 of the
  // packed words; lanes with tig >= 2 (groups 4..7) splice low 4 bits and high 2 bits
  uint32_t m_lo, m_hi;      // 0x3F3F3F3F / 0 for groups 0..3, 0x0F0F0F0F / 0x30303030 for groups 4..7
  uint32_t sel0, sel1;      // PRMT selectors that turn byte 2*(tig&1) (+1) into the float 2^23 + byte
  bool upper;
};

__device__ __forceinline__ float prmt_float(uint32_t v, uint32_t selector) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, selector)) - 8388608.f;
}

__device__ __forceinline__ void q4k_item_groups(const SmemMap& sm, uint32_t stage, int sbl,
                                                const GroupLane& gl, float& accA, float& accB) {
  const uint32_t blkA = stage + gl.row_off + sbl * 144;
  const uint32_t blkB = blkA + gl.row8;
  const uint4 hdrA = ptx::lds128(blkA), hdrB = ptx::lds128(blkB);
  const uint4 su = ptx::lds128(gl.sxu + sbl * 64);  // {Sx, u} of groups 2*tig and 2*tig+1
  float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};  // two independent MMA chains
#pragma unroll
  for (int ci = 0; ci < 2; ++ci) {
    const uint4 qa = ptx::lds128(blkA + gl.quant_off + 64 * ci);
    const uint4 qb = ptx::lds128(blkB + gl.quant_off + 64 * ci);
    const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
    const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
    const uint32_t pl = gl.xbase[2 * ci] + sbl * gl.xstep[2 * ci];
    const uint32_t ph = gl.xbase[2 * ci + 1] + sbl * gl.xstep[2 * ci + 1];
    const uint4 l0 = ptx::lds128(pl), l1 = ptx::lds128(pl + 16);
    const uint4 h0 = ptx::lds128(ph), h1 = ptx::lds128(ph + 16);
    const uint32_t xlo[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
    const uint32_t xhi[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const Nibbles na = split_nibbles(wa[i], sm.nc), nb = split_nibbles(wb[i], sm.nc);
      ptx::mma16816<true>(c0, na.lo02, nb.lo02, na.lo13, nb.lo13, xlo[2 * i], xlo[2 * i + 1], c0);
      ptx::mma16816<true>(c1, na.hi02, nb.hi02, na.hi13, nb.hi13, xhi[2 * i], xhi[2 * i + 1], c1);
    }
  }
  // c0 collects the even groups (columns 0, 2, 4, 6), c1 the odd ones.  c[0], c[1]: row gid,
  // groups 2*tig, 2*tig+1; c[2], c[3]: row gid+8.
  const float sx0 = __uint_as_float(su.x), u0 = __uint_as_float(su.y);
  const float sx1 = __uint_as_float(su.z), u1 = __uint_as_float(su.w);
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const uint4 hdr = rr ? hdrB : hdrA;
    const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&hdr.x));  // d, dmin
    // 6-bit scales / mins of the lane's two groups, all four packed bytes at once
    const uint32_t sc_src = gl.upper ? hdr.w : hdr.y;
    const uint32_t mn_src = gl.upper ? (hdr.w >> 4) : hdr.z;
    const uint32_t scv = and_or(sc_src, gl.m_lo, (hdr.y >> 2) & gl.m_hi);
    const uint32_t mnv = and_or(mn_src, gl.m_lo, (hdr.z >> 2) & gl.m_hi);
    const float dsc0 = dd.x * prmt_float(scv, gl.sel0);              // even group: low nibbles
    const float dsc1 = dd.x * 0.0625f * prmt_float(scv, gl.sel1);    // odd group: 16 * high nibble
    const float e0 = fmaf(kOffset, dsc0, dd.y * prmt_float(mnv, gl.sel0));
    const float e1 = fmaf(kOffset, dsc1, dd.y * prmt_float(mnv, gl.sel1));
    const float t0 = fmaf(dsc0, c0[2 * rr], -e0 * sx0);      // even column: low-nibble MMAs only
    const float t1 = fmaf(dsc1, c1[2 * rr + 1], -e1 * sx1);  // odd column: high-nibble MMAs only
    float v = rr ? accB : accA;
    v = fmaf(u0, t0, v);
    v = fmaf(u1, t1, v);
    if (rr) accB = v; else accA = v;
  }
}

template <int FMT, bool F16, int NT, bool GROUPS>
__device__ __forceinline__ void gemv_mma_body(const GemvArgs& a, const CUtensorMap* wmap) {
  static_assert(FMT == kQ4_K, "only Q4_K is pipelined so far");
  constexpr int NTB = GROUPS ? 1 : NT * 8;
  constexpr int kBlockBytes = Fmt<FMT>::kBytes;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);
  uint64_t* empty = full + kMaxStages;
  uint64_t* cbar = empty + kMaxStages;  // consumer-only barrier for the staging phase (bounded)
  uint64_t* red_full = cbar + 1;        // [2] consumers -> reducer: partial sums of a tile are in place
  uint64_t* red_empty = red_full + 2;   // [2] reducer -> consumers: buffer may be overwritten
  uint64_t* xbar = red_empty + 2;       // activation rows have landed in shared memory
  uint64_t* fin = xbar + 1;             // reducer -> consumers: whether this CTA adds the K ranges
  __shared__ int s_last;
  __shared__ int s_exit;  // warps of this CTA that have stored everything they will store

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int W = a.consumer_warps;
  const int ks = blockIdx.x % a.k_splits;
  const int rg = blockIdx.x / a.k_splits;
  const int sb0 = ks * a.sb_per_split;
  const int nsb_local = min(a.sb_per_split, a.nsb - sb0);
  const uint32_t range_bytes = (uint32_t)nsb_local * kBlockBytes;
  const int S = a.stages;
  float* red = reinterpret_cast<float*>(smem + a.off_red);
  constexpr int kRedPerWarp = NTB * kTileRows;
  const int red_per_buf = W * kRedPerWarp;
  volatile float* unscale_slot = reinterpret_cast<volatile float*>(smem + a.off_misc);

  if (threadIdx.x == 0) {
    s_exit = 0;
    // all CTAs of this grid are resident at once, so the next kernel on the stream may be
    // scheduled as CTAs of this one retire
    ptx::grid_launch_dependents();
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(&full[s], 1);
      ptx::mbar_init(&empty[s], W);
    }
    ptx::mbar_init(cbar, W);
    ptx::mbar_init(xbar, 1);
    ptx::mbar_init(fin, 1);
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&red_full[b], W);
      ptx::mbar_init(&red_empty[b], 1);
    }
    ptx::fence_mbar_init();
  }
  if (threadIdx.x < 128) reinterpret_cast<uint32_t*>(smem + a.off_zero)[threadIdx.x] = 0u;
#ifdef TB200_GEMV_TRACE
  // slots per traced CTA (blockIdx % 100 == 0): 0 start, 1 staged, 8+i tile data ready, 24+i tile decoded,
  // 40+i tile reduced, 56+i tile copy issued
  unsigned long long* trace = (a.trace && blockIdx.x % 100 == 0) ? a.trace + (blockIdx.x / 100) * 80 : nullptr;
  if (trace && threadIdx.x == 0) trace[0] = ptx::global_timer_ns();
#define TB200_TRACE(cond, slot) do { if (trace && (cond) && (slot) < 80) trace[slot] = ptx::global_timer_ns(); } while (0)
#else
#define TB200_TRACE(cond, slot) do { } while (0)
#endif
  __syncthreads();

  // K split over CTAs: the last CTA of a group to finish adds every K range's partial sums, in K
  // order (deterministic).  Work items = (row tile of the group, column, 4 consecutive rows), spread
  // over all helper lanes (consumer warps + reducer) so many independent 16-byte loads are in flight.
  auto add_partials = [&](int helper, int helpers) {
    __threadfence();
    const long long plane = (long long)a.m * a.n;
    const int my_tiles = (a.row_tiles - rg + a.row_groups - 1) / a.row_groups;
    const int per_tile = a.m * 4;
    const bool vec = (a.n & 3) == 0;
    for (int item = helper * 32 + lane; item < my_tiles * per_tile; item += helpers * 32) {
      const int t = item / per_tile, rem = item - t * per_tile;
      const int col = rem >> 2, r4 = (rem & 3) * 4;
      const long long grow = ((long long)rg + (long long)t * a.row_groups) * kTileRows + r4;
      if (grow >= a.n) continue;
      const long long idx = (long long)col * a.n + grow;
      const long long oidx = (long long)col * a.out_ld + grow;
      if (vec) {
        float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int q = 0; q < a.k_splits; ++q) {
          const float4 p = __ldcg(reinterpret_cast<const float4*>(&a.partials[q * plane + idx]));
          tot.x += p.x;
          tot.y += p.y;
          tot.z += p.z;
          tot.w += p.w;
        }
        if (a.out_vec) {
          for (int d = 0; d < a.n_out; ++d) *reinterpret_cast<float4*>(&a.outs[d][oidx]) = tot;
        } else {
          const float e[4] = {tot.x, tot.y, tot.z, tot.w};
          for (int d = 0; d < a.n_out; ++d)
            for (int r = 0; r < 4; ++r) a.outs[d][oidx + r] = e[r];
        }
      } else {
        for (int r = 0; r < 4 && grow + r < a.n; ++r) {
          float total = 0.f;
          for (int q = 0; q < a.k_splits; ++q) total += __ldcg(&a.partials[q * plane + idx + r]);
          for (int d = 0; d < a.n_out; ++d) a.outs[d][oidx + r] = total;
        }
      }
    }
  };

  // Peers (N-sharded runs).  wait_peers: one warp polls this rank's pad until every peer's count
  // has reached this rank's own count of signals sent (bounded; gives up with status 0x80000|peer).
  auto wait_peers = [&]() {
    if (!(a.sync & 1)) return;
    const unsigned int* mine = a.pads[a.rank];
    const unsigned int expected = *reinterpret_cast<const volatile unsigned int*>(mine + 32);
    if (lane < a.world && lane != a.rank) {
      const unsigned long long t0 = ptx::global_timer_ns();
      for (;;) {
        unsigned int seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + lane) : "memory");
        if ((int)(seen - expected) >= 0) break;
        if (ptx::global_timer_ns() - t0 > a.wait_limit_ns) {
          report_timeout(0x80000u | (unsigned)lane);
          break;
        }
        __nanosleep(200);
      }
    }
    __syncwarp();
  };
  // cta_done: every warp calls it on its normal way out.  The last warp of the CTA counts the CTA
  // in; the last CTA of the grid bumps this rank's count and stores it into every peer's pad.
  // Ordering is handed along that chain (CTA-scope fence -> shared counter -> GPU-scope fence ->
  // global counter -> ONE system-scope fence -> flags): a system-scope fence per warp costs
  // microseconds once a few thousand of them queue up.
  auto cta_done = [&]() {
    if (!(a.sync & 2)) return;
    __syncwarp();
    unsigned int last = 0;
    if (lane == 0) {
      __threadfence_block();
      last = atomicAdd(&s_exit, 1) == W + 1;
    }
    if (!__shfl_sync(0xffffffffu, last, 0)) return;
    if (lane != 0) return;
    unsigned int* mine = a.pads[a.rank];
    __threadfence();
    if (atomicAdd(mine + 34, 1u) != gridDim.x - 1) return;
    __threadfence_system();
    mine[34] = 0u;
    const unsigned int epoch = mine[32] + 1u;
    mine[32] = epoch;
    for (int p = 0; p < a.world; ++p)
      if (p != a.rank)
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(a.pads[p] + a.rank), "r"(epoch) : "memory");
  };

  if (warp == W) {
    // ---------------- producer: bulk copies of the tile's weight rows ----------------
    const uint8_t* src0 = a.w + (long long)sb0 * kBlockBytes;
    // Weights never depend on the kernel before this one, activations may: the ring is filled
    // first (while the previous kernel drains, if this launch overlaps it), then the dependency
    // wait, then the activation rows.
    auto fetch_activations = [&]() {
      ptx::grid_dependency_wait();
      // one poller per CTA: thousands of warps polling the same pad would queue the peers' flag
      // stores behind their loads
      wait_peers();
      if constexpr (GROUPS) {
        if ((a.sync & 1) && lane == 0) ptx::mbar_arrive(xbar);  // releases the decode warps
      } else {
        asm volatile("fence.proxy.async.global;" ::: "memory");  // the copies below read through the async proxy
        const uint32_t x_row_bytes = (uint32_t)nsb_local * 512;
        const uint32_t table_bytes = a.x16 ? (uint32_t)nsb_local * 8 * NTB * 4 : 0u;
        const uint32_t unscale_bytes = a.x16 ? (uint32_t)nsb_local * NTB * 4 : 0u;
        const uint16_t* src = a.x16 ? a.x16 : static_cast<const uint16_t*>(a.x);
        if (lane == 0) ptx::mbar_arrive_expect_tx(xbar, (uint32_t)a.m * x_row_bytes + table_bytes + unscale_bytes);
        __syncwarp();
        if (lane < a.m)
          ptx::bulk_g2s(smem + a.off_xs + (size_t)lane * a.xs_stride, src + (long long)lane * a.k + sb0 * 256,
                        x_row_bytes, xbar);
        if (a.x16 && lane == 31)
          ptx::bulk_g2s(smem + a.off_sx, a.x_table + (long long)sb0 * 8 * NTB, table_bytes, xbar);
        if (a.x16 && lane == 30)  // the factors sit behind the (half-size) table of group sums
          ptx::bulk_g2s(smem + a.off_sx + (size_t)a.sb_per_split * 8 * NTB * 4, a.x_unscale + (long long)sb0 * NTB,
                        unscale_bytes, xbar);
      }
    };
    int i = 0;
    for (int rt = rg; rt < a.row_tiles; rt += a.row_groups, ++i) {
      const int s = i % S;
      // the dependency wait and the activation requests come after the first tile(s), see kTilesBeforeWait
      if (i == min(S, kTilesBeforeWait)) fetch_activations();
      if (i >= S && !ptx::mbar_wait(&empty[s], ((i / S) - 1) & 1)) {
        report_timeout(0x10000u | (unsigned)s);
        break;
      }
      const long long row0 = (long long)rt * kTileRows;
      const int rows = (int)min((long long)kTileRows, a.n - row0);
      uint8_t* dst = smem + a.off_stage + (size_t)s * kTileRows * a.stride_s;
      TB200_TRACE(lane == 0 && i < 16, 56 + i);
      // which weight the tile's rows live in (grouped launches), and its first row there
      const bool second = a.w2 != nullptr && row0 >= a.n1;
      const uint8_t* wsrc = second ? a.w2 + (long long)sb0 * kBlockBytes : src0;
      const long long wrow0 = second ? row0 - a.n1 : row0;
      if (a.contiguous) {
        // the K range is the whole row and rows are packed back to back: one copy per tile
        if (lane == 0) {
          ptx::mbar_arrive_expect_tx(&full[s], (uint32_t)rows * range_bytes);
          ptx::bulk_g2s(dst, wsrc + wrow0 * a.row_bytes, (uint32_t)rows * range_bytes, &full[s]);
        }
      } else if (a.use_tma) {
        // K is split: one tiled copy fetches the K range of all 16 rows (rows past N and
        // super-blocks past K arrive as zeros, and count towards the transaction bytes)
        if (lane == 0) {
          ptx::mbar_arrive_expect_tx(&full[s], (uint32_t)(kTileRows * a.stride_s));
          ptx::tma_load_2d(dst, wmap, sb0 * (kBlockBytes / 8), (int)row0, &full[s]);
        }
      } else {
        if (lane == 0) ptx::mbar_arrive_expect_tx(&full[s], (uint32_t)rows * range_bytes);
        __syncwarp();
        if (lane < rows)
          ptx::bulk_g2s(dst + (size_t)lane * a.stride_s, wsrc + (wrow0 + lane) * a.row_bytes, range_bytes, &full[s]);
      }
    }
    if (i <= min(S, kTilesBeforeWait)) fetch_activations();
    cta_done();
    return;
  }

  if (warp == W + 1) {
    // ---------------- reducer: sum the consumer warps' partials in warp order, write out ----------------
    ptx::grid_dependency_wait();  // outputs and scratch may still be in use by the kernel before
    int i = 0;
    for (int rt = rg; rt < a.row_tiles; rt += a.row_groups, ++i) {
      const int b = a.red_bufs == 2 ? (i & 1) : 0;
      const int use = a.red_bufs == 2 ? (i >> 1) : i;
      if (!ptx::mbar_wait(&red_full[b], use & 1)) {
        report_timeout(0x40000u | (unsigned)b);
        return;
      }
      const float unscale = *unscale_slot;
      // Four consecutive rows of one column per lane and step: 16-byte shared loads, independent
      // across steps, added in warp order.
      const float4* buf4 = reinterpret_cast<const float4*>(red + b * red_per_buf);
      constexpr int kQuads = kRedPerWarp / 4;                 // float4 per warp partial
      constexpr int kPerLane = (kQuads + 31) / 32;
      float4 sum[kPerLane];
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) sum[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
      for (int w8 = 0; w8 < W; ++w8) {
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) {
          const int f = lane + 32 * j;
          if (f < kQuads) {
            const float4 p = buf4[w8 * kQuads + f];
            sum[j].x += p.x;
            sum[j].y += p.y;
            sum[j].z += p.z;
            sum[j].w += p.w;
          }
        }
      }
      __syncwarp();
      TB200_TRACE(lane == 0 && i < 16, 40 + i);
      if (lane == 0) ptx::mbar_arrive(&red_empty[b]);  // partials are in registers now
      const bool final_out = a.k_splits == 1;
      float* part = a.partials + (long long)ks * a.m * a.n;
      const bool vec = final_out ? a.out_vec != 0 : (a.n & 3) == 0;
      const long long ld = final_out ? a.out_ld : a.n;
      const int dests = final_out ? a.n_out : 1;
#pragma unroll
      for (int j = 0; j < kPerLane; ++j) {
        const int f = lane + 32 * j;  // (column f / 4, rows 4 * (f % 4) ..)
        const int col = f >> 2, r4 = (f & 3) * 4;
        const long long grow = (long long)rt * kTileRows + r4;
        if (f >= kQuads || col >= a.m || grow >= a.n) continue;
        const float4 v = make_float4(sum[j].x * unscale, sum[j].y * unscale, sum[j].z * unscale, sum[j].w * unscale);
        for (int d = 0; d < dests; ++d) {
          float* p;
          if (!final_out) p = part + (long long)col * ld + grow;
          else if (a.w2 != nullptr && grow >= a.n1) p = a.outs2[d] + (long long)col * ld + (grow - a.n1);
          else p = a.outs[d] + (long long)col * ld + grow;
          if (vec) {
            *reinterpret_cast<float4*>(p) = v;
          } else {
            const float e[4] = {v.x, v.y, v.z, v.w};
            for (int r = 0; r < 4 && grow + r < a.n; ++r) p[r] = e[r];
          }
        }
      }
    }
    if (a.k_splits > 1) {
      // K is split over CTAs: the CTAs that share this set of row tiles count themselves in; the
      // last one to arrive adds everybody's partial sums in K order (deterministic) and writes out.
      __threadfence();
      __syncwarp();
      unsigned int last = 0;
      if (lane == 0) {
        const unsigned int old = atomicAdd(&a.counters[rg], 1u);
        last = old == (unsigned)(a.k_splits - 1);
        if (last) a.counters[rg] = 0u;  // every other K range has already arrived: ready for the next call
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (lane == 0) {
        s_last = (int)last;
        __threadfence_block();
        ptx::mbar_arrive(fin);  // the consumer warps are waiting for this decision
      }
      if (last) add_partials(W, W + 1);
    }
    TB200_TRACE(lane == 0, 72);
    cta_done();
    return;
  }

  // ---------------- consumers ----------------
  const int cw = warp;
  if (cw >= W) return;
  ptx::grid_dependency_wait();  // activations may come from the kernel before
  TB200_TRACE(threadIdx.x == 0, 7);
  if constexpr (GROUPS) {
    // the decode warps read the activations themselves: hold them until the producer warp has
    // seen the peers' signals
    if ((a.sync & 1) && !ptx::mbar_wait(xbar, 0)) {
      report_timeout(0x60000u);
      return;
    }
  }
  const int ctid = threadIdx.x;
  uint32_t cphase = 0;
  // All consumer warps meet here; returns false if the (bounded) wait gave up.
  auto consumer_sync = [&]() -> bool {
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive(cbar);
    const bool ok = ptx::mbar_wait(cbar, cphase & 1);
    ++cphase;
    if (!ok) report_timeout(0x30000u);
    return ok;
  };
  if constexpr (GROUPS) {
    stage_activations_groups<F16>(a, smem, ctid, sb0 * 256, nsb_local * 256);
    if (ctid == 0) *unscale_slot = 1.f;  // scaling is undone per group inside the item
  } else {
    if (a.x16) {
      if (!stage_prepared<NTB>(a, smem, ctid, nsb_local * 256, xbar)) return;
    } else if (!stage_activations<F16, NTB>(a, smem, ctid, sb0 * 256, nsb_local * 256, xbar)) {
      return;
    }
    if (ctid == 0) *unscale_slot = 1.f;  // scaling is undone per group inside the item
  }
  if (!consumer_sync()) return;
  TB200_TRACE(ctid == 0, 1);

  const int gid = lane >> 2, tig = lane & 3;
  const uint32_t smem_base = ptx::smem_addr(smem);
  SmemMap sm;
  sm.xs = pin(smem_base + a.off_xs);
  sm.sx = pin(smem_base + a.off_sx);
  sm.scl = pin(smem_base + a.off_scl + cw * (kTileRows * kSclRowFloats * 4));
  sm.zero = pin(smem_base + a.off_zero);
  sm.su = pin(smem_base + a.off_sx + a.sb_per_split * 8 * NTB * 4);
  sm.m = pin(a.m);
  sm.stride_s = pin(a.stride_s);
  sm.xs_stride = pin(a.xs_stride);
  sm.nc = nibble_consts();
  GroupLane gl;
  if constexpr (GROUPS) {
    // this lane's slice of x: group gid, 16 values starting at 16 * (tig & 1)
    const uint32_t mine = sm.xs + ((32 * gid + 16 * (tig & 1)) << 1);
    const uint32_t zeros = smem_base + a.off_zero;
#pragma unroll
    for (int ci = 0; ci < 2; ++ci)
#pragma unroll
      for (int nib = 0; nib < 2; ++nib) {
        const bool live = gid == 2 * (tig >> 1) + 4 * ci + nib;
        gl.xbase[2 * ci + nib] = pin(live ? mine : zeros);
        gl.xstep[2 * ci + nib] = pin(live ? 512 : 0);
      }
    gl.row_off = pin((uint32_t)(gid * a.stride_s));
    gl.row8 = pin((uint32_t)(8 * a.stride_s));
    gl.quant_off = pin((uint32_t)(16 + 16 * tig));
    gl.sxu = pin(sm.sx + 2 * tig * 8);
    gl.upper = tig >= 2;
    gl.m_lo = gl.upper ? 0x0F0F0F0Fu : 0x3F3F3F3Fu;
    gl.m_hi = gl.upper ? 0x30303030u : 0u;
    gl.sel0 = 0x7540u | (uint32_t)(2 * (tig & 1));
    gl.sel1 = gl.sel0 + 1;
  }

  const uint32_t stage0 = pin(smem_base + a.off_stage);
  const uint32_t stage_step = pin((uint32_t)(kTileRows * a.stride_s));
  const int row_tiles = pin(a.row_tiles), row_groups = pin(a.row_groups);
  const int nsb_l = pin(nsb_local), Wp = pin(W), Sp = pin(S);
  int i = 0, s = 0, phase = 0;
  for (int rt = rg; rt < row_tiles; rt += row_groups, ++i) {
    if (!ptx::mbar_wait(&full[s], phase)) {
      report_timeout(0x20000u | (unsigned)s);
      return;
    }
    TB200_TRACE(ctid == 0 && i < 16, 8 + i);
    const uint32_t stage = stage0 + s * stage_step;
    const int rb = a.red_bufs == 2 ? (i & 1) : 0;
    const int ruse = a.red_bufs == 2 ? (i >> 1) : i;
    float* redbuf = red + rb * red_per_buf + cw * kRedPerWarp;
    if constexpr (GROUPS) {
      float accA = 0.f, accB = 0.f;
      for (int sbl = cw; sbl < nsb_l; sbl += Wp)
        q4k_item_groups(sm, stage, sbl, gl, accA, accB);

      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&empty[s]);
      accA += __shfl_xor_sync(0xffffffffu, accA, 1);
      accA += __shfl_xor_sync(0xffffffffu, accA, 2);
      accB += __shfl_xor_sync(0xffffffffu, accB, 1);
      accB += __shfl_xor_sync(0xffffffffu, accB, 2);
      if (ruse >= 1 && !ptx::mbar_wait(&red_empty[rb], (ruse - 1) & 1)) {
        report_timeout(0x50000u);
        return;
      }
      if (tig == 0) {
        redbuf[gid] = accA;
        redbuf[gid + 8] = accB;
      }
    } else {
      float acc[NT][4];
      const bool partial_batch = sm.m < NTB;
      const bool uniform_scale = a.x16 != nullptr;
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[t][j] = 0.f;
      for (int sbl = cw; sbl < nsb_l; sbl += Wp)
        if (uniform_scale) {
          if (partial_batch) q4k_item_batch<NT, true, true>(sm, stage, sbl, lane, acc);
          else q4k_item_batch<NT, false, true>(sm, stage, sbl, lane, acc);
        } else {
          if (partial_batch) q4k_item_batch<NT, true, false>(sm, stage, sbl, lane, acc);
          else q4k_item_batch<NT, false, false>(sm, stage, sbl, lane, acc);
        }
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&empty[s]);
      if (ruse >= 1 && !ptx::mbar_wait(&red_empty[rb], (ruse - 1) & 1)) {
        report_timeout(0x50000u);
        return;
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        const int col = 8 * t + 2 * tig;
        redbuf[col * kTileRows + gid] = acc[t][0];
        redbuf[(col + 1) * kTileRows + gid] = acc[t][1];
        redbuf[col * kTileRows + gid + 8] = acc[t][2];
        redbuf[(col + 1) * kTileRows + gid + 8] = acc[t][3];
      }
    }
    __syncwarp();
    TB200_TRACE(ctid == 0 && i < 16, 24 + i);
    if (lane == 0) ptx::mbar_arrive(&red_full[rb]);
    if (++s == Sp) {
      s = 0;
      phase ^= 1;
    }
  }
  if (a.k_splits > 1) {
    if (!ptx::mbar_wait(fin, 0)) {
      report_timeout(0x70000u);
      return;
    }
    if (*reinterpret_cast<volatile int*>(&s_last)) add_partials(cw, W + 1);
  }
  cta_done();
}

template <int FMT, bool F16, int NT, bool GROUPS, bool WIDE>
__global__ void __launch_bounds__(WIDE ? kThreadsWide : kThreadsNarrow, WIDE ? 1 : 2)
    gemv_mma_kernel(const GemvArgs a, const __grid_constant__ CUtensorMap wmap) {
  gemv_mma_body<FMT, F16, NT, GROUPS>(a, &wmap);
}

inline int round_up(int v, int to) { return (v + to - 1) / to * to; }
inline int groups_limit(int slots, int splits) { return slots / splits; }
// as many decode warps as divide the super-blocks of a K range most evenly (ties: more warps)
inline int choose_warps(int sb_per_split, int max_warps) {
  int best_w = max_warps;
  double best_eff = 0;
  for (int w = max_warps; w >= 4; --w) {
    const int rounds = (sb_per_split + w - 1) / w;
    const double eff = (double)sb_per_split / (rounds * w) * (0.9 + 0.1 * w / max_warps);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best_w = w;
    }
  }
  return best_w;
}
// a tiled copy with 8-byte elements covers at most 256 elements = 2048 bytes per row
inline bool tma_ok(int fmt, int sb_per_split) { return sb_per_split * block_bytes(fmt) <= 2048; }

// smallest s >= bytes with s % 128 == want (want a multiple of 16)
inline int pad_stride(int bytes, int want) {
  int s = round_up(bytes, 16);
  while (s % 128 != want) s += 16;
  return s;
}

struct Layout {
  int stride_s, xs_stride, stage_bytes, off_stage, off_xs, off_sx, off_red, off_scl, off_zero, off_misc, total;
};

Layout make_layout(int fmt, int m, int sb_per_split, int stages, bool packed, int warps, int red_bufs) {
  const bool groups = m == 1;
  const int ntb = groups ? 1 : (m <= 8 ? 8 : 16);
  Layout L;
  L.stride_s = packed ? sb_per_split * block_bytes(fmt)
                          : pad_stride(sb_per_split * block_bytes(fmt), groups ? 64 : 32);
  L.xs_stride = pad_stride(sb_per_split * 512, 64);
  L.stage_bytes = kTileRows * L.stride_s;
  int off = 256;  // mbarriers: full[8], empty[8], consumer barrier, red_full[2], red_empty[2]
  L.off_stage = off;
  off += stages * L.stage_bytes;
  L.off_xs = off;
  off += (groups ? 1 : m) * L.xs_stride;  // only the live rows are kept
  L.off_sx = off;
  off += round_up(sb_per_split * 8 * ntb * 8, 128);  // {group sum, unscale} per group and column
  L.off_red = off;
  off += red_bufs * warps * ntb * kTileRows * 4;
  L.off_scl = off;
  off += groups ? 0 : warps * kTileRows * kSclRowFloats * 4;
  L.off_zero = off;  // zero bytes: the B fragments of lanes whose weights feed another column (m == 1)
  off += 512;        // or whose batch column is past m (one 16-byte load at each of the 8 group offsets)
  L.off_misc = off;  // the factor that undoes the activation scaling
  off += 64;
  L.total = round_up(off, 128);
  return L;
}

}  // namespace

// ---- static-shape entry used by generated .tbin wrappers ------------------------------------------
// A .tbin kernel is launched by the reference's provider with nothing but its declared buffers, so
// the launch plan is baked in as constants (GemvStatic) by the packaging step.
struct GemvStatic {
  int nsb, sb_per_split, k_splits, row_groups, row_tiles, stages, stride_s, xs_stride;
  int off_stage, off_xs, off_sx, off_red, off_scl, off_zero, off_misc, contiguous, use_tma, consumer_warps;
  int red_bufs;
};
template <int FMT, bool F16, int NT, bool GROUPS>
__device__ __forceinline__ void gemv_static_entry(const GemvStatic& s, const void* x, const uint8_t* w,
                                                  const CUtensorMap* wmap, float* out, unsigned char* scratch,
                                                  int m, long long n, int k, int counter_bytes) {
  GemvArgs a;
  a.x = x;
  a.w = w;
  a.outs[0] = out;
  a.n_out = 1;
  a.out_ld = n;
  a.out_vec = (n & 3) == 0;
  a.rank = 0;
  a.world = 1;
  a.sync = 0;
  a.x16 = nullptr;
  a.x_table = nullptr;
  a.x_unscale = nullptr;
  a.w2 = nullptr;
  a.n1 = n;
  a.counters = reinterpret_cast<unsigned int*>(scratch);
  a.partials = reinterpret_cast<float*>(scratch + counter_bytes);
  a.m = m;
  a.n = n;
  a.k = k;
  a.row_bytes = row_bytes(FMT, k);
  a.nsb = s.nsb;
  a.sb_per_split = s.sb_per_split;
  a.k_splits = s.k_splits;
  a.row_groups = s.row_groups;
  a.row_tiles = s.row_tiles;
  a.stages = s.stages;
  a.stride_s = s.stride_s;
  a.xs_stride = s.xs_stride;
  a.off_stage = s.off_stage;
  a.off_xs = s.off_xs;
  a.off_sx = s.off_sx;
  a.off_red = s.off_red;
  a.off_scl = s.off_scl;
  a.off_zero = s.off_zero;
  a.off_misc = s.off_misc;
  a.contiguous = s.contiguous;
  a.use_tma = s.use_tma;
  a.consumer_warps = s.consumer_warps;
  a.red_bufs = s.red_bufs;
  gemv_mma_body<FMT, F16, NT, GROUPS>(a, wmap);
}

#ifndef TB200_TBIN_WRAPPER
TB200_DEFINE_STATUS_READER(read_gemv_status)

GemvPlan plan_gemv_fast(int fmt, int xt, long long m, long long n, long long k,
                        long long scratch_bytes_available, const DeviceInfo& dev, bool allow_prep,
                        const Schedule* sched) {
  GemvPlan best;
  if (!sched) sched = lookup_schedule(kOpGemv, fmt, m, n, k);
  const Schedule none{};
  if (!sched) sched = &none;
  if (fmt != kQ4_K) return best;
  if (xt != kBF16 && xt != kF16) return best;
  if (m < 1 || m > 16 || n < 1 || k < 256 || k % 256 || k > (1 << 24)) return best;
  const long long rb = row_bytes(fmt, k);
  if (rb % 16) return best;
  const int nsb = (int)(k / 256);
  const long long row_tiles = (n + kTileRows - 1) / kTileRows;
  if (row_tiles > 0x7fffffffLL) return best;
  // converted activations + table, placed after the counters and the partial sums
  const int ntb = m <= 8 ? 8 : 16;
  const long long prep_x_bytes = (m * k * 2 + 255) / 256 * 256;
  // (measured at batch 4 and 8 as well: the extra launch, which starts while the previous kernel
  // drains, costs less than every CTA converting its K range: 48.6 -> 46.9 us for gate+up and down)
  const bool ahead = allow_prep && m > 1 && sched->convert_ahead != 2;
  const long long prep_bytes = ahead ? prep_x_bytes + ((k / 32) * ntb * 8 + 255) / 256 * 256 : 0;
  double best_cost = 1e300;
  const int force_splits = sched->k_splits, force_per_sm = sched->ctas_per_sm;
  if (force_splits < 0 || force_per_sm < 0 || force_per_sm > 2) return best;
  // Two CTAs per SM hide each other's barriers and reductions when the shared memory allows it.
  for (int per_sm = 2; per_sm >= 1; --per_sm) {
    if (force_per_sm && per_sm != force_per_sm) continue;
    const int slots = dev.sm_count * per_sm;
    const int smem_limit = per_sm == 1 ? dev.max_smem_optin : (dev.max_smem_optin + 1024) / 2 - 1024;
    for (int splits = 1; splits <= nsb && splits <= 64; ++splits) {
      if (force_splits && splits != force_splits) continue;
      const int per = (nsb + splits - 1) / splits;
      if ((splits - 1) * per >= nsb) continue;  // an empty K range
      const long long need =
          splits > 1 ? (kCounterBytes + (long long)splits * m * n * 4) : 0;
      if (need > scratch_bytes_available) continue;
      int stages = 0, red_bufs = 2;
      const int warps = choose_warps(per, per_sm == 1 ? kMaxConsumerWarps : kNarrowWarps);
      Layout L{};
      // two partial-sum buffers when that still leaves a ring of four stages, else whichever
      // choice gives the deeper ring
      for (int rbufs = 2; rbufs >= 1 && stages < 4; --rbufs)
        for (int s = kMaxStages; s > stages && s >= 2; --s) {
          const Layout cand = make_layout(fmt, (int)m, per, s, splits == 1 || tma_ok(fmt, per), warps, rbufs);
          if (cand.total <= smem_limit) {
            L = cand;
            stages = s;
            red_bufs = rbufs;
            break;
          }
        }
      if (!stages) continue;
      // splitting K so finely that the ring holds little data cannot keep HBM busy
      if (splits > 1 && (long long)stages * L.stage_bytes * per_sm < 96 * 1024 && stages < kMaxStages) continue;
      if (groups_limit(slots, splits) > 1024) continue;
      int groups = (int)((long long)slots / splits < row_tiles ? slots / splits : row_tiles);
      if (groups < 1) continue;
      const long long tiles_per_cta = (row_tiles + groups - 1) / groups;
      // time ~ bytes the busiest SM streams, plus the partial-sum traffic and sync of a split
      double cost = (double)per_sm * tiles_per_cta * per * block_bytes(fmt) * kTileRows;
      if (splits > 1) cost += per_sm * ((double)tiles_per_cta * kTileRows * m * 4 * 2 + 2000.0 * tiles_per_cta);
      // ... and the latency of its extra phase (partial sums out, counter, the last CTA's sum): about 2 us,
      // in bytes an SM streams meanwhile (fewer at larger batches, where the decode sets the pace).  Measured
      // at batch 1: 3072 x 4096 runs 4.4 us unsplit and 11.6 us on the split this term now rules out.
      if (splits > 1) cost += m == 1 ? 50000.0 : m <= 4 ? 40000.0 : m <= 8 ? 30000.0 : 20000.0;
      // per-row bulk copies of ~2 KB run far below HBM speed (each costs a few hundred cycles)
      if (splits > 1 && !tma_ok(fmt, per)) cost *= 3.0;
      // the decode warps are latency-bound: a second CTA on the SM is worth more than a perfect split
      if (per_sm == 1 && m == 1) cost *= 1.3;
      if (cost < best_cost) {
        best_cost = cost;
        best.supported = true;
        best.k_splits = splits;
        best.row_groups = groups;
        best.sb_per_split = per;
        best.stages = stages;
        best.stage_bytes = L.stage_bytes;
        best.smem_bytes = L.total;
        best.scratch_bytes = need;
        best.prep_x_offset = best.prep_table_offset = 0;
        if (prep_bytes) {
          const long long base = need ? need : kCounterBytes;  // keep the counter page even without a split
          if (base + prep_bytes <= scratch_bytes_available) {
            best.prep_x_offset = base;
            best.prep_table_offset = base + prep_x_bytes;
            best.scratch_bytes = base + prep_bytes;
          }
        }
        best.ctas_per_sm = per_sm;
        best.consumer_warps = warps;
        best.red_bufs = red_bufs;
        best.overlap = sched->overlap == 2 ? 0 : 1;
      }
    }
  }
  // a caller that asked for conversion ahead of the launch must have got it
  if (best.supported && sched->convert_ahead == 1 && m > 1 && !best.prep_x_offset) best.supported = false;
  return best;
}

#ifdef TB200_GEMV_TRACE
// Trace builds: a pinned host buffer the traced CTAs stamp, printed when the process exits.
static unsigned long long* gemv_trace_buffer() {
    static unsigned long long* host = nullptr;
    if (!host) {
      cudaHostAlloc((void**)&host, 80 * 8 * 8, cudaHostAllocMapped);
      memset(host, 0, 80 * 8 * 8);
      atexit([] {
        for (int c = 0; c < 3; ++c) {
          const unsigned long long* d = host + c * 80;
          if (!d[0]) continue;
          printf("trace cta %d (start %llu): dependency resolved +%llu ns, activations landed +%llu ns, staged +%llu ns; conversion rounds at +%llu +%llu +%llu +%llu; last warp out +%llu\n",
                 c * 100, d[0] % 1000000ull, d[7] ? d[7] - d[0] : 0ull, d[2] ? d[2] - d[0] : 0ull, d[1] - d[0], d[3] - d[0], d[4] - d[0], d[5] - d[0], d[6] - d[0],
                 d[72] ? d[72] - d[0] : 0ull);
          for (int i = 0; i < 16 && d[8 + i]; ++i)
            printf("  tile %2d: copy issued +%6llu  data ready +%6llu  decoded +%6llu  reduced +%6llu\n", i,
                   d[56 + i] - d[0], d[8 + i] - d[0], d[24 + i] - d[0], d[40 + i] - d[0]);
        }
      });
    }
    return host;
}
#endif

template <int FMT, bool F16, int NT, bool GROUPS, bool WIDE>
static cudaError_t launch_variant(GemvArgs& a, int grid, int smem, cudaStream_t stream, bool overlap) {
  auto kernel = gemv_mma_kernel<FMT, F16, NT, GROUPS, WIDE>;
  cudaError_t e = allow_full_shared_memory(kernel);
  if (e != cudaSuccess) return e;
  alignas(64) CUtensorMap wmap;
  memset(&wmap, 0, sizeof(wmap));
  if (a.use_tma) {
    // the weight as [n rows] x [row_bytes / 8] opaque 8-byte words; box = K range x 16 rows
    const unsigned box_inner = (unsigned)(a.sb_per_split * Fmt<FMT>::kBytes / 8);
    if (!make_tensor_map_2d(&wmap, TmaType::kU64, a.w, (unsigned long long)a.row_bytes / 8, (unsigned long long)a.n,
                            (unsigned long long)a.row_bytes, box_inner, kTileRows, false))
      return cudaErrorNotSupported;
  }
  // Programmatic serialization: this kernel may start (barrier setup, filling its weight ring)
  // while the previous kernel on the stream drains; it waits for that kernel before it touches
  // activations, outputs or scratch.  Works the same inside a stream capture.
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)((a.consumer_warps + 2) * 32));
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, a, wmap);
}

static int fill_args(GemvArgs& a, const GemvPlan& plan, int fmt, long long m, long long n, long long k);

bool gemv_launch_config(const GemvPlan& plan, int fmt, long long m, long long n, long long k, int* out32) {
  if (!plan.supported || fmt != kQ4_K) return false;
  GemvArgs a{};
  const int smem = fill_args(a, plan, fmt, m, n, k);
  const int vals[] = {plan.k_splits * plan.row_groups, (a.consumer_warps + 2) * 32, smem, a.k_splits, a.row_groups, a.row_tiles,
                      a.sb_per_split, a.nsb, a.stages, a.stride_s, a.xs_stride, a.off_stage, a.off_xs, a.off_sx,
                      a.off_red, a.off_scl, a.off_zero, a.off_misc, a.contiguous, a.use_tma, a.consumer_warps,
                      (int)(plan.scratch_bytes > 0x7fffffff ? 0x7fffffff : plan.scratch_bytes), plan.ctas_per_sm,
                      kCounterBytes, a.red_bufs};
  for (int i = 0; i < 32; ++i) out32[i] = i < (int)(sizeof(vals) / sizeof(int)) ? vals[i] : 0;
  return true;
}

cudaError_t launch_gemv_prepare_jobs(const PrepJobs& jobs, const PeerSync* peers, cudaStream_t stream) {
  if (jobs.count < 1) return cudaSuccess;
  if (jobs.count > kMaxPrepJobs) return cudaErrorInvalidValue;
  PrepJobsArg arg{};
  arg.jobs = jobs;
  arg.wait_limit_ns = peer_wait_limit_ns();
  if (peers && (peers->flags & kPeerWait)) {
    if (peers->world < 1 || peers->world > kMaxOutputs || peers->rank < 0 || peers->rank >= peers->world)
      return cudaErrorInvalidValue;
    arg.pad = peers->pads[peers->rank];
    arg.rank = peers->rank;
    arg.world = peers->world;
  }
  long long blocks = 0;
  for (int i = 0; i < jobs.count; ++i) blocks += jobs.job[i].blocks;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)blocks);
  cfg.blockDim = dim3(256);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemv_prepare_multi_kernel, arg);
}

cudaError_t launch_gemv_fast(const GemvPlan& plan, int fmt, int xt, const void* x, const uint8_t* w,
                             const OutSpec& out, long long m, long long n, long long k, void* scratch,
                             cudaStream_t stream, const PeerSync* peers, const uint8_t* w2, long long n1,
                             int prep_mode, PrepJobs* collect) {
  if (!plan.supported || fmt != kQ4_K) return cudaErrorInvalidValue;
  if (prep_mode == kPrepOnly && !plan.prep_x_offset) return cudaSuccess;  // this plan converts inside the GEMV
  // a second weight is fetched tile by tile from its own base: K must not be split (the split
  // path addresses rows through one tensor map) and the first weight must end on a tile boundary
  if (w2 && (plan.k_splits != 1 || n1 <= 0 || n1 >= n || n1 % kTileRows)) return cudaErrorInvalidValue;
  if (out.count < 1 || out.count > kMaxOutputs) return cudaErrorInvalidValue;
  if (out.ld < (w2 ? (n1 > n - n1 ? n1 : n - n1) : n)) return cudaErrorInvalidValue;
  GemvArgs a{};
  if (peers && peers->flags) {
    if (peers->world < 1 || peers->world > kMaxOutputs || peers->rank < 0 || peers->rank >= peers->world)
      return cudaErrorInvalidValue;
    for (int i = 0; i < peers->world; ++i) a.pads[i] = peers->pads[i];
    a.rank = peers->rank;
    a.world = peers->world;
    a.sync = peers->flags;
  }
  a.wait_limit_ns = peer_wait_limit_ns();
  const int smem_total = fill_args(a, plan, fmt, m, n, k);
  a.x = x;
  a.w = w;
  a.w2 = w2;
  a.n1 = w2 ? n1 : n;
  a.n_out = out.count;
  a.out_ld = out.ld;
  a.out_vec = (n & 3) == 0 && (out.ld & 3) == 0;
  for (int d = 0; d < out.count; ++d) {
    a.outs[d] = out.ptr[d];
    if (reinterpret_cast<uintptr_t>(out.ptr[d]) & 15) a.out_vec = 0;
    if (w2) {
      if (!out.ptr2[d]) return cudaErrorInvalidValue;
      a.outs2[d] = out.ptr2[d];
      if (reinterpret_cast<uintptr_t>(out.ptr2[d]) & 15) a.out_vec = 0;
    }
  }
#ifdef TB200_GEMV_TRACE
  a.trace = gemv_trace_buffer();
#endif
  if (plan.k_splits > 1) {
    if (!scratch) return cudaErrorInvalidValue;
    a.counters = static_cast<unsigned int*>(scratch);
    a.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + kCounterBytes);
  }
  if (plan.prep_x_offset) {
    if (!scratch || m < 2) return cudaErrorInvalidValue;
    uint16_t* x16 = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(scratch) + plan.prep_x_offset);
    float* table = reinterpret_cast<float*>(static_cast<uint8_t*>(scratch) + plan.prep_table_offset);
    const int ntb = m <= 8 ? 8 : 16;
    float* unscale = table + (k / 32) * ntb;  // behind the group sums (the region is sized for pairs)
    const long long threads = m * (k / 8);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)((threads + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = plan.overlap ? 1 : 0;
    const uint16_t* xin = static_cast<const uint16_t*>(x);
    if (prep_mode != kPrepDone && collect) {
      // the caller issues the collected conversions as one launch (launch_gemv_prepare_jobs)
      if (collect->count >= kMaxPrepJobs) return cudaErrorInvalidValue;
      PrepJob& job = collect->job[collect->count++];
      job.x = x;
      job.x16 = x16;
      job.table = table;
      job.unscale = unscale;
      job.m = (int)m;
      job.k = (int)k;
      job.ntb = ntb;
      job.f16 = xt == kF16;
      job.blocks = (int)cfg.gridDim.x;
    } else if (prep_mode != kPrepDone) {
      const unsigned int* pad = (a.sync & kPeerWait) ? a.pads[a.rank] : nullptr;
      cudaError_t e = xt == kF16 ? cudaLaunchKernelEx(&cfg, gemv_prepare_kernel<true>, xin, x16, table, unscale, (int)m,
                                                      (int)k, ntb, pad, a.rank, a.world, a.wait_limit_ns)
                                 : cudaLaunchKernelEx(&cfg, gemv_prepare_kernel<false>, xin, x16, table, unscale, (int)m,
                                                      (int)k, ntb, pad, a.rank, a.world, a.wait_limit_ns);
      if (e != cudaSuccess) return e;
    }
    if (prep_mode == kPrepOnly) return cudaSuccess;
    a.x16 = x16;
    a.x_table = table;
    a.x_unscale = unscale;
  }
  const int grid = plan.k_splits * plan.row_groups;
  const bool f16 = xt == kF16;
  const bool wide = plan.ctas_per_sm == 1;
#define TB200_GEMV_DISPATCH(NT, GROUPS)                                                                    \
  (f16 ? (wide ? launch_variant<kQ4_K, true, NT, GROUPS, true>(a, grid, smem_total, stream, plan.overlap != 0)   \
               : launch_variant<kQ4_K, true, NT, GROUPS, false>(a, grid, smem_total, stream, plan.overlap != 0)) \
       : (wide ? launch_variant<kQ4_K, false, NT, GROUPS, true>(a, grid, smem_total, stream, plan.overlap != 0)  \
               : launch_variant<kQ4_K, false, NT, GROUPS, false>(a, grid, smem_total, stream, plan.overlap != 0)))
  if (m == 1) return TB200_GEMV_DISPATCH(1, true);
  if (m <= 8) return TB200_GEMV_DISPATCH(1, false);
  return TB200_GEMV_DISPATCH(2, false);
#undef TB200_GEMV_DISPATCH
}

// Everything of GemvArgs that follows from the plan and the shape; returns the dynamic shared memory.
static int fill_args(GemvArgs& a, const GemvPlan& plan, int fmt, long long m, long long n, long long k) {
  a.m = (int)m;
  a.n = n;
  a.k = (int)k;
  a.row_bytes = row_bytes(fmt, k);
  a.nsb = (int)(k / 256);
  a.sb_per_split = plan.sb_per_split;
  a.k_splits = plan.k_splits;
  a.row_groups = plan.row_groups;
  a.row_tiles = (int)((n + kTileRows - 1) / kTileRows);
  a.stages = plan.stages;
  const bool tma = plan.k_splits > 1 && tma_ok(fmt, plan.sb_per_split);
  const Layout L = make_layout(fmt, (int)m, plan.sb_per_split, plan.stages, plan.k_splits == 1 || tma,
                               plan.consumer_warps, plan.red_bufs);
  a.contiguous = plan.k_splits == 1;
  a.use_tma = tma;
  a.stride_s = L.stride_s;
  a.xs_stride = L.xs_stride;
  a.off_stage = L.off_stage;
  a.off_xs = L.off_xs;
  a.off_sx = L.off_sx;
  a.off_red = L.off_red;
  a.off_scl = L.off_scl;
  a.off_zero = L.off_zero;
  a.off_misc = L.off_misc;
  a.consumer_warps = plan.consumer_warps;
  a.red_bufs = plan.red_bufs;
  return L.total;
}
#endif  // TB200_TBIN_WRAPPER

}  // namespace tb200
