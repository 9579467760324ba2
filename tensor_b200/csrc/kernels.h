// Internal launch interface between the C-ABI layer (cabi.cu) and the kernel files.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb200 {

struct DeviceInfo {
  int ordinal = -1;
  int sm_count = 0;
  int max_smem_optin = 0;
  int cc_major = 0, cc_minor = 0;
};
// Properties of the current device (cached per ordinal).  Returns nullptr on a CUDA error.
const DeviceInfo* device_info(cudaError_t* err);

// Opts a kernel in to the device's whole dynamic shared memory, once per kernel and device.  The
// attribute belongs to the function, not to a launch: setting it to each launch's own size would
// let a later, smaller plan shrink it under launches that were captured into a graph earlier (a
// replay of such a node as a plain launch is then checked against the smaller value and fails).
// Always the same value, so concurrent callers cannot undo one another.
cudaError_t allow_full_shared_memory(const void* kernel);
template <typename Kernel>
inline cudaError_t allow_full_shared_memory(Kernel* kernel) {
  return allow_full_shared_memory(reinterpret_cast<const void*>(kernel));
}

cudaError_t launch_dequant(int fmt, const uint8_t* w, float* out, long long n, long long k,
                           cudaStream_t stream);

// Where a GEMV writes its [m, n] result: element (row, col) goes to ptr[i][row * ld + col] for every
// i < count.  One destination with ld == n is the plain case; an N-sharded projection passes the
// same column window of every rank's full-width output (ptr[1..] are peer-mapped addresses), so
// the all-gather happens in the kernel's own stores.
constexpr int kMaxOutputs = 8;
struct OutSpec {
  float* ptr[kMaxOutputs];
  int count;
  long long ld;
  // grouped launches (two weights): where the second weight's columns go, column 0 of that weight
  // at ptr2[i][row * ld]; unused (null) for a single weight
  float* ptr2[kMaxOutputs];
};
inline OutSpec single_output(float* out, long long n) {
  OutSpec o{};
  o.ptr[0] = out;
  o.count = 1;
  o.ld = n;
  return o;
}

// SIMT fallback: any m, any K that is a multiple of the block size.  weights_bf16 rounds each
// decoded weight to bf16 first (the GEMM operand contract).
cudaError_t launch_gemv_simple(int fmt, int xt, const void* x, const uint8_t* w, const OutSpec& out,
                               long long m, long long n, long long k, bool weights_bf16,
                               cudaStream_t stream);
inline cudaError_t launch_gemv_simple(int fmt, int xt, const void* x, const uint8_t* w, float* out,
                                      long long m, long long n, long long k, bool weights_bf16,
                                      cudaStream_t stream) {
  return launch_gemv_simple(fmt, xt, x, w, single_output(out, n), m, n, k, weights_bf16, stream);
}

// A schedule: the launch choices a caller may pin instead of letting the library derive them.  Zero in
// a field means "derive".  Plays the role of the reference's schedule dictionaries
// (src/tensor/compiler/cuda/schedules.py:3-52).
struct Schedule {
  int k_splits = 0;       // GEMV: CTAs along K per row tile
  int ctas_per_sm = 0;    // GEMV: 1 or 2
  int convert_ahead = 0;  // GEMV, m > 1: 1 = activations converted by a kernel ahead of the GEMV, 2 = by every CTA
  int overlap = 0;        // 1 = launch with programmatic stream serialization (default), 2 = fully serialized
  int gemm_shape = 0;     // GEMM: 11, 12 or 22 = <256-token tiles per CTA, decode warp groups>
};
// Schedules recorded for a shape (by a search) that the default entry points consult; nullptr if none.
enum ScheduleOp : int { kOpGemv = 1, kOpGemm = 2 };
const Schedule* lookup_schedule(int op, int fmt, long long m, long long n, long long k);
void record_schedule(int op, int fmt, long long m, long long n, long long k, const Schedule& s);
void clear_schedules();

// Bulk-copy pipeline + mma.sync GEMV for m <= 16.
struct GemvPlan {
  bool supported = false;
  int k_splits = 1;        // CTAs along K per row tile
  int row_groups = 0;      // CTAs along N
  int sb_per_split = 0;    // 256-weight super-blocks per K range (last may be shorter)
  int stages = 0;
  int stage_bytes = 0;
  int smem_bytes = 0;
  long long scratch_bytes = 0;
  int ctas_per_sm = 1;
  int consumer_warps = 8;
  int red_bufs = 2;
  // Batch plans (1 < m <= 16) with scratch to spare: a small kernel ahead of the GEMV converts the
  // activations once (fp16, scaled per 32-value group, fragment order) and every CTA copies the
  // result, instead of every CTA converting all of them.  Offsets into the scratch buffer; 0 = the
  // CTAs convert on their own.
  long long prep_x_offset = 0;
  long long prep_table_offset = 0;
  int overlap = 1;  // 1: the launch may start while its predecessor drains (programmatic dependent launch)
};
// sched: pinned choices (nullptr: the schedule recorded for the shape, else derived).  A pinned choice
// that is not legal at the shape (shared memory, scratch, empty K ranges) yields supported == false.
GemvPlan plan_gemv_fast(int fmt, int xt, long long m, long long n, long long k,
                        long long scratch_bytes_available, const DeviceInfo& dev, bool allow_prep = true,
                        const Schedule* sched = nullptr);
// All launch constants of a plan (grid, threads, shared memory, ring layout ...): see tbin.py.
bool gemv_launch_config(const GemvPlan& plan, int fmt, long long m, long long n, long long k, int* out32);
// Cross-GPU ordering folded into a GEMV launch (N-sharded runs): pads[i] is rank i's signal pad as
// mapped here; flags bit 0 = wait for the peers before reading activations, bit 1 = signal the
// peers after the last output store.
constexpr int kPeerWait = 1, kPeerSignal = 2;
struct PeerSync {
  unsigned int* pads[kMaxOutputs];
  int rank;
  int world;
  int flags;
};
// How a plan that converts the activations ahead of the GEMV (m > 1) does so: with a launch of its own right
// before the GEMV (normal), only that launch (a list issues the conversions of all its projections first, so
// that its GEMVs follow one another directly), or not at all because that launch has been made already.
enum PrepMode : int { kPrepNormal = 0, kPrepOnly = 1, kPrepDone = 2 };
// With kPrepOnly and a collector the conversion is not launched but noted; launch_gemv_prepare_jobs then runs all
// noted conversions as one launch (which waits for the peers first where `peers` asks for it).
constexpr int kMaxPrepJobs = 12;
struct PrepJob {
  const void* x;   // [m, k] activations
  void* x16;       // converted activations, group sums and factors: inside the launch's scratch slice
  float* table;
  float* unscale;
  int m, k, ntb, f16, blocks;
};
struct PrepJobs {
  PrepJob job[kMaxPrepJobs];
  int count;
};
cudaError_t launch_gemv_prepare_jobs(const PrepJobs& jobs, const PeerSync* peers, cudaStream_t stream);
cudaError_t launch_gemv_fast(const GemvPlan& plan, int fmt, int xt, const void* x, const uint8_t* w,
                             const OutSpec& out, long long m, long long n, long long k, void* scratch,
                             cudaStream_t stream, const PeerSync* peers = nullptr, const uint8_t* w2 = nullptr,
                             long long n1 = 0, int prep_mode = kPrepNormal, PrepJobs* collect = nullptr);
// the first bytes of a GEMV scratch buffer: arrival counters that must read zero when a call starts
constexpr int kGemvCounterBytes = 4096;
constexpr int kGemvTileRows = 16;  // rows per weight tile of the pipelined GEMV (n1 of a grouped launch is a multiple)
inline cudaError_t launch_gemv_fast(const GemvPlan& plan, int fmt, int xt, const void* x, const uint8_t* w,
                                    float* out, long long m, long long n, long long k, void* scratch,
                                    cudaStream_t stream) {
  return launch_gemv_fast(plan, fmt, xt, x, w, single_output(out, n), m, n, k, scratch, stream);
}

// Persistent tcgen05 / TMEM GEMV over a list of projections (gemv_tc.cu): one launch (plus one small
// activation-conversion launch) serves up to kTcMaxItems independent GEMVs of one format, each with its
// own batch (1..16), shape and destinations.  x_share >= 0 names an earlier item of the list that
// reads the same activations (gate and up of an MLP): they are converted once.
constexpr int kTcMaxItems = 12;
struct TcLaunchItem {
  int fmt, xt;
  const void* x;
  const uint8_t* w;
  OutSpec out;
  long long m, n, k;
  int x_share;
};
// Q6_K and Q4_K at batch 1 on the integer dot-product units (gemv_dp4a.cu): activations as three exact 8-bit
// limbs; no scratch.
bool gemv_dp4a_supported(int fmt, int xt, long long m, long long n, long long k);
cudaError_t launch_gemv_dp4a(int fmt, int xt, const void* x, const uint8_t* w, const OutSpec& out, long long n,
                             long long k, cudaStream_t stream, const PeerSync* peers = nullptr);

bool gemv_tc_supported(int fmt, int xt, long long m, long long n, long long k);
// Scratch a list needs (arrival counters, partial sums of row tiles that span CTAs, converted
// activations); zero before the first use, 256-byte aligned.
long long gemv_tc_scratch_bytes(const TcLaunchItem* items, int count, const DeviceInfo& dev);
cudaError_t launch_gemv_tc(const TcLaunchItem* items, int count, void* scratch, long long scratch_bytes,
                           cudaStream_t stream, const PeerSync* peers = nullptr);
// How long a kernel waits for a peer GPU's signal before it records a status code and returns.
void set_peer_wait_limit_ns(unsigned long long ns);
unsigned long long peer_wait_limit_ns();

// The steps either side of a decode projection (glue.cu); every pointer 16-byte aligned, k and width
// multiples of 4.  All three are launched so that the kernel behind them may start early.
cudaError_t launch_rmsnorm(const float* x, const float* weight, void* out_bf16, long long m, long long k, float eps,
                           cudaStream_t stream);
cudaError_t launch_swiglu(const float* gate_up, void* out_bf16, long long m, long long width, cudaStream_t stream);
cudaError_t launch_residual_add(float* stream_buffer, const float* delta, long long count, cudaStream_t stream);

// Cross-GPU barrier over peer-mapped signal pads (one pad of kSignalWords uint32 per rank, zeroed
// once): every rank tells every peer that all work it enqueued before is complete and visible,
// then waits (bounded) until every peer has said the same.  pads[i] is rank i's pad as mapped here.
constexpr int kSignalWords = 64;
// mode: kPeerSignal | kPeerWait (a full barrier), or one of them alone
cudaError_t launch_peer_barrier(unsigned int* const* pads, int rank, int world, int mode, cudaStream_t stream);

// tcgen05 / TMEM prefill GEMM (bf16 operands, fp32 accumulate).
// {grid.x, grid.y, threads, dynamic shared memory, token tile, k per stage, 0, 0}
void gemm_launch_config(long long m, long long n, int* out8);
bool gemm_fast_supported(int fmt, long long m, long long n, long long k, const DeviceInfo& dev);
cudaError_t launch_gemm_fast(int fmt, const void* x, const uint8_t* w, float* out, long long m,
                             long long n, long long k, cudaStream_t stream, const char** detail,
                             const Schedule* sched = nullptr);
bool gemm_shape_legal(int shape, long long m, const DeviceInfo& dev);

// 2-D tiled TMA tensor map (128 bytes, 64-byte aligned) over a row-major matrix; elements are bf16
// or opaque 8-byte words.  Returns false if the driver entry point is unavailable or rejects it.
enum class TmaType { kBF16, kU64 };
bool make_tensor_map_2d(void* map_out, TmaType type, const void* base, unsigned long long inner,
                        unsigned long long outer, unsigned long long row_stride_bytes, unsigned box_inner,
                        unsigned box_outer, bool swizzle_128b);

// Sticky status words of the pipelined kernels (bounded waits that gave up); these synchronise.
// Base address and size of the device allocation that contains ptr (driver cuMemGetAddressRange).
bool allocation_range(const void* ptr, void** base, size_t* size);

cudaError_t read_gemv_status(unsigned int* value, bool clear);
cudaError_t read_gemv_tc_status(unsigned int* value, bool clear);
cudaError_t read_gemm_status(unsigned int* value, bool clear);
cudaError_t read_barrier_status(unsigned int* value, bool clear);

}  // namespace tb200
