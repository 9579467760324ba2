// C-ABI entry points of libtensor_b200_gguf.so (declared in include/tensor_b200_gguf.h).
//
// Layer 1: plain device pointers + sizes + stream.  Layer 2 (`*_v1`): the reference's
// `int32_t fn(const TensorCallV1*, TensorErrorV1*)` convention (src/tensor/include/tensor/abi.h:141),
// validated the way the reference's CPU image wrappers validate a call before touching data
// (src/tensor/compiler/cpu.py:60-155): abi version, struct size, argument count / kind / dtype,
// byte sizes, alignment, device.  Errors are status codes + a message, never C++ exceptions
// (abi.h:135-141).  There is no CPU fallback: every path below ends in a CUDA launch or an error.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <utility>
#include <vector>

#include "../../include/tensor_b200_gguf.h"
#include "common.cuh"
#include "kernels.h"

static_assert(sizeof(TensorBufferV1) == 48, "TensorBufferV1 layout");
static_assert(sizeof(TensorArgumentV1) == 64, "TensorArgumentV1 layout");
static_assert(sizeof(TensorStreamV1) == 16, "TensorStreamV1 layout");
static_assert(sizeof(TensorCallV1) == 72, "TensorCallV1 layout");
static_assert(sizeof(TensorErrorV1) == 512, "TensorErrorV1 layout");
static_assert(tb200::kPeerWait == TB200_PEER_WAIT && tb200::kPeerSignal == TB200_PEER_SIGNAL, "sync bits");
static_assert(tb200::kMaxOutputs == TB200_MAX_PEERS && tb200::kSignalWords * 4 == TB200_SIGNAL_PAD_BYTES, "peer limits");

namespace tb200 {

const DeviceInfo* device_info(cudaError_t* err) {
  static DeviceInfo table[64];
  static std::mutex lock;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess && (dev < 0 || dev >= 64)) e = cudaErrorInvalidDevice;
  if (e != cudaSuccess) {
    if (err) *err = e;
    return nullptr;
  }
  std::lock_guard<std::mutex> guard(lock);
  DeviceInfo& d = table[dev];
  if (d.ordinal != dev) {
    int sm = 0, smem = 0, major = 0, minor = 0;
    if ((e = cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev)) != cudaSuccess) {
      if (err) *err = e;
      return nullptr;
    }
    d.sm_count = sm;
    d.max_smem_optin = smem;
    d.cc_major = major;
    d.cc_minor = minor;
    d.ordinal = dev;
  }
  if (err) *err = cudaSuccess;
  return &d;
}

namespace {
struct ScheduleEntry {
  int op, fmt;
  long long m, n, k;
  Schedule schedule;
};
std::mutex g_schedule_lock;
std::vector<ScheduleEntry> g_schedules;  // entries are never moved once handed out: see record_schedule
}  // namespace

const Schedule* lookup_schedule(int op, int fmt, long long m, long long n, long long k) {
  std::lock_guard<std::mutex> guard(g_schedule_lock);
  for (const ScheduleEntry& e : g_schedules)
    if (e.op == op && e.fmt == fmt && e.m == m && e.n == n && e.k == k) return &e.schedule;
  return nullptr;
}
void record_schedule(int op, int fmt, long long m, long long n, long long k, const Schedule& s) {
  std::lock_guard<std::mutex> guard(g_schedule_lock);
  for (ScheduleEntry& e : g_schedules)
    if (e.op == op && e.fmt == fmt && e.m == m && e.n == n && e.k == k) {
      e.schedule = s;
      return;
    }
  if (g_schedules.capacity() == 0) g_schedules.reserve(4096);  // pointers handed out by lookup stay valid
  if (g_schedules.size() < g_schedules.capacity()) g_schedules.push_back(ScheduleEntry{op, fmt, m, n, k, s});
}
void clear_schedules() {
  std::lock_guard<std::mutex> guard(g_schedule_lock);
  for (ScheduleEntry& e : g_schedules) e.schedule = Schedule{};  // entries stay in place; "derive everything"
}

cudaError_t allow_full_shared_memory(const void* kernel) {
  static std::mutex lock;
  static std::vector<std::pair<const void*, int>> done;  // (kernel, device) pairs already opted in
  cudaError_t e;
  const DeviceInfo* dev = device_info(&e);
  if (!dev) return e;
  std::lock_guard<std::mutex> guard(lock);
  for (const auto& entry : done)
    if (entry.first == kernel && entry.second == dev->ordinal) return cudaSuccess;
  cudaFuncAttributes attr;
  e = cudaFuncGetAttributes(&attr, kernel);
  if (e != cudaSuccess) return e;
  // statically declared shared memory counts against the same limit
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           dev->max_smem_optin - (int)attr.sharedSizeBytes);
  if (e == cudaSuccess) done.emplace_back(kernel, dev->ordinal);
  return e;
}

}  // namespace tb200

namespace {

using namespace tb200;

int32_t fail(TensorErrorV1* error, int32_t code, const char* fmt, ...) {
  if (error) {
    error->code = code;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error->message, sizeof(error->message), fmt, ap);
    va_end(ap);
    error->message[sizeof(error->message) - 1] = 0;
  }
  return code;
}

int32_t ok(TensorErrorV1* error) {
  if (error) {
    error->code = TENSOR_OK;
    error->message[0] = 0;
  }
  return TENSOR_OK;
}

int32_t cuda_fail(TensorErrorV1* error, const char* what, cudaError_t e) {
  return fail(error, TENSOR_ERROR_PROVIDER, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

// The kernels are sm_100a-only; refuse anything else before a launch can fail obscurely.
int32_t require_device(TensorErrorV1* error, const DeviceInfo** out) {
  cudaError_t e;
  const DeviceInfo* dev = device_info(&e);
  if (!dev) return cuda_fail(error, "no usable CUDA device", e);
  if (dev->cc_major != 10)
    return fail(error, TENSOR_ERROR_PROVIDER,
                "device %d has compute capability %d.%d; this library is built for sm_100a only", dev->ordinal,
                dev->cc_major, dev->cc_minor);
  *out = dev;
  return TENSOR_OK;
}

int32_t check_shape(TensorErrorV1* error, int32_t format, int64_t m, int64_t n, int64_t k) {
  if (!valid_format(format))
    return fail(error, TENSOR_ERROR_ARGUMENT, "unknown GGUF format id %d (expected 2, 8, 12 or 14)", format);
  if (m < 0 || n < 0 || k < 0) return fail(error, TENSOR_ERROR_ARGUMENT, "negative extent m=%lld n=%lld k=%lld",
                                           (long long)m, (long long)n, (long long)k);
  if (k % block_weights(format))
    return fail(error, TENSOR_ERROR_ARGUMENT, "K=%lld is not a multiple of the block size %d of format %d",
                (long long)k, block_weights(format), format);
  if (k > (1ll << 30) || n > (1ll << 31) || m > (1ll << 24))
    return fail(error, TENSOR_ERROR_ARGUMENT, "extent too large: m=%lld n=%lld k=%lld", (long long)m,
                (long long)n, (long long)k);
  return TENSOR_OK;
}

int32_t check_pointer(TensorErrorV1* error, const char* name, const void* p, size_t alignment, bool needed) {
  if (!p && needed) return fail(error, TENSOR_ERROR_ARGUMENT, "%s is NULL", name);
  if (reinterpret_cast<uintptr_t>(p) % alignment)
    return fail(error, TENSOR_ERROR_ARGUMENT, "%s (%p) is not %zu-byte aligned", name, p, alignment);
  return TENSOR_OK;
}

int dtype_bytes(int32_t dtype) {
  switch (dtype) {
    case TENSOR_FLOAT16:
    case TENSOR_BFLOAT16: return 2;
    case TENSOR_FLOAT32: return 4;
    case TENSOR_UINT8: return 1;
  }
  return 0;
}

}  // namespace

extern "C" {

int32_t tb200_gguf_version(void) { return (1 << 16) | 0; }

int64_t tb200_gguf_weight_bytes(int32_t format, int64_t n, int64_t k) {
  if (!valid_format(format) || n < 0 || k < 0 || k % block_weights(format)) return -1;
  return n * row_bytes(format, k);
}

int64_t tb200_gguf_gemv_scratch_bytes(int32_t format, int64_t m, int64_t n, int64_t k) {
  if (!valid_format(format) || m < 1 || n < 1 || k < 0 || k % block_weights(format)) return 0;
  cudaError_t e;
  const DeviceInfo* dev = device_info(&e);
  if (!dev) return 0;
  // The plan does not depend on the 2-byte activation type.
  GemvPlan plan = plan_gemv_fast(format, kBF16, m, n, k, (long long)1 << 40, *dev);
  if (plan.supported) return plan.scratch_bytes;
  if (format == kQ6_K && gemv_tc_supported(format, kBF16, m, n, k)) {  // served by the tensor-memory kernel
    TcLaunchItem item{};
    item.fmt = format;
    item.xt = kBF16;
    item.m = m;
    item.n = n;
    item.k = k;
    item.x_share = -1;
    return gemv_tc_scratch_bytes(&item, 1, *dev);
  }
  return 0;
}

int32_t tb200_gguf_gemv_plan(int32_t format, int64_t m, int64_t n, int64_t k, int64_t scratch_bytes,
                             int32_t* plan_out) {
  if (!plan_out) return TENSOR_ERROR_ARGUMENT;
  for (int i = 0; i < 8; ++i) plan_out[i] = 0;
  if (!valid_format(format) || m < 1 || n < 1 || k < 0 || k % block_weights(format)) return TENSOR_ERROR_ARGUMENT;
  DeviceInfo b200;  // without a device, plan for a B200: 148 SMs, 227 KB of opt-in shared memory
  b200.ordinal = 0;
  b200.sm_count = 148;
  b200.max_smem_optin = 232448;
  b200.cc_major = 10;
  cudaError_t e;
  const DeviceInfo* dev = device_info(&e);
  if (!dev) {
    cudaGetLastError();
    dev = &b200;
  }
  GemvPlan plan = plan_gemv_fast(format, kBF16, m, n, k, scratch_bytes, *dev);
  plan_out[0] = plan.supported ? 1 : 0;
  plan_out[1] = plan.k_splits;
  plan_out[2] = plan.row_groups;
  plan_out[3] = plan.sb_per_split;
  plan_out[4] = plan.stages;
  plan_out[5] = plan.smem_bytes;
  plan_out[6] = (int32_t)(plan.scratch_bytes > 0x7fffffff ? 0x7fffffff : plan.scratch_bytes);
  plan_out[7] = plan.ctas_per_sm;
  return TENSOR_OK;
}

int32_t tb200_gguf_gemv_launch_config(int32_t format, int32_t x_dtype, int64_t m, int64_t n, int64_t k,
                                      int64_t scratch_bytes, int32_t* out32) {
  if (!out32) return TENSOR_ERROR_ARGUMENT;
  if (!valid_format(format) || m < 1 || n < 1 || k < 0 || k % block_weights(format)) return TENSOR_ERROR_ARGUMENT;
  DeviceInfo b200;  // packaging usually happens on a machine without a GPU: plan for a B200
  b200.ordinal = 0;
  b200.sm_count = 148;
  b200.max_smem_optin = 232448;
  b200.cc_major = 10;
  // a packaged kernel is a single launch: no conversion kernel ahead of it
  GemvPlan plan = plan_gemv_fast(format, x_dtype, m, n, k, scratch_bytes, b200, false);
  return gemv_launch_config(plan, format, m, n, k, out32) ? TENSOR_OK : TENSOR_ERROR_ARGUMENT;
}

int32_t tb200_gguf_gemm_launch_config(int32_t format, int64_t m, int64_t n, int64_t k, int32_t* out8) {
  if (!out8) return TENSOR_ERROR_ARGUMENT;
  DeviceInfo b200;
  b200.ordinal = 0;
  b200.sm_count = 148;
  b200.max_smem_optin = 232448;
  b200.cc_major = 10;
  if (!gemm_fast_supported(format, m, n, k, b200)) return TENSOR_ERROR_ARGUMENT;
  gemm_launch_config(m, n, out8);
  return TENSOR_OK;
}

int32_t tb200_gguf_device_status(uint32_t* status, TensorErrorV1* error) {
  unsigned int a = 0, b = 0, c = 0, t = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return cuda_fail(error, "cudaDeviceSynchronize", e);
  if ((e = read_gemv_tc_status(&t, true)) != cudaSuccess) return cuda_fail(error, "reading GEMV status", e);
  if ((e = read_gemv_status(&a, true)) != cudaSuccess) return cuda_fail(error, "reading GEMV status", e);
  if (!a) a = t;
  if ((e = read_gemm_status(&b, true)) != cudaSuccess) return cuda_fail(error, "reading GEMM status", e);
  if ((e = read_barrier_status(&c, true)) != cudaSuccess) return cuda_fail(error, "reading barrier status", e);
  if (status) *status = a ? a : (b ? b : c);
  if (a || b || c)
    return fail(error, TENSOR_ERROR_PROVIDER,
                "a bounded device-side wait gave up (gemv 0x%x, gemm 0x%x, peer barrier 0x%x)", a, b, c);
  return ok(error);
}

int32_t tb200_gguf_dequant(int32_t format, const void* w, float* out, int64_t n, int64_t k, void* stream,
                           TensorErrorV1* error) {
  if (int32_t s = check_shape(error, format, 0, n, k)) return s;
  if (n == 0 || k == 0) return ok(error);
  if (int32_t s = check_pointer(error, "w", w, 2, true)) return s;
  if (int32_t s = check_pointer(error, "out", out, 16, true)) return s;
  const DeviceInfo* dev;
  if (int32_t s = require_device(error, &dev)) return s;
  cudaError_t e = launch_dequant(format, static_cast<const uint8_t*>(w), out, n, k, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(error, "dequant launch", e);
  return ok(error);
}

}  // extern "C"

namespace {
// Shared by the plain and the sharded entry points: `out` says where the [m, n] result goes.
int32_t gemv_common(int32_t format, int32_t x_dtype, const void* x, const void* w, const OutSpec& out, int64_t m,
                    int64_t n, int64_t k, void* scratch, int64_t scratch_bytes, int32_t variant, void* stream,
                    TensorErrorV1* error, const PeerSync* peers = nullptr, const Schedule* sched = nullptr,
                    int prep_mode = kPrepNormal, PrepJobs* collect = nullptr) {
  if (int32_t s = check_pointer(error, "x", x, 16, k > 0)) return s;
  if (int32_t s = check_pointer(error, "w", w, 16, k > 0)) return s;
  for (int i = 0; i < out.count; ++i)
    if (int32_t s = check_pointer(error, "out", out.ptr[i], 4, true)) return s;
  if (int32_t s = check_pointer(error, "scratch", scratch, 256, false)) return s;
  if (scratch_bytes < 0) return fail(error, TENSOR_ERROR_ARGUMENT, "negative scratch size");
  const DeviceInfo* dev;
  if (int32_t s = require_device(error, &dev)) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* wp = static_cast<const uint8_t*>(w);
  if (prep_mode == kPrepOnly) {
    // only the conversion launch of the pipelined kernel, where this call would take that kernel and its plan
    // converts ahead (the same conditions as below lead there)
    if (format != kQ4_K || m < 2 || variant == TB200_VARIANT_SIMPLE || variant == TB200_VARIANT_TC ||
        variant == TB200_VARIANT_DP4A)
      return ok(error);
    GemvPlan plan = plan_gemv_fast(format, x_dtype, m, n, k, scratch ? scratch_bytes : 0, *dev, true, sched);
    if (plan.supported) {
      cudaError_t e = launch_gemv_fast(plan, format, x_dtype, x, wp, out, m, n, k, scratch, st, peers, nullptr, 0, kPrepOnly,
                                       collect);
      if (e != cudaSuccess) return cuda_fail(error, "activation conversion launch", e);
    }
    return ok(error);
  }
  // Batch 1 of Q6_K, Q8_0 and Q4_0 (and of Q4_K on request, variant "dp4a"): the integer dot-product kernel,
  // measured about 2.4 times as fast as the tensor-memory kernel for Q6_K (for Q4_K the mma.sync pipeline stays
  // ahead; FAST / MMA still name the bulk-copy ring for the formats it covers).
  const bool dp_default = (format == kQ6_K && (variant == TB200_VARIANT_AUTO || variant == TB200_VARIANT_FAST)) ||
                          ((format == kQ8_0 || format == kQ4_0) && variant == TB200_VARIANT_AUTO);
  if ((dp_default || variant == TB200_VARIANT_DP4A) && gemv_dp4a_supported(format, x_dtype, m, n, k)) {
    cudaError_t e = launch_gemv_dp4a(format, x_dtype, x, wp, out, n, k, st, peers);
    if (e == cudaSuccess) return ok(error);
    if (e != cudaErrorInvalidValue) return cuda_fail(error, "integer dot-product GEMV launch", e);
  }
  if (variant == TB200_VARIANT_DP4A)
    return fail(error, TENSOR_ERROR_ARGUMENT,
                "the integer dot-product GEMV takes m = 1 with 2-byte activations, K a multiple of 256 "
                "(2048 for Q6_K) up to 32768 (format %d, dtype %d, m=%lld, n=%lld, k=%lld)",
                format, x_dtype, (long long)m, (long long)n, (long long)k);
  // The tensor-memory kernel: on request, and by default for Q6_K, which has no other pipelined GEMV
  // (measured 1.0x .. 10x faster than the SIMT kernels there).  For Q4_K it is measured slower than the
  // mma.sync pipeline at every batch on B200, so the default never picks it.
  const bool tc_default = format == kQ6_K && (variant == TB200_VARIANT_AUTO || variant == TB200_VARIANT_FAST) &&
                          gemv_tc_supported(format, x_dtype, m, n, k);
  if (variant == TB200_VARIANT_TC || tc_default) {
    TcLaunchItem item{};
    item.fmt = format;
    item.xt = x_dtype;
    item.x = x;
    item.w = wp;
    item.out = out;
    item.m = m;
    item.n = n;
    item.k = k;
    item.x_share = -1;
    const long long need = gemv_tc_scratch_bytes(&item, 1, *dev);  // 0: the shape is not covered
    if (need && scratch && scratch_bytes >= need) {
      cudaError_t e = launch_gemv_tc(&item, 1, scratch, scratch_bytes, st, peers);
      if (e != cudaSuccess) return cuda_fail(error, "tensor-memory GEMV launch", e);
      return ok(error);
    }
    if (variant == TB200_VARIANT_TC)
    return fail(error, TENSOR_ERROR_ARGUMENT,
                "the tensor-memory GEMV needs format 12 or 14 (K a multiple of 2048), 2-byte activations, m <= 16 and %lld bytes of scratch "
                "(format %d, dtype %d, m=%lld, n=%lld, k=%lld, scratch %lld)",
                need, format, x_dtype, (long long)m, (long long)n, (long long)k,
                (long long)(scratch ? scratch_bytes : 0));
  }
  if (variant != TB200_VARIANT_SIMPLE) {
    GemvPlan plan = plan_gemv_fast(format, x_dtype, m, n, k, scratch ? scratch_bytes : 0, *dev, true, sched);
    if (plan.supported) {
      // (a conversion launch reads the activations ahead of the GEMV's folded wait: it carries the wait too)
      cudaError_t e = launch_gemv_fast(plan, format, x_dtype, x, wp, out, m, n, k, scratch, st, peers, nullptr, 0, prep_mode);
      if (e != cudaSuccess) return cuda_fail(error, "pipelined GEMV launch", e);
      return ok(error);
    }
    if (sched)
      return fail(error, TENSOR_ERROR_ARGUMENT,
                  "the schedule {k_splits %d, ctas_per_sm %d, convert_ahead %d} is not legal for format %d, m=%lld, "
                  "n=%lld, k=%lld with %lld bytes of scratch", sched->k_splits, sched->ctas_per_sm, sched->convert_ahead,
                  format, (long long)m, (long long)n, (long long)k, (long long)(scratch ? scratch_bytes : 0));
    if (variant == TB200_VARIANT_FAST || variant == TB200_VARIANT_MMA)
      return fail(error, TENSOR_ERROR_ARGUMENT,
                  "the pipelined GEMV does not cover format %d, dtype %d, m=%lld, n=%lld, k=%lld", format, x_dtype,
                  (long long)m, (long long)n, (long long)k);
  }
  // the fallback kernel knows nothing of peers: order it with separate launches
  if (peers && (peers->flags & kPeerWait)) {
    cudaError_t e = launch_peer_barrier(peers->pads, peers->rank, peers->world, kPeerWait, st);
    if (e != cudaSuccess) return cuda_fail(error, "peer wait launch", e);
  }
  cudaError_t e = launch_gemv_simple(format, x_dtype, x, wp, out, m, n, k, false, st);
  if (e != cudaSuccess) return cuda_fail(error, "GEMV launch", e);
  if (peers && (peers->flags & kPeerSignal)) {
    e = launch_peer_barrier(peers->pads, peers->rank, peers->world, kPeerSignal, st);
    if (e != cudaSuccess) return cuda_fail(error, "peer signal launch", e);
  }
  return ok(error);
}

int32_t check_pads(TensorErrorV1* error, uint32_t* const* pads, int32_t rank, int32_t world) {
  if (!pads) return fail(error, TENSOR_ERROR_ARGUMENT, "pads is null");
  if (world < 1 || world > TB200_MAX_PEERS || rank < 0 || rank >= world)
    return fail(error, TENSOR_ERROR_ARGUMENT, "rank %d of world %d (at most %d ranks)", rank, world, TB200_MAX_PEERS);
  for (int i = 0; i < world; ++i)
    if (int32_t s = check_pointer(error, "pad", pads[i], 4, true)) return s;
  return TENSOR_OK;
}

int32_t check_gemv_scalars(TensorErrorV1* error, int32_t format, int32_t x_dtype, int64_t m, int64_t n, int64_t k,
                           int32_t variant) {
  if (int32_t s = check_shape(error, format, m, n, k)) return s;
  if (x_dtype != TENSOR_FLOAT16 && x_dtype != TENSOR_BFLOAT16 && x_dtype != TENSOR_FLOAT32)
    return fail(error, TENSOR_ERROR_ARGUMENT, "activation dtype %d is not float16, bfloat16 or float32", x_dtype);
  if (variant < 0 || variant > TB200_VARIANT_DP4A) return fail(error, TENSOR_ERROR_ARGUMENT, "unknown variant %d", variant);
  return TENSOR_OK;
}

// Several projections as ONE persistent launch of the tensor-memory kernel; false if the list does
// not qualify (the caller then launches them one by one).
bool try_list(const TcLaunchItem* items, int count, void* scratch, int64_t scratch_bytes, const DeviceInfo& dev,
              cudaStream_t st, const PeerSync* peers, cudaError_t* launch_error) {
  *launch_error = cudaSuccess;
  const long long need = gemv_tc_scratch_bytes(items, count, dev);
  if (!need || !scratch || scratch_bytes < need) return false;
  *launch_error = launch_gemv_tc(items, count, scratch, scratch_bytes, st, peers);
  return true;
}
}  // namespace

extern "C" {

int32_t tb200_gguf_gemv(int32_t format, int32_t x_dtype, const void* x, const void* w, float* out, int64_t m,
                        int64_t n, int64_t k, void* scratch, int64_t scratch_bytes, int32_t variant, void* stream,
                        TensorErrorV1* error) {
  if (int32_t s = check_gemv_scalars(error, format, x_dtype, m, n, k, variant)) return s;
  if (m == 0 || n == 0) return ok(error);
  return gemv_common(format, x_dtype, x, w, single_output(out, n), m, n, k, scratch, scratch_bytes, variant, stream,
                     error);
}

static int32_t gemv_sharded_impl(int32_t format, int32_t x_dtype, const void* x, const void* w,
                                 float* const* outs, int32_t out_count, int64_t out_ld, int64_t col_offset,
                                 int64_t m, int64_t n, int64_t k, void* scratch, int64_t scratch_bytes,
                                 int32_t variant, uint32_t* const* pads, int32_t rank, int32_t world,
                                 int32_t sync, void* stream, TensorErrorV1* error, int prep_mode,
                                 PrepJobs* collect = nullptr) {
  if (int32_t s = check_gemv_scalars(error, format, x_dtype, m, n, k, variant)) return s;
  if (!outs) return fail(error, TENSOR_ERROR_ARGUMENT, "outs is null");
  if (out_count < 1 || out_count > TB200_MAX_PEERS)
    return fail(error, TENSOR_ERROR_ARGUMENT, "out_count %d is not in 1..%d", out_count, TB200_MAX_PEERS);
  if (col_offset < 0 || out_ld < col_offset + n)
    return fail(error, TENSOR_ERROR_ARGUMENT, "columns %lld..%lld do not fit a row of %lld", (long long)col_offset,
                (long long)(col_offset + n), (long long)out_ld);
  if (sync & ~(TB200_PEER_WAIT | TB200_PEER_SIGNAL)) return fail(error, TENSOR_ERROR_ARGUMENT, "unknown sync bits 0x%x", sync);
  PeerSync peers{};
  if (sync) {
    if (int32_t s = check_pads(error, pads, rank, world)) return s;
    for (int i = 0; i < world; ++i) peers.pads[i] = pads[i];
    peers.rank = rank;
    peers.world = world;
    peers.flags = world > 1 ? sync : 0;
  }
  OutSpec spec{};
  spec.count = out_count;
  spec.ld = out_ld;
  for (int i = 0; i < out_count; ++i) {
    if (!outs[i]) return fail(error, TENSOR_ERROR_ARGUMENT, "outs[%d] is null", i);
    spec.ptr[i] = outs[i] + col_offset;
  }
  if (m == 0 || n == 0) {
    // nothing to compute, but the peers still count on this rank's signal
    if (peers.flags) {
      const DeviceInfo* dev;
      if (int32_t s = require_device(error, &dev)) return s;
      cudaError_t e = launch_peer_barrier(peers.pads, rank, world, peers.flags, static_cast<cudaStream_t>(stream));
      if (e != cudaSuccess) return cuda_fail(error, "peer sync launch", e);
    }
    return ok(error);
  }
  return gemv_common(format, x_dtype, x, w, spec, m, n, k, scratch, scratch_bytes, variant, stream, error,
                     peers.flags ? &peers : nullptr, nullptr, prep_mode, collect);
}

int32_t tb200_gguf_gemv_sharded_sync(int32_t format, int32_t x_dtype, const void* x, const void* w,
                                     float* const* outs, int32_t out_count, int64_t out_ld, int64_t col_offset,
                                     int64_t m, int64_t n, int64_t k, void* scratch, int64_t scratch_bytes,
                                     int32_t variant, uint32_t* const* pads, int32_t rank, int32_t world,
                                     int32_t sync, void* stream, TensorErrorV1* error) {
  return gemv_sharded_impl(format, x_dtype, x, w, outs, out_count, out_ld, col_offset, m, n, k, scratch, scratch_bytes,
                           variant, pads, rank, world, sync, stream, error, kPrepNormal);
}

int32_t tb200_gguf_gemv_sharded(int32_t format, int32_t x_dtype, const void* x, const void* w, float* const* outs,
                                int32_t out_count, int64_t out_ld, int64_t col_offset, int64_t m, int64_t n,
                                int64_t k, void* scratch, int64_t scratch_bytes, int32_t variant, void* stream,
                                TensorErrorV1* error) {
  return tb200_gguf_gemv_sharded_sync(format, x_dtype, x, w, outs, out_count, out_ld, col_offset, m, n, k, scratch,
                                      scratch_bytes, variant, nullptr, 0, 1, 0, stream, error);
}

int32_t tb200_gguf_gemv_pair(int32_t format, int32_t x_dtype, const void* x, const void* w1, int64_t n1,
                             const void* w2, int64_t n2, float* out, int64_t m, int64_t k, void* scratch,
                             int64_t scratch_bytes, int32_t variant, void* stream, TensorErrorV1* error) {
  if (int32_t s = check_gemv_scalars(error, format, x_dtype, m, n1, k, variant)) return s;
  if (int32_t s = check_gemv_scalars(error, format, x_dtype, m, n2, k, variant)) return s;
  if (m == 0 || n1 + n2 == 0) return ok(error);
  const int64_t n = n1 + n2;
  if (n1 > 0 && n2 > 0 && variant != TB200_VARIANT_SIMPLE) {
    // one launch over both weights when the pipelined kernel takes the concatenated shape unsplit
    if (int32_t s = check_pointer(error, "x", x, 16, k > 0)) return s;
    if (int32_t s = check_pointer(error, "w1", w1, 16, k > 0)) return s;
    if (int32_t s = check_pointer(error, "w2", w2, 16, k > 0)) return s;
    if (int32_t s = check_pointer(error, "out", out, 4, true)) return s;
    if (int32_t s = check_pointer(error, "scratch", scratch, 256, false)) return s;
    if (scratch_bytes < 0) return fail(error, TENSOR_ERROR_ARGUMENT, "negative scratch size");
    const DeviceInfo* dev;
    if (int32_t s = require_device(error, &dev)) return s;
    if (variant == TB200_VARIANT_TC) {
      TcLaunchItem pair[2]{};
      for (int i = 0; i < 2; ++i) {
        pair[i].fmt = format;
        pair[i].xt = x_dtype;
        pair[i].x = x;
        pair[i].m = m;
        pair[i].k = k;
        pair[i].x_share = i - 1;
      }
      pair[0].w = static_cast<const uint8_t*>(w1);
      pair[0].n = n1;
      pair[0].out = single_output(out, n);
      pair[1].w = static_cast<const uint8_t*>(w2);
      pair[1].n = n2;
      pair[1].out = single_output(out + n1, n);
      cudaError_t e;
      if (try_list(pair, 2, scratch, scratch_bytes, *dev, static_cast<cudaStream_t>(stream), nullptr, &e)) {
        if (e != cudaSuccess) return cuda_fail(error, "tensor-memory GEMV launch (two weights)", e);
        return ok(error);
      }
    }
    GemvPlan plan = plan_gemv_fast(format, x_dtype, m, n, k, scratch ? scratch_bytes : 0, *dev);
    if (plan.supported && plan.k_splits == 1 && n1 % kGemvTileRows == 0) {
      OutSpec both = single_output(out, n);
      both.ptr2[0] = out + n1;
      cudaError_t e = launch_gemv_fast(plan, format, x_dtype, x, static_cast<const uint8_t*>(w1), both, m,
                                       n, k, scratch, static_cast<cudaStream_t>(stream), nullptr,
                                       static_cast<const uint8_t*>(w2), n1);
      if (e != cudaSuccess) return cuda_fail(error, "pipelined GEMV launch (two weights)", e);
      return ok(error);
    }
  }
  // otherwise two launches, each into its own column window of the same [m, n1 + n2] output
  OutSpec first = single_output(out, n), second = single_output(out + n1, n);
  if (n1 > 0)
    if (int32_t s = gemv_common(format, x_dtype, x, w1, first, m, n1, k, scratch, scratch_bytes, variant, stream, error))
      return s;
  if (n2 > 0)
    if (int32_t s = gemv_common(format, x_dtype, x, w2, second, m, n2, k, scratch, scratch_bytes, variant, stream, error))
      return s;
  return ok(error);
}

static int32_t gemv_pair_sharded_impl(int32_t format, int32_t x_dtype, const void* x, const void* w1, int64_t n1,
                                      const void* w2, int64_t n2, float* const* outs1, float* const* outs2,
                                      int32_t out_count, int64_t out_ld, int64_t col_offset1, int64_t col_offset2,
                                      int64_t m, int64_t k, void* scratch, int64_t scratch_bytes, int32_t variant,
                                      uint32_t* const* pads, int32_t rank, int32_t world, int32_t sync,
                                      void* stream, TensorErrorV1* error, int prep_mode,
                                      PrepJobs* collect = nullptr) {
  if (int32_t s = check_gemv_scalars(error, format, x_dtype, m, n1, k, variant)) return s;
  if (int32_t s = check_gemv_scalars(error, format, x_dtype, m, n2, k, variant)) return s;
  if (!outs1 || !outs2) return fail(error, TENSOR_ERROR_ARGUMENT, "outs1 and outs2 are required");
  if (out_count < 1 || out_count > TB200_MAX_PEERS)
    return fail(error, TENSOR_ERROR_ARGUMENT, "out_count %d is not in 1..%d", out_count, TB200_MAX_PEERS);
  if (col_offset1 < 0 || col_offset2 < 0 || out_ld < col_offset1 + n1 || out_ld < col_offset2 + n2)
    return fail(error, TENSOR_ERROR_ARGUMENT, "column windows %lld+%lld / %lld+%lld do not fit a row of %lld",
                (long long)col_offset1, (long long)n1, (long long)col_offset2, (long long)n2, (long long)out_ld);
  if (sync & ~(TB200_PEER_WAIT | TB200_PEER_SIGNAL)) return fail(error, TENSOR_ERROR_ARGUMENT, "unknown sync bits 0x%x", sync);
  for (int i = 0; i < out_count; ++i)
    if (!outs1[i] || !outs2[i]) return fail(error, TENSOR_ERROR_ARGUMENT, "a destination of rank slot %d is null", i);
  const int64_t n = n1 + n2;
  if (m > 0 && n1 > 0 && n2 > 0 && variant != TB200_VARIANT_SIMPLE && variant != TB200_VARIANT_DP4A) {
    PeerSync peers{};
    if (sync) {
      if (int32_t s = check_pads(error, pads, rank, world)) return s;
      for (int i = 0; i < world; ++i) peers.pads[i] = pads[i];
      peers.rank = rank;
      peers.world = world;
      peers.flags = world > 1 ? sync : 0;
    }
    if (int32_t s = check_pointer(error, "x", x, 16, k > 0)) return s;
    if (int32_t s = check_pointer(error, "w1", w1, 16, k > 0)) return s;
    if (int32_t s = check_pointer(error, "w2", w2, 16, k > 0)) return s;
    if (int32_t s = check_pointer(error, "scratch", scratch, 256, false)) return s;
    if (scratch_bytes < 0) return fail(error, TENSOR_ERROR_ARGUMENT, "negative scratch size");
    const DeviceInfo* dev;
    if (int32_t s = require_device(error, &dev)) return s;
    if (variant == TB200_VARIANT_TC && prep_mode == kPrepNormal) {
      TcLaunchItem pair[2]{};
      for (int i = 0; i < 2; ++i) {
        pair[i].fmt = format;
        pair[i].xt = x_dtype;
        pair[i].x = x;
        pair[i].m = m;
        pair[i].k = k;
        pair[i].x_share = i - 1;
        pair[i].out.count = out_count;
        pair[i].out.ld = out_ld;
      }
      pair[0].w = static_cast<const uint8_t*>(w1);
      pair[0].n = n1;
      pair[1].w = static_cast<const uint8_t*>(w2);
      pair[1].n = n2;
      for (int i = 0; i < out_count; ++i) {
        pair[0].out.ptr[i] = outs1[i] + col_offset1;
        pair[1].out.ptr[i] = outs2[i] + col_offset2;
      }
      cudaError_t e;
      if (try_list(pair, 2, scratch, scratch_bytes, *dev, static_cast<cudaStream_t>(stream),
                   peers.flags ? &peers : nullptr, &e)) {
        if (e != cudaSuccess) return cuda_fail(error, "tensor-memory GEMV launch (two weights, sharded)", e);
        return ok(error);
      }
    }
    GemvPlan plan = plan_gemv_fast(format, x_dtype, m, n, k, scratch ? scratch_bytes : 0, *dev);
    if (plan.supported && plan.k_splits == 1 && n1 % kGemvTileRows == 0) {
      OutSpec spec{};
      spec.count = out_count;
      spec.ld = out_ld;
      for (int i = 0; i < out_count; ++i) {
        spec.ptr[i] = outs1[i] + col_offset1;
        spec.ptr2[i] = outs2[i] + col_offset2;
      }
      cudaError_t e = launch_gemv_fast(plan, format, x_dtype, x, static_cast<const uint8_t*>(w1), spec, m, n, k, scratch,
                                       static_cast<cudaStream_t>(stream), peers.flags ? &peers : nullptr,
                                       static_cast<const uint8_t*>(w2), n1, prep_mode, collect);
      if (e != cudaSuccess) return cuda_fail(error, "pipelined GEMV launch (two weights, sharded)", e);
      return ok(error);
    }
  }
  // two launches: the first waits for the peers, the second signals them
  if (int32_t s = gemv_sharded_impl(format, x_dtype, x, w1, outs1, out_count, out_ld, col_offset1, m, n1, k, scratch,
                                    scratch_bytes, variant, pads, rank, world, sync & TB200_PEER_WAIT, stream, error,
                                    prep_mode, collect))
    return s;
  return gemv_sharded_impl(format, x_dtype, x, w2, outs2, out_count, out_ld, col_offset2, m, n2, k, scratch, scratch_bytes,
                           variant, pads, rank, world, sync & TB200_PEER_SIGNAL, stream, error, prep_mode, collect);
}

int32_t tb200_gguf_gemv_pair_sharded_sync(int32_t format, int32_t x_dtype, const void* x, const void* w1, int64_t n1,
                                          const void* w2, int64_t n2, float* const* outs1, float* const* outs2,
                                          int32_t out_count, int64_t out_ld, int64_t col_offset1, int64_t col_offset2,
                                          int64_t m, int64_t k, void* scratch, int64_t scratch_bytes, int32_t variant,
                                          uint32_t* const* pads, int32_t rank, int32_t world, int32_t sync,
                                          void* stream, TensorErrorV1* error) {
  return gemv_pair_sharded_impl(format, x_dtype, x, w1, n1, w2, n2, outs1, outs2, out_count, out_ld, col_offset1,
                                col_offset2, m, k, scratch, scratch_bytes, variant, pads, rank, world, sync, stream, error,
                                kPrepNormal);
}

int32_t tb200_peer_sync(uint32_t* const* pads, int32_t rank, int32_t world, int32_t mode, void* stream,
                        TensorErrorV1* error) {
  if (int32_t s = check_pads(error, pads, rank, world)) return s;
  if (!(mode & (TB200_PEER_WAIT | TB200_PEER_SIGNAL)) || (mode & ~(TB200_PEER_WAIT | TB200_PEER_SIGNAL)))
    return fail(error, TENSOR_ERROR_ARGUMENT, "mode 0x%x is not TB200_PEER_WAIT, TB200_PEER_SIGNAL or both", mode);
  const DeviceInfo* dev;
  if (int32_t s = require_device(error, &dev)) return s;
  cudaError_t e = launch_peer_barrier(pads, rank, world, mode, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(error, "peer sync launch", e);
  return ok(error);
}

int32_t tb200_peer_barrier(uint32_t* const* pads, int32_t rank, int32_t world, void* stream, TensorErrorV1* error) {
  return tb200_peer_sync(pads, rank, world, TB200_PEER_WAIT | TB200_PEER_SIGNAL, stream, error);
}

int32_t tb200_peer_export(const void* ptr, uint8_t* handle, int64_t* offset, TensorErrorV1* error) {
  static_assert(sizeof(cudaIpcMemHandle_t) == TB200_PEER_HANDLE_BYTES, "IPC handle size");
  if (!ptr || !handle || !offset) return fail(error, TENSOR_ERROR_ARGUMENT, "ptr, handle and offset are required");
  void* base = nullptr;
  size_t size = 0;
  if (!allocation_range(ptr, &base, &size))
    return fail(error, TENSOR_ERROR_PROVIDER, "%p is not inside a device allocation of this process", ptr);
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, base);
  if (e != cudaSuccess) return cuda_fail(error, "cudaIpcGetMemHandle", e);
  memcpy(handle, &h, sizeof(h));
  *offset = (int64_t)(static_cast<const char*>(ptr) - static_cast<const char*>(base));
  return ok(error);
}

int32_t tb200_peer_open(const uint8_t* handle, void** base, TensorErrorV1* error) {
  if (!handle || !base) return fail(error, TENSOR_ERROR_ARGUMENT, "handle and base are required");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(error, "cudaIpcOpenMemHandle", e);
  *base = p;
  return ok(error);
}

int32_t tb200_peer_close(void* base, TensorErrorV1* error) {
  if (!base) return ok(error);
  cudaError_t e = cudaIpcCloseMemHandle(base);
  if (e != cudaSuccess) return cuda_fail(error, "cudaIpcCloseMemHandle", e);
  return ok(error);
}

}  // extern "C"

namespace {
Schedule to_schedule(const TB200Schedule* in) {
  Schedule s;
  if (in) {
    s.k_splits = in->k_splits;
    s.ctas_per_sm = in->ctas_per_sm;
    s.convert_ahead = in->convert_ahead;
    s.overlap = in->overlap;
    s.gemm_shape = in->gemm_shape;
  }
  return s;
}
int32_t gemm_common(int32_t format, int32_t x_dtype, const void* x, const void* w, float* out, int64_t m, int64_t n,
                    int64_t k, int32_t variant, void* stream, TensorErrorV1* error, const Schedule* sched);
}  // namespace

extern "C" {

int32_t tb200_gguf_gemm(int32_t format, int32_t x_dtype, const void* x, const void* w, float* out, int64_t m,
                        int64_t n, int64_t k, int32_t variant, void* stream, TensorErrorV1* error) {
  return gemm_common(format, x_dtype, x, w, out, m, n, k, variant, stream, error, nullptr);
}

int32_t tb200_gguf_gemm_scheduled(int32_t format, int32_t x_dtype, const void* x, const void* w, float* out, int64_t m,
                                  int64_t n, int64_t k, const TB200Schedule* schedule, void* stream,
                                  TensorErrorV1* error) {
  if (!schedule) return fail(error, TENSOR_ERROR_ARGUMENT, "schedule is null");
  const Schedule s = to_schedule(schedule);
  return gemm_common(format, x_dtype, x, w, out, m, n, k, TB200_VARIANT_FAST, stream, error, &s);
}

int32_t tb200_gguf_gemv_scheduled(int32_t format, int32_t x_dtype, const void* x, const void* w, float* out, int64_t m,
                                  int64_t n, int64_t k, void* scratch, int64_t scratch_bytes,
                                  const TB200Schedule* schedule, void* stream, TensorErrorV1* error) {
  if (!schedule) return fail(error, TENSOR_ERROR_ARGUMENT, "schedule is null");
  if (int32_t s = check_gemv_scalars(error, format, x_dtype, m, n, k, TB200_VARIANT_FAST)) return s;
  if (m == 0 || n == 0) return ok(error);
  const Schedule s = to_schedule(schedule);
  return gemv_common(format, x_dtype, x, w, single_output(out, n), m, n, k, scratch, scratch_bytes, TB200_VARIANT_MMA,
                     stream, error, nullptr, &s);
}

int32_t tb200_gguf_schedule_legal(int32_t op, int32_t format, int64_t m, int64_t n, int64_t k, int64_t scratch_bytes,
                                  const TB200Schedule* schedule) {
  if (!schedule || !valid_format(format) || m < 1 || n < 1 || k < 1 || k % block_weights(format)) return 0;
  DeviceInfo b200;  // without a device, judge legality for a B200
  b200.ordinal = 0;
  b200.sm_count = 148;
  b200.max_smem_optin = 232448;
  b200.cc_major = 10;
  cudaError_t e;
  const DeviceInfo* dev = device_info(&e);
  if (!dev) {
    cudaGetLastError();
    dev = &b200;
  }
  const Schedule s = to_schedule(schedule);
  if (s.overlap < 0 || s.overlap > 2 || s.convert_ahead < 0 || s.convert_ahead > 2) return 0;
  if (op == TB200_OP_GEMV) return plan_gemv_fast(format, kBF16, m, n, k, scratch_bytes, *dev, true, &s).supported ? 1 : 0;
  if (op == TB200_OP_GEMM) return gemm_fast_supported(format, m, n, k, *dev) && gemm_shape_legal(s.gemm_shape, m, *dev) ? 1 : 0;
  return 0;
}

int32_t tb200_gguf_schedule_record(int32_t op, int32_t format, int64_t m, int64_t n, int64_t k,
                                   const TB200Schedule* schedule) {
  if ((op != TB200_OP_GEMV && op != TB200_OP_GEMM) || !valid_format(format)) return TENSOR_ERROR_ARGUMENT;
  record_schedule(op, format, m, n, k, to_schedule(schedule));
  return TENSOR_OK;
}

void tb200_gguf_schedule_clear(void) { clear_schedules(); }

}  // extern "C"

namespace {
int32_t gemm_common(int32_t format, int32_t x_dtype, const void* x, const void* w, float* out, int64_t m, int64_t n,
                    int64_t k, int32_t variant, void* stream, TensorErrorV1* error, const Schedule* sched) {
  if (int32_t s = check_shape(error, format, m, n, k)) return s;
  if (x_dtype != TENSOR_BFLOAT16)
    return fail(error, TENSOR_ERROR_ARGUMENT, "the GEMM takes bfloat16 activations (dtype 13), got %d", x_dtype);
  if (variant < 0 || variant > TB200_VARIANT_FAST) return fail(error, TENSOR_ERROR_ARGUMENT, "unknown variant %d", variant);
  if (m == 0 || n == 0) return ok(error);
  if (int32_t s = check_pointer(error, "x", x, 16, k > 0)) return s;
  if (int32_t s = check_pointer(error, "w", w, 16, k > 0)) return s;
  if (int32_t s = check_pointer(error, "out", out, 16, true)) return s;
  const DeviceInfo* dev;
  if (int32_t s = require_device(error, &dev)) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const uint8_t* wp = static_cast<const uint8_t*>(w);
  if (variant != TB200_VARIANT_SIMPLE) {
    if (gemm_fast_supported(format, m, n, k, *dev)) {
      const char* detail = "";
      if (sched && !gemm_shape_legal(sched->gemm_shape, m, *dev))
        return fail(error, TENSOR_ERROR_ARGUMENT, "GEMM shape %d is not legal on this device", sched->gemm_shape);
      cudaError_t e = launch_gemm_fast(format, x, wp, out, m, n, k, st, &detail, sched);
      if (e != cudaSuccess) return cuda_fail(error, detail && *detail ? detail : "tcgen05 GEMM launch", e);
      return ok(error);
    }
    if (variant == TB200_VARIANT_FAST)
      return fail(error, TENSOR_ERROR_ARGUMENT, "the tcgen05 GEMM does not cover format %d, m=%lld, n=%lld, k=%lld",
                  format, (long long)m, (long long)n, (long long)k);
  }
  cudaError_t e = launch_gemv_simple(format, x_dtype, x, wp, out, m, n, k, true, st);
  if (e != cudaSuccess) return cuda_fail(error, "GEMM launch", e);
  return ok(error);
}
}  // namespace

extern "C" {

namespace {
int32_t check_list(TensorErrorV1* error, const TB200GemvItem* items, int32_t count) {
  if (!items) return fail(error, TENSOR_ERROR_ARGUMENT, "items is null");
  if (count < 1 || count > TB200_GEMV_LIST_MAX)
    return fail(error, TENSOR_ERROR_ARGUMENT, "a list holds 1..%d projections, got %d", TB200_GEMV_LIST_MAX, count);
  for (int i = 0; i < count; ++i) {
    const TB200GemvItem& it = items[i];
    if (int32_t s = check_gemv_scalars(error, it.format, it.x_dtype, it.m, it.n, it.k, TB200_VARIANT_AUTO)) return s;
    if (it.m < 1 || it.n < 1) return fail(error, TENSOR_ERROR_ARGUMENT, "item %d: empty projection", i);
    if (it.out_count < 1 || it.out_count > TB200_MAX_PEERS)
      return fail(error, TENSOR_ERROR_ARGUMENT, "item %d: out_count %d is not in 1..%d", i, it.out_count, TB200_MAX_PEERS);
    if (it.out_ld < it.n) return fail(error, TENSOR_ERROR_ARGUMENT, "item %d: out_ld %lld < n %lld", i, (long long)it.out_ld, (long long)it.n);
  }
  return TENSOR_OK;
}
void to_launch_items(const TB200GemvItem* items, int count, TcLaunchItem* out) {
  for (int i = 0; i < count; ++i) {
    const TB200GemvItem& it = items[i];
    TcLaunchItem& o = out[i];
    o = TcLaunchItem{};
    o.fmt = it.format;
    o.xt = it.x_dtype;
    o.x = it.x;
    o.w = static_cast<const uint8_t*>(it.w);
    o.m = it.m;
    o.n = it.n;
    o.k = it.k;
    o.out.count = it.out_count;
    o.out.ld = it.out_ld;
    for (int d = 0; d < it.out_count && d < kMaxOutputs; ++d) o.out.ptr[d] = it.outs[d];
    o.x_share = -1;
    for (int j = 0; j < i; ++j)
      if (items[j].x == it.x && items[j].m == it.m && items[j].k == it.k && items[j].x_dtype == it.x_dtype) {
        o.x_share = out[j].x_share >= 0 ? out[j].x_share : j;
        break;
      }
  }
}
}  // namespace

namespace {
// The launches a list becomes when its projections go out one by one: neighbours that share their activations
// (and format, and output layout) as one grouped launch.  need[u] = scratch of unit u (the larger of the grouped
// launch's and its members'), rounded up to 256 bytes.
struct ListUnits {
  int count;
  int first[kTcMaxItems];
  bool pair[kTcMaxItems];
  long long need[kTcMaxItems];
  long long total, largest;
};
ListUnits list_units(const TB200GemvItem* items, int count, const TcLaunchItem* list, int variant,
                     const DeviceInfo& dev) {
  ListUnits u{};
  for (int i = 0; i < count;) {
    bool pair = i + 1 < count && list[i + 1].x_share == i && items[i + 1].format == items[i].format &&
                items[i + 1].out_count == items[i].out_count && items[i + 1].out_ld == items[i].out_ld &&
                variant != TB200_VARIANT_SIMPLE && variant != TB200_VARIANT_DP4A;
    long long need = tb200_gguf_gemv_scratch_bytes(items[i].format, items[i].m, items[i].n, items[i].k);
    if (pair) {
      // only where the two really run as ONE launch (the pipelined kernel, K not split, the first weight ending on
      // a tile boundary); otherwise they are two units with a slice each
      const GemvPlan both = plan_gemv_fast(items[i].format, kBF16, items[i].m, items[i].n + items[i + 1].n, items[i].k,
                                           (long long)1 << 40, dev);
      pair = both.supported && both.k_splits == 1 && items[i].n % kGemvTileRows == 0;
      if (pair) need = both.scratch_bytes;
    }
    need = (need + 255) / 256 * 256;
    u.first[u.count] = i;
    u.pair[u.count] = pair;
    u.need[u.count] = need;
    u.total += need;
    u.largest = std::max(u.largest, need);
    ++u.count;
    i += pair ? 2 : 1;
  }
  return u;
}
}  // namespace

int64_t tb200_gguf_gemv_list_scratch_bytes(const TB200GemvItem* items, int32_t count) {
  if (!items || count < 1 || count > TB200_GEMV_LIST_MAX) return 0;
  cudaError_t e;
  const DeviceInfo* dev = device_info(&e);
  if (!dev) return 0;
  TcLaunchItem list[kTcMaxItems];
  to_launch_items(items, count, list);
  // Launched one by one (or two by two) every unit gets a slice of its own, so that the activation conversions
  // of all units can run ahead of the first GEMV; a buffer that only holds the largest unit still works (the
  // units then share it and every conversion runs right before its GEMV).
  const ListUnits units = list_units(items, count, list, TB200_VARIANT_AUTO, *dev);
  return std::max<long long>(gemv_tc_scratch_bytes(list, count, *dev), units.total);
}

int32_t tb200_gguf_gemv_list(const TB200GemvItem* items, int32_t count, void* scratch, int64_t scratch_bytes,
                             int32_t variant, uint32_t* const* pads, int32_t rank, int32_t world, int32_t sync,
                             void* stream, TensorErrorV1* error) {
  static_assert(TB200_GEMV_LIST_MAX == kTcMaxItems, "list length");
  if (int32_t s = check_list(error, items, count)) return s;
  if (variant < 0 || variant > TB200_VARIANT_DP4A) return fail(error, TENSOR_ERROR_ARGUMENT, "unknown variant %d", variant);
  if (int32_t s = check_pointer(error, "scratch", scratch, 256, false)) return s;
  if (scratch_bytes < 0) return fail(error, TENSOR_ERROR_ARGUMENT, "negative scratch size");
  if (sync & ~(TB200_PEER_WAIT | TB200_PEER_SIGNAL)) return fail(error, TENSOR_ERROR_ARGUMENT, "unknown sync bits 0x%x", sync);
  for (int i = 0; i < count; ++i) {
    if (int32_t s = check_pointer(error, "x", items[i].x, 16, true)) return s;
    if (int32_t s = check_pointer(error, "w", items[i].w, 16, true)) return s;
    for (int d = 0; d < items[i].out_count; ++d)
      if (int32_t s = check_pointer(error, "out", items[i].outs[d], 4, true)) return s;
  }
  PeerSync peers{};
  if (sync) {
    if (int32_t s = check_pads(error, pads, rank, world)) return s;
    for (int i = 0; i < world; ++i) peers.pads[i] = pads[i];
    peers.rank = rank;
    peers.world = world;
    peers.flags = world > 1 ? sync : 0;
  }
  const DeviceInfo* dev;
  if (int32_t s = require_device(error, &dev)) return s;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  TcLaunchItem list[kTcMaxItems];
  to_launch_items(items, count, list);
  if (variant == TB200_VARIANT_TC) {
    cudaError_t e;
    if (!try_list(list, count, scratch, scratch_bytes, *dev, st, peers.flags ? &peers : nullptr, &e))
      return fail(error, TENSOR_ERROR_ARGUMENT,
                  "the persistent tensor-memory kernel takes Q4_K or Q6_K lists with 2-byte activations, m <= 16 and %lld "
                  "bytes of scratch", (long long)gemv_tc_scratch_bytes(list, count, *dev));
    if (e != cudaSuccess) return cuda_fail(error, "tensor-memory GEMV launch (list)", e);
    return ok(error);
  }
  // Pipelined launches back to back (each overlaps its predecessor's tail); neighbours that share
  // their activations go out as one grouped launch.  The first launch waits for the peers, the last
  // one signals them.  Where the scratch holds a slice per unit, the activation conversions of all
  // units (batches above 1) go out first, as ONE launch, so that no small launch sits between two GEMVs; it
  // reads the activations, so on an N-sharded list it waits for the peers as the first GEMV does.
  const ListUnits units = list_units(items, count, list, variant, *dev);
  const bool slices = scratch && units.total <= scratch_bytes && units.count > 1;
  uint8_t* const base = static_cast<uint8_t*>(scratch);
  PrepJobs conversions{};
  auto launch_unit = [&](int u, long long offset, long long bytes, int flags, int prep_mode) -> int32_t {
    PrepJobs* collect = prep_mode == kPrepOnly ? &conversions : nullptr;
    const int i = units.first[u];
    void* sc = scratch ? base + offset : nullptr;
    if (units.pair[u])
      return gemv_pair_sharded_impl(items[i].format, items[i].x_dtype, items[i].x, items[i].w, items[i].n, items[i + 1].w,
                                    items[i + 1].n, items[i].outs, items[i + 1].outs, items[i].out_count, items[i].out_ld,
                                    0, 0, items[i].m, items[i].k, sc, bytes, variant, pads, rank, world > 0 ? world : 1,
                                    flags, stream, error, prep_mode, collect);
    PeerSync each = peers;
    each.flags = flags;
    return gemv_common(items[i].format, items[i].x_dtype, items[i].x, items[i].w, list[i].out, items[i].m, items[i].n,
                       items[i].k, sc, bytes, variant, stream, error, each.flags ? &each : nullptr, nullptr, prep_mode,
                       collect);
  };
  bool hoist = false;
  if (slices)
    for (int i = 0; i < count; ++i) hoist |= items[i].m > 1 && items[i].format == kQ4_K;
  const int wait_flag = peers.flags & kPeerWait;
  if (hoist) {
    long long offset = 0;
    for (int u = 0; u < units.count; ++u) {  // notes the conversions ...
      if (int32_t s = launch_unit(u, offset, units.need[u], 0, kPrepOnly)) return s;
      offset += units.need[u];
    }
    PeerSync first = peers;  // ... and ONE launch runs them, after waiting for the peers like the first GEMV
    first.flags = wait_flag;
    cudaError_t e = launch_gemv_prepare_jobs(conversions, wait_flag ? &first : nullptr, st);
    if (e != cudaSuccess) return cuda_fail(error, "activation conversion launch (list)", e);
  }
  long long offset = 0;
  for (int u = 0; u < units.count; ++u) {
    const int flags = (u == 0 ? wait_flag : 0) | (u + 1 == units.count ? peers.flags & kPeerSignal : 0);
    if (int32_t s = launch_unit(u, slices ? offset : 0, slices ? units.need[u] : scratch_bytes, flags,
                                hoist ? kPrepDone : kPrepNormal))
      return s;
    offset += units.need[u];
  }
  return ok(error);
}

int32_t tb200_rmsnorm_bf16(const float* x, const float* weight, void* out, int64_t m, int64_t k, float eps, void* stream,
                           TensorErrorV1* error) {
  if (m < 1 || k < 4 || k % 4) return fail(error, TENSOR_ERROR_ARGUMENT, "rmsnorm needs m >= 1 and k a multiple of 4");
  if (int32_t s = check_pointer(error, "x", x, 16, true)) return s;
  if (int32_t s = check_pointer(error, "weight", weight, 16, true)) return s;
  if (int32_t s = check_pointer(error, "out", out, 8, true)) return s;
  const DeviceInfo* dev;
  if (int32_t s = require_device(error, &dev)) return s;
  cudaError_t e = launch_rmsnorm(x, weight, out, m, k, eps, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(error, "rmsnorm launch", e);
  return ok(error);
}

int32_t tb200_swiglu_bf16(const float* gate_up, void* out, int64_t m, int64_t width, void* stream, TensorErrorV1* error) {
  if (m < 1 || width < 4 || width % 4) return fail(error, TENSOR_ERROR_ARGUMENT, "swiglu needs m >= 1 and a width that is a multiple of 4");
  if (int32_t s = check_pointer(error, "gate_up", gate_up, 16, true)) return s;
  if (int32_t s = check_pointer(error, "out", out, 8, true)) return s;
  const DeviceInfo* dev;
  if (int32_t s = require_device(error, &dev)) return s;
  cudaError_t e = launch_swiglu(gate_up, out, m, width, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(error, "swiglu launch", e);
  return ok(error);
}

int32_t tb200_residual_add(float* stream_buffer, const float* delta, int64_t count, void* stream, TensorErrorV1* error) {
  if (count < 4 || count % 4) return fail(error, TENSOR_ERROR_ARGUMENT, "residual add needs a count that is a multiple of 4");
  if (int32_t s = check_pointer(error, "stream_buffer", stream_buffer, 16, true)) return s;
  if (int32_t s = check_pointer(error, "delta", delta, 16, true)) return s;
  const DeviceInfo* dev;
  if (int32_t s = require_device(error, &dev)) return s;
  cudaError_t e = launch_residual_add(stream_buffer, delta, count, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(error, "residual add launch", e);
  return ok(error);
}

int32_t tb200_peer_set_wait_limit(uint64_t nanoseconds) {
  set_peer_wait_limit_ns(nanoseconds);
  return TENSOR_OK;
}

// ---- descriptor forms ----------------------------------------------------------------------------

}  // extern "C"

namespace {

struct Parsed {
  const TensorBufferV1* buffers[4] = {nullptr, nullptr, nullptr, nullptr};
  int buffer_count = 0;
  int64_t scalars[5] = {0, 0, 0, 0, 0};
  int scalar_count = 0;
};

int32_t parse_call(const TensorCallV1* call, TensorErrorV1* error, int min_buffers, int max_buffers,
                   int min_scalars, int max_scalars, Parsed* out) {
  if (!call) return fail(error, TENSOR_ERROR_ABI, "call descriptor is NULL");
  if (call->abi_version != TENSOR_ABI_VERSION)
    return fail(error, TENSOR_ERROR_ABI, "unsupported ABI version %u (expected %u)", call->abi_version,
                TENSOR_ABI_VERSION);
  if (call->struct_size != sizeof(TensorCallV1))
    return fail(error, TENSOR_ERROR_ABI, "TensorCallV1 struct_size %u, expected %zu", call->struct_size,
                sizeof(TensorCallV1));
  if (call->flags != 0) return fail(error, TENSOR_ERROR_ABI, "call flags must be zero");
  if (call->stream.device_type != TENSOR_DEVICE_CUDA)
    return fail(error, TENSOR_ERROR_ARGUMENT, "stream device type %u is not CUDA", call->stream.device_type);
  if (!call->arguments && call->argument_count)
    return fail(error, TENSOR_ERROR_ARGUMENT, "argument array is NULL");
  for (uint32_t i = 0; i < call->argument_count; ++i) {
    const TensorArgumentV1& a = call->arguments[i];
    if (a.kind == TENSOR_ARG_BUFFER) {
      if (out->scalar_count) return fail(error, TENSOR_ERROR_ARGUMENT, "argument %u: buffers must precede scalars", i);
      if (out->buffer_count == max_buffers) return fail(error, TENSOR_ERROR_ARGUMENT, "too many buffer arguments");
      if (a.buffer.device_type != TENSOR_DEVICE_CUDA)
        return fail(error, TENSOR_ERROR_ARGUMENT, "argument %u: buffer is not on a CUDA device", i);
      if (a.buffer.device_ordinal != call->stream.device_ordinal)
        return fail(error, TENSOR_ERROR_ARGUMENT, "argument %u: buffer on device %d, stream on device %d", i,
                    a.buffer.device_ordinal, call->stream.device_ordinal);
      if (a.dtype != a.buffer.dtype)
        return fail(error, TENSOR_ERROR_ARGUMENT, "argument %u: dtype %u does not match its buffer's %u", i, a.dtype,
                    a.buffer.dtype);
      if (a.scalar != 0) return fail(error, TENSOR_ERROR_ARGUMENT, "argument %u: buffer with a scalar payload", i);
      out->buffers[out->buffer_count++] = &a.buffer;
    } else if (a.kind == TENSOR_ARG_SCALAR) {
      if (out->scalar_count == max_scalars) return fail(error, TENSOR_ERROR_ARGUMENT, "too many scalar arguments");
      int64_t v;
      if (a.dtype == TENSOR_INT32) {
        int32_t t;
        memcpy(&t, &a.scalar, 4);
        v = t;
      } else if (a.dtype == TENSOR_INT64) {
        memcpy(&v, &a.scalar, 8);
      } else {
        return fail(error, TENSOR_ERROR_ARGUMENT, "argument %u: scalar dtype %u is not int32 or int64", i, a.dtype);
      }
      out->scalars[out->scalar_count++] = v;
    } else {
      return fail(error, TENSOR_ERROR_ARGUMENT, "argument %u: unsupported kind %u", i, a.kind);
    }
  }
  if (out->buffer_count < min_buffers || out->scalar_count < min_scalars)
    return fail(error, TENSOR_ERROR_ARGUMENT, "expected at least %d buffers and %d scalars, got %d and %d", min_buffers,
                min_scalars, out->buffer_count, out->scalar_count);
  return TENSOR_OK;
}

int32_t check_buffer(TensorErrorV1* error, const char* name, const TensorBufferV1* b, int32_t dtype_a,
                     int32_t dtype_b, int64_t elements) {
  if ((int32_t)b->dtype != dtype_a && (int32_t)b->dtype != dtype_b)
    return fail(error, TENSOR_ERROR_ARGUMENT, "%s has dtype %u", name, b->dtype);
  const int64_t need = elements * dtype_bytes((int32_t)b->dtype);
  if ((int64_t)b->byte_size != need)
    return fail(error, TENSOR_ERROR_ARGUMENT, "%s holds %llu bytes, the shape needs %lld", name,
                (unsigned long long)b->byte_size, (long long)need);
  if (!b->address && need) return fail(error, TENSOR_ERROR_ARGUMENT, "%s has a NULL address", name);
  return TENSOR_OK;
}

// Run on the stream's device, restoring the caller's current device afterwards.
struct DeviceScope {
  int previous = -1;
  cudaError_t status;
  explicit DeviceScope(int ordinal) {
    status = cudaGetDevice(&previous);
    if (status == cudaSuccess && previous != ordinal) status = cudaSetDevice(ordinal);
  }
  ~DeviceScope() {
    if (previous >= 0) cudaSetDevice(previous);
  }
};

}  // namespace

extern "C" {

int32_t tb200_gguf_dequant_v1(const TensorCallV1* call, TensorErrorV1* error) {
  Parsed p;
  if (int32_t s = parse_call(call, error, 2, 2, 3, 3, &p)) return s;
  const int64_t n = p.scalars[0], k = p.scalars[1];
  const int32_t format = (int32_t)p.scalars[2];
  if (int32_t s = check_shape(error, format, 0, n, k)) return s;
  if (int32_t s = check_buffer(error, "w", p.buffers[0], TENSOR_UINT8, TENSOR_UINT8, n * row_bytes(format, k))) return s;
  if (int32_t s = check_buffer(error, "out", p.buffers[1], TENSOR_FLOAT32, TENSOR_FLOAT32, n * k)) return s;
  DeviceScope scope(call->stream.device_ordinal);
  if (scope.status != cudaSuccess) return cuda_fail(error, "selecting the stream's device", scope.status);
  return tb200_gguf_dequant(format, (const void*)p.buffers[0]->address, (float*)p.buffers[1]->address, n, k,
                            (void*)call->stream.handle, error);
}

int32_t tb200_gguf_gemv_v1(const TensorCallV1* call, TensorErrorV1* error) {
  Parsed p;
  if (int32_t s = parse_call(call, error, 3, 4, 4, 5, &p)) return s;
  const int64_t m = p.scalars[0], n = p.scalars[1], k = p.scalars[2];
  const int32_t format = (int32_t)p.scalars[3];
  const int32_t variant = p.scalar_count > 4 ? (int32_t)p.scalars[4] : 0;
  if (int32_t s = check_shape(error, format, m, n, k)) return s;
  const TensorBufferV1* x = p.buffers[0];
  if (x->dtype != TENSOR_FLOAT16 && x->dtype != TENSOR_BFLOAT16 && x->dtype != TENSOR_FLOAT32)
    return fail(error, TENSOR_ERROR_ARGUMENT, "x has dtype %u; expected float16, bfloat16 or float32", x->dtype);
  if (int32_t s = check_buffer(error, "x", x, (int32_t)x->dtype, (int32_t)x->dtype, m * k)) return s;
  if (int32_t s = check_buffer(error, "w", p.buffers[1], TENSOR_UINT8, TENSOR_UINT8, n * row_bytes(format, k))) return s;
  if (int32_t s = check_buffer(error, "out", p.buffers[2], TENSOR_FLOAT32, TENSOR_FLOAT32, m * n)) return s;
  void* scratch = nullptr;
  int64_t scratch_bytes = 0;
  if (p.buffer_count == 4) {
    if (p.buffers[3]->dtype != TENSOR_UINT8) return fail(error, TENSOR_ERROR_ARGUMENT, "scratch must be uint8");
    scratch = (void*)p.buffers[3]->address;
    scratch_bytes = (int64_t)p.buffers[3]->byte_size;
  }
  DeviceScope scope(call->stream.device_ordinal);
  if (scope.status != cudaSuccess) return cuda_fail(error, "selecting the stream's device", scope.status);
  return tb200_gguf_gemv(format, (int32_t)x->dtype, (const void*)x->address, (const void*)p.buffers[1]->address,
                         (float*)p.buffers[2]->address, m, n, k, scratch, scratch_bytes, variant,
                         (void*)call->stream.handle, error);
}

int32_t tb200_gguf_gemm_v1(const TensorCallV1* call, TensorErrorV1* error) {
  Parsed p;
  if (int32_t s = parse_call(call, error, 3, 3, 4, 5, &p)) return s;
  const int64_t m = p.scalars[0], n = p.scalars[1], k = p.scalars[2];
  const int32_t format = (int32_t)p.scalars[3];
  const int32_t variant = p.scalar_count > 4 ? (int32_t)p.scalars[4] : 0;
  if (int32_t s = check_shape(error, format, m, n, k)) return s;
  if (int32_t s = check_buffer(error, "x", p.buffers[0], TENSOR_BFLOAT16, TENSOR_BFLOAT16, m * k)) return s;
  if (int32_t s = check_buffer(error, "w", p.buffers[1], TENSOR_UINT8, TENSOR_UINT8, n * row_bytes(format, k))) return s;
  if (int32_t s = check_buffer(error, "out", p.buffers[2], TENSOR_FLOAT32, TENSOR_FLOAT32, m * n)) return s;
  DeviceScope scope(call->stream.device_ordinal);
  if (scope.status != cudaSuccess) return cuda_fail(error, "selecting the stream's device", scope.status);
  return tb200_gguf_gemm(format, TENSOR_BFLOAT16, (const void*)p.buffers[0]->address,
                         (const void*)p.buffers[1]->address, (float*)p.buffers[2]->address, m, n, k, variant,
                         (void*)call->stream.handle, error);
}

}  // extern "C"
