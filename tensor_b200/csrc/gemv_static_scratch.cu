// tb200_gguf_gemv_static: the decode GEMV for callers that are not allowed to allocate.
//
// Some hosts of this library cannot hand it scratch memory and cannot let it call cudaMalloc either:
// a launch adapter that only forwards the buffers an artifact declares (the reference runtime's
// contract has no hidden workspace), a serving loop that owns all device memory through its own
// arena, or code running between cudaStreamBeginCapture and EndCapture, where an allocation is an
// error.  For them the split-K partial sums and arrival counters live in the array below, which
// is part of the library image: every GPU that loads the library holds these bytes until the
// process exits, whether the entry point is ever called or not.
//
// What the caller must know:
//   * shapes whose plan wants more scratch than kStaticScratchBytes are rejected (status 2) rather
//     than silently run with another plan;
//   * the first call on each device looks up the array's device address
//     (cudaGetSymbolAddress); make that first call outside any stream capture;
//   * all calls on a device share the one array.  Two calls that overlap on the GPU (different
//     streams, no ordering between them) would add into each other's partial sums -- keep them
//     ordered.  The arrival counters are cleared on the stream at the start of every call, so a call
//     never inherits state from an earlier one.
// Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#include <mutex>

#include "../../include/tensor_b200_gguf.h"
#include "common.cuh"
#include "kernels.h"

namespace {

constexpr size_t kStaticScratchBytes = TB200_GEMV_STATIC_SCRATCH_BYTES;  // 4 MiB: Q4_K 3584 x 18944 at batch 16 needs 1.6 MB
constexpr size_t kCounterRegionBytes = tb200::kGemvCounterBytes;  // the part of the scratch that must start at zero

// In host code this name is only a handle for the runtime, never a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct PerDevice {
  bool ready = false;
  void* address = nullptr;
};

// Device address of the array on the current device, resolved once per device.
cudaError_t static_scratch_address(void** out) {
  static PerDevice table[64];
  static std::mutex lock;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> guard(lock);
  if (!table[dev].ready) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return e;
    table[dev].address = ptr;
    table[dev].ready = true;
  }
  *out = table[dev].address;
  return cudaSuccess;
}

int32_t report(TensorErrorV1* error, int32_t code, const char* text) {
  if (error) {
    error->code = code;
    size_t i = 0;
    for (; text[i] && i + 1 < sizeof(error->message); ++i) error->message[i] = text[i];
    error->message[i] = 0;
  }
  return code;
}

}  // namespace

extern "C" {

int32_t tb200_gguf_gemv_static(int32_t format, int32_t x_dtype, const void* x, const void* w, float* out, int64_t m,
                               int64_t n, int64_t k, void* stream, TensorErrorV1* error) {
  // How much scratch would the regular entry point like at this shape?  (0: its plan never splits K.)
  const int64_t wanted = tb200_gguf_gemv_scratch_bytes(format, m, n, k);
  if (wanted > (int64_t)kStaticScratchBytes)
    return report(error, TENSOR_ERROR_ARGUMENT,
                  "tb200_gguf_gemv_static: this shape wants more scratch than the 4 MiB built into the library; "
                  "use tb200_gguf_gemv with caller-provided scratch");
  void* scratch = nullptr;
  cudaError_t e = static_scratch_address(&scratch);
  if (e != cudaSuccess)
    return report(error, TENSOR_ERROR_PROVIDER, "tb200_gguf_gemv_static: cudaGetSymbolAddress failed for the scratch array");
  if (wanted > 0) {
    e = cudaMemsetAsync(scratch, 0, kCounterRegionBytes, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess)
      return report(error, TENSOR_ERROR_PROVIDER, "tb200_gguf_gemv_static: clearing the arrival counters failed");
  }
  return tb200_gguf_gemv(format, x_dtype, x, w, out, m, n, k, scratch, (int64_t)kStaticScratchBytes,
                         TB200_VARIANT_AUTO, stream, error);
}

}  // extern "C"
