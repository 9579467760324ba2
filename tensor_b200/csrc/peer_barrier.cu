// Cross-GPU barrier for N-sharded projections whose kernels store their columns straight into
// every rank's output (peer-mapped memory over NVLink).  The reference has no collective; this is
// the exchange step that replaces an all-gather call when the data has already been written by the
// producing kernel.
//
// One signal pad per rank (kSignalWords uint32, zeroed once before the first use, never reset):
//   word j < world : epoch last announced by rank j (written by rank j through its peer mapping)
//   word 32        : this rank's own epoch counter = signals it has sent (device-resident so that
//                    a captured launch can be replayed: nothing about the epoch is baked into it)
//   word 34        : CTAs of the running GEMV that have stored their outputs (used when the signal
//                    is folded into the GEMV, see gemv_mma.cu; back to zero after every launch)
// The two halves can be used apart: a signal (count up, tell the peers) once this rank's stores are
// done, and a wait (until every peer's count has reached this rank's own) before anything reads
// what the peers stored; the pipelined GEMV does both inside its own launch.
// A launch on rank r: epoch = ++pad_r[32]; fence; release-store epoch into pad_j[r] for every peer j;
// then wait until pad_r[j] has reached epoch for every j.  Epochs only grow, so a peer that is
// already one barrier ahead satisfies the wait.  Everything enqueued on the stream before the
// barrier (the GEMV's peer stores) is complete when the kernel starts; the system-scope fence and
// release order it before the flag at the peer, and the acquire load orders the peer's data after
// the flag for whatever this rank enqueues next.
//
// The wait is bounded (two seconds of the global timer unless tb200_peer_set_wait_limit chose another
// limit): on expiry the kernel records status 0x90000 | peer in the library's sticky status word and
// returns, so a missing rank surfaces as a host-visible error instead of a hung GPU.  A rank that gave
// up does not signal for that launch either, so its peers' next waits run out in turn.  Every rank must run on its own GPU: kernels that
// wait on one another must never share a device.
#include "kernels.h"
#include "ptx.cuh"

namespace tb200 {

namespace {

struct BarrierArgs {
  unsigned int* pads[kMaxOutputs];
  int rank;
  int world;
  int mode;
  unsigned long long wait_limit_ns;
};

__global__ void __launch_bounds__(32) peer_barrier_kernel(const BarrierArgs a) {
  // launched with programmatic serialization: let the kernel after start its own independent
  // prologue right away (it waits for this kernel's completion before it reads anything), then wait
  // for the kernel before, whose peer stores this barrier publishes
  if (threadIdx.x == 0) ptx::grid_launch_dependents();
  ptx::grid_dependency_wait();
  unsigned int* mine = a.pads[a.rank];
  unsigned int epoch = 0;
  if (threadIdx.x == 0) {
    epoch = mine[32];
    if (a.mode & kPeerSignal) mine[32] = ++epoch;
  }
  epoch = __shfl_sync(0xffffffffu, epoch, 0);
  const int peer = (int)threadIdx.x;
  if (peer >= a.world || peer == a.rank) return;
  if (a.mode & kPeerSignal) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.pads[peer] + a.rank), "r"(epoch) : "memory");
  }
  if (!(a.mode & kPeerWait)) return;
  const unsigned long long t0 = ptx::global_timer_ns();
  const unsigned int* slot = mine + peer;
  for (;;) {
    unsigned int seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(slot) : "memory");
    if ((int)(seen - epoch) >= 0) break;
    if (ptx::global_timer_ns() - t0 > a.wait_limit_ns) {
      report_timeout(0x90000u | (unsigned)peer);
      break;
    }
    __nanosleep(100);
  }
}

}  // namespace

cudaError_t launch_peer_barrier(unsigned int* const* pads, int rank, int world, int mode, cudaStream_t stream) {
  if (world < 1 || world > kMaxOutputs || rank < 0 || rank >= world) return cudaErrorInvalidValue;
  if (!(mode & (kPeerSignal | kPeerWait))) return cudaErrorInvalidValue;
  if (world == 1) return cudaSuccess;
  BarrierArgs a{};
  for (int i = 0; i < world; ++i) a.pads[i] = pads[i];
  a.rank = rank;
  a.world = world;
  a.mode = mode;
  a.wait_limit_ns = peer_wait_limit_ns();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, peer_barrier_kernel, a);
}

TB200_DEFINE_STATUS_READER(read_barrier_status)

}  // namespace tb200
