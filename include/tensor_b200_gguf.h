/* C ABI of libtensor_b200_gguf.so: B200 (sm_100a) GGUF dequant-fused GEMV / GEMM.
 *
 * This is the drop-in boundary for the one path the reference runs through
 * benchmarks/kernels/showcase/kernels.py:114-119 (`gguf(m, n, k, encoding)`:
 * `gemv_packed` for m == 1, `_packed` for m > 1), whose device kernels present the
 * signature `kernel(x, w, out)` with flat, 64-byte aligned buffers to the runtime
 * (src/tensor/runtime/executable.py:87-149 -> src/tensor/providers/cuda/device.py:211-229).
 *
 * Two layers are exported:
 *   1. plain-pointer entry points (device pointers, sizes, a CUstream as void*);
 *   2. `*_v1` entry points with the reference's C calling convention
 *      `int32_t fn(const TensorCallV1*, TensorErrorV1*)` (src/tensor/include/tensor/abi.h:141),
 *      which validate the descriptors before touching memory, as the reference's CPU image
 *      wrappers do (src/tensor/compiler/cpu.py:60-155), and then call layer 1.
 *
 * The structs below re-declare the reference's frozen ABI 1.3 layouts
 * (src/tensor/include/tensor/abi.h:37-85: 48 / 64 / 16 / 72 / 512 bytes); the library
 * static-asserts the sizes.  Status codes are abi.h:20-23.  Nothing is allocated by the
 * library on these paths: scratch memory is an explicit argument (the reference's ABI allows no
 * hidden workspace, src/tensor/runtime/abi.py:135-152).  All work is enqueued on the given
 * stream and returns without synchronising.  There is no CPU fallback.
 */
#ifndef TENSOR_B200_GGUF_H
#define TENSOR_B200_GGUF_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- reference ABI 1.3 layouts (abi.h:10-85) ---------------------------------------------- */
#ifndef TENSOR_ABI_H
#define TENSOR_ABI_VERSION 1u
#define TENSOR_DEVICE_CUDA 2u
#define TENSOR_ARG_BUFFER 1u
#define TENSOR_ARG_SCALAR 2u
#define TENSOR_OK 0
#define TENSOR_ERROR_ABI 1
#define TENSOR_ERROR_ARGUMENT 2
#define TENSOR_ERROR_PROVIDER 3
#define TENSOR_UINT8 3
#define TENSOR_INT32 6
#define TENSOR_INT64 8
#define TENSOR_FLOAT16 10
#define TENSOR_FLOAT32 11
#define TENSOR_BFLOAT16 13

typedef struct TensorBufferV1 {
  uint64_t address;
  uint64_t byte_size;
  const int64_t *shape;
  const int64_t *strides; /* bytes */
  uint32_t rank;
  uint32_t dtype;
  uint32_t device_type;
  int32_t device_ordinal;
} TensorBufferV1;

typedef struct TensorArgumentV1 {
  uint32_t kind;
  uint32_t dtype;
  TensorBufferV1 buffer;
  uint64_t scalar;
} TensorArgumentV1;

typedef struct TensorStreamV1 {
  uint32_t device_type;
  int32_t device_ordinal;
  uint64_t handle; /* CUstream */
} TensorStreamV1;

typedef struct TensorCallV1 {
  uint32_t abi_version;
  uint32_t struct_size;
  const TensorArgumentV1 *arguments;
  uint32_t argument_count;
  uint32_t flags;
  uint32_t grid[3];  /* ignored: the library sizes its own launches */
  uint32_t block[3]; /* ignored */
  uint64_t shared_memory_bytes; /* ignored */
  TensorStreamV1 stream;
} TensorCallV1;

typedef struct TensorErrorV1 {
  int32_t code;
  char message[508];
} TensorErrorV1;
#endif /* TENSOR_ABI_H */

/* ---- block formats: GGML type ids, the `encoding` of showcase/benchmark.py:122 ------------- */
#define TB200_Q4_0 2
#define TB200_Q8_0 8
#define TB200_Q4_K 12
#define TB200_Q6_K 14

/* kernel selection: 0 lets the library choose */
#define TB200_VARIANT_AUTO 0
#define TB200_VARIANT_SIMPLE 1 /* SIMT fp32 kernels, any shape */
#define TB200_VARIANT_FAST 2   /* a pipelined tensor-core kernel or an error: GEMV bulk-copy ring + mma.sync, GEMM tcgen05 */
#define TB200_VARIANT_MMA 3    /* GEMV only: the same as FAST */
#define TB200_VARIANT_TC 4     /* GEMV only: the persistent tcgen05 / TMEM kernel (Q4_K, Q6_K; needs scratch), or an
                                * error.  AUTO picks it for Q6_K above one activation row; for Q4_K the mma.sync
                                * pipeline measures faster */
#define TB200_VARIANT_DP4A 5   /* GEMV only, m = 1, every format: integer dot products against the activations split into
                                * three exact 8-bit limbs (no scratch), or an error.  AUTO picks it at m = 1 for Q6_K,
                                * Q8_0 and Q4_0 */

/* Library / ABI version: (major << 16) | minor. */
int32_t tb200_gguf_version(void);

/* Bytes of an [n, k] weight in `format`; -1 if k is not a multiple of the block size or the
 * format id is unknown.  Row stride is k / block * bytes (triton_kernels.py:136,144,164). */
int64_t tb200_gguf_weight_bytes(int32_t format, int64_t n, int64_t k);

/* Scratch bytes the GEMV can use at this shape on the current device: arrival counters and
 * split-K partial sums where K is split across CTAs, and for 1 < m <= 16 the activations converted
 * once per call (fp16 in fragment order, group sums, scale factors).  0 when neither applies.
 * Passing less (or NULL) is legal: the library then picks a plan that fits what it is given. */
int64_t tb200_gguf_gemv_scratch_bytes(int32_t format, int64_t m, int64_t n, int64_t k);

/* The launch plan the pipelined GEMV would use with `scratch_bytes` of scratch available:
 * plan_out[0..7] = {covered by the pipelined kernel (0/1), CTAs along K, CTAs along N,
 * 256-weight super-blocks per K range, ring stages, dynamic shared memory bytes, scratch bytes
 * needed, CTAs per SM}.  Without a CUDA device the plan is made for a B200 (148 SMs).  This is the
 * schedule the library derives (or the one recorded for the shape); TB200Schedule below pins one. */
int32_t tb200_gguf_gemv_plan(int32_t format, int64_t m, int64_t n, int64_t k, int64_t scratch_bytes,
                             int32_t *plan_out);

/* A schedule: the launch choices of the pipelined kernels that a caller may pin; a zero field means
 * "let the library derive it".  This is the counterpart of the reference's schedule dictionaries and
 * their legality predicate (src/tensor/compiler/cuda/schedules.py:3-52) for kernels that are written by
 * hand instead of generated: tb200_gguf_schedule_legal answers whether a schedule can run at a shape,
 * tb200_gguf_*_scheduled runs it, tb200_gguf_schedule_record makes it the default for that exact shape
 * in this process (what a search stores in its profile; src/tensor/compiler/search.py:29-159). */
#define TB200_OP_GEMV 1
#define TB200_OP_GEMM 2
typedef struct TB200Schedule {
  int32_t k_splits;      /* GEMV: CTAs along K per 16-row tile (1 .. 64) */
  int32_t ctas_per_sm;   /* GEMV: 1 (up to 16 decode warps) or 2 (8 decode warps each) */
  int32_t convert_ahead; /* GEMV, m > 1: 1 = activations converted by a kernel ahead of the GEMV (needs scratch), 2 = by every CTA */
  int32_t overlap;       /* 1 = the launch may start while its predecessor drains (default), 2 = fully serialized */
  int32_t gemm_shape;    /* GEMM: 11, 12 or 22 = <256-token tiles per CTA, decode warp groups> */
  int32_t reserved[3];
} TB200Schedule;
int32_t tb200_gguf_schedule_legal(int32_t op, int32_t format, int64_t m, int64_t n, int64_t k,
                                  int64_t scratch_bytes, const TB200Schedule *schedule);
int32_t tb200_gguf_schedule_record(int32_t op, int32_t format, int64_t m, int64_t n, int64_t k,
                                   const TB200Schedule *schedule);
void tb200_gguf_schedule_clear(void);
/* The pipelined GEMV / the tcgen05 GEMM with a pinned schedule; status 2 if it is not legal at the shape. */
int32_t tb200_gguf_gemv_scheduled(int32_t format, int32_t x_dtype, const void *x, const void *w, float *out,
                                  int64_t m, int64_t n, int64_t k, void *scratch, int64_t scratch_bytes,
                                  const TB200Schedule *schedule, void *stream, TensorErrorV1 *error);
int32_t tb200_gguf_gemm_scheduled(int32_t format, int32_t x_dtype, const void *x, const void *w, float *out,
                                  int64_t m, int64_t n, int64_t k, const TB200Schedule *schedule, void *stream,
                                  TensorErrorV1 *error);

/* Launch constants for packaging a static-shape kernel as a `.tbin` artifact of the reference
 * (src/tensor/artifacts/format.py), planned for a B200: the reference's provider launches with the
 * manifest's grid / block / shared memory and passes only the declared buffers, so the plan is baked
 * into the cubin.  gemv: out32 = {grid, threads, smem, k_splits, row_groups, row_tiles, sb_per_split,
 * nsb, stages, ring / staging layout ..., scratch bytes, CTAs per SM, counter bytes};
 * gemm: out8 = {grid.x, grid.y, threads, smem, token tile, k per stage, 0, 0}. */
int32_t tb200_gguf_gemv_launch_config(int32_t format, int32_t x_dtype, int64_t m, int64_t n, int64_t k,
                                      int64_t scratch_bytes, int32_t *out32);
int32_t tb200_gguf_gemm_launch_config(int32_t format, int64_t m, int64_t n, int64_t k, int32_t *out8);

/* Synchronises the current device and reads the sticky status words of the pipelined kernels.
 * Every device-side wait in this library is bounded (about two seconds); a wait that gives up
 * records a code there and the kernel returns instead of hanging.  Returns TENSOR_OK and
 * *status == 0 when nothing was recorded; the words are cleared by the call.  No counterpart in
 * the reference (its generated kernels do not wait on anything). */
int32_t tb200_gguf_device_status(uint32_t *status, TensorErrorV1 *error);

/* out[n, k] (fp32) = dequant(w).  Replaces the decode the reference states in
 * benchmarks/kernels/showcase/triton_kernels.py:133-181; results are bit-identical to it. */
int32_t tb200_gguf_dequant(int32_t format, const void *w, float *out, int64_t n, int64_t k,
                           void *stream, TensorErrorV1 *error);

/* Decode GEMV: out[m, n] (fp32) = x[m, k] . dequant(w[n, k])^T with fp32 weights and fp32
 * accumulation, 1 <= m.  Replaces `gemv_packed` (showcase/kernels.py:116-119; contract
 * showcase/benchmark.py:468-470, triton_kernels.py:213-222).  x_dtype is TENSOR_FLOAT16,
 * TENSOR_BFLOAT16 or TENSOR_FLOAT32.  If scratch is used, it must start zeroed before the first
 * call; every call leaves its counters zeroed again (the rest is overwritten before it is read).
 * Calls that share scratch must not overlap. */
int32_t tb200_gguf_gemv(int32_t format, int32_t x_dtype, const void *x, const void *w, float *out,
                        int64_t m, int64_t n, int64_t k, void *scratch, int64_t scratch_bytes,
                        int32_t variant, void *stream, TensorErrorV1 *error);

/* The same GEMV for callers that may neither pass scratch nor let the library allocate: launch
 * adapters that forward only an artifact's declared buffers, hosts that own all device memory in
 * their own arena, code inside a stream capture.  The split-K scratch is a 4 MiB array built into
 * the library image (held by every GPU that loads the library, until exit).  Shapes that want more
 * are rejected with status 2.  The first call on a device resolves the array's address: make it
 * outside any stream capture.  All calls on a device share the array, so calls must not overlap on
 * the GPU; each call clears the counters it needs first.  Calls no allocator.  This entry point
 * has no counterpart in the reference. */
#define TB200_GEMV_STATIC_SCRATCH_BYTES (4u << 20)
int32_t tb200_gguf_gemv_static(int32_t format, int32_t x_dtype, const void *x, const void *w, float *out,
                               int64_t m, int64_t n, int64_t k, void *stream, TensorErrorV1 *error);

/* Two weights of the same format and K applied to the same activations in ONE launch (gate and up
 * of an MLP, or q/k/v): out[m, n1 + n2] holds x . dequant(w1)^T in columns 0 .. n1 and
 * x . dequant(w2)^T in columns n1 .. n1 + n2, exactly as two calls of tb200_gguf_gemv would have
 * produced them.  A decode GEMV costs several microseconds of launch, staging and tail whatever its
 * size; grouping pays them once.  Where the pipelined kernel cannot take the pair in one launch
 * (K split across CTAs, n1 not a multiple of 16, other formats) the call issues two launches into
 * the same output.  scratch: as tb200_gguf_gemv for the shape (m, n1 + n2, k).  The reference
 * launches one kernel per weight (showcase/kernels.py:114-119); no counterpart there. */
int32_t tb200_gguf_gemv_pair(int32_t format, int32_t x_dtype, const void *x, const void *w1, int64_t n1,
                             const void *w2, int64_t n2, float *out, int64_t m, int64_t k,
                             void *scratch, int64_t scratch_bytes, int32_t variant, void *stream,
                             TensorErrorV1 *error);

/* N-sharded GEMV: this rank holds n of the projection's rows (w is [n, k]) and writes its n result
 * columns into `out_count` destinations: element (row, col) goes to
 * outs[i][row * out_ld + col_offset + col].  outs is a HOST array of device addresses; outs[0] is
 * normally this rank's own full-width output and outs[1..] the other ranks' outputs as mapped into
 * this process (CUDA IPC / peer access), so the all-gather of the reference-side plan "shard along
 * N, gather `out`" happens in the kernel's own stores over NVLink.  Follow it (once per group of
 * projections) with tb200_peer_barrier before anything reads the outputs.  out_count <= 8,
 * out_ld >= col_offset + n.  The reference has no multi-GPU path; the per-shard call is an
 * ordinary launch(x, w_shard, out_shard) (src/tensor/providers/cuda/device.py:30-39). */
#define TB200_MAX_PEERS 8
int32_t tb200_gguf_gemv_sharded(int32_t format, int32_t x_dtype, const void *x, const void *w,
                                float *const *outs, int32_t out_count, int64_t out_ld,
                                int64_t col_offset, int64_t m, int64_t n, int64_t k, void *scratch,
                                int64_t scratch_bytes, int32_t variant, void *stream,
                                TensorErrorV1 *error);

/* The same with the cross-GPU ordering folded into the launch, so that a decode step needs no
 * barrier kernels: with TB200_PEER_WAIT the kernel waits, after filling its weight ring and before
 * it reads x, until every peer has signalled as often as this rank has; with TB200_PEER_SIGNAL
 * the last CTA to store its outputs signals every peer.  pads / rank / world are those of
 * tb200_peer_barrier, and both forms count on the same pads, so they can be mixed: a signal by
 * one and the matching wait by the other.  Typical step: gate (wait), up (signal), down (wait and
 * signal).  The waits are bounded like the barrier's (status 0x80000 | peer).  Where the shape is
 * served by the fallback kernel the same ordering is enforced with separate wait / signal launches. */
#define TB200_PEER_WAIT 1
#define TB200_PEER_SIGNAL 2
int32_t tb200_gguf_gemv_sharded_sync(int32_t format, int32_t x_dtype, const void *x, const void *w,
                                     float *const *outs, int32_t out_count, int64_t out_ld,
                                     int64_t col_offset, int64_t m, int64_t n, int64_t k,
                                     void *scratch, int64_t scratch_bytes, int32_t variant,
                                     uint32_t *const *pads, int32_t rank, int32_t world,
                                     int32_t sync, void *stream, TensorErrorV1 *error);

/* tb200_gguf_gemv_pair for an N-sharded rank: this rank's n1 rows of the first weight and n2 rows of
 * the second (same format, K and activations) in one launch; the first weight's columns go to
 * outs1[i][row * out_ld + col_offset1 + col], the second's to outs2[i][row * out_ld + col_offset2 +
 * col], for every destination i (own buffers first, then the peers').  pads / rank / world / sync as
 * in tb200_gguf_gemv_sharded_sync.  Falls back to two sharded launches (wait on the first, signal on
 * the second) where the pair cannot share a launch. */
int32_t tb200_gguf_gemv_pair_sharded_sync(int32_t format, int32_t x_dtype, const void *x, const void *w1,
                                          int64_t n1, const void *w2, int64_t n2, float *const *outs1,
                                          float *const *outs2, int32_t out_count, int64_t out_ld,
                                          int64_t col_offset1, int64_t col_offset2, int64_t m, int64_t k,
                                          void *scratch, int64_t scratch_bytes, int32_t variant,
                                          uint32_t *const *pads, int32_t rank, int32_t world,
                                          int32_t sync, void *stream, TensorErrorV1 *error);

/* Several independent decode GEMVs in one call: what a decoder layer issues back to back -- q/k/v,
 * gate/up, or one projection at several batches.  The reference launches one kernel per projection
 * (showcase/kernels.py:114-119, showcase/benchmark.py:276-290) and pays its host path per launch
 * (runtime/executable.py:87-149); here the host path is paid once and the launches overlap each
 * other's tails.  Item i computes outs[d][row * out_ld + col] = x_i . dequant(w_i)^T for every
 * destination d < out_count (outs[1..] are peer-mapped outputs of other ranks in N-sharded runs, with
 * the column window already added to the pointers).  Items must not depend on one another.
 * Neighbouring items with the same x pointer, m, k and format run as one grouped launch.
 * variant: TB200_VARIANT_AUTO ... as for tb200_gguf_gemv; TB200_VARIANT_TC runs the whole list as ONE
 * persistent tcgen05 / TMEM launch (Q4_K or Q6_K, 2-byte activations, m <= 16).
 * scratch: tb200_gguf_gemv_list_scratch_bytes (a slice per launch), 256-byte aligned, zeroed before first
 * use, not shared with a call that may overlap.  With a slice per launch the activation conversions of
 * all batched items (m > 1) are issued ahead of the first GEMV, so that the GEMVs follow one another
 * directly; a smaller buffer that holds the largest single need is accepted (the launches then share it
 * and every conversion runs right before its GEMV).  pads / rank / world / sync as in
 * tb200_gguf_gemv_sharded_sync (sync 0 on one GPU): the first launch waits (and so does every conversion
 * launch, which reads activations ahead of it), the last one signals. */
#define TB200_GEMV_LIST_MAX 12
typedef struct TB200GemvItem {
  int32_t format;  /* TB200_Q4_K ... */
  int32_t x_dtype; /* TENSOR_FLOAT16 / TENSOR_BFLOAT16 / TENSOR_FLOAT32 */
  const void *x;   /* [m, k] */
  const void *w;   /* [n, k] raw blocks */
  float *outs[TB200_MAX_PEERS];
  int32_t out_count;
  int32_t reserved;
  int64_t out_ld;
  int64_t m, n, k;
} TB200GemvItem;
int64_t tb200_gguf_gemv_list_scratch_bytes(const TB200GemvItem *items, int32_t count);
int32_t tb200_gguf_gemv_list(const TB200GemvItem *items, int32_t count, void *scratch,
                             int64_t scratch_bytes, int32_t variant, uint32_t *const *pads, int32_t rank,
                             int32_t world, int32_t sync, void *stream, TensorErrorV1 *error);

/* The steps either side of a decode projection, launched so that they chain with the GEMVs without a gap
 * (programmatic dependent launch): RMS normalisation of the fp32 residual stream into the bf16
 * activations of the next projection, SwiGLU of the fp32 [m, 2 * width] output of a grouped gate + up launch
 * into the bf16 activations of the down projection, and the residual add behind a projection.  The
 * reference states these as generated kernels (packages/tensor-nn/src/tensor_nn/kernels/normalization.py)
 * or matmul epilogues (tensor_nn/kernels/linear.py:6-100).  Pointers 16-byte aligned, k / width / count
 * multiples of 4. */
int32_t tb200_rmsnorm_bf16(const float *x, const float *weight, void *out_bf16, int64_t m, int64_t k, float eps,
                           void *stream, TensorErrorV1 *error);
int32_t tb200_swiglu_bf16(const float *gate_up, void *out_bf16, int64_t m, int64_t width, void *stream,
                          TensorErrorV1 *error);
int32_t tb200_residual_add(float *stream_buffer, const float *delta, int64_t count, void *stream,
                           TensorErrorV1 *error);

/* How long a kernel of this library waits for another GPU's signal before it gives up, records
 * 0x80000 | peer (GEMV) or 0x90000 | peer (barrier) in the status word and returns; 0 restores the
 * default of two seconds.  Process-wide; applies to launches made after the call.  A rank whose wait
 * ran out does not signal for that launch, so its peers' waits run out in turn: read
 * tb200_gguf_device_status on every rank and re-zero the pads before going on. */
int32_t tb200_peer_set_wait_limit(uint64_t nanoseconds);

/* Barrier between the GPUs of one box over peer-mapped signal pads.  pads is a HOST array of
 * `world` device addresses: pads[i] is rank i's pad (TB200_SIGNAL_PAD_BYTES, 4-byte aligned,
 * zero-filled once before the first use) as mapped into this process.  The kernel announces on
 * every peer's pad that all work enqueued on `stream` before it is complete, then waits until
 * every peer has announced the same; the wait gives up after two seconds and leaves
 * 0x90000 | peer in the device status word (tb200_gguf_device_status).  Every rank must call it
 * the same number of times, each rank on its own GPU.  No counterpart in the reference. */
#define TB200_SIGNAL_PAD_BYTES 256
int32_t tb200_peer_barrier(uint32_t *const *pads, int32_t rank, int32_t world, void *stream,
                           TensorErrorV1 *error);
/* One half of the barrier: mode TB200_PEER_SIGNAL announces, TB200_PEER_WAIT waits until every peer
 * has announced as often as this rank has; both together are tb200_peer_barrier. */
int32_t tb200_peer_sync(uint32_t *const *pads, int32_t rank, int32_t world, int32_t mode,
                        void *stream, TensorErrorV1 *error);

/* Peer mapping of host-owned device memory between the processes of one box (one process per
 * GPU), for the two entry points above.  tb200_peer_export writes the 64-byte CUDA IPC handle of
 * the allocation that contains ptr and ptr's byte offset inside it; the host sends both to the other
 * ranks by its own means.  tb200_peer_open maps such an allocation into the calling process on the
 * current device (peer access is enabled as a side effect) and returns its base: the peer's ptr is
 * base + offset.  An allocation can be opened once per process; tb200_peer_close unmaps it.  The
 * library allocates nothing here either: the memory stays the exporting host's.  The exporting
 * allocation must come from cudaMalloc (for PyTorch: the default caching allocator, not expandable
 * segments).  No counterpart in the reference. */
#define TB200_PEER_HANDLE_BYTES 64
int32_t tb200_peer_export(const void *ptr, uint8_t *handle, int64_t *offset, TensorErrorV1 *error);
int32_t tb200_peer_open(const uint8_t *handle, void **base, TensorErrorV1 *error);
int32_t tb200_peer_close(void *base, TensorErrorV1 *error);

/* Prefill GEMM: out[m, n] (fp32) = x[m, k] . dequant(w[n, k])^T with both operands rounded to
 * bf16 and fp32 accumulation.  Replaces `_packed` (showcase/kernels.py:116-119; contract
 * showcase/benchmark.py:471-477, triton_kernels.py:184-210, there with fp16 operands).
 * x_dtype must be TENSOR_BFLOAT16. */
int32_t tb200_gguf_gemm(int32_t format, int32_t x_dtype, const void *x, const void *w, float *out,
                        int64_t m, int64_t n, int64_t k, int32_t variant, void *stream,
                        TensorErrorV1 *error);

/* Descriptor forms (reference convention, abi.h:141).  Arguments, in order:
 *   dequant: buffers w (uint8), out (float32); scalars n, k, format.
 *   gemv:    buffers x, w (uint8), out (float32)[, scratch (uint8)]; scalars m, n, k, format[, variant].
 *   gemm:    buffers x (bfloat16), w (uint8), out (float32); scalars m, n, k, format[, variant].
 * Scalars are TENSOR_INT32 or TENSOR_INT64.  call->stream.handle is the CUstream. */
int32_t tb200_gguf_dequant_v1(const TensorCallV1 *call, TensorErrorV1 *error);
int32_t tb200_gguf_gemv_v1(const TensorCallV1 *call, TensorErrorV1 *error);
int32_t tb200_gguf_gemm_v1(const TensorCallV1 *call, TensorErrorV1 *error);

#ifdef __cplusplus
}
#endif
#endif
