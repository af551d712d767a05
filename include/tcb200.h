/*
 * tcb200 — C ABI of the sm_100a kernel library behind the Tensor Comprehensions
 * execution backend.
 *
 * This is the boundary a replacement for the reference's device runtime binds:
 * where the reference JIT-compiles CUDA-C and launches it with cuLaunchKernel
 * (tc/core/cuda/cuda_rtc.cc:299-387, reached from CudaTcExecutor::uncheckedRun,
 * tc/core/cuda/cuda_tc_executor.cc:111-126), the new executor describes the
 * pattern-matched comprehension as a tcb200_problem_t and calls into this
 * library.  Plain C types, status codes, caller-owned memory, stream-ordered,
 * re-entrant: no function here throws, aborts or calls exit().
 *
 * All tensor pointers are DEVICE pointers to dense row-major float32 data owned
 * by the caller (the reference's layout: docs/source/semantics.rst:17-19).
 */
#ifndef TCB200_H_
#define TCB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TCB200_ABI_VERSION 3

/* Opaque CUDA stream handle; identical to cudaStream_t / CUstream. */
typedef struct CUstream_st* tcb200_stream_t;

/* Kernel families a comprehension can be matched to. */
enum {
  TCB200_FAMILY_CONTRACTION = 1, /* C(b,m,n) (+)= sum_k A(b,m,k) * B(b,n,k)  [+bias] [relu] */
  TCB200_FAMILY_TENSORDOT = 2,   /* O(n,c1,c3,p) = sum_c2 I0(n,c1,c2,p) * I1(n,c2,c3,p), tiny C2,C3 */
  TCB200_FAMILY_GROUP_CONV = 3,  /* O(n,g,f,h,w) = sum_{c,kh,kw} I(n,g,c,h+kh,w+kw) * W(g,f,c,kh,kw) [+B(g,f)] */
  TCB200_FAMILY_REDUCTION = 4,   /* O(a,b) (+)= sum_c I(a,c,b): one input, sum over a contiguous group of its indices
                                    (sum1D / sum2D of test/test_tc_mapper_harness-inl.h:60-146) */
  TCB200_FAMILY_COPY = 5         /* O(i...) = I(i...): a whole-tensor copy (red[0] = number of elements), what a
                                    statement such as d_Bias(m) = Bias(m) is (python/tests/test_tc.py:403-407) */
};

/* Elementwise statements fused after the reduction (how the reference's TCs
 * spell bias and ReLU: tc/library/fcrelu.h:24-26). */
enum {
  TCB200_EPI_NONE = 0,
  TCB200_EPI_BIAS = 1,      /* O = O + bias             */
  TCB200_EPI_BIAS_RELU = 2, /* O = fmax(O + bias, 0)    */
  TCB200_EPI_RELU = 3       /* O = fmax(O, 0)           */
};

/* Kernel variants inside a family (the tile sweep behind ATenAutotuner::tune
 * enumerates them; tc/aten/aten_autotuner.h:73-78 only promises "best first"). */
enum {
  TCB200_VARIANT_AUTO = 0,
  TCB200_VARIANT_SIMT = 1,       /* fp32 FMA, shared-memory tiled                                */
  TCB200_VARIANT_SIMT_SMALL = 2, /* fp32 FMA, one whole small matrix pair per CTA (batched)      */
  TCB200_VARIANT_TCGEN05 = 3,    /* tcgen05/TMEM tiles fed by TMA, TF32 with optional 3x split   */
  TCB200_VARIANT_TCGEN05_TS = 4, /* same, 3xTF32 with the A operand staged in tensor memory     */
  TCB200_VARIANT_TCGEN05_PAIR = 5 /* same on CTA pairs (cta_group::2): 256-row tiles, B split over the pair; an output of
                                     at most 128 rows runs as C^T = B A^T with its tiles written transposed */
};

/* Status codes (0 = success, negative = error). */
enum {
  TCB200_OK = 0,
  TCB200_ERR_INVALID_ARGUMENT = -1,
  TCB200_ERR_UNSUPPORTED = -2,   /* no kernel of the library covers this problem/tile: hard error, no fallback */
  TCB200_ERR_CUDA = -3,          /* a CUDA runtime/driver call failed; tcb200_last_cuda_error() has the code   */
  TCB200_ERR_ALIGNMENT = -4,     /* a pointer or leading dimension breaks the kernel's alignment rule          */
  TCB200_ERR_DEVICE_TIMEOUT = -5,/* a bounded device-side wait gave up (reported through dev_status)           */
  TCB200_ERR_NO_DEVICE = -6,
  TCB200_ERR_TOO_LARGE = -7
};

enum { TCB200_REDUCE_SUM = 0, TCB200_REDUCE_MAX = 1, TCB200_REDUCE_MIN = 2, TCB200_REDUCE_PROD = 3 };

typedef struct tcb200_problem {
  int32_t family;
  int32_t epilogue;
  int32_t accumulate;  /* 0: "+=!" the output is overwritten; 1: "+=" added to what the output holds
                          (test/cuda/test_compile_and_run.cc:181-200) */
  int32_t a_k_major;   /* contraction: 1 if A's reduction index is innermost (A(m,k)), 0 if A(k,m) */
  int32_t b_k_major;   /* contraction: 1 if B's reduction index is innermost (B(n,k)), 0 if B(k,n) */
  int32_t bias_on_m;   /* contraction: 0 bias is indexed by n (columns), 1 by m (rows) */
  int64_t batch, M, N, K;
  int64_t lda, ldb, ldc;                /* leading dimensions, in elements */
  int64_t stride_a, stride_b, stride_c; /* batch strides, in elements (0 = shared by all batches) */
  int64_t conv[8];                      /* group conv: N, G, C, F, H, W, KH, KW (valid window) */
  int64_t td[5];                        /* tensordot: N, C1, C2, C3, P (P = product of trailing shared dims) */
  int64_t conv_stride[2];               /* group conv: SH, SW of I(.., SH*h+kh, SW*w+kw) (tc/library/convolution.h:27-31);
                                           0 reads as 1.  Output extent: (H - KH) / SH + 1 by (W - KW) / SW + 1 */
  int64_t red[3];                       /* reduction: A, C, B of the [A][C][B] view of the input (C is reduced) */
  int32_t reduce_op;                    /* reduction: TCB200_REDUCE_SUM (+=), _MAX (max=), _MIN (min=), _PROD (*=) */
  int32_t batch_reduce;                 /* contraction: 1 = the batch index is reduced too,
                                           C(m,n) (+)= sum_b sum_k A(b,m,k) * B(b,n,k)  (stride_c is ignored).  Runs as a
                                           batched contraction into one plane of partial sums per batch entry (scratch
                                           memory owned by the plan) and a second pass that adds the planes in order. */
} tcb200_problem_t;

/* One point of a family's tile sweep.  Fields a variant does not use are 0. */
typedef struct tcb200_tile {
  int32_t variant;
  int32_t bm, bn, bk;  /* CTA tile (contraction); bm = rows of C1 per CTA (tensordot) */
  int32_t stages;      /* TMA pipeline depth (tcgen05 contraction).  Group convolution: which kernel of the family
                          (SIMT: 0 band / rows, 4 item, 5 run of items, 6 channel-split item; tcgen05_ts: 3 = filters
                          stationary in tensor memory with the filter rows as accumulator rows, 4 = pixels x F) */
  int32_t threads;     /* CTA size */
  int32_t split_tf32;  /* tcgen05: 1 = one TF32 pass, 3 = 3xTF32 split keeping fp32 accuracy, 4 = the same with
                          every accumulator drained after each of its k-blocks (strict accumulation: meets the
                          reference's checkRtol on all-positive operands too; slower) */
  int32_t split_k;     /* tensor-memory contraction tiles: CTAs that share the reduction of one output tile
                          (0 or 1 = none).  A split contraction keeps S x M x N partial sums in scratch memory
                          owned by the plan and adds them in a fixed order in a second small kernel. */
} tcb200_tile_t;

typedef struct tcb200_plan tcb200_plan_t;

/* Library / device probes. */
int tcb200_abi_version(void);
const char* tcb200_strerror(int status);
int tcb200_last_cuda_error(void); /* cudaError_t of the last TCB200_ERR_CUDA on this thread */
int tcb200_device_count(int* count);

/* Candidate tiles for a problem, preferred first.  Writes at most `max`
 * entries to `out` and the number available to *n.  Replaces the search space
 * of the reference's genetic autotuner (tc/autotuner/autotuner-inl.h:326-404). */
int tcb200_query(const tcb200_problem_t* problem, tcb200_tile_t* out, int max, int* n);

/* Validates problem+tile and records launch geometry for `device`.  tile may be
 * NULL (family default).  No kernel is launched and no device memory is
 * allocated.  Replaces CudaBackend::compileWithTcMapper + CudaRTCFunction::Compile
 * (tc/core/cuda/cuda_tc_executor.cc:71-109, tc/core/cuda/cuda_rtc.cc:265-287). */
int tcb200_plan_create(const tcb200_problem_t* problem, const tcb200_tile_t* tile,
                       int device, tcb200_plan_t** plan);
int tcb200_plan_destroy(tcb200_plan_t* plan);

/* Grid / block the plan launches with (CudaTcExecutor::grid()/block(),
 * tc/core/cuda/cuda_tc_executor.h:27-66) and a one-line human-readable
 * description (what TcExecutor::compiledSource holds, tc/core/tc_executor.h:104-106). */
int tcb200_plan_geometry(const tcb200_plan_t* plan, int64_t grid[3], int64_t block[3]);
int tcb200_plan_describe(const tcb200_plan_t* plan, char* buf, size_t buflen);
int tcb200_plan_tile(const tcb200_plan_t* plan, tcb200_tile_t* tile);

/* Enqueues the plan on `stream` of the CURRENT device (which must be the plan's
 * device) and returns without synchronising.  Replaces CudaRTCFunction::Launch
 * (tc/core/cuda/cuda_rtc.cc:299-387).
 *   inputs : contraction {A, B[, bias]}; tensordot {I0, I1}; group conv {I, W[, bias]}; reduction {I}; copy {I}
 *   outputs: {O}
 *   dev_status: optional device int; a kernel whose bounded wait gives up stores a
 *               nonzero code there instead of spinning (NULL: not reported).
 * The plan is immutable: it may be launched concurrently from several host threads
 * and streams.  One exception: a reduction plan that splits the reduced range over several CTAs
 * (tile.bn > 1) and a contraction plan that splits its reduction (tile.split_k > 1) keep partial sums in
 * scratch memory owned by the plan, allocated and zeroed by its
 * first launch (cudaMalloc is a synchronous call: not inside a stream capture; the counters are zeroed on
 * `stream`, ahead of the kernel) and freed by tcb200_plan_destroy; launches of one such plan must not
 * overlap in time. */
int tcb200_launch(const tcb200_plan_t* plan, const void* const* inputs, int n_inputs,
                  void* const* outputs, int n_outputs, tcb200_stream_t stream,
                  int* dev_status);

/* The same launch for a reduction plan, with its scratch (tickets + partial sums) taken from a fixed
 * array in device memory that is part of the library image instead of memory the plan allocates: no
 * allocation happens in this call, at the first launch or ever.  No counterpart in the reference (it
 * generates single-pass reductions and has no scratch memory to place).
 *   - Limit: TCB200_STATIC_SCRATCH_TICKETS counters and TCB200_STATIC_SCRATCH_FLOATS partial sums
 *     (the array is 1 MiB + 16 KiB per device); a plan that needs more is refused with
 *     TCB200_ERR_TOO_LARGE and nothing is launched.  Plans of other families: TCB200_ERR_INVALID_ARGUMENT.
 *   - The first call on a device looks the array's address up (cudaGetSymbolAddress, which may load the
 *     module and synchronise): make that call before any stream capture begins.
 *   - Every call, and every plan, uses the same array of its device: two calls whose kernels can overlap
 *     in time (different streams, or host threads) race on it and give wrong sums.  Calls on one stream
 *     are ordered and safe.  The counters the launch uses are cleared on `stream` ahead of the kernel. */
#define TCB200_STATIC_SCRATCH_TICKETS 4096
#define TCB200_STATIC_SCRATCH_FLOATS (256 * 1024)
int tcb200_reduce_launch_static(const tcb200_plan_t* plan, const void* input, void* output,
                                tcb200_stream_t stream);


/* Device plumbing for hosts that do not link the CUDA runtime themselves (the C++ host library
 * reaches CUDA only through this ABI).  tcb200_set_device / tcb200_get_device wrap the calling
 * thread's current device (the reference's WithCudaDevice, tc/core/cuda/cuda.h:79-96);
 * tcb200_device_name is the device string tuned configurations are keyed by
 * (CudaGPUInfo::getCudaDeviceStr, tc/core/cuda/cuda.h:98-118). */
int tcb200_get_device(int* device);
int tcb200_set_device(int device);
int tcb200_device_name(int device, char* buf, size_t buflen);
int tcb200_stream_synchronize(tcb200_stream_t stream);

/* Event timer around any number of launches on `stream`: start records an event, stop records a
 * second one, waits for it and returns the elapsed device time in microseconds (what
 * CudaRTCFunction::Launch does when profiling, tc/core/cuda/cuda_rtc.cc:373-386, without
 * truncating to whole microseconds).  stop destroys the timer. */
typedef struct tcb200_timer tcb200_timer_t;
int tcb200_timer_start(tcb200_stream_t stream, tcb200_timer_t** timer);
int tcb200_timer_stop(tcb200_timer_t* timer, tcb200_stream_t stream, float* elapsed_us);

/* Device status word: a device int that the kernels' bounded waits report into (the dev_status argument of
 * tcb200_launch).  create allocates and zeroes one on the current device; check waits for `stream`, copies the
 * word to *code, clears it, and returns TCB200_OK when it was zero, TCB200_ERR_DEVICE_TIMEOUT otherwise (the
 * context stays usable: a wait that gives up makes its kernel stop issuing work and leave through its normal
 * exit).  This is how a failed launch reaches the host, where the reference's enforce macros throw
 * (tc/core/cuda/cuda.h:38-73) and its tuner discards the candidate (tc/autotuner/autotuner-inl.h:204-214). */
int tcb200_status_create(int** dev_status);
int tcb200_status_destroy(int* dev_status);
int tcb200_status_check(int* dev_status, tcb200_stream_t stream, int* code);

/* Self-test of the bounded waits: launches one warp that waits on an mbarrier nothing ever arrives on, through
 * the same wait routine the kernels use, with the limit set to `limit_cycles` SM cycles (the kernels use ~4e9).
 * The wait runs out, the warp records TCB200_SELFTEST_WAIT_CODE in *dev_status and the kernel returns.  No
 * counterpart in the reference (its generated kernels never wait on one another). */
#define TCB200_SELFTEST_WAIT_CODE 99
int tcb200_selftest_wait(long long limit_cycles, int* dev_status, tcb200_stream_t stream);

/* Device time of very short launches.  begin creates a private stream and starts capturing it (thread-local
 * capture mode); the caller enqueues any number of launches on *capture_stream; end closes the capture,
 * instantiates the graph, replays it once untimed and `timed_replays` times between two events, and returns
 * the device time of ONE replay in microseconds.  A kernel of a few microseconds is then timed at the
 * device's pace, not at the host's launch rate (the reference times one launch between two events,
 * tc/core/cuda/cuda_rtc.cc:373-386, which its whole-microsecond Duration then truncates).  Everything the
 * launches need to allocate or configure must have happened before (one plain launch does that).  end
 * destroys the object whether it succeeds or not. */
typedef struct tcb200_replay tcb200_replay_t;
int tcb200_replay_begin(tcb200_replay_t** replay, tcb200_stream_t* capture_stream);
int tcb200_replay_end(tcb200_replay_t* replay, int timed_replays, float* elapsed_us_per_replay);

/* Assembles an all-gathered output on `stream`.  `gathered` holds the shards of `world` ranks one after the
 * other, each padded to the largest shard: [world][rows][max_count * inner] floats, where the sharded
 * dimension has `total` entries split as total / world per rank with the remainder on the first ranks,
 * `rows` is the product of the dimensions in front of it and `inner` of those behind it.  `out` receives the
 * unsharded row-major tensor [rows][total * inner].  rows = 1 trims the padding of a dimension-0 shard;
 * rows = M turns the transposed matmul's [world][M][N / world] into C[M][N].  No counterpart in the
 * reference, which runs a comprehension on one device (its only multi-GPU code is the tuner's,
 * tc/autotuner/autotuner-inl.h:279-295). */
int tcb200_assemble_shards(const void* gathered, void* out, int world, int64_t rows, int64_t total,
                           int64_t inner, tcb200_stream_t stream);

/* Writes `bytes` of a rotating pattern to `buf` on `stream`: the bench uses it to
 * evict L2 between timed launches of the small problems. */
int tcb200_l2_flush(void* buf, size_t bytes, tcb200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TCB200_H_ */
