// Shared declarations of the tcb200 kernel library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <algorithm>
#include <utility>
#include <atomic>

#include "tcb200.h"

namespace tcb200 {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; used only when no device can be asked
// Multiprocessors of `device` (< 0: the calling thread's current device), asked once per device and cached;
// kNumSMs when there is no usable device (plans can be created and inspected on a host without a GPU).
// Persistent grids are sized from this, so a MIG slice or another Blackwell part is neither over- nor
// under-subscribed.
int sm_count(int device);

// Launch geometry + resolved tile of one plan.
struct Launch {
  dim3 grid{1, 1, 1};
  dim3 block{1, 1, 1};
  size_t smem = 0;
};

struct Plan {
  tcb200_problem_t p;
  tcb200_tile_t tile;
  int device;
  int sms = kNumSMs;  // multiprocessors of `device`, filled in by tcb200_plan_create
  Launch launch;
  int kernel_id;  // family-private selector of the instantiated kernel
  // Scratch global memory the launches of this plan need (reduction family, when the reduced range is
  // split over several CTAs): partial sums and one ticket counter per output tile.  0 = none.
  size_t scratch_floats = 0, scratch_tickets = 0;
};

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }
// Convolution strides (0 in the problem reads as 1) and the extents of the valid output window.
inline int64_t conv_sh(const tcb200_problem_t& p) { return p.conv_stride[0] > 0 ? p.conv_stride[0] : 1; }
inline int64_t conv_sw(const tcb200_problem_t& p) { return p.conv_stride[1] > 0 ? p.conv_stride[1] : 1; }
inline int64_t conv_oh(const tcb200_problem_t& p) { return (p.conv[4] - p.conv[6]) / conv_sh(p) + 1; }
inline int64_t conv_ow(const tcb200_problem_t& p) { return (p.conv[5] - p.conv[7]) / conv_sw(p) + 1; }

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device): the call costs tens of
// microseconds, more than the small kernels themselves.  `flags` is a per-kernel static bit set.
template <typename Fn>
inline cudaError_t ensure_dynamic_smem(Fn fn, int bytes, int device, std::atomic<uint64_t>& flags) {
  const uint64_t bit = 1ull << (device & 63);
  if (flags.load(std::memory_order_acquire) & bit) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) flags.fetch_or(bit, std::memory_order_release);
  return e;
}

// Programmatic dependent launch.  A kernel launched through launch_pdl() may be scheduled while the
// kernel before it in the stream is still running (as soon as SMs free up); it must call pdl_sync()
// before its first access to global memory: that releases its own dependents for early scheduling and
// then waits until the preceding kernel has completed and its writes are visible.  What a kernel does
// before pdl_sync() (barrier and tensor-memory set-up, descriptor prefetch) overlaps the tail of its
// predecessor; measured on the three MLP3 launches, same GPU: 360.9 us against 365.0 us per step.
// Both instructions are no-ops in a launch without the attribute.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_sync() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

// Thread-local record of the last failing CUDA call.
void set_last_cuda_error(cudaError_t e);

#define TCB200_CUDA_TRY(expr)                 \
  do {                                        \
    cudaError_t _e = (expr);                  \
    if (_e != cudaSuccess) {                  \
      ::tcb200::set_last_cuda_error(_e);      \
      return TCB200_ERR_CUDA;                 \
    }                                         \
  } while (0)

// ---- family entry points (each in its own .cu) ----------------------------------------
// *_query: append candidate tiles (preferred first); *_plan: validate + fill Launch;
// *_launch: enqueue.

int tensordot_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n);
int tensordot_plan(Plan& plan);
int tensordot_launch(const Plan& plan, const float* I0, const float* I1, float* O, cudaStream_t s,
                     int* dev_status);

int contraction_simt_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n);
int contraction_simt_plan(Plan& plan);
int contraction_simt_launch(const Plan& plan, const float* A, const float* B, const float* bias,
                            float* C, cudaStream_t s);

int contraction_tc_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n);
bool contraction_tc_preferred(const tcb200_problem_t& p);  // tensor-core tiles ahead of the SIMT ones
int contraction_tc_plan(Plan& plan);
// scratch: plan.scratch_floats floats when the plan splits the reduction (tile.split_k > 1), else unused;
// map_cache: a cache made by tc_map_cache_new() (may be null: the tensor maps are then encoded per launch)
int contraction_tc_launch(const Plan& plan, const float* A, const float* B, const float* bias,
                          float* C, cudaStream_t s, int* dev_status, float* scratch, void* map_cache);
// C = epilogue([C +] sum_s P[s]) over S dense planes P[s][M][N] of partial sums (splitk.cu)
int partial_planes_reduce(const float* P, float* C, const float* bias, int M, int N, int S, int64_t ldc, int epi,
                          int bias_on_m, int accumulate, int sms, cudaStream_t s);
// the same for the split tail of a CTA-pair launch: tail tile j = output tile tile0 + j (256 x 128, column tiles
// fastest), its S partial tiles dense at P[(s * tail_tiles + j) * 256 * 128]
int tail_tiles_reduce(const float* P, float* C, const float* bias, int M, int N, int S, int tail_tiles, int tile0,
                      int64_t ldc, int epi, int bias_on_m, int accumulate, cudaStream_t s);
constexpr int kTcMapSlots = 8;
void* tc_map_cache_new();
void tc_map_cache_delete(void* cache);

int group_conv_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n);
int group_conv_plan(Plan& plan);
int group_conv_launch(const Plan& plan, const float* I, const float* W, const float* bias,
                      float* O, cudaStream_t s, int* dev_status);
// reduction family (reduce.cu); partial / tickets: scratch of plan.scratch_floats floats and
// plan.scratch_tickets zeroed counters (may be null when the plan needs none)
constexpr int kReduceMaxSegments = 4096;
int reduce_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n);
int reduce_plan(Plan& plan);
int reduce_launch(const Plan& plan, const float* I, float* O, float* partial, unsigned* tickets, cudaStream_t s);
// The plan behind the opaque handle (abi.cu owns the handle type).
const Plan* plan_of(const tcb200_plan_t* handle);

// tensor-core variant with the filter rows as accumulator rows (group_conv_tap_rows.cu)
bool group_conv_tap_rows_ok(const tcb200_problem_t& p);
int group_conv_tap_rows_plan(Plan& plan);
bool group_conv_tap_rows_aligned(const float* I, const float* W, const float* O);
int group_conv_tap_rows_launch(const Plan& plan, const float* I, const float* W, const float* bias, float* O,
                               cudaStream_t s, int* dev_status);
// tensor-core variant (group_conv_tcgen05.cu)
bool group_conv_tc_ok(const tcb200_problem_t& p);
int group_conv_tc_plan(Plan& plan);
int group_conv_tc_launch(const Plan& plan, const float* I, const float* W, const float* bias,
                         float* O, cudaStream_t s, int* dev_status);

// ---- small device helpers ---------------------------------------------------------------

__device__ __forceinline__ float4 ldg_stream4(const float4* p) {
  // Read-once data: bypass L1 allocation so the streamed operand does not evict the reused one.
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void stg_stream4(float4* p, const float4& v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w)
               : "memory");
}

// Asynchronous global -> shared copies (LDGSTS): the data never passes through registers, so a
// thread can have many in flight instead of stalling on each load's first use.
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(
                   (uint32_t)__cvta_generic_to_shared(smem_dst)),
               "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                   (uint32_t)__cvta_generic_to_shared(smem_dst)),
               "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;" ::: "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
// waits until at most N of this thread's committed groups are still in flight
template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int EPI>
__device__ __forceinline__ float apply_epilogue(float acc, float bias) {
  if (EPI == TCB200_EPI_BIAS) return acc + bias;
  if (EPI == TCB200_EPI_BIAS_RELU) return fmaxf(acc + bias, 0.0f);
  if (EPI == TCB200_EPI_RELU) return fmaxf(acc, 0.0f);
  return acc;
}

__device__ __forceinline__ float apply_epilogue_rt(int epi, float acc, float bias) {
  if (epi == TCB200_EPI_BIAS) return acc + bias;
  if (epi == TCB200_EPI_BIAS_RELU) return fmaxf(acc + bias, 0.0f);
  if (epi == TCB200_EPI_RELU) return fmaxf(acc, 0.0f);
  return acc;
}

}  // namespace tcb200
