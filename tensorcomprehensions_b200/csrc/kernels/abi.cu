// extern "C" surface of the tcb200 kernel library (declared in include/tcb200.h).
// Validates arguments, owns the immutable plan objects and dispatches to the
// kernel families.  Nothing here throws or aborts; every failure is a status code.
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <new>

#include "async.cuh"
#include "common.cuh"

namespace tcb200 {

static thread_local cudaError_t g_last_cuda_error = cudaSuccess;
void set_last_cuda_error(cudaError_t e) { g_last_cuda_error = e; }

int sm_count(int device) {
  static std::atomic<int> cached[64];
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) {
    (void)cudaGetLastError();
    return kNumSMs;
  }
  if (device < 0 || device >= 64) return kNumSMs;
  int n = cached[device].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    return kNumSMs;
  }
  cached[device].store(n, std::memory_order_relaxed);
  return n;
}

namespace {

__global__ void l2_flush_kernel(float4* buf, size_t n4, float v) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4;
       i += (size_t)gridDim.x * blockDim.x)
    buf[i] = make_float4(v, v, v, v);
}

// One warp waits on a barrier that nothing arrives on; the bounded wait gives up after `limit` cycles.
__global__ void selftest_wait_kernel(long long limit, int* dev_status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  mbar_wait_slow(&bar, 0, TCB200_SELFTEST_WAIT_CODE, dev_status, &abort_flag, limit);
}

int n_inputs_expected(const tcb200_problem_t& p) {
  if (p.family == TCB200_FAMILY_REDUCTION || p.family == TCB200_FAMILY_COPY) return 1;
  const bool has_bias = p.epilogue == TCB200_EPI_BIAS || p.epilogue == TCB200_EPI_BIAS_RELU;
  return 2 + (has_bias ? 1 : 0);
}

const char* variant_name(int v) {
  switch (v) {
    case TCB200_VARIANT_SIMT: return "simt";
    case TCB200_VARIANT_SIMT_SMALL: return "simt_small";
    case TCB200_VARIANT_TCGEN05: return "tcgen05";
    case TCB200_VARIANT_TCGEN05_TS: return "tcgen05_ts";
    case TCB200_VARIANT_TCGEN05_PAIR: return "tcgen05_pair";
    default: return "auto";
  }
}

const char* epilogue_name(int e) {
  switch (e) {
    case TCB200_EPI_BIAS: return "+bias";
    case TCB200_EPI_BIAS_RELU: return "+bias,relu";
    case TCB200_EPI_RELU: return "relu";
    default: return "none";
  }
}

}  // namespace
}  // namespace tcb200

using namespace tcb200;

struct tcb200_plan {
  Plan impl;
  // Scratch of a plan that needs some (impl.scratch_*): allocated and zeroed at the first launch,
  // freed with the plan.  Launches of one such plan share it, so they must not overlap in time.
  std::mutex scratch_mu;
  std::atomic<void*> scratch{nullptr};
  // tensor-core contraction plans: tensor maps of the last few sets of base pointers
  void* map_cache = nullptr;
  // a contraction that also reduces over its batch index: `impl` is the batched contraction into planes of
  // partial sums, `outer` the problem as the caller stated it (its epilogue runs in the second pass)
  bool batch_reduce = false;
  tcb200_problem_t outer;
};

namespace tcb200 {
const Plan* plan_of(const tcb200_plan_t* handle) { return handle ? &handle->impl : nullptr; }
}  // namespace tcb200

struct tcb200_timer {
  cudaEvent_t start = nullptr, stop = nullptr;
};

struct tcb200_replay {
  cudaStream_t stream = nullptr;
  bool capturing = false;
};

extern "C" {

int tcb200_abi_version(void) { return TCB200_ABI_VERSION; }

const char* tcb200_strerror(int status) {
  switch (status) {
    case TCB200_OK: return "success";
    case TCB200_ERR_INVALID_ARGUMENT: return "invalid argument";
    case TCB200_ERR_UNSUPPORTED: return "no kernel of this library covers the requested problem/tile";
    case TCB200_ERR_CUDA: return "a CUDA call failed (see tcb200_last_cuda_error)";
    case TCB200_ERR_ALIGNMENT: return "pointer or leading dimension violates the kernel's alignment rule";
    case TCB200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case TCB200_ERR_NO_DEVICE: return "no usable CUDA device";
    case TCB200_ERR_TOO_LARGE: return "problem exceeds the kernel's size limits";
    default: return "unknown tcb200 status";
  }
}

int tcb200_last_cuda_error(void) { return (int)g_last_cuda_error; }

int tcb200_device_count(int* count) {
  if (!count) return TCB200_ERR_INVALID_ARGUMENT;
  int c = 0;
  cudaError_t e = cudaGetDeviceCount(&c);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    *count = 0;
    return TCB200_ERR_NO_DEVICE;
  }
  *count = c;
  return TCB200_OK;
}

int tcb200_query(const tcb200_problem_t* problem, tcb200_tile_t* out, int max, int* n) {
  if (!problem || !n || max < 0 || (max > 0 && !out)) return TCB200_ERR_INVALID_ARGUMENT;
  *n = 0;
  switch (problem->family) {
    case TCB200_FAMILY_TENSORDOT:
      return tensordot_query(*problem, out, max, n);
    case TCB200_FAMILY_GROUP_CONV:
      return group_conv_query(*problem, out, max, n);
    case TCB200_FAMILY_REDUCTION:
      return reduce_query(*problem, out, max, n);
    case TCB200_FAMILY_COPY:
      if (max > 0 && out) out[0] = tcb200_tile_t{TCB200_VARIANT_SIMT, 0, 0, 0, 0, 0, 0, 0};
      *n = 1;
      return problem->red[0] > 0 ? TCB200_OK : TCB200_ERR_INVALID_ARGUMENT;
    case TCB200_FAMILY_CONTRACTION: {
      if (problem->batch_reduce && problem->batch > 1) {  // the candidates of the batched contraction into planes
        tcb200_problem_t inner = *problem;
        inner.batch_reduce = 0;
        inner.epilogue = TCB200_EPI_NONE;
        inner.accumulate = 0;
        inner.ldc = inner.N;
        inner.stride_c = inner.M * inner.N;
        return tcb200_query(&inner, out, max, n);
      }
      // The first candidate is the family default: the tensor-core tiles when the contraction is
      // large enough to prefer them, else the SIMT ones.
      int n_first = 0, n_second = 0;
      const bool tc_first = contraction_tc_preferred(*problem);
      auto list = [&](bool tc, tcb200_tile_t* o, int room, int* cnt) {
        return tc ? contraction_tc_query(*problem, o, room, cnt) : contraction_simt_query(*problem, o, room, cnt);
      };
      int st = list(tc_first, out, max, &n_first);
      if (st != TCB200_OK) return st;
      const int used = n_first < max ? n_first : max;
      st = list(!tc_first, out ? out + used : nullptr, max - used, &n_second);
      if (st != TCB200_OK) return st;
      *n = n_first + n_second;
      return TCB200_OK;
    }
    default:
      return TCB200_ERR_INVALID_ARGUMENT;
  }
}

int tcb200_plan_create(const tcb200_problem_t* problem, const tcb200_tile_t* tile, int device,
                       tcb200_plan_t** plan) {
  if (!problem || !plan || device < 0) return TCB200_ERR_INVALID_ARGUMENT;
  *plan = nullptr;
  tcb200_plan_t* pl = new (std::nothrow) tcb200_plan_t();
  if (!pl) return TCB200_ERR_INVALID_ARGUMENT;
  Plan& P = pl->impl;
  P.p = *problem;
  if (tile) P.tile = *tile; else memset(&P.tile, 0, sizeof(P.tile));
  P.device = device;
  P.sms = sm_count(device);
  P.kernel_id = 0;
  pl->outer = *problem;
  if (problem->family == TCB200_FAMILY_CONTRACTION && problem->batch_reduce && problem->batch > 1) {
    if (problem->M <= 0 || problem->N <= 0 || (double)problem->batch * problem->M * problem->N > 1e9) {
      delete pl;
      return TCB200_ERR_TOO_LARGE;
    }
    pl->batch_reduce = true;
    P.p.batch_reduce = 0;
    P.p.epilogue = TCB200_EPI_NONE;
    P.p.accumulate = 0;
    P.p.ldc = P.p.N;
    P.p.stride_c = P.p.M * P.p.N;
  }
  problem = &P.p;
  int st = TCB200_ERR_INVALID_ARGUMENT;
  switch (problem->family) {
    case TCB200_FAMILY_COPY:
      st = problem->red[0] > 0 ? TCB200_OK : TCB200_ERR_INVALID_ARGUMENT;
      P.tile.variant = TCB200_VARIANT_SIMT;
      break;
    case TCB200_FAMILY_TENSORDOT:
      st = tensordot_plan(P);
      break;
    case TCB200_FAMILY_GROUP_CONV:
      st = group_conv_plan(P);
      break;
    case TCB200_FAMILY_REDUCTION:
      st = reduce_plan(P);
      break;
    case TCB200_FAMILY_CONTRACTION:
      if (P.tile.variant == TCB200_VARIANT_AUTO) {
        // Family default = first candidate of the sweep.
        tcb200_tile_t first;
        int n = 0;
        st = tcb200_query(problem, &first, 1, &n);
        if (st != TCB200_OK) break;
        if (n == 0) { st = TCB200_ERR_UNSUPPORTED; break; }
        P.tile = first;
      }
      if (P.tile.variant == TCB200_VARIANT_TCGEN05 || P.tile.variant == TCB200_VARIANT_TCGEN05_TS ||
          P.tile.variant == TCB200_VARIANT_TCGEN05_PAIR) {
        st = contraction_tc_plan(P);
        if (st == TCB200_OK) pl->map_cache = tc_map_cache_new();
      } else {
        st = contraction_simt_plan(P);
      }
      break;
    default:
      break;
  }
  if (st != TCB200_OK) {
    if (pl->map_cache) tc_map_cache_delete(pl->map_cache);
    delete pl;
    return st;
  }
  if (pl->batch_reduce) {
    if (P.scratch_floats != 0) {  // (a split-K tile never applies to a batched problem; keep the two scratch uses apart)
      if (pl->map_cache) tc_map_cache_delete(pl->map_cache);
      delete pl;
      return TCB200_ERR_UNSUPPORTED;
    }
    P.scratch_floats = (size_t)P.p.batch * (size_t)P.p.M * (size_t)P.p.N;
  }
  *plan = pl;
  return TCB200_OK;
}

int tcb200_plan_destroy(tcb200_plan_t* plan) {
  if (plan) {
    if (void* s = plan->scratch.load()) cudaFree(s);
    if (plan->map_cache) tc_map_cache_delete(plan->map_cache);
    delete plan;
  }
  return TCB200_OK;
}

namespace {
// Device scratch of the plan: tickets first (zeroed), then the partial sums.  The allocation is a
// synchronous host call: the first launch of such a plan must not be inside a stream capture.  The tickets
// are zeroed on the launch stream `s`, so the kernel that follows on `s` is ordered behind the zeroing
// whatever kind of stream `s` is (a memset on the legacy default stream would not be ordered against a
// non-blocking stream).
int plan_scratch(const tcb200_plan_t* cplan, float** partial, unsigned** tickets, cudaStream_t s) {
  *partial = nullptr;
  *tickets = nullptr;
  const Plan& P = cplan->impl;
  if (P.scratch_floats == 0 && P.scratch_tickets == 0) return TCB200_OK;
  tcb200_plan_t* plan = const_cast<tcb200_plan_t*>(cplan);
  const size_t ticket_bytes = (P.scratch_tickets * sizeof(unsigned) + 255) / 256 * 256;
  void* base = plan->scratch.load(std::memory_order_acquire);
  if (!base) {
    std::lock_guard<std::mutex> lock(plan->scratch_mu);
    base = plan->scratch.load(std::memory_order_relaxed);
    if (!base) {
      TCB200_CUDA_TRY(cudaMalloc(&base, ticket_bytes + P.scratch_floats * sizeof(float)));
      cudaError_t e = ticket_bytes ? cudaMemsetAsync(base, 0, ticket_bytes, s) : cudaSuccess;
      if (e != cudaSuccess) {
        cudaFree(base);
        set_last_cuda_error(e);
        return TCB200_ERR_CUDA;
      }
      plan->scratch.store(base, std::memory_order_release);
    }
  }
  *tickets = static_cast<unsigned*>(base);
  *partial = reinterpret_cast<float*>(static_cast<char*>(base) + ticket_bytes);
  return TCB200_OK;
}
}  // namespace

int tcb200_plan_geometry(const tcb200_plan_t* plan, int64_t grid[3], int64_t block[3]) {
  if (!plan || !grid || !block) return TCB200_ERR_INVALID_ARGUMENT;
  const Launch& l = plan->impl.launch;
  grid[0] = l.grid.x; grid[1] = l.grid.y; grid[2] = l.grid.z;
  block[0] = l.block.x; block[1] = l.block.y; block[2] = l.block.z;
  return TCB200_OK;
}

int tcb200_plan_tile(const tcb200_plan_t* plan, tcb200_tile_t* tile) {
  if (!plan || !tile) return TCB200_ERR_INVALID_ARGUMENT;
  *tile = plan->impl.tile;
  return TCB200_OK;
}

int tcb200_plan_describe(const tcb200_plan_t* plan, char* buf, size_t buflen) {
  if (!plan || !buf || buflen == 0) return TCB200_ERR_INVALID_ARGUMENT;
  const Plan& P = plan->impl;
  const tcb200_problem_t& p = P.p;
  const tcb200_tile_t& t = P.tile;
  const Launch& l = P.launch;
  char head[256];
  switch (p.family) {
    case TCB200_FAMILY_TENSORDOT:
      snprintf(head, sizeof(head), "tcb200::tensordot N=%lld C1=%lld C2=%lld C3=%lld P=%lld",
               (long long)p.td[0], (long long)p.td[1], (long long)p.td[2], (long long)p.td[3],
               (long long)p.td[4]);
      break;
    case TCB200_FAMILY_REDUCTION:
      snprintf(head, sizeof(head), "tcb200::reduction %s A=%lld C=%lld B=%lld%s",
               p.reduce_op == TCB200_REDUCE_MAX ? "max" : p.reduce_op == TCB200_REDUCE_MIN ? "min"
               : p.reduce_op == TCB200_REDUCE_PROD ? "prod" : "sum",
               (long long)p.red[0], (long long)p.red[1], (long long)p.red[2], p.accumulate ? " accumulate" : "");
      break;
    case TCB200_FAMILY_COPY:
      snprintf(head, sizeof(head), "tcb200::copy elements=%lld", (long long)p.red[0]);
      break;
    case TCB200_FAMILY_GROUP_CONV:
      snprintf(head, sizeof(head),
               "tcb200::group_conv N=%lld G=%lld C=%lld F=%lld H=%lld W=%lld KH=%lld KW=%lld epilogue=%s",
               (long long)p.conv[0], (long long)p.conv[1], (long long)p.conv[2],
               (long long)p.conv[3], (long long)p.conv[4], (long long)p.conv[5],
               (long long)p.conv[6], (long long)p.conv[7], epilogue_name(p.epilogue));
      if (conv_sh(p) != 1 || conv_sw(p) != 1) {
        const size_t used = strlen(head);
        snprintf(head + used, sizeof(head) - used, " stride=%lldx%lld", (long long)conv_sh(p), (long long)conv_sw(p));
      }
      break;
    default:
      snprintf(head, sizeof(head),
               "tcb200::contraction batch=%lld%s M=%lld N=%lld K=%lld A=%s B=%s epilogue=%s%s",
               (long long)p.batch, plan->batch_reduce ? " (reduced)" : "", (long long)p.M, (long long)p.N, (long long)p.K,
               p.a_k_major ? "k-major" : "m-major", p.b_k_major ? "k-major" : "n-major",
               epilogue_name(plan->outer.epilogue), plan->outer.accumulate ? " accumulate" : "");
      break;
  }
  char split[32] = "";
  if (t.split_k > 100) snprintf(split, sizeof(split), " tail_split=%d", t.split_k - 100);
  else if (t.split_k > 1) snprintf(split, sizeof(split), " split_k=%d", t.split_k);
  snprintf(buf, buflen,
           "%s | variant=%s tile=%dx%dx%d stages=%d threads=%d split_tf32=%d%s | grid=(%u,%u,%u) "
           "block=(%u,%u,%u) smem=%zu",
           head, variant_name(t.variant), t.bm, t.bn, t.bk, t.stages, t.threads, t.split_tf32, split,
           l.grid.x, l.grid.y, l.grid.z, l.block.x, l.block.y, l.block.z, l.smem);
  return TCB200_OK;
}

int tcb200_launch(const tcb200_plan_t* plan, const void* const* inputs, int n_inputs,
                  void* const* outputs, int n_outputs, tcb200_stream_t stream, int* dev_status) {
  if (!plan || !inputs || !outputs) return TCB200_ERR_INVALID_ARGUMENT;
  const Plan& P = plan->impl;
  if (n_inputs != n_inputs_expected(plan->outer) || n_outputs != 1) return TCB200_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < n_inputs; ++i)
    if (!inputs[i]) return TCB200_ERR_INVALID_ARGUMENT;
  if (!outputs[0]) return TCB200_ERR_INVALID_ARGUMENT;
  int cur = -1;
  TCB200_CUDA_TRY(cudaGetDevice(&cur));
  if (cur != P.device) return TCB200_ERR_INVALID_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const float* in0 = static_cast<const float*>(inputs[0]);
  const float* in1 = n_inputs > 1 ? static_cast<const float*>(inputs[1]) : nullptr;
  const float* bias = n_inputs > 2 ? static_cast<const float*>(inputs[2]) : nullptr;
  float* out = static_cast<float*>(outputs[0]);
  if (plan->batch_reduce) {
    // batched contraction into one plane per batch entry, then the planes are added in order
    float* planes;
    unsigned* tickets;
    int st = plan_scratch(plan, &planes, &tickets, s);
    if (st != TCB200_OK) return st;
    if (P.tile.variant == TCB200_VARIANT_TCGEN05 || P.tile.variant == TCB200_VARIANT_TCGEN05_TS ||
        P.tile.variant == TCB200_VARIANT_TCGEN05_PAIR)
      st = contraction_tc_launch(P, in0, in1, nullptr, planes, s, dev_status, nullptr, plan->map_cache);
    else
      st = contraction_simt_launch(P, in0, in1, nullptr, planes, s);
    if (st != TCB200_OK) return st;
    const tcb200_problem_t& o = plan->outer;
    return partial_planes_reduce(planes, out, bias, (int)o.M, (int)o.N, (int)o.batch, o.ldc, o.epilogue, o.bias_on_m,
                                 o.accumulate, P.sms, s);
  }
  switch (P.p.family) {
    case TCB200_FAMILY_COPY:
      TCB200_CUDA_TRY(cudaMemcpyAsync(out, in0, (size_t)P.p.red[0] * sizeof(float), cudaMemcpyDeviceToDevice, s));
      return TCB200_OK;
    case TCB200_FAMILY_TENSORDOT:
      return tensordot_launch(P, in0, in1, out, s, dev_status);
    case TCB200_FAMILY_GROUP_CONV:
      return group_conv_launch(P, in0, in1, bias, out, s, dev_status);
    case TCB200_FAMILY_REDUCTION: {
      float* partial;
      unsigned* tickets;
      const int st = plan_scratch(plan, &partial, &tickets, s);
      if (st != TCB200_OK) return st;
      return reduce_launch(P, in0, out, partial, tickets, s);
    }
    case TCB200_FAMILY_CONTRACTION:
      if (P.tile.variant == TCB200_VARIANT_TCGEN05 || P.tile.variant == TCB200_VARIANT_TCGEN05_TS ||
          P.tile.variant == TCB200_VARIANT_TCGEN05_PAIR) {
        float* partial;
        unsigned* tickets;
        const int st = plan_scratch(plan, &partial, &tickets, s);
        if (st != TCB200_OK) return st;
        return contraction_tc_launch(P, in0, in1, bias, out, s, dev_status, partial, plan->map_cache);
      }
      return contraction_simt_launch(P, in0, in1, bias, out, s);
    default:
      return TCB200_ERR_INVALID_ARGUMENT;
  }
}

int tcb200_get_device(int* device) {
  if (!device) return TCB200_ERR_INVALID_ARGUMENT;
  TCB200_CUDA_TRY(cudaGetDevice(device));
  return TCB200_OK;
}

int tcb200_set_device(int device) {
  TCB200_CUDA_TRY(cudaSetDevice(device));
  return TCB200_OK;
}

int tcb200_device_name(int device, char* buf, size_t buflen) {
  if (!buf || buflen == 0) return TCB200_ERR_INVALID_ARGUMENT;
  cudaDeviceProp prop;
  TCB200_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  snprintf(buf, buflen, "%s", prop.name);
  return TCB200_OK;
}

int tcb200_stream_synchronize(tcb200_stream_t stream) {
  TCB200_CUDA_TRY(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  return TCB200_OK;
}

int tcb200_timer_start(tcb200_stream_t stream, tcb200_timer_t** timer) {
  if (!timer) return TCB200_ERR_INVALID_ARGUMENT;
  *timer = nullptr;
  tcb200_timer_t* t = new (std::nothrow) tcb200_timer_t();
  if (!t) return TCB200_ERR_INVALID_ARGUMENT;
  cudaError_t e = cudaEventCreate(&t->start);
  if (e == cudaSuccess) e = cudaEventCreate(&t->stop);
  if (e == cudaSuccess) e = cudaEventRecord(t->start, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    if (t->start) cudaEventDestroy(t->start);
    if (t->stop) cudaEventDestroy(t->stop);
    delete t;
    return TCB200_ERR_CUDA;
  }
  *timer = t;
  return TCB200_OK;
}

int tcb200_timer_stop(tcb200_timer_t* timer, tcb200_stream_t stream, float* elapsed_us) {
  if (!timer || !elapsed_us) return TCB200_ERR_INVALID_ARGUMENT;
  float ms = 0.f;
  cudaError_t e = cudaEventRecord(timer->stop, reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = cudaEventSynchronize(timer->stop);
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, timer->start, timer->stop);
  cudaEventDestroy(timer->start);
  cudaEventDestroy(timer->stop);
  delete timer;
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    return TCB200_ERR_CUDA;
  }
  *elapsed_us = ms * 1000.f;
  return TCB200_OK;
}

int tcb200_status_create(int** dev_status) {
  if (!dev_status) return TCB200_ERR_INVALID_ARGUMENT;
  *dev_status = nullptr;
  int* p = nullptr;
  TCB200_CUDA_TRY(cudaMalloc(&p, sizeof(int)));
  cudaError_t e = cudaMemset(p, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(p);
    set_last_cuda_error(e);
    return TCB200_ERR_CUDA;
  }
  *dev_status = p;
  return TCB200_OK;
}

int tcb200_status_destroy(int* dev_status) {
  if (dev_status) cudaFree(dev_status);
  return TCB200_OK;
}

int tcb200_status_check(int* dev_status, tcb200_stream_t stream, int* code) {
  if (!dev_status) return TCB200_ERR_INVALID_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int v = 0;
  TCB200_CUDA_TRY(cudaMemcpyAsync(&v, dev_status, sizeof(int), cudaMemcpyDeviceToHost, s));
  TCB200_CUDA_TRY(cudaStreamSynchronize(s));
  if (code) *code = v;
  if (v == 0) return TCB200_OK;
  TCB200_CUDA_TRY(cudaMemsetAsync(dev_status, 0, sizeof(int), s));
  TCB200_CUDA_TRY(cudaStreamSynchronize(s));
  return TCB200_ERR_DEVICE_TIMEOUT;
}

int tcb200_selftest_wait(long long limit_cycles, int* dev_status, tcb200_stream_t stream) {
  // the limit is capped at the kernels' own, so the call cannot be used to keep an SM busy for long
  if (limit_cycles <= 0 || limit_cycles > kWaitLimitCycles) return TCB200_ERR_INVALID_ARGUMENT;
  selftest_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(limit_cycles, dev_status);
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}

int tcb200_replay_begin(tcb200_replay_t** replay, tcb200_stream_t* capture_stream) {
  if (!replay || !capture_stream) return TCB200_ERR_INVALID_ARGUMENT;
  *replay = nullptr;
  *capture_stream = nullptr;
  tcb200_replay_t* r = new (std::nothrow) tcb200_replay_t();
  if (!r) return TCB200_ERR_INVALID_ARGUMENT;
  cudaError_t e = cudaStreamCreateWithFlags(&r->stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamBeginCapture(r->stream, cudaStreamCaptureModeThreadLocal);
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    if (r->stream) cudaStreamDestroy(r->stream);
    delete r;
    return TCB200_ERR_CUDA;
  }
  r->capturing = true;
  *replay = r;
  *capture_stream = reinterpret_cast<tcb200_stream_t>(r->stream);
  return TCB200_OK;
}

int tcb200_replay_end(tcb200_replay_t* r, int timed_replays, float* elapsed_us_per_replay) {
  if (!r) return TCB200_ERR_INVALID_ARGUMENT;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaError_t e = cudaStreamEndCapture(r->stream, &graph);  // always: leaves the stream out of capture mode
  r->capturing = false;
  if (e == cudaSuccess && (!elapsed_us_per_replay || timed_replays <= 0)) e = cudaErrorInvalidValue;
  if (e == cudaSuccess) e = cudaGraphInstantiate(&exec, graph, 0);
  if (e == cudaSuccess) e = cudaEventCreate(&e0);
  if (e == cudaSuccess) e = cudaEventCreate(&e1);
  if (e == cudaSuccess) e = cudaGraphLaunch(exec, r->stream);  // untimed: uploads the graph, warms the caches
  if (e == cudaSuccess) e = cudaEventRecord(e0, r->stream);
  for (int i = 0; e == cudaSuccess && i < timed_replays; ++i) e = cudaGraphLaunch(exec, r->stream);
  if (e == cudaSuccess) e = cudaEventRecord(e1, r->stream);
  if (e == cudaSuccess) e = cudaEventSynchronize(e1);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (exec) cudaGraphExecDestroy(exec);
  if (graph) cudaGraphDestroy(graph);
  cudaStreamDestroy(r->stream);
  delete r;
  if (e != cudaSuccess) {
    set_last_cuda_error(e);
    (void)cudaGetLastError();
    return TCB200_ERR_CUDA;
  }
  *elapsed_us_per_replay = ms * 1000.f / (float)timed_replays;
  return TCB200_OK;
}

int tcb200_l2_flush(void* buf, size_t bytes, tcb200_stream_t stream) {
  if (!buf || bytes < 16 || ((uintptr_t)buf & 15)) return TCB200_ERR_INVALID_ARGUMENT;
  static unsigned counter = 0;
  const float v = (float)(++counter & 1023);
  l2_flush_kernel<<<sm_count(-1) * 4, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<float4*>(buf), bytes / 16, v);
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}

}  // extern "C"
