// K4 — reductions (sum, max, min, product) of one tensor over a contiguous group of its indices:
//   O(a, b) (op)= reduce_c I(a, c, b)        I viewed as [A][C][B], O as [A][B]
// with A / B the products of the kept leading / trailing dimensions (either may be 1).  These are the
// comprehensions the reference's mapper tests exercise as sum1D / sum2D
// (test/test_tc_mapper_harness-inl.h:60-146: C +=! A(r_m), C(m) +=! A(m, r_n)) and the building
// blocks of its moment / normalisation examples; they replace the kernels it generates for them,
// including the CUB block reductions those call (tc/core/cuda/cuda_libraries.h:128-282).
//
// All of it is HBM streaming (4 * (A*C*B + A*B) bytes, one add per element).  Two kernels:
//  * tile kernel (any shape): a CTA of 256 threads owns CP output columns (a power of two, one warp
//    wide by default: narrow tiles give many CTAs and few segments) of one row a and one of S
//    interleaved shares ("segments") of the reduced range; thread (tx, ty) of the CP x (256 / CP)
//    layout adds elements ty, ty + TY, ... of column tx, so a warp reads consecutive addresses
//    whatever B is (B = 1: consecutive c; B >= 32: consecutive columns).  The TY partial sums of a
//    column are combined through shared memory in a fixed order.
//    When the output alone gives too few CTAs to fill 148 SMs, S > 1 (grid.y): each CTA leaves its
//    partial sums in scratch memory, takes a ticket, and the CTA that draws the last ticket of a tile
//    adds the S partials in a fixed order and writes the output.  Same bits on every run, one launch,
//    no atomics on data.
//  * warp-rows kernel (B = 1, short rows): one warp per row, 128-bit loads when the rows allow.
#include <atomic>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace tcb200 {
namespace {

constexpr int kThreads = 256;

struct ReduceArgs {
  const float* I;
  float* O;
  long long A, C, B;  // in elements of the kernel's value type (see reduce_tile_kernel)
  long long tiles_b;  // column tiles per row a
  int S;              // segments
  int cp_log2;        // log2 of the columns per CTA
  int accumulate;
  float* partial;     // [tile][S][CP] output values
  unsigned* tickets;  // [tile], zero between launches
};

// The reduction operator (TCB200_REDUCE_*) and its identity (tc/core/tc2halide.cc:573-601: 0 for +=,
// 1 for *=, the type's lowest / largest value for max= / min=).
template <int OP>
__device__ __forceinline__ float rop(float a, float b) {
  if (OP == TCB200_REDUCE_MAX) return fmaxf(a, b);
  if (OP == TCB200_REDUCE_MIN) return fminf(a, b);
  if (OP == TCB200_REDUCE_PROD) return a * b;
  return a + b;
}
template <int OP>
__device__ __forceinline__ float4 rop(float4 a, float4 b) {
  return make_float4(rop<OP>(a.x, b.x), rop<OP>(a.y, b.y), rop<OP>(a.z, b.z), rop<OP>(a.w, b.w));
}
template <int OP>
__device__ __forceinline__ float identity() {
  return OP == TCB200_REDUCE_MAX ? -3.402823466e38f : OP == TCB200_REDUCE_MIN ? 3.402823466e38f
       : OP == TCB200_REDUCE_PROD ? 1.f : 0.f;
}
template <int OP> __device__ __forceinline__ void vinit(float& a) { a = identity<OP>(); }
template <int OP> __device__ __forceinline__ void vinit(float4& a) {
  const float i = identity<OP>();
  a = make_float4(i, i, i, i);
}
template <int OP> __device__ __forceinline__ float hred(float4 a) { return rop<OP>(rop<OP>(a.x, a.y), rop<OP>(a.z, a.w)); }

// T = float: the plain form.  T = float4, HSUM = false: four adjacent output columns per thread
// (B a multiple of 4; A.B counts float4 columns).  T = float4, HSUM = true: B = 1 and the reduced range
// itself is read four elements at a time (C a multiple of 4; A.C counts float4 elements), the four
// lanes of a thread's sum are added at the end.  16 to 64 bytes of loads per thread are in flight.
template <typename T, bool HSUM, int OP>
__global__ void __launch_bounds__(kThreads) reduce_tile_kernel(ReduceArgs a) {
  using OutT = typename std::conditional<HSUM, float, T>::type;
  constexpr int UNROLL = sizeof(T) == 4 ? 8 : 4;
  __shared__ T red[kThreads];
  __shared__ int is_last;
  const int CP = 1 << a.cp_log2, TY = kThreads >> a.cp_log2;
  const int tid = threadIdx.x, tx = tid & (CP - 1), ty = tid >> a.cp_log2;
  const long long tile = blockIdx.x;
  const int s = blockIdx.y;
  const long long arow = tile / a.tiles_b, ct = tile - arow * a.tiles_b;
  const long long col = ct * CP + tx;
  // Segment s takes the blocks s, s + S, s + 2S, ... of UNROLL * TY reduced elements: interleaved, so
  // that all segments of a tile end within one block of each other whatever the number of CTAs per SM.
  const long long BLK = (long long)UNROLL * TY;
  T acc[UNROLL];
#pragma unroll
  for (int k = 0; k < UNROLL; ++k) vinit<OP>(acc[k]);
  if (col < a.B) {
    const T* base = reinterpret_cast<const T*>(a.I) + (size_t)arow * a.C * a.B + col;
    for (long long b0 = (long long)s * BLK; b0 < a.C; b0 += (long long)a.S * BLK) {
      const long long c = b0 + ty;
      if (b0 + BLK <= a.C) {
        T v[UNROLL];
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) v[k] = __ldg(base + (size_t)(c + (long long)k * TY) * a.B);
#pragma unroll
        for (int k = 0; k < UNROLL; ++k) acc[k] = rop<OP>(acc[k], v[k]);
      } else {  // the last, ragged block of the range
#pragma unroll
        for (int k = 0; k < UNROLL; ++k)
          if (c + (long long)k * TY < a.C) acc[k] = rop<OP>(acc[k], __ldg(base + (size_t)(c + (long long)k * TY) * a.B));
      }
    }
  }
#pragma unroll
  for (int h = UNROLL / 2; h > 0; h >>= 1)
#pragma unroll
    for (int k = 0; k < h; ++k) acc[k] = rop<OP>(acc[k], acc[k + h]);
  red[tid] = acc[0];
  __syncthreads();
  // rows of the CP x TY layout are ty-major: element (ty, tx) sits at ty * CP + tx = tid
  for (int h = TY >> 1; h > 0; h >>= 1) {
    if (ty < h) red[tid] = rop<OP>(red[tid], red[tid + h * CP]);
    __syncthreads();
  }
  const bool writer = ty == 0 && col < a.B;
  OutT mine_v;
  if constexpr (HSUM) mine_v = hred<OP>(red[tid]); else mine_v = red[tid];
  OutT* out = reinterpret_cast<OutT*>(a.O) + (size_t)arow * a.B + col;
  if (a.S == 1) {
    if (writer) *out = a.accumulate ? rop<OP>(*out, mine_v) : mine_v;
    return;
  }
  OutT* part = reinterpret_cast<OutT*>(a.partial) + (size_t)tile * a.S * CP;
  if (ty == 0) part[(size_t)s * CP + tx] = mine_v;
  __threadfence();  // the partial sums are visible device-wide before the ticket is drawn
  __syncthreads();
  if (tid == 0) is_last = atomicAdd(a.tickets + tile, 1u) == (unsigned)(a.S - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // The S partial sums of every column, added by the same thread layout in the same fixed order:
  // thread (tx, ty) takes segments ty, ty + TY, ..., then the TY rows are combined as above.
  OutT* redo = reinterpret_cast<OutT*>(red);
  OutT sum;
  vinit<OP>(sum);
  for (int k = ty; k < a.S; k += TY) sum = rop<OP>(sum, __ldcg(part + (size_t)k * CP + tx));  // L2: written by other SMs
  redo[tid] = sum;
  __syncthreads();
  for (int h = TY >> 1; h > 0; h >>= 1) {
    if (ty < h) redo[tid] = rop<OP>(redo[tid], redo[tid + h * CP]);
    __syncthreads();
  }
  if (writer) *out = a.accumulate ? rop<OP>(*out, redo[tid]) : redo[tid];
  if (tid == 0) a.tickets[tile] = 0;  // the next launch on this scratch starts from zero again
}

// B = 1: O(a) = sum_c I(a, c), one warp per row.
template <bool VEC, int OP>
__global__ void __launch_bounds__(kThreads) reduce_rows_warp_kernel(ReduceArgs a) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int WARPS = kThreads / 32;
  for (long long r = (long long)blockIdx.x * WARPS + warp; r < a.A; r += (long long)gridDim.x * WARPS) {
    const float* row = a.I + (size_t)r * a.C;
    float s0 = identity<OP>(), s1 = identity<OP>();
    if (VEC) {
      const float4* row4 = reinterpret_cast<const float4*>(row);
      const long long n4 = a.C >> 2;
      long long i = lane;
      for (; i + 32 < n4; i += 64) {
        const float4 u = __ldg(row4 + i), v = __ldg(row4 + i + 32);
        s0 = rop<OP>(s0, hred<OP>(u));
        s1 = rop<OP>(s1, hred<OP>(v));
      }
      if (i < n4) {
        const float4 u = __ldg(row4 + i);
        s0 = rop<OP>(s0, hred<OP>(u));
      }
    } else {
      long long i = lane;
      for (; i + 32 < a.C; i += 64) {
        s0 = rop<OP>(s0, __ldg(row + i));
        s1 = rop<OP>(s1, __ldg(row + i + 32));
      }
      if (i < a.C) s0 = rop<OP>(s0, __ldg(row + i));
    }
    float s = rop<OP>(s0, s1);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s = rop<OP>(s, __shfl_xor_sync(0xffffffffu, s, off));
    if (lane == 0) a.O[r] = a.accumulate ? rop<OP>(a.O[r], s) : s;
  }
}

bool valid(const tcb200_problem_t& p) {
  for (int i = 0; i < 3; ++i)
    if (p.red[i] <= 0 || p.red[i] > (1ll << 40)) return false;
  if (p.reduce_op < TCB200_REDUCE_SUM || p.reduce_op > TCB200_REDUCE_PROD) return false;
  return (double)p.red[0] * (double)p.red[1] * (double)p.red[2] < 9.0e18;
}

int pow2_ceil_log2(long long v, int cap_log2) {
  int l = 0;
  while (l < cap_log2 && (1ll << l) < v) ++l;
  return l;
}

// The problem in units of the tile kernel's value type.  vec = 4: float4 loads, along the reduced range
// when B = 1 (C a multiple of 4), else along the columns (B a multiple of 4); vec = 1: plain floats.
struct Units { long long A, C, B; bool hsum; };
bool vec_ok(const tcb200_problem_t& p) { return p.red[2] == 1 ? p.red[1] % 4 == 0 : p.red[2] % 4 == 0; }
Units units(const tcb200_problem_t& p, int vec) {
  if (vec != 4) return Units{p.red[0], p.red[1], p.red[2], false};
  if (p.red[2] == 1) return Units{p.red[0], p.red[1] / 4, 1, true};
  return Units{p.red[0], p.red[1], p.red[2] / 4, false};
}

// Segments of the tile kernel: enough CTAs for eight per SM, at least 32 reduced elements per thread row.
int auto_segments(const Units& u, int cp_log2, int sms) {
  const long long CP = 1ll << cp_log2, TY = kThreads / CP;
  const long long tiles = u.A * ceil_div(u.B, CP);
  const long long want = ceil_div(8 * sms, tiles);
  const long long most = std::max<long long>(1, u.C / (32 * TY));
  return (int)std::max<long long>(1, std::min<long long>({want, most, (long long)kReduceMaxSegments}));
}

bool warp_rows_ok(const tcb200_problem_t& p) { return p.red[2] == 1 && p.red[1] <= (1 << 20); }

template <int OP>
int launch_tile_op(bool vec, bool hsum, const Plan& plan, const ReduceArgs& a, cudaStream_t s) {
  if (vec && hsum) reduce_tile_kernel<float4, true, OP><<<plan.launch.grid, plan.launch.block, 0, s>>>(a);
  else if (vec) reduce_tile_kernel<float4, false, OP><<<plan.launch.grid, plan.launch.block, 0, s>>>(a);
  else reduce_tile_kernel<float, false, OP><<<plan.launch.grid, plan.launch.block, 0, s>>>(a);
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}
int launch_tile(int op, bool vec, bool hsum, const Plan& plan, const ReduceArgs& a, cudaStream_t s) {
  switch (op) {
    case TCB200_REDUCE_MAX: return launch_tile_op<TCB200_REDUCE_MAX>(vec, hsum, plan, a, s);
    case TCB200_REDUCE_MIN: return launch_tile_op<TCB200_REDUCE_MIN>(vec, hsum, plan, a, s);
    case TCB200_REDUCE_PROD: return launch_tile_op<TCB200_REDUCE_PROD>(vec, hsum, plan, a, s);
    default: return launch_tile_op<TCB200_REDUCE_SUM>(vec, hsum, plan, a, s);
  }
}
template <int OP>
int launch_rows_op(bool vec, const Plan& plan, const ReduceArgs& a, cudaStream_t s) {
  if (vec) reduce_rows_warp_kernel<true, OP><<<plan.launch.grid, plan.launch.block, 0, s>>>(a);
  else reduce_rows_warp_kernel<false, OP><<<plan.launch.grid, plan.launch.block, 0, s>>>(a);
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}
int launch_rows(int op, bool vec, const Plan& plan, const ReduceArgs& a, cudaStream_t s) {
  switch (op) {
    case TCB200_REDUCE_MAX: return launch_rows_op<TCB200_REDUCE_MAX>(vec, plan, a, s);
    case TCB200_REDUCE_MIN: return launch_rows_op<TCB200_REDUCE_MIN>(vec, plan, a, s);
    case TCB200_REDUCE_PROD: return launch_rows_op<TCB200_REDUCE_PROD>(vec, plan, a, s);
    default: return launch_rows_op<TCB200_REDUCE_SUM>(vec, plan, a, s);
  }
}

}  // namespace

int reduce_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n) {
  if (!valid(p)) return TCB200_ERR_INVALID_ARGUMENT;
  int cnt = 0;
  auto add = [&](int cp, int s, int mode, int vec) {
    if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_SIMT, cp, s, mode, vec, kThreads, 0};
    ++cnt;
  };
  const int vec = vec_ok(p) ? 4 : 1;
  const int cp = 1 << pow2_ceil_log2(units(p, vec).B, 5);
  // short rows, many of them: a warp per row first; else the tile kernel
  const bool warp_first = warp_rows_ok(p) && p.red[1] <= 4096 && p.red[0] >= 2 * sm_count(-1);
  if (warp_first) add(1, 1, 1, 0);
  add(cp, 0, 0, vec);
  if (warp_rows_ok(p) && !warp_first) add(1, 1, 1, 0);
  if (units(p, vec).B > 64) add(64, 0, 0, vec);  // two warps wide: half the tiles, longer row pieces
  if (vec == 4) add(1 << pow2_ceil_log2(p.red[2], 5), 0, 0, 1);  // plain floats: no alignment rule
  *n = cnt;
  return TCB200_OK;
}

// tile: bm = columns per CTA in units of the value type (power of two), bn = segments (0 = chosen here),
// bk = 1 for the warp-rows kernel, stages = 4 for 128-bit loads (pointers must then be 16-byte aligned)
int reduce_plan(Plan& plan) {
  const tcb200_problem_t& p = plan.p;
  if (!valid(p)) return TCB200_ERR_INVALID_ARGUMENT;
  if (p.epilogue != TCB200_EPI_NONE) return TCB200_ERR_UNSUPPORTED;
  tcb200_tile_t& t = plan.tile;
  if (t.variant == TCB200_VARIANT_AUTO) {
    tcb200_tile_t first;
    int n = 0;
    reduce_query(p, &first, 1, &n);
    t = first;
  }
  if (t.variant != TCB200_VARIANT_SIMT) return TCB200_ERR_UNSUPPORTED;
  t.threads = kThreads;
  t.split_tf32 = 0;
  plan.scratch_floats = 0;
  plan.scratch_tickets = 0;
  if (t.bk == 1) {
    if (!warp_rows_ok(p)) return TCB200_ERR_UNSUPPORTED;
    t.bm = 1; t.bn = 1; t.stages = 0;
    plan.launch.grid = dim3((unsigned)std::min<long long>(ceil_div(p.red[0], kThreads / 32), 8 * plan.sms), 1, 1);
    plan.launch.block = dim3(kThreads, 1, 1);
    plan.kernel_id = 2;
    return TCB200_OK;
  }
  if (t.bk != 0) return TCB200_ERR_INVALID_ARGUMENT;
  if (t.stages == 0) t.stages = vec_ok(p) ? 4 : 1;
  if (t.stages != 1 && !(t.stages == 4 && vec_ok(p))) return TCB200_ERR_UNSUPPORTED;
  const Units u = units(p, t.stages);
  int cp_log2 = 0;
  if (t.bm <= 0) cp_log2 = pow2_ceil_log2(u.B, 5);
  else {
    while ((1 << cp_log2) < t.bm) ++cp_log2;
    if ((1 << cp_log2) != t.bm || cp_log2 > 8) return TCB200_ERR_INVALID_ARGUMENT;
  }
  t.bm = 1 << cp_log2;
  const long long tiles = u.A * ceil_div(u.B, t.bm);
  if (tiles > 0x7fffffffll) return TCB200_ERR_TOO_LARGE;
  int S = t.bn > 0 ? t.bn : auto_segments(u, cp_log2, plan.sms);
  if (S > kReduceMaxSegments) return TCB200_ERR_INVALID_ARGUMENT;
  const long long unroll = t.stages == 4 ? 4 : 8, TY = kThreads >> cp_log2;
  S = (int)std::min<long long>(S, ceil_div(u.C, unroll * TY));  // no segment without a block
  t.bn = S;
  plan.launch.grid = dim3((unsigned)tiles, (unsigned)S, 1);
  plan.launch.block = dim3(kThreads, 1, 1);
  plan.kernel_id = 1;
  if (S > 1) {
    plan.scratch_floats = (size_t)tiles * S * t.bm * (u.hsum ? 1 : t.stages);
    plan.scratch_tickets = (size_t)tiles;
  }
  return TCB200_OK;
}

int reduce_launch(const Plan& plan, const float* I, float* O, float* partial, unsigned* tickets, cudaStream_t s) {
  const tcb200_problem_t& p = plan.p;
  ReduceArgs a;
  a.I = I; a.O = O;
  a.A = p.red[0]; a.C = p.red[1]; a.B = p.red[2];
  a.accumulate = p.accumulate;
  a.partial = partial; a.tickets = tickets;
  if (plan.kernel_id == 2) {
    a.S = 1; a.cp_log2 = 0; a.tiles_b = 1;
    const bool vec = (a.C & 3) == 0 && (((uintptr_t)I) & 15) == 0;
    return launch_rows(p.reduce_op, vec, plan, a, s);
  }
  const int vec = plan.tile.stages;
  const Units u = units(p, vec);
  if (vec == 4 && ((((uintptr_t)I) & 15) || (!u.hsum && (((uintptr_t)O) & 15)))) return TCB200_ERR_ALIGNMENT;
  a.A = u.A; a.C = u.C; a.B = u.B;
  a.cp_log2 = 0;
  while ((1 << a.cp_log2) < plan.tile.bm) ++a.cp_log2;
  a.tiles_b = ceil_div(a.B, plan.tile.bm);
  a.S = plan.tile.bn;
  if (a.S > 1 && (!partial || !tickets)) return TCB200_ERR_INVALID_ARGUMENT;
  return launch_tile(p.reduce_op, vec == 4, u.hsum, plan, a, s);
}

// ------------------------------------------------------------------------------------------------
// Launch with the scratch in a fixed array of the library image (no allocation, see tcb200.h)
// ------------------------------------------------------------------------------------------------
namespace {

// Tickets first (as 32-bit counters), then the partial sums.  Part of the module image: zero when the
// module is loaded; the kernel leaves every ticket it used at zero again.
constexpr size_t kStaticWords = TCB200_STATIC_SCRATCH_TICKETS + TCB200_STATIC_SCRATCH_FLOATS;
static __device__ __align__(256) float g_static_scratch[kStaticWords];

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
std::atomic<float*> g_static_ptr[kMaxDevices];  // address of the array on each device, looked up once

// Once per device: the device address of g_static_scratch.
int static_scratch(int device, float** ptr) {
  if (device < 0 || device >= kMaxDevices) return TCB200_ERR_INVALID_ARGUMENT;
  float* p = g_static_ptr[device].load(std::memory_order_acquire);
  if (!p) {
    std::lock_guard<std::mutex> lock(g_static_mu);
    p = g_static_ptr[device].load(std::memory_order_relaxed);
    if (!p) {
      TCB200_CUDA_TRY(cudaGetSymbolAddress((void**)&p, g_static_scratch));
      if (!p) return TCB200_ERR_CUDA;
      g_static_ptr[device].store(p, std::memory_order_release);
    }
  }
  *ptr = p;
  return TCB200_OK;
}

}  // namespace
}  // namespace tcb200

extern "C" int tcb200_reduce_launch_static(const tcb200_plan_t* handle, const void* input, void* output,
                                           tcb200_stream_t stream) {
  using namespace tcb200;
  const Plan* plan = plan_of(handle);
  if (!plan || !input || !output || plan->p.family != TCB200_FAMILY_REDUCTION) return TCB200_ERR_INVALID_ARGUMENT;
  if (plan->scratch_tickets > (size_t)TCB200_STATIC_SCRATCH_TICKETS ||
      plan->scratch_floats > (size_t)TCB200_STATIC_SCRATCH_FLOATS)
    return TCB200_ERR_TOO_LARGE;  // the fixed array cannot hold this plan's partial sums: nothing is launched
  int cur = -1;
  TCB200_CUDA_TRY(cudaGetDevice(&cur));
  if (cur != plan->device) return TCB200_ERR_INVALID_ARGUMENT;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  float* base = nullptr;
  unsigned* tickets = nullptr;
  float* partial = nullptr;
  if (plan->scratch_tickets > 0) {
    const int st = static_scratch(cur, &base);
    if (st != TCB200_OK) return st;
    tickets = reinterpret_cast<unsigned*>(base);
    partial = base + TCB200_STATIC_SCRATCH_TICKETS;
    // the counters must start at zero even if an earlier kernel on this array did not run to its end
    TCB200_CUDA_TRY(cudaMemsetAsync(tickets, 0, plan->scratch_tickets * sizeof(unsigned), s));
  }
  return reduce_launch(*plan, static_cast<const float*>(input), static_cast<float*>(output), partial, tickets, s);
}
