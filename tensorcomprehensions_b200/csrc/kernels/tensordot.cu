// K2 — bandwidth-bound tensordot with a tiny reduction:
//   O(n,c1,c3,p) = sum_{c2} I0(n,c1,c2,p) * I1(n,c2,c3,p)       (p = flattened h,w; innermost, contiguous)
//
// Replaces the kernel the reference generates for tc/examples/tensordot.cc:41-47
// (and its CubReduceAlongX helper, tc/core/cuda/cuda_libraries.h:227-282).
//
// At the benchmark size (N=32, C1=512, C2=8, C3=2, P=784) the arithmetic intensity
// is 0.8 flop/byte, so the only thing that matters is streaming I0 (411 MB) and O
// (103 MB) at HBM speed:
//   * p is the contiguous index of all three tensors, so a warp reads/writes
//     32 consecutive float4 (512 B) per access: fully coalesced 128-bit accesses;
//   * the reduction index c2 lives in one thread's registers (no cross-thread
//     reduction is needed when C2 is this small, so no shuffle or shared memory);
//   * I1 (1.6 MB, reused C1 = 512 times) is held in registers: each thread loads its
//     C2*C3 float4 of I1 once and sweeps `bm` rows of c1 with them;
//   * I0/O use streaming cache hints so they do not evict I1 from L1/L2.
//
// Two kernels implement this:
//   * tensordot_bulk_kernel (default): persistent CTAs; one producer thread streams I0 through a
//     ring of shared-memory stages with 1-D bulk copies (cp.async.bulk, mbarrier completion), so
//     ~200 KB per SM are in flight regardless of register pressure; 7 consumer warps read the
//     stage with conflict-free 128-bit shared loads and write O with 128-bit streaming stores.
//     The rows (n, c1) of I0 are contiguous blocks of C2*P floats, so every copy is one linear
//     transfer of a few tens of KB.
//   * tensordot_vec4_kernel: direct 128-bit global loads, one CTA per (n, chunk of c1).
#include "async.cuh"
#include "common.cuh"

namespace tcb200 {
namespace {

template <int C2, int C3>
__global__ void __launch_bounds__(256)
tensordot_vec4_kernel(const float4* __restrict__ I0, const float4* __restrict__ I1,
                      float4* __restrict__ O, int C1, int P4, int c1_per_cta) {
  const int p4 = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.z;
  if (p4 >= P4) return;

  float4 w[C2][C3];
  {
    const float4* i1 = I1 + (size_t)n * C2 * C3 * P4 + p4;
#pragma unroll
    for (int c2 = 0; c2 < C2; ++c2)
#pragma unroll
      for (int c3 = 0; c3 < C3; ++c3) w[c2][c3] = __ldg(i1 + (size_t)(c2 * C3 + c3) * P4);
  }

  const int c1_begin = blockIdx.y * c1_per_cta;
  const int c1_end = min(C1, c1_begin + c1_per_cta);
#pragma unroll 2
  for (int c1 = c1_begin + threadIdx.y; c1 < c1_end; c1 += blockDim.y) {
    const float4* x = I0 + ((size_t)n * C1 + c1) * C2 * P4 + p4;
    float4 xv[C2];
#pragma unroll
    for (int c2 = 0; c2 < C2; ++c2) xv[c2] = ldg_stream4(x + (size_t)c2 * P4);
    float4* o = O + ((size_t)n * C1 + c1) * C3 * P4 + p4;
#pragma unroll
    for (int c3 = 0; c3 < C3; ++c3) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int c2 = 0; c2 < C2; ++c2) {  // reduction in textual order, like the loop nest
        acc.x = fmaf(xv[c2].x, w[c2][c3].x, acc.x);
        acc.y = fmaf(xv[c2].y, w[c2][c3].y, acc.y);
        acc.z = fmaf(xv[c2].z, w[c2][c3].z, acc.z);
        acc.w = fmaf(xv[c2].w, w[c2][c3].w, acc.w);
      }
      stg_stream4(o + (size_t)c3 * P4, acc);
    }
  }
}

// Persistent bulk-copy variant.  Work item = `R` consecutive rows c1 of one n (a contiguous block
// of I0); items are split evenly over the CTAs.  Thread layout of the 224 consumers:
// px = float4 column of p, ry = which of the RY rows handled in parallel.
constexpr int kBulkThreads = 256;
constexpr int kBulkConsumers = 224;

struct BulkArgs {
  const float* I0;
  const float* I1;
  float* O;
  int N, C1, P4;
  int R, RY, stages;
  uint32_t stage_bytes;
  int* dev_status;
};

template <int C2, int C3>
__global__ void __launch_bounds__(kBulkThreads, 1) tensordot_bulk_kernel(BulkArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)a.stages * a.stage_bytes);
  uint64_t* empty = full + a.stages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + a.stages);

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kBulkConsumers);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int groups = (a.C1 + a.R - 1) / a.R;          // work items per n
  const int64_t items = (int64_t)a.N * groups;
  const int64_t begin = items * blockIdx.x / gridDim.x;
  const int64_t end = items * (blockIdx.x + 1) / gridDim.x;
  const uint32_t row_bytes = (uint32_t)C2 * a.P4 * 16;
  if (threadIdx.x == 32) {
    // The first stages of this CTA are asked into L2 before the wait for the preceding kernel: a prefetch uses
    // no value, and L2 is where that kernel's writes land, so the bulk copies below read what it wrote.
    int it = 0;
    for (int64_t item = begin; item < end && it < a.stages; ++item, ++it) {
      const int n = (int)(item / groups), c1 = (int)(item % groups) * a.R;
      const uint32_t bytes = min(a.R, a.C1 - c1) * row_bytes;
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a.I0 + ((size_t)n * a.C1 + c1) * C2 * a.P4 * 4),
                   "r"(bytes)
                   : "memory");
    }
  }
  __syncthreads();
  pdl_sync();  // nothing above uses a value from global memory

  if (threadIdx.x < 32) {
    if (threadIdx.x == 0) {
      int it = 0;
      for (int64_t item = begin; item < end; ++item, ++it) {
        const int s = it % a.stages;
        const uint32_t ph = (it / a.stages) & 1;
        if (!mbar_wait(&empty[s], ph ^ 1, 1, a.dev_status, abort_flag)) break;
        const int n = (int)(item / groups), c1 = (int)(item % groups) * a.R;
        const int rows = min(a.R, a.C1 - c1);
        const uint32_t bytes = rows * row_bytes;
        mbar_expect_tx(&full[s], bytes);
        bulk_load(smem + (size_t)s * a.stage_bytes,
                  a.I0 + ((size_t)n * a.C1 + c1) * C2 * a.P4 * 4, bytes, &full[s]);
      }
    }
    return;
  }

  const int ct = threadIdx.x - 32;
  const int ry = ct / a.P4, px = ct - ry * a.P4;
  const bool active = ry < a.RY;
  float4 w[C2][C3];
  int cur_n = -1;
  int it = 0;
  for (int64_t item = begin; item < end; ++item, ++it) {
    const int s = it % a.stages;
    const uint32_t ph = (it / a.stages) & 1;
    const int n = (int)(item / groups), c1 = (int)(item % groups) * a.R;
    const int rows = min(a.R, a.C1 - c1);
    if (active && n != cur_n) {
      cur_n = n;
      const float4* i1 = reinterpret_cast<const float4*>(a.I1) + (size_t)n * C2 * C3 * a.P4 + px;
#pragma unroll
      for (int c2 = 0; c2 < C2; ++c2)
#pragma unroll
        for (int c3 = 0; c3 < C3; ++c3) w[c2][c3] = __ldg(i1 + (size_t)(c2 * C3 + c3) * a.P4);
    }
    if (!mbar_wait(&full[s], ph, 2, a.dev_status, abort_flag)) break;
    if (active) {
      const float4* st = reinterpret_cast<const float4*>(smem + (size_t)s * a.stage_bytes);
      for (int r = ry; r < rows; r += a.RY) {
        const float4* x = st + (size_t)r * C2 * a.P4 + px;
        float4 xv[C2];
#pragma unroll
        for (int c2 = 0; c2 < C2; ++c2) xv[c2] = x[(size_t)c2 * a.P4];
        float4* o = reinterpret_cast<float4*>(a.O) + ((size_t)n * a.C1 + c1 + r) * C3 * a.P4 + px;
#pragma unroll
        for (int c3 = 0; c3 < C3; ++c3) {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int c2 = 0; c2 < C2; ++c2) {
            acc.x = fmaf(xv[c2].x, w[c2][c3].x, acc.x);
            acc.y = fmaf(xv[c2].y, w[c2][c3].y, acc.y);
            acc.z = fmaf(xv[c2].z, w[c2][c3].z, acc.z);
            acc.w = fmaf(xv[c2].w, w[c2][c3].w, acc.w);
          }
          stg_stream4(o + (size_t)c3 * a.P4, acc);
        }
      }
    }
    mbar_arrive(&empty[s]);  // this thread is done reading the stage
  }
}

// Any C2, C3, P (odd P, large C3, unaligned pointers): one thread per (n, c1, p),
// still coalesced along p; I0's C2 values are re-read from L1 for every c3.
__global__ void __launch_bounds__(256)
tensordot_generic_kernel(const float* __restrict__ I0, const float* __restrict__ I1,
                         float* __restrict__ O, int64_t N, int C1, int C2, int C3, int P) {
  const int64_t total = N * (int64_t)C1 * P;
  for (int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int p = (int)(idx % P);
    const int64_t nc1 = idx / P;
    const int64_t n = nc1 / C1;
    const float* x = I0 + nc1 * C2 * P + p;
    const float* w = I1 + n * C2 * C3 * P + p;
    float* o = O + nc1 * C3 * P + p;
    for (int c3 = 0; c3 < C3; ++c3) {
      float acc = 0.f;
      for (int c2 = 0; c2 < C2; ++c2)
        acc = fmaf(__ldg(x + (size_t)c2 * P), __ldg(w + (size_t)(c2 * C3 + c3) * P), acc);
      o[(size_t)c3 * P] = acc;
    }
  }
}

typedef void (*vec4_fn)(const float4*, const float4*, float4*, int, int, int);
typedef void (*bulk_fn)(BulkArgs);

// The (C2, C3) pairs with register-resident I1 (C2*C3 float4 per thread).
#define TD_FOR_EACH(X) \
  X(8, 2) X(8, 1) X(8, 4) X(4, 1) X(4, 2) X(4, 4) X(16, 1) X(16, 2) X(2, 1) X(2, 2) X(2, 4) X(1, 1)

vec4_fn pick_vec4(int c2, int c3) {
#define TD_CASE(a, b) \
  if (c2 == a && c3 == b) return tensordot_vec4_kernel<a, b>;
  TD_FOR_EACH(TD_CASE)
#undef TD_CASE
  return nullptr;
}

bulk_fn pick_bulk(int c2, int c3) {
#define TD_CASE(a, b) \
  if (c2 == a && c3 == b) return tensordot_bulk_kernel<a, b>;
  TD_FOR_EACH(TD_CASE)
#undef TD_CASE
  return nullptr;
}

bool valid(const tcb200_problem_t& p) {
  for (int i = 0; i < 5; ++i)
    if (p.td[i] <= 0) return false;
  return p.td[1] < (1ll << 31) && p.td[2] < (1 << 20) && p.td[3] < (1 << 20) &&
         p.td[4] < (1ll << 31) && p.td[0] <= 65535;
}

constexpr int64_t kBulkSmemBudget = 200 * 1024;
constexpr int64_t kBulkMaxStage = 64 * 1024;

bool vec_ok(const tcb200_problem_t& p) {
  return p.td[4] % 4 == 0 && pick_vec4((int)p.td[2], (int)p.td[3]) != nullptr;
}
// The bulk kernel keeps one float4 column of p per consumer thread and one row per stage slot.
bool bulk_ok(const tcb200_problem_t& p) {
  return vec_ok(p) && p.td[4] / 4 <= kBulkConsumers && p.td[2] * p.td[4] * 4 <= kBulkMaxStage / 2;
}

// Rows per stage / rows in parallel / ring depth of the bulk kernel.
void bulk_geometry(const tcb200_problem_t& p, int want_rows, int want_stages, int* R, int* RY,
                   int* stages, int64_t* stage_bytes) {
  const int64_t P4 = p.td[4] / 4, C1 = p.td[1];
  const int64_t row_bytes = p.td[2] * P4 * 16;
  int64_t ry = std::max<int64_t>(1, std::min<int64_t>(kBulkConsumers / P4, C1));
  int64_t r = want_rows > 0 ? want_rows : ry * std::max<int64_t>(1, (16 * 1024) / (ry * row_bytes));
  r = std::max<int64_t>(ry, std::min<int64_t>(r, C1));
  while (r > ry && r * row_bytes > kBulkMaxStage) r -= ry;
  if (r * row_bytes > kBulkMaxStage) { r = std::max<int64_t>(1, kBulkMaxStage / row_bytes); ry = std::min(ry, r); }
  const int64_t sb = round_up(r * row_bytes, 128);
  // four stages (~100 KB in flight per SM) measured faster than a deeper ring on B200
  int64_t st = want_stages > 0 ? want_stages : std::min<int64_t>(4, kBulkSmemBudget / sb);
  st = std::max<int64_t>(2, std::min<int64_t>(st, std::min<int64_t>(8, kBulkSmemBudget / sb)));
  *R = (int)r; *RY = (int)ry; *stages = (int)st; *stage_bytes = sb;
}

}  // namespace

int tensordot_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n) {
  if (!valid(p)) return TCB200_ERR_INVALID_ARGUMENT;
  int cnt = 0;
  auto push = [&](int variant, int bm, int stages, int threads) {
    if (cnt < max && out) out[cnt] = tcb200_tile_t{variant, bm, 0, 0, stages, threads, 0};
    ++cnt;
  };
  if (bulk_ok(p)) {
    int R, RY, st;
    int64_t sb;
    bulk_geometry(p, 0, 0, &R, &RY, &st, &sb);
    push(TCB200_VARIANT_SIMT, R, st, kBulkThreads);
    if (2 * R <= p.td[1] && 2 * sb <= kBulkMaxStage) push(TCB200_VARIANT_SIMT, 2 * R, st / 2 > 2 ? st / 2 : 2, kBulkThreads);
    if (kBulkSmemBudget / sb >= 8) push(TCB200_VARIANT_SIMT, R, 8, kBulkThreads);
  }
  if (vec_ok(p)) {
    const int bms[] = {8, 16, 4, 32};
    for (int bm : bms)
      if (bm <= p.td[1] || bm == 8) push(TCB200_VARIANT_SIMT, bm, 0, 256);
  }
  push(TCB200_VARIANT_SIMT, 0, 0, 256);  // generic kernel
  *n = cnt;
  return TCB200_OK;
}

// tile encoding: stages > 0 -> bulk kernel (bm = rows per stage); stages == 0 && bm > 0 -> direct
// vec4 kernel (bm = rows of c1 per CTA); bm == 0 -> generic scalar kernel.
int tensordot_plan(Plan& plan) {
  const tcb200_problem_t& p = plan.p;
  if (!valid(p)) return TCB200_ERR_INVALID_ARGUMENT;
  if (p.epilogue != TCB200_EPI_NONE || p.accumulate) return TCB200_ERR_UNSUPPORTED;
  tcb200_tile_t& t = plan.tile;
  const int64_t N = p.td[0], C1 = p.td[1], P = p.td[4];
  if (t.variant == TCB200_VARIANT_AUTO) {
    tcb200_tile_t first;
    int n = 0;
    tensordot_query(p, &first, 1, &n);
    t = first;
  }
  if (t.variant != TCB200_VARIANT_SIMT) return TCB200_ERR_UNSUPPORTED;
  if (t.stages > 0) {
    if (!bulk_ok(p)) return TCB200_ERR_UNSUPPORTED;
    int R, RY, st;
    int64_t sb;
    bulk_geometry(p, t.bm, t.stages, &R, &RY, &st, &sb);
    t.bm = R; t.stages = st; t.threads = kBulkThreads; t.bn = RY;
    const int64_t items = N * ceil_div(C1, R);
    plan.launch.grid = dim3((unsigned)std::min<int64_t>(items, plan.sms), 1, 1);
    plan.launch.block = dim3(kBulkThreads, 1, 1);
    plan.launch.smem = (size_t)st * sb + 16 * st + 16;
    plan.kernel_id = 2;
    return TCB200_OK;
  }
  if (t.bm > 0 && !vec_ok(p)) return TCB200_ERR_UNSUPPORTED;
  if (t.threads <= 0) t.threads = 256;
  if (t.threads > 256 || t.threads % 32) return TCB200_ERR_INVALID_ARGUMENT;
  if (t.bm > 0) {
    const int64_t P4 = P / 4;
    // x: float4 columns of p (rounded to warps); y: rows of c1 swept together.
    int bx = (int)std::min<int64_t>(round_up(P4, 32), t.threads);
    int by = std::max(1, t.threads / bx);
    by = (int)std::min<int64_t>(by, t.bm);
    plan.launch.block = dim3(bx, by, 1);
    plan.launch.grid = dim3((unsigned)ceil_div(P4, bx), (unsigned)ceil_div(C1, t.bm), (unsigned)N);
    if (plan.launch.grid.y > 65535) return TCB200_ERR_TOO_LARGE;
    plan.kernel_id = 1;
  } else {
    const int64_t total = N * C1 * P;
    plan.launch.block = dim3(t.threads, 1, 1);
    plan.launch.grid =
        dim3((unsigned)std::min<int64_t>(ceil_div(total, t.threads), (int64_t)plan.sms * 32), 1, 1);
    plan.kernel_id = 0;
  }
  plan.launch.smem = 0;
  return TCB200_OK;
}

int tensordot_launch(const Plan& plan, const float* I0, const float* I1, float* O,
                     cudaStream_t s, int* dev_status) {
  const tcb200_problem_t& p = plan.p;
  const bool aligned =
      (((uintptr_t)I0 | (uintptr_t)I1 | (uintptr_t)O) & 15) == 0;
  if (plan.kernel_id == 2 && aligned) {
    bulk_fn fn = pick_bulk((int)p.td[2], (int)p.td[3]);
    BulkArgs a;
    a.I0 = I0; a.I1 = I1; a.O = O;
    a.N = (int)p.td[0]; a.C1 = (int)p.td[1]; a.P4 = (int)(p.td[4] / 4);
    a.R = plan.tile.bm; a.RY = plan.tile.bn; a.stages = plan.tile.stages;
    a.stage_bytes = (uint32_t)round_up((int64_t)a.R * p.td[2] * a.P4 * 16, 128);
    a.dev_status = dev_status;
    static std::atomic<uint64_t> configured[17][5];  // one flag word per (C2 <= 16, C3 <= 4) instantiation
    TCB200_CUDA_TRY(ensure_dynamic_smem(fn, (int)kBulkSmemBudget + 1024, plan.device,
                                        configured[p.td[2]][p.td[3]]));
    TCB200_CUDA_TRY(launch_pdl(fn, plan.launch.grid, plan.launch.block, plan.launch.smem, s, a));
  } else if (plan.kernel_id >= 1 && aligned) {
    vec4_fn fn = pick_vec4((int)p.td[2], (int)p.td[3]);
    dim3 grid = plan.launch.grid, block = plan.launch.block;
    const int bm = plan.tile.bm;
    fn<<<grid, block, 0, s>>>(
        reinterpret_cast<const float4*>(I0), reinterpret_cast<const float4*>(I1),
        reinterpret_cast<float4*>(O), (int)p.td[1], (int)(p.td[4] / 4), bm);
  } else {
    // Unaligned base pointers (a view into a larger buffer) take the scalar kernel.
    const int64_t total = p.td[0] * p.td[1] * p.td[4];
    dim3 block(256, 1, 1);
    dim3 grid((unsigned)std::min<int64_t>(ceil_div(total, 256), (int64_t)plan.sms * 32), 1, 1);
    tensordot_generic_kernel<<<grid, block, 0, s>>>(I0, I1, O, p.td[0], (int)p.td[1],
                                                    (int)p.td[2], (int)p.td[3], (int)p.td[4]);
  }
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}

}  // namespace tcb200
