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

vec4_fn pick_vec4(int c2, int c3) {
#define TD_CASE(a, b) \
  if (c2 == a && c3 == b) return tensordot_vec4_kernel<a, b>;
  TD_CASE(8, 2) TD_CASE(8, 1) TD_CASE(8, 4) TD_CASE(4, 1) TD_CASE(4, 2) TD_CASE(4, 4)
  TD_CASE(16, 1) TD_CASE(16, 2) TD_CASE(2, 1) TD_CASE(2, 2) TD_CASE(2, 4) TD_CASE(1, 1)
#undef TD_CASE
  return nullptr;
}

bool valid(const tcb200_problem_t& p) {
  for (int i = 0; i < 5; ++i)
    if (p.td[i] <= 0) return false;
  return p.td[1] < (1ll << 31) && p.td[2] < (1 << 20) && p.td[3] < (1 << 20) &&
         p.td[4] < (1ll << 31) && p.td[0] <= 65535;
}

}  // namespace

int tensordot_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n) {
  if (!valid(p)) return TCB200_ERR_INVALID_ARGUMENT;
  int cnt = 0;
  auto push = [&](int variant, int bm, int threads) {
    if (cnt < max && out) out[cnt] = tcb200_tile_t{variant, bm, 0, 0, 0, threads, 0};
    ++cnt;
  };
  const bool vec = p.td[4] % 4 == 0 && pick_vec4((int)p.td[2], (int)p.td[3]) != nullptr;
  if (vec) {
    const int bms[] = {8, 16, 4, 32};
    for (int bm : bms)
      if (bm <= p.td[1] || bm == 8) push(TCB200_VARIANT_SIMT, bm, 256);
  }
  push(TCB200_VARIANT_SIMT, 0, 256);  // generic kernel
  *n = cnt;
  return TCB200_OK;
}

int tensordot_plan(Plan& plan) {
  const tcb200_problem_t& p = plan.p;
  if (!valid(p)) return TCB200_ERR_INVALID_ARGUMENT;
  if (p.epilogue != TCB200_EPI_NONE || p.accumulate) return TCB200_ERR_UNSUPPORTED;
  tcb200_tile_t& t = plan.tile;
  const int64_t N = p.td[0], C1 = p.td[1], P = p.td[4];
  const bool vec_ok = P % 4 == 0 && pick_vec4((int)p.td[2], (int)p.td[3]) != nullptr;
  if (t.variant == TCB200_VARIANT_AUTO) {
    t.variant = TCB200_VARIANT_SIMT;
    t.bm = vec_ok ? 8 : 0;
    t.threads = 256;
  }
  if (t.variant != TCB200_VARIANT_SIMT) return TCB200_ERR_UNSUPPORTED;
  if (t.bm > 0 && !vec_ok) return TCB200_ERR_UNSUPPORTED;
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
        dim3((unsigned)std::min<int64_t>(ceil_div(total, t.threads), (int64_t)kNumSMs * 32), 1, 1);
    plan.kernel_id = 0;
  }
  plan.launch.smem = 0;
  return TCB200_OK;
}

int tensordot_launch(const Plan& plan, const float* I0, const float* I1, float* O,
                     cudaStream_t s) {
  const tcb200_problem_t& p = plan.p;
  const bool aligned =
      (((uintptr_t)I0 | (uintptr_t)I1 | (uintptr_t)O) & 15) == 0;
  if (plan.kernel_id == 1 && aligned) {
    vec4_fn fn = pick_vec4((int)p.td[2], (int)p.td[3]);
    fn<<<plan.launch.grid, plan.launch.block, 0, s>>>(
        reinterpret_cast<const float4*>(I0), reinterpret_cast<const float4*>(I1),
        reinterpret_cast<float4*>(O), (int)p.td[1], (int)(p.td[4] / 4), plan.tile.bm);
  } else {
    // Unaligned base pointers (a view into a larger buffer) take the scalar kernel.
    const int64_t total = p.td[0] * p.td[1] * p.td[4];
    dim3 block(256, 1, 1);
    dim3 grid((unsigned)std::min<int64_t>(ceil_div(total, 256), (int64_t)kNumSMs * 32), 1, 1);
    tensordot_generic_kernel<<<grid, block, 0, s>>>(I0, I1, O, p.td[0], (int)p.td[1],
                                                    (int)p.td[2], (int)p.td[3], (int)p.td[4]);
  }
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}

}  // namespace tcb200
