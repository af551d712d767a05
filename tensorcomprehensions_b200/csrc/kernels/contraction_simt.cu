// K1 (SIMT variants) — strided-batched contraction in plain fp32 FMA:
//   C(b,m,n) (+)= sum_k A(b,m,k) * B(b,n,k)   [+ bias] [relu]
//
// Two kernels:
//   * simt_small: one whole (A_b, B_b) pair per CTA in shared memory.  This is the path
//     for the reference's batchmatmul benchmark (tc/benchmarks/batchmatmul.cc:80-84:
//     500 x [26x72]·[72x26]) where each matrix is far below one tensor-core tile and
//     the problem is bound by HBM and launch latency, not by math.
//   * simt_tiled: 64x64x16 shared-memory tiles, 4x4 register blocking, any operand
//     major-ness, any size.  Exact-fp32 path for contractions the tcgen05 kernel does
//     not take (reduction too short, K not a multiple of 4, "+=" accumulation into
//     unaligned outputs) and one point of the tile sweep.
// Both follow the loop nest's semantics (test/test_core.cc:93-127): zero-initialised
// accumulator, reduction in increasing k.
#include "async.cuh"
#include "common.cuh"

namespace tcb200 {
namespace {

struct GemmArgs {
  const float* A;
  const float* B;
  const float* bias;
  float* C;
  int M, N, K;
  int64_t lda, ldb, ldc, sa, sb, sc;
  int epi, bias_on_m, accumulate;
};

__device__ __forceinline__ void store_out(const GemmArgs& g, float* Cb, int m, int n, float acc) {
  float bias = 0.f;
  if (g.epi == TCB200_EPI_BIAS || g.epi == TCB200_EPI_BIAS_RELU)
    bias = __ldg(g.bias + (g.bias_on_m ? m : n));
  float* c = Cb + (int64_t)m * g.ldc + n;
  if (g.accumulate) acc += *c;
  *c = apply_epilogue_rt(g.epi, acc, bias);
}

// ------------------------------------------------------------------------------------
// simt_tiled
// ------------------------------------------------------------------------------------
constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

// Loads a (64 rows of the free index) x (16 of k) tile into smem as T[k][row].
// `kmaj`: the operand's k is its innermost (contiguous) index.
template <bool KMAJ>
__device__ __forceinline__ void load_tile(const float* __restrict__ base, int64_t ld, int rows,
                                          int K, int row0, int k0, bool vec_ok,
                                          float (*T)[BM + PAD], int tid) {
  if (KMAJ) {
    const int r = tid >> 2, kk = (tid & 3) << 2;
    const int row = row0 + r, k = k0 + kk;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (row < rows) {
      const float* src = base + (int64_t)row * ld + k;
      if (vec_ok && k + 3 < K) {
        float4 q = __ldg(reinterpret_cast<const float4*>(src));
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (k + i < K) v[i] = __ldg(src + i);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) T[kk + i][r] = v[i];
  } else {
    const int kk = tid >> 4, r = (tid & 15) << 2;
    const int row = row0 + r, k = k0 + kk;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (k < K) {
      const float* src = base + (int64_t)k * ld + row;
      if (vec_ok && row + 3 < rows) {
        float4 q = __ldg(reinterpret_cast<const float4*>(src));
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (row + i < rows) v[i] = __ldg(src + i);
      }
    }
    *reinterpret_cast<float4*>(&T[kk][r]) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

template <bool AK, bool BKM>
__global__ void __launch_bounds__(256) simt_tiled_kernel(GemmArgs g, int a_vec, int b_vec) {
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Bs[BK][BN + PAD];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int64_t b = blockIdx.z;
  const float* A = g.A + b * g.sa;
  const float* B = g.B + b * g.sb;
  float* C = g.C + b * g.sc;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < g.K; k0 += BK) {
    load_tile<AK>(A, g.lda, g.M, g.K, m0, k0, a_vec, As, tid);
    load_tile<BKM>(B, g.ldb, g.N, g.K, n0, k0, b_vec, Bs, tid);
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 bq = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w};
      const float bv[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < g.N) store_out(g, C, m, n, acc[i][j]);
    }
  }
}

// ------------------------------------------------------------------------------------
// simt_small: whole matrices of one batch entry in shared memory; 2x2 outputs per thread.
// The kernel is instruction-bound (profiled: 2.5 IPC, integer index math and scalar shared loads
// dominated), so the FAST form avoids divisions (one warp stages one row at a time, a lane per
// 16-byte / 8-byte chunk), stages with asynchronous copies, and consumes four k per step with
// 128-bit loads of A and 64-bit loads of B: 6 shared loads per 16 FMAs.
//   FAST needs: K % 4 == 0, lda % 4 == 0, 16-byte aligned A slabs; ldb % 2 == 0, 8-byte aligned B slabs.
//   BULK (MODE 2) is FAST for dense operands (lda == K, ldb == N, even N, slabs that are multiples of
//   16 bytes): one thread brings each slab in with a single 1-D bulk copy (cp.async.bulk + mbarrier)
//   instead of ~1400 small asynchronous copies with their index arithmetic per CTA.
// smem: As[M][lda_s], Bs[K][ldb_s];  FAST: lda_s = K + 4, ldb_s = even(N) + 2;  else K + 1, N | 1.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_8(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(
                   (uint32_t)__cvta_generic_to_shared(smem_dst)),
               "l"(gmem_src)
               : "memory");
}

template <int MODE>  // 0: any layout, 1: FAST, 2: BULK
__global__ void __launch_bounds__(256) simt_small_kernel(GemmArgs g, int ldas, int ldbs) {
  constexpr bool FAST = MODE >= 1;
  extern __shared__ __align__(16) float smem[];
  const int M = g.M, N = g.N, K = g.K;
  float* As = smem;
  float* Bs = smem + (size_t)M * ldas;
  const int64_t b = blockIdx.x;
  const float* A = g.A + b * g.sa;
  const float* B = g.B + b * g.sb;
  float* C = g.C + b * g.sc;
  const int tid = threadIdx.x, nt = blockDim.x;
  if (MODE == 2 && tid == 32) {
    // Both slabs are asked into L2 before the wait for the preceding kernel: a prefetch uses no value, and L2
    // is where that kernel's writes land, so the later bulk copies read what it wrote.  The kernel is one DRAM
    // round trip and a few microseconds of work; this takes the round trip out of its start.
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(A), "r"((uint32_t)M * K * 4) : "memory");
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(B), "r"((uint32_t)K * N * 4) : "memory");
  }
  pdl_sync();  // launched as a programmatic dependent: wait for the preceding kernel before any use of global memory

  // Only the A(m,k) / B(k,n) row-major form reaches this kernel (checked by the plan).
  if (MODE == 2) {
    // the barrier sits behind both slabs (their sizes are multiples of 16 bytes)
    uint64_t* bar = reinterpret_cast<uint64_t*>(Bs + (size_t)K * ldbs);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar + 1);
    if (tid == 0) {
      mbar_init(bar, 1);
      *abort_flag = 0;
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      const uint32_t bytes_a = (uint32_t)M * K * 4, bytes_b = (uint32_t)K * N * 4;
      mbar_expect_tx(bar, bytes_a + bytes_b);
      bulk_load(As, A, bytes_a, bar);
      bulk_load(Bs, B, bytes_b, bar);
    }
    __syncthreads();  // the barrier is initialised before anyone polls it
    if (!mbar_wait(bar, 0, 9, nullptr, abort_flag)) return;
  } else if (FAST) {
    const int warp = tid >> 5, lane = tid & 31, nw = nt >> 5;
    const int ka = K >> 2, nb = (N + 1) >> 1;
    for (int m = warp; m < M; m += nw)
      for (int q = lane; q < ka; q += 32)
        cp_async_16(As + m * ldas + 4 * q, A + (int64_t)m * g.lda + 4 * q);
    for (int k = warp; k < K; k += nw)
      for (int q = lane; q < nb; q += 32) {
        if (2 * q + 1 < N) cp_async_8(Bs + k * ldbs + 2 * q, B + (int64_t)k * g.ldb + 2 * q);
        else cp_async_4(Bs + k * ldbs + 2 * q, B + (int64_t)k * g.ldb + 2 * q);
      }
  } else {
    for (int i = tid; i < M * K; i += nt) {
      const int m = i / K, k = i - m * K;
      cp_async_4(As + m * ldas + k, A + (int64_t)m * g.lda + k);
    }
    for (int i = tid; i < K * N; i += nt) {
      const int k = i / N, n = i - k * N;
      cp_async_4(Bs + k * ldbs + n, B + (int64_t)k * g.ldb + n);
    }
  }
  if (MODE != 2) {
    cp_async_wait_all();
    __syncthreads();
  }

  const int tm = (M + 1) >> 1, tn = (N + 1) >> 1;
  for (int t = tid; t < tm * tn; t += nt) {
    const int mi = (t / tn) * 2, ni = (t % tn) * 2;
    const bool m1 = mi + 1 < M, n1 = ni + 1 < N;
    const float* a0 = As + mi * ldas;
    const float* a1 = As + (m1 ? mi + 1 : mi) * ldas;
    const float* b0 = Bs + ni;
    float c00 = 0.f, c01 = 0.f, c10 = 0.f, c11 = 0.f;
    if (FAST) {
      // b0 + 1 may be the padding column when N is odd: its products only reach c01/c11, which are
      // not stored then.
#pragma unroll 2
      for (int k = 0; k < K; k += 4) {
        const float4 x0 = *reinterpret_cast<const float4*>(a0 + k);
        const float4 x1 = *reinterpret_cast<const float4*>(a1 + k);
        const float2 y0 = *reinterpret_cast<const float2*>(b0 + (k + 0) * ldbs);
        const float2 y1 = *reinterpret_cast<const float2*>(b0 + (k + 1) * ldbs);
        const float2 y2 = *reinterpret_cast<const float2*>(b0 + (k + 2) * ldbs);
        const float2 y3 = *reinterpret_cast<const float2*>(b0 + (k + 3) * ldbs);
        c00 = fmaf(x0.x, y0.x, c00); c01 = fmaf(x0.x, y0.y, c01);
        c10 = fmaf(x1.x, y0.x, c10); c11 = fmaf(x1.x, y0.y, c11);
        c00 = fmaf(x0.y, y1.x, c00); c01 = fmaf(x0.y, y1.y, c01);
        c10 = fmaf(x1.y, y1.x, c10); c11 = fmaf(x1.y, y1.y, c11);
        c00 = fmaf(x0.z, y2.x, c00); c01 = fmaf(x0.z, y2.y, c01);
        c10 = fmaf(x1.z, y2.x, c10); c11 = fmaf(x1.z, y2.y, c11);
        c00 = fmaf(x0.w, y3.x, c00); c01 = fmaf(x0.w, y3.y, c01);
        c10 = fmaf(x1.w, y3.x, c10); c11 = fmaf(x1.w, y3.y, c11);
      }
    } else {
      const int nj = n1 ? 1 : 0;
#pragma unroll 8
      for (int k = 0; k < K; ++k) {
        const float x0 = a0[k], x1 = a1[k];
        const float y0 = b0[k * ldbs], y1 = b0[k * ldbs + nj];
        c00 = fmaf(x0, y0, c00);
        c01 = fmaf(x0, y1, c01);
        c10 = fmaf(x1, y0, c10);
        c11 = fmaf(x1, y1, c11);
      }
    }
    store_out(g, C, mi, ni, c00);
    if (n1) store_out(g, C, mi, ni + 1, c01);
    if (m1) store_out(g, C, mi + 1, ni, c10);
    if (m1 && n1) store_out(g, C, mi + 1, ni + 1, c11);
  }
}

// ------------------------------------------------------------------------------------
// simt_small, 4x4 register tiles (dense operands only).  The 2x2 form above moves one shared-memory word
// per multiply-add into registers and is bound by that (shared memory returns 32 words per clock per SM
// against 128 FMA lanes); a 4x4 tile moves half a word per multiply-add.  Per step of four k: four 128-bit
// loads of A (rows tm, tm + TM, tm + 2 TM, tm + 3 TM: rows TM apart fall into different banks where
// adjacent rows of a 72-float pitch would collide) and eight 64-bit loads of B (four consecutive columns of
// four rows; a B row of 26 floats is only 8-byte aligned), then 64 FMAs.  Both slabs arrive by one bulk copy
// each.  Threads past the edge of the tile grid read clamped rows / the next row's first columns and do not
// store.
// A 26 x 26 output has only 49 such tiles, two warps where the 2x2 form runs eight, and with a few matrices per
// SM nothing then hides the latency of a step (measured: 8.7 us against 7.5 us).  So the reduction is split over
// `ks` thread groups as well (72 = 3 x 24): group q runs k in [q K/ks, (q+1) K/ks), the ks partial tiles meet in
// shared memory and are added in the fixed order q = 0 .. ks-1 by the threads that store the output, one element
// per thread, consecutive threads on consecutive addresses.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) simt_small4_kernel(GemmArgs g, int ks) {
  extern __shared__ __align__(16) float smem[];
  pdl_sync();  // launched as a programmatic dependent: wait for the preceding kernel before any global access
  const int M = g.M, N = g.N, K = g.K;
  float* As = smem;                    // [M][K], dense
  float* Bs = smem + (size_t)M * K;    // [K][N], dense, followed by 16 bytes of slack for the last row's overrun
  uint64_t* bar = reinterpret_cast<uint64_t*>(Bs + (size_t)K * N + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar + 1);
  float* Ps = Bs + (size_t)K * N + 8;  // [ks][4 TM][4 TN] partial tiles (ks > 1)
  const int64_t b = blockIdx.x;
  const int tid = threadIdx.x, nt = blockDim.x;
  if (tid == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const uint32_t bytes_a = (uint32_t)M * K * 4, bytes_b = (uint32_t)K * N * 4;
    mbar_expect_tx(bar, bytes_a + bytes_b);
    bulk_load(As, g.A + b * g.sa, bytes_a, bar);
    bulk_load(Bs, g.B + b * g.sb, bytes_b, bar);
  }
  const int TM = (M + 3) >> 2, TN = (N + 3) >> 2, tasks = TM * TN;
  const int q = tid / tasks, task = tid - q * tasks;
  const int tm = task / TN, tn = task - tm * TN;
  const bool active = q < ks;
  const float* arow[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) arow[i] = As + (size_t)min(tm + TM * i, M - 1) * K;
  const float* bcol = Bs + 4 * tn;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  __syncthreads();  // the barrier is initialised before anyone polls it
  const bool loaded = mbar_wait(bar, 0, 9, nullptr, abort_flag);
  if (loaded && active) {
    const int kq = K / ks;  // a multiple of 4 (checked by the plan)
#pragma unroll 2
    for (int k = q * kq; k < (q + 1) * kq; k += 4) {
      float a[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(arow[i] + k);
        a[i][0] = v.x; a[i][1] = v.y; a[i][2] = v.z; a[i][3] = v.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 b0 = *reinterpret_cast<const float2*>(bcol + (size_t)(k + j) * N);
        const float2 b1 = *reinterpret_cast<const float2*>(bcol + (size_t)(k + j) * N + 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[i][0] = fmaf(a[i][j], b0.x, acc[i][0]);
          acc[i][1] = fmaf(a[i][j], b0.y, acc[i][1]);
          acc[i][2] = fmaf(a[i][j], b1.x, acc[i][2]);
          acc[i][3] = fmaf(a[i][j], b1.y, acc[i][3]);
        }
      }
    }
  }
  float* C = g.C + b * g.sc;
  if (ks == 1) {
    if (!(loaded && active)) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = tm + TM * i;
      if (m >= M) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = 4 * tn + j;
        if (n < N) store_out(g, C, m, n, acc[i][j]);
      }
    }
    return;
  }
  const int MP = 4 * TM, NP = 4 * TN;
  if (loaded && active) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      *reinterpret_cast<float4*>(Ps + ((size_t)q * MP + tm + TM * i) * NP + 4 * tn) =
          make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
  }
  __syncthreads();
  if (!loaded) return;
  for (int i = tid; i < M * N; i += nt) {
    const int m = i / N, n = i - m * N;
    float v = Ps[(size_t)m * NP + n];
    for (int s2 = 1; s2 < ks; ++s2) v += Ps[((size_t)s2 * MP + m) * NP + n];
    store_out(g, C, m, n, v);
  }
}

bool valid(const tcb200_problem_t& p) {
  return p.batch > 0 && p.M > 0 && p.N > 0 && p.K > 0 && p.M < (1ll << 31) &&
         p.N < (1ll << 31) && p.K < (1ll << 31) && p.batch <= 0x7fffffffll && p.lda > 0 &&
         p.ldb > 0 && p.ldc >= p.N && p.stride_a >= 0 && p.stride_b >= 0 && p.stride_c >= 0;
}

// Shape part of the FAST conditions (pointer alignment is checked at launch).
bool small_fast_shape(const tcb200_problem_t& p) {
  return p.K % 4 == 0 && p.lda % 4 == 0 && p.stride_a % 4 == 0 && p.ldb % 2 == 0 && p.stride_b % 2 == 0;
}
// Shared-memory pitches: the larger (FAST) ones are always reserved so the launch can pick either form.
void small_pitches(const tcb200_problem_t& p, bool fast, int* ldas, int* ldbs) {
  *ldas = fast ? (int)p.K + 4 : (int)p.K + 1;
  *ldbs = fast ? (int)((p.N + 1) / 2 * 2 + 2) : ((int)p.N | 1);  // odd pitch keeps k-strided reads off one bank
}
size_t small_smem_bytes(const tcb200_problem_t& p) {
  return sizeof(float) * ((size_t)p.M * (p.K + 4) + (size_t)p.K * ((p.N + 1) / 2 * 2 + 2)) + 16;
}
// Shape part of the conditions of the bulk-copy forms: dense operands whose slabs are multiples of 16 bytes.
bool small_dense_shape(const tcb200_problem_t& p) {
  return small_fast_shape(p) && p.lda == p.K && p.ldb == p.N && p.N % 2 == 0 && (p.M * p.K) % 4 == 0 &&
         (p.K * p.N) % 4 == 0 && p.stride_b % 4 == 0 && p.M * p.K * 4 < (1 << 20) && p.K * p.N * 4 < (1 << 20);
}
// The 4x4-tile form: one thread per (4x4 tile of the output, share of the reduction).
int small4_tasks(const tcb200_problem_t& p) { return (int)(((p.M + 3) / 4) * ((p.N + 3) / 4)); }
// Shares of the reduction: as many as keep every share a multiple of four k and the CTA within 256 threads.
int small4_ksplit(const tcb200_problem_t& p) {
  for (int ks = 4; ks > 1; --ks)
    if (p.K % (4 * ks) == 0 && small4_tasks(p) * ks <= 256) return ks;
  return 1;
}
int small4_threads(const tcb200_problem_t& p, int ks) { return (int)round_up((int64_t)small4_tasks(p) * ks, 32); }
size_t small4_smem(const tcb200_problem_t& p, int ks) {
  const size_t partial = ks > 1 ? (size_t)ks * 16 * small4_tasks(p) : 0;
  return sizeof(float) * ((size_t)p.M * p.K + (size_t)p.K * p.N + 8 + partial) + 16;
}
bool small4_ok(const tcb200_problem_t& p) {
  return small_dense_shape(p) && small4_tasks(p) <= 256 && small4_smem(p, small4_ksplit(p)) <= 48 * 1024;
}

// simt_small reads A as (m,k) row-major and B as (k,n) row-major: the batchmatmul form.
bool small_ok(const tcb200_problem_t& p) {
  return p.a_k_major && !p.b_k_major && small_smem_bytes(p) <= 48 * 1024 &&
         p.M * p.N <= 4096;
}

}  // namespace

int contraction_simt_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n) {
  if (!valid(p)) return TCB200_ERR_INVALID_ARGUMENT;
  int cnt = 0;
  auto push = [&](int variant, int bm, int bn, int bk, int threads) {
    if (cnt < max && out) out[cnt] = tcb200_tile_t{variant, bm, bn, bk, 0, threads, 0};
    ++cnt;
  };
  if (small_ok(p)) {
    push(TCB200_VARIANT_SIMT_SMALL, (int)p.M, (int)p.N, (int)p.K, 256);
    // bk = 4: 4x4 register tiles with the reduction shared by up to four thread groups (stages = groups);
    // stages = 1 is the unsplit form (two warps per 26 x 26 matrix: 8.7 us against 7.5 us for the 2x2 form)
    if (small4_ok(p)) {
      const int ks = small4_ksplit(p);
      if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_SIMT_SMALL, (int)p.M, (int)p.N, 4, ks, small4_threads(p, ks), 0};
      ++cnt;
      if (ks > 1) {
        if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_SIMT_SMALL, (int)p.M, (int)p.N, 4, 1, small4_threads(p, 1), 0};
        ++cnt;
      }
    }
    push(TCB200_VARIANT_SIMT_SMALL, (int)p.M, (int)p.N, (int)p.K, 192);
    push(TCB200_VARIANT_SIMT_SMALL, (int)p.M, (int)p.N, (int)p.K, 128);
  }
  push(TCB200_VARIANT_SIMT, BM, BN, BK, 256);
  *n = cnt;
  return TCB200_OK;
}

int contraction_simt_plan(Plan& plan) {
  const tcb200_problem_t& p = plan.p;
  if (!valid(p)) return TCB200_ERR_INVALID_ARGUMENT;
  tcb200_tile_t& t = plan.tile;
  if (t.variant == TCB200_VARIANT_SIMT_SMALL) {
    if (!small_ok(p)) return TCB200_ERR_UNSUPPORTED;
    if (t.bk == 4 && p.K != 4) {  // 4x4 register tiles; stages = thread groups that share the reduction
      if (!small4_ok(p)) return TCB200_ERR_UNSUPPORTED;
      int ks = t.stages > 0 ? t.stages : small4_ksplit(p);
      if (ks > 4 || p.K % (4 * ks) != 0 || small4_tasks(p) * ks > 256 || small4_smem(p, ks) > 48 * 1024)
        return TCB200_ERR_UNSUPPORTED;
      t.bm = (int)p.M; t.bn = (int)p.N; t.stages = ks; t.threads = small4_threads(p, ks);
      plan.launch.grid = dim3((unsigned)p.batch, 1, 1);
      plan.launch.block = dim3(t.threads, 1, 1);
      plan.launch.smem = small4_smem(p, ks);
      plan.kernel_id = 11;
      return TCB200_OK;
    }
    if (t.threads <= 0) t.threads = 256;
    if (t.threads > 256 || t.threads % 32) return TCB200_ERR_INVALID_ARGUMENT;
    t.bm = (int)p.M; t.bn = (int)p.N; t.bk = (int)p.K;
    plan.launch.grid = dim3((unsigned)p.batch, 1, 1);
    plan.launch.block = dim3(t.threads, 1, 1);
    plan.launch.smem = small_smem_bytes(p);
    plan.kernel_id = 10;
    return TCB200_OK;
  }
  if (t.variant != TCB200_VARIANT_SIMT) return TCB200_ERR_UNSUPPORTED;
  t.bm = BM; t.bn = BN; t.bk = BK; t.threads = 256;
  if (p.batch > 65535) return TCB200_ERR_TOO_LARGE;
  if (ceil_div(p.M, BM) > 65535) return TCB200_ERR_TOO_LARGE;
  plan.launch.grid = dim3((unsigned)ceil_div(p.N, BN), (unsigned)ceil_div(p.M, BM), (unsigned)p.batch);
  plan.launch.block = dim3(256, 1, 1);
  plan.launch.smem = 0;
  plan.kernel_id = (p.a_k_major ? 1 : 0) | (p.b_k_major ? 2 : 0);
  return TCB200_OK;
}

int contraction_simt_launch(const Plan& plan, const float* A, const float* B, const float* bias,
                            float* C, cudaStream_t s) {
  const tcb200_problem_t& p = plan.p;
  GemmArgs g{A, B, bias, C, (int)p.M, (int)p.N, (int)p.K, p.lda, p.ldb, p.ldc,
             p.stride_a, p.stride_b, p.stride_c, p.epilogue, p.bias_on_m, p.accumulate};
  if (plan.kernel_id == 11 && (((uintptr_t)A | (uintptr_t)B) & 15) == 0) {
    TCB200_CUDA_TRY(launch_pdl(simt_small4_kernel, plan.launch.grid, plan.launch.block, plan.launch.smem, s, g,
                               plan.tile.stages));
  } else if (plan.kernel_id == 10 || plan.kernel_id == 11) {
    // (a 4x4-tile plan whose operands are views at an odd offset runs the forms that take any alignment)
    const dim3 block = plan.kernel_id == 11 ? dim3(256, 1, 1) : plan.launch.block;
    const size_t smem_bytes = plan.kernel_id == 11 ? small_smem_bytes(p) : plan.launch.smem;
    const bool fast = small_fast_shape(p) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)B % 8 == 0);
    int ldas = 0, ldbs = 0;
    small_pitches(p, fast, &ldas, &ldbs);
    const bool bulk = fast && small_dense_shape(p) && ((uintptr_t)B % 16 == 0);
    if (bulk)
      TCB200_CUDA_TRY(launch_pdl(simt_small_kernel<2>, plan.launch.grid, block, smem_bytes, s, g,
                                 (int)p.K, (int)p.N));
    else if (fast)
      TCB200_CUDA_TRY(launch_pdl(simt_small_kernel<1>, plan.launch.grid, block, smem_bytes, s, g, ldas, ldbs));
    else
      TCB200_CUDA_TRY(launch_pdl(simt_small_kernel<0>, plan.launch.grid, block, smem_bytes, s, g, ldas, ldbs));
  } else {
    // 128-bit loads need a 16-byte aligned base, leading dimension and batch stride.
    const int a_vec = ((uintptr_t)A % 16 == 0) && p.lda % 4 == 0 && p.stride_a % 4 == 0;
    const int b_vec = ((uintptr_t)B % 16 == 0) && p.ldb % 4 == 0 && p.stride_b % 4 == 0;
    switch (plan.kernel_id) {
      case 0: simt_tiled_kernel<false, false><<<plan.launch.grid, plan.launch.block, 0, s>>>(g, a_vec, b_vec); break;
      case 1: simt_tiled_kernel<true, false><<<plan.launch.grid, plan.launch.block, 0, s>>>(g, a_vec, b_vec); break;
      case 2: simt_tiled_kernel<false, true><<<plan.launch.grid, plan.launch.block, 0, s>>>(g, a_vec, b_vec); break;
      default: simt_tiled_kernel<true, true><<<plan.launch.grid, plan.launch.block, 0, s>>>(g, a_vec, b_vec); break;
    }
  }
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}

}  // namespace tcb200
