// K1 (tensor-core variant) — C(b,m,n) (+)= sum_k A(b,m,k) * B(b,n,k) [+bias][relu], both operands
// k-major ("NT" form: the reference's transposed matmul tc/benchmarks/tmm.cc:79-83 and the
// fully-connected layers of tc/library/fcrelu.h:22-28, tc/benchmarks/MLP_model.cc:547-560).
//
// Blackwell execution model, one 128 x BN output tile per CTA:
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the fp32 A (128x32) and B (BNx32)
//               k-blocks into 128B-swizzled shared memory, completion on an mbarrier (no multicast)
//   warps 2-5   3xTF32 split (when split_tf32 == 3): for every fp32 value v of the stage,
//               lo = tf32(v - trunc_tf32(v)) goes to a second buffer with the same (swizzled)
//               layout; the raw tile serves as hi because the tensor core truncates fp32 words to
//               TF32 itself; then the stage is handed to the MMA warp
//   warp 1      one elected thread issues tcgen05.mma.kind::tf32 (M=128, N=BN, K=8) with the
//               accumulator in TMEM: per k-slice  lo*hi, hi*lo, hi*hi  (small terms first), and
//               tcgen05.commit releases the stage back to the producer
//   epilogue    tcgen05.ld of the fp32 accumulator (lane = row), + bias, ReLU, 128-bit stores
//
// Why the split: kind::tf32 keeps 10 mantissa bits of each operand.  With v = hi + lo
// (hi, lo both exactly representable in TF32 up to 2^-21 |v|) the three products recover
// fp32-level accuracy (the dropped lo*lo term is 2^-22 relative) at 3x the tensor work.
//
// Every wait on an mbarrier is bounded: when it gives up the thread records a code in
// *dev_status, stops issuing work and falls through to the common exit, where TMEM is freed.
#include <cuda.h>

#include <atomic>
#include <mutex>

#include "async.cuh"
#include "common.cuh"
#include "tcgen05.cuh"

namespace tcb200 {
namespace {

constexpr int BM = 128;       // UMMA M (cta_group::1)
constexpr int BK = 32;        // fp32 elements per 128-byte swizzle row
constexpr int UMMA_K = 8;     // kind::tf32
constexpr int kSmemBudget = 200 * 1024;

__host__ __device__ constexpr int raw_bytes(int bn) { return (BM + bn) * BK * 4; }
__host__ __device__ constexpr int stage_bytes(int bn, int split) {
  return raw_bytes(bn) * (split == 3 ? 2 : 1);
}
__host__ __device__ constexpr int num_stages(int bn, int split) {
  return (kSmemBudget / stage_bytes(bn, split)) > 8 ? 8 : (kSmemBudget / stage_bytes(bn, split));
}
constexpr int kBarrierBytes = 512;
__host__ __device__ constexpr int smem_bytes(int bn, int split) {
  return num_stages(bn, split) * stage_bytes(bn, split) + kBarrierBytes + 1024 /*alignment slack*/;
}

struct TcArgs {
  float* C;
  const float* bias;
  int M, N, K, batch;
  int64_t ldc, stride_c;
  int epi, bias_on_m, accumulate;
  int a_batched, b_batched;  // 0: operand shared by all batch entries
  int c_vec;                 // 128-bit stores allowed
  int tma_store;             // pair kernel: epilogue through the staging tile and tiled TMA stores
  int c_transposed;          // pair kernel: the kernel's (row, column) is C's (column, row): C = (B A^T)^T, operands swapped
  int tail_S, tail_tiles, tail_kb;  // pair kernel: the last tail_tiles tiles split tail_S ways, tail_kb k-blocks each
                                    // (tail_S = 0: none)
  int ksplit_kb;             // split-K launch (TS and pair kernels): k-blocks per split, the "batch" index is the
                             // split and selects the k range, not an operand slab; 0 = the whole reduction
  int* dev_status;
};

// Shared-memory matrix descriptor: k-major operand, 128-byte swizzle, rows of 128 B, groups of
// 8 rows 1024 B apart (SBO); LBO is unused for swizzled k-major; descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);   // start address, 16-byte units
  d |= (uint64_t)1 << 16;                    // leading byte offset (ignored)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset
  d |= (uint64_t)1 << 46;                    // version
  d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D=f32, A=B=tf32, both k-major, M=128, N=BN.
__host__ __device__ constexpr uint32_t make_idesc(int bn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(bn >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}

// ---------------------------------------------------------------------------------- kernel
// Warp roles.  With the 3xTF32 split: 0 = TMA, 1 = MMA, 2-5 = split, 6-13 = drain/epilogue (448
// threads); with a single TF32 pass the split warps do not exist (320 threads).  The eight drain
// warps have warp%4 = {2,3,0,1,2,3,0,1} in both cases: two per TMEM lane quarter, each taking one
// half of the tile's columns.
template <int SPLIT>
__host__ __device__ constexpr int num_threads() { return SPLIT == 3 ? 448 : 320; }

// K elements accumulated inside TMEM before the partial sum is drained into fp32 registers.
// The tensor core adds into its fp32 accumulator with truncation, so a long chain of accumulations
// drifts towards zero by up to half an ulp per MMA; draining every 256 K elements and summing the
// chunks with round-to-nearest FADDs keeps the result at SIMT-fp32 accuracy.
constexpr int kChunkKB = 8;  // k-blocks of 32
// Own k-blocks per issuer between drains.  The error the truncation leaves is proportional to the
// chunk length (all-positive U[0,1) operands, K = 2048: mean error -1.2e-3 of a sum of 511 with chunks
// of 4, -2.3e-3 with 8).  Measured with the library swapped between runs on one GPU: the single-CTA kernel
// on the transposed matmul 84.5 / 85.8 / 90.6 us at 8 / 4 / 2, the CTA-pair kernel on MLP3 360 / 376 / 386 us at
// 8 / 6 / 4 (and 358 us at 12).
constexpr int kTsChunkKB = 4;
constexpr int kPairChunkKB = 8;

template <int BN, int SPLIT>
__global__ void __launch_bounds__(num_threads<SPLIT>(), 1)
contraction_tc_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, TcArgs a) {
  constexpr int STAGES = num_stages(BN, SPLIT);
  constexpr int RAW = raw_bytes(BN);
  constexpr int STAGE = stage_bytes(BN, SPLIT);
  constexpr int A_BYTES = BM * BK * 4;
  constexpr uint32_t IDESC = make_idesc(BN);
  constexpr bool CHUNKED = BN <= 128;  // register budget of the drain warps: BN fp32 per thread
  constexpr int SPLIT_WARPS = SPLIT == 3 ? 4 : 0;
  constexpr int DRAIN_WARP0 = 2 + SPLIT_WARPS;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators: MMA fills one while the other drains
  static_assert(STAGES >= 2, "pipeline needs two stages");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE);
  uint64_t* ready = full + STAGES;
  uint64_t* empty = ready + STAGES;
  uint64_t* acc_full = empty + STAGES;   // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (a.K + BK - 1) / BK;
  const int chunk_kb = CHUNKED ? kChunkKB : num_kb;
  const int num_chunks = (num_kb + chunk_kb - 1) / chunk_kb;
  const int tiles_n = (a.N + BN - 1) / BN, tiles_m = (a.M + BM - 1) / BM;
  const int64_t num_tiles = (int64_t)tiles_n * tiles_m * a.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&ready[s], 128);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 256);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Static persistent schedule: tile t -> (batch, m-tile, n-tile) with n fastest, so the CTAs that
  // run at the same time share rows of A (L2 hits) while B tiles differ.
  auto tile_coords = [&](int64_t t, int* m0, int* n0, int* bz) {
    *n0 = (int)(t % tiles_n) * BN;
    *m0 = (int)((t / tiles_n) % tiles_m) * BM;
    *bz = (int)(t / ((int64_t)tiles_n * tiles_m));
  };

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int64_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        int m0, n0, bz;
        tile_coords(t, &m0, &n0, &bz);
        const int za = a.a_batched ? bz : 0, zb = a.b_batched ? bz : 0;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(&empty[s], ph ^ 1, 1, a.dev_status, abort_flag);
          if (!ok) break;
          uint8_t* st = smem + s * STAGE;
          mbar_expect_tx(&full[s], RAW);
          tma_load_3d(st, &tmA, kb * BK, m0, za, &full[s]);
          tma_load_3d(st + A_BYTES, &tmB, kb * BK, n0, zb, &full[s]);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t it = 0, cc = 0;
      bool ok = true;
      for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int c = 0; c < num_chunks && ok; ++c, ++cc) {
          const uint32_t buf = cc & 1;
          ok = mbar_wait(&acc_empty[buf], ((cc >> 1) & 1) ^ 1, 5, a.dev_status, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + buf * BN;
          uint32_t accumulate = 0;
          const int kb_end = min(num_kb, (c + 1) * chunk_kb);
          for (int kb = c * chunk_kb; kb < kb_end; ++kb, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            ok = mbar_wait(SPLIT == 3 ? &ready[s] : &full[s], ph, 2, a.dev_status, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * STAGE);
            const uint32_t sb = sa + A_BYTES;
#pragma unroll
            for (int ks = 0; ks < BK / UMMA_K; ++ks) {
              const uint32_t koff = ks * UMMA_K * 4;
              const uint64_t a_hi = make_desc(sa + koff), b_hi = make_desc(sb + koff);
              if (SPLIT == 3) {
                const uint64_t a_lo = make_desc(sa + RAW + koff), b_lo = make_desc(sb + RAW + koff);
                umma_tf32(tmem_d, a_lo, b_hi, IDESC, accumulate);
                umma_tf32(tmem_d, a_hi, b_lo, IDESC, 1);
                umma_tf32(tmem_d, a_hi, b_hi, IDESC, 1);
              } else {
                umma_tf32(tmem_d, a_hi, b_hi, IDESC, accumulate);
              }
              accumulate = 1;
            }
            umma_commit(&empty[s]);  // frees the stage once the MMAs above have read it
          }
          if (ok) umma_commit(&acc_full[buf]);
        }
      }
    }
  } else if (warp < DRAIN_WARP0) {
    // ------------------------------------------------ 3xTF32 split (exists only when SPLIT == 3)
    const int tt = threadIdx.x - 64;  // 0..127
    uint32_t it = 0;
    bool ok = true;
    for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        ok = mbar_wait(&full[s], ph, 3, a.dev_status, abort_flag);
        if (!ok) break;
        float4* hi = reinterpret_cast<float4*>(smem + s * STAGE);
        float4* lo = reinterpret_cast<float4*>(smem + s * STAGE + RAW);
#pragma unroll 4
        for (int i = tt; i < RAW / 16; i += 128) {
          // kind::tf32 reads an fp32 word by dropping its 13 low mantissa bits (truncation, measured),
          // so the raw tile already IS the hi operand; only lo = v - trunc(v) has to be written.
          const float4 v = hi[i];
          float4 l;
          l.x = tf32_lo(v.x); l.y = tf32_lo(v.y);
          l.z = tf32_lo(v.z); l.w = tf32_lo(v.w);
          lo[i] = l;
        }
        // make the generic-proxy writes visible to the tensor core (async proxy)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(&ready[s]);
      }
    }
  } else {
    // ------------------------------------------------ drain + epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    constexpr int HALF = BN / 2;                       // columns this warp drains
    const int col0 = ((warp - DRAIN_WARP0) >> 2) * HALF;
    const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
    uint32_t cc = 0;
    bool ok = true;
    for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      int m0, n0, bz;
      tile_coords(t, &m0, &n0, &bz);
      const int row = m0 + q * 32 + lane;
      float* crow = a.C + (int64_t)bz * a.stride_c + (int64_t)row * a.ldc;
      const float bias_m = (has_bias && a.bias_on_m && row < a.M) ? __ldg(a.bias + row) : 0.f;

      auto store32 = [&](const float* v, int c0) {
        const int nb = n0 + c0;
        if (row >= a.M || nb >= a.N) return;
        if (a.c_vec && nb + 32 <= a.N) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 b4 = make_float4(bias_m, bias_m, bias_m, bias_m);
            if (has_bias && !a.bias_on_m) b4 = __ldg(reinterpret_cast<const float4*>(a.bias + nb + j));
            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            float4* dst = reinterpret_cast<float4*>(crow + nb + j);
            if (a.accumulate) {
              const float4 old = *dst;
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            o.x = apply_epilogue_rt(a.epi, o.x, b4.x);
            o.y = apply_epilogue_rt(a.epi, o.y, b4.y);
            o.z = apply_epilogue_rt(a.epi, o.z, b4.z);
            o.w = apply_epilogue_rt(a.epi, o.w, b4.w);
            *dst = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int n = nb + j;
            if (n < a.N) {
              float o = v[j];
              if (a.accumulate) o += crow[n];
              const float bb = has_bias ? (a.bias_on_m ? bias_m : __ldg(a.bias + n)) : 0.f;
              crow[n] = apply_epilogue_rt(a.epi, o, bb);
            }
          }
        }
      };

      if (CHUNKED) {
        constexpr int G = CHUNKED ? HALF / 32 : 1;
        float acc[G][32];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
          for (int j = 0; j < 32; ++j) acc[g][j] = 0.f;
        for (int c = 0; c < num_chunks; ++c, ++cc) {
          const uint32_t buf = cc & 1;
          ok = mbar_wait(&acc_full[buf], (cc >> 1) & 1, 4, a.dev_status, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int g = 0; g < G; ++g) {
            float v[32];
            tmem_ld32(tmem_base + buf * BN + lane_base + col0 + g * 32, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[g][j] += v[j];
          }
          tc_fence_before();
          mbar_arrive(&acc_empty[buf]);  // the MMA warp may overwrite this accumulator
        }
        if (!ok) break;
#pragma unroll
        for (int g = 0; g < G; ++g) store32(acc[g], col0 + g * 32);
      } else {
        const uint32_t buf = cc & 1;
        ok = mbar_wait(&acc_full[buf], (cc >> 1) & 1, 4, a.dev_status, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c0 = col0; c0 < col0 + HALF; c0 += 32) {
          float v[32];
          tmem_ld32(tmem_base + buf * BN + lane_base + c0, v);
          store32(v, c0);
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[buf]);
        ++cc;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------- kernel (TS)
// Same pipeline with the A operand staged in TENSOR MEMORY instead of shared memory (3xTF32 only).
// Shared-memory bandwidth, not the tensor pipe, bounds the all-shared-memory kernel: per k-block
// the tensor core re-reads both operands for each of the three MMAs.  Here the split warps write
// A's hi and lo halves into TMEM columns (tcgen05.st, lane = row) and the MMAs read A from there,
// so shared memory only carries B: its traffic per k-block drops from 192 KB to 128 KB (BN = 128)
// and a stage shrinks to 48 KB (A raw + B raw + B lo), which doubles the pipeline depth.
// TMEM columns: [0, 128) and [128, 256) two accumulators, [256, 512) ring of 4 x (A hi: 32, A lo: 32).
//
// Three rings in shared memory plus one in TMEM, each as deep as its buffer's life needs:
//   raw A     4 x 16 KB   TMA load -> read by the split (~1600 cycles)
//   raw B     6 x BN*128  TMA load -> last MMA that reads it as "B hi" (~4000 cycles)
//   B lo      4 x BN*128  written by the split -> last MMA (~2400 cycles)
//   A hi/lo   4 x 64 TMEM columns, same life and same slot index as B lo ("processed" slot)
// 224 KB at BN = 128.  One ring of whole stages (A raw + B raw + B lo = 48 KB) fits only four
// times.
//
// Every ring has an EVEN number of slots.  Even and odd k-blocks are handled by different warps
// (split sets, MMA issuers) that can drift apart by more than a ring; with an even ring a slot
// always belongs to the same set, which therefore sees its barrier phases one by one.  With an
// odd ring a set could test a parity that the other set's phase has not yet flipped and take a
// stale "complete" for its own.
constexpr int kTsASlots = 4;
constexpr int kTsPSlots = 4;      // processed slots: A hi/lo in TMEM + B lo in shared memory
constexpr int kTsBarrierBytes = 512;
constexpr int kTsSmemLimit = 227 * 1024;
__host__ __device__ constexpr int ts_b_bytes(int bn) { return bn * BK * 4; }
__host__ __device__ constexpr int ts_b_slots(int bn) {
  const int n = (kTsSmemLimit - kTsBarrierBytes - 1024 - kTsASlots * BM * BK * 4 - kTsPSlots * ts_b_bytes(bn)) /
                ts_b_bytes(bn);
  return n >= 8 ? 8 : (n & ~1);
}
__host__ __device__ constexpr int ts_smem_bytes(int bn) {
  return kTsASlots * BM * BK * 4 + (ts_b_slots(bn) + kTsPSlots) * ts_b_bytes(bn) + kTsBarrierBytes + 1024;
}

// Warps: 0 = TMA, 1-2 = MMA issuers, 3-10 = split (two sets of four that alternate k-blocks, so one
// set's shared-load / tcgen05.st latencies overlap the other set's work), 11-18 = drain/epilogue.
//
// Two MMA issuers: measured on B200, a thread that has just issued tcgen05.mma instructions pays
// about 230 cycles for its next mbarrier wait (and ~100 for any other instruction) while the tensor
// pipe holds at most one or two MMAs in its queue, so a single issuer that waits once per k-block
// leaves the pipe idle a quarter of the time (1030 cycles per 12 MMAs of 128x128x8 instead of 768).
// Two issuers in different warps that alternate k-blocks hide each other's waits (769 cycles per
// 12 MMAs in the same microbenchmark).  Their MMAs reach the pipe in no fixed order, so each issuer
// owns one TMEM accumulator: the additions inside an accumulator keep their order and the result is
// the same bits on every run.  An accumulator is drained into fp32 registers every kTsChunkKB of its
// issuer's k-blocks (the tensor core's own fp32 accumulation truncates); the second issuer's chunk
// boundaries are shifted by half a chunk so that while one issuer waits for its drain the other
// keeps the tensor pipe busy.
constexpr int kTsThreads = 608;

template <int BN, int CHUNK>
__global__ void __launch_bounds__(kTsThreads, 1)
contraction_ts_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, TcArgs a) {
  constexpr int A_SLOTS = kTsASlots, P_SLOTS = kTsPSlots, B_SLOTS = ts_b_slots(BN);
  constexpr int A_BYTES = BM * BK * 4;
  constexpr int B_BYTES = BN * BK * 4;
  constexpr int B_RING = A_SLOTS * A_BYTES;          // byte offset of the raw B ring
  constexpr int LO_RING = B_RING + B_SLOTS * B_BYTES;  // byte offset of the B lo ring
  constexpr uint32_t A_RING = 256;         // first TMEM column of the A ring
  constexpr uint32_t ACC_STRIDE = 128;     // TMEM columns between the two accumulators
  static_assert(BN <= 128 && BN % 16 == 0, "two accumulators and the A ring share 512 TMEM columns");
  constexpr uint32_t IDESC = make_idesc(BN);
  constexpr int SPLIT_WARP0 = 3;  // after the TMA warp and the two MMA issuer warps
  constexpr int SPLIT_WARPS = 8;
  constexpr int DRAIN_WARP0 = SPLIT_WARP0 + SPLIT_WARPS;  // 8 warps from here cover every TMEM lane quarter twice
  constexpr int FIRST = ((BN / 2 + 15) / 16) * 16;         // columns of the first drain warp of a quarter
  constexpr int PIECES = FIRST / 16;
  constexpr uint32_t TMEM_COLS = 512;
  static_assert(B_SLOTS >= 2 && B_SLOTS <= 8 && A_SLOTS <= 4 && P_SLOTS == 4, "barrier arrays / TMEM ring sizes");
  static_assert(A_SLOTS % 2 == 0 && B_SLOTS % 2 == 0 && P_SLOTS % 2 == 0, "a slot must stay with one set");
  static_assert(B_BYTES % 1024 == 0, "128-byte swizzle atoms must stay 1024-byte aligned");
  static_assert((kTsChunkKB & (kTsChunkKB - 1)) == 0 && (kPairChunkKB & (kPairChunkKB - 1)) == 0, "chunk lengths are powers of two");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_a = reinterpret_cast<uint64_t*>(smem + LO_RING + P_SLOTS * B_BYTES);  // [4]
  uint64_t* empty_a = full_a + 4;        // [4] raw A slot read by the split warps
  uint64_t* pfree = empty_a + 4;         // [4] processed slot (A hi/lo, B lo) read by its MMAs
  uint64_t* ready = pfree + 4;           // [4] processed slot filled
  uint64_t* full_b = ready + 4;          // [8]
  uint64_t* empty_b = full_b + 8;        // [8] raw B slot read by its MMAs
  uint64_t* acc_full = empty_b + 8;      // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // split-K: every split runs the same number of k-blocks; those past the end of K read zeros (TMA fill)
  const int num_kb = a.ksplit_kb > 0 ? a.ksplit_kb : (a.K + BK - 1) / BK;
  const int tiles_n = (a.N + BN - 1) / BN, tiles_m = (a.M + BM - 1) / BM;
  const int64_t num_tiles = (int64_t)tiles_n * tiles_m * a.batch;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 4; ++s) {
      mbar_init(&full_a[s], 1);
      mbar_init(&empty_a[s], 4);  // one elected arrival per warp of the split set
      mbar_init(&pfree[s], 1);
      mbar_init(&ready[s], 4);
    }
    for (int s = 0; s < 8; ++s) {
      mbar_init(&full_b[s], 1);
      mbar_init(&empty_b[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 256);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_sync();  // nothing above touches global memory
  const uint32_t tmem_base = *tmem_slot;
  const bool second_half = warp >= DRAIN_WARP0 + 4;  // drain warps: which column range of the quarter

  // Issuer i takes the k-blocks whose running number (counted over all tiles of this CTA) has
  // parity i.  Within a tile that starts at running number it0 these are kb = first + 2j,
  // j = 0 .. count-1; own k-block j closes a chunk when (j + 1 + skew) % kTsChunkKB == 0 (skew 0 for
  // issuer 0, kTsChunkKB / 2 for issuer 1) or when it is the issuer's last k-block of the tile.
  auto own_first = [](uint32_t it0, int i) { return (int)((it0 ^ (uint32_t)i) & 1u); };
  auto own_count = [&](uint32_t it0, int i) {
    const int f = own_first(it0, i);
    return num_kb > f ? (num_kb - f + 1) / 2 : 0;
  };
  // chunk length CHUNK: kTsChunkKB, or 1 for the strict-accumulation tiles (a compile-time constant: the test sits
  // on the single issuing thread's critical path)
  auto closes_chunk = [](int j, int count, int i) {
    return j == count - 1 || (j + 1 + (i ? CHUNK / 2 : 0)) % CHUNK == 0;
  };

  // Static persistent schedule: tile t -> (batch, m-tile, n-tile) with n fastest, so the CTAs that
  // run at the same time share rows of A (L2 hits) while B tiles differ.
  auto tile_coords = [&](int64_t t, int* m0, int* n0, int* bz) {
    *n0 = (int)(t % tiles_n) * BN;
    *m0 = (int)((t / tiles_n) % tiles_m) * BM;
    *bz = (int)(t / ((int64_t)tiles_n * tiles_m));
  };

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int64_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        int m0, n0, bz;
        tile_coords(t, &m0, &n0, &bz);
        const int za = a.a_batched ? bz : 0, zb = a.b_batched ? bz : 0;
        const int k0 = a.ksplit_kb > 0 ? bz * a.ksplit_kb * BK : 0;  // first k of this split
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int sa = it % A_SLOTS, sb = it % B_SLOTS;
          ok = mbar_wait(&empty_a[sa], ((it / A_SLOTS) & 1) ^ 1, 1, a.dev_status, abort_flag);
          if (!ok) break;
          mbar_expect_tx(&full_a[sa], A_BYTES);
          tma_load_3d(smem + sa * A_BYTES, &tmA, k0 + kb * BK, m0, za, &full_a[sa]);
          ok = mbar_wait(&empty_b[sb], ((it / B_SLOTS) & 1) ^ 1, 1, a.dev_status, abort_flag);
          if (!ok) break;
          mbar_expect_tx(&full_b[sb], B_BYTES);
          tma_load_3d(smem + B_RING + sb * B_BYTES, &tmB, k0 + kb * BK, n0, zb, &full_b[sb]);
        }
        if (!ok) break;
      }
    }
  } else if (warp < SPLIT_WARP0) {
    // ------------------------------------------------ MMA issuers
    const int issuer = warp - 1;
    if (lane == 0) {
      uint32_t it0 = 0, cc = 0;  // running k-block number at the start of the tile; chunks of this issuer
      bool ok = true;
      const uint32_t tmem_d = tmem_base + issuer * ACC_STRIDE;
      for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, it0 += (uint32_t)num_kb) {
        const int first = own_first(it0, issuer), count = own_count(it0, issuer);
        bool opens = true;
        for (int j = 0; j < count; ++j) {
          const uint32_t it = it0 + (uint32_t)(first + 2 * j);
          uint32_t accumulate = 1;
          if (opens) {  // the drain warps have read the previous chunk out of this accumulator
            ok = mbar_wait(&acc_empty[issuer], (cc & 1) ^ 1, 5, a.dev_status, abort_flag);
            if (!ok) break;
            accumulate = 0;
            opens = false;
          }
          const int s = it % B_SLOTS, sp = it % P_SLOTS;
          ok = mbar_wait(&ready[sp], (it / P_SLOTS) & 1, 2, a.dev_status, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sb = smem_u32(smem + B_RING + s * B_BYTES);
          const uint32_t sl = smem_u32(smem + LO_RING + sp * B_BYTES);
          const uint32_t ta_hi = tmem_base + A_RING + sp * 64, ta_lo = ta_hi + 32;
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            const uint32_t koff = ks * UMMA_K * 4;
            const uint64_t b_hi = make_desc(sb + koff), b_lo = make_desc(sl + koff);
            umma_tf32_ts(tmem_d, ta_lo + ks * UMMA_K, b_hi, IDESC, accumulate);
            umma_tf32_ts(tmem_d, ta_hi + ks * UMMA_K, b_lo, IDESC, 1);
            umma_tf32_ts(tmem_d, ta_hi + ks * UMMA_K, b_hi, IDESC, 1);
            accumulate = 1;
          }
          umma_commit(&empty_b[s]);  // both fire once the MMAs above have read their operands
          umma_commit(&pfree[sp]);
          if (closes_chunk(j, count, issuer)) {
            umma_commit(&acc_full[issuer]);
            ++cc;
            opens = true;
          }
        }
      }
    }
  } else if (warp < DRAIN_WARP0) {
    // ------------------------------------------------ 3xTF32 split: A -> TMEM, B lo -> smem
    const int set = (warp - SPLIT_WARP0) >> 2;             // which of the two alternating sets
    const int tt = (threadIdx.x - SPLIT_WARP0 * 32) & 127;  // 0..127 within the set
    const int arow = (warp & 3) * 32 + lane;          // TMEM lane quarter of this warp
    uint32_t it = 0;
    bool ok = true;
    for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        if ((int)(it & 1) != set) continue;
        const int sa = it % A_SLOTS, sp = it % P_SLOTS, s = it % B_SLOTS;
        ok = mbar_wait(&pfree[sp], ((it / P_SLOTS) & 1) ^ 1, 6, a.dev_status, abort_flag) &&
             mbar_wait(&full_a[sa], (it / A_SLOTS) & 1, 3, a.dev_status, abort_flag);
        if (!ok) break;
        tc_fence_after();
        // A: this thread owns row `arow` of the 128 x 32 tile (TMEM lane = row).  The tile sits in
        // shared memory with the 128-byte swizzle: 16-byte chunk c of row r is stored at c ^ (r & 7).
        {
          const float4* arow_p = reinterpret_cast<const float4*>(smem + sa * A_BYTES + arow * 128);
          float hi[32], lo[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 v = arow_p[c ^ (arow & 7)];
            hi[4 * c + 0] = v.x; hi[4 * c + 1] = v.y; hi[4 * c + 2] = v.z; hi[4 * c + 3] = v.w;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) lo[j] = tf32_lo(hi[j]);
          const uint32_t ta = tmem_base + A_RING + sp * 64 + ((uint32_t)(arow & ~31) << 16);
          tmem_st32(ta, hi);        // the tensor core truncates the fp32 words itself
          tmem_st32(ta + 32, lo);
          // Free the raw A slot only once the stores have consumed the registers the shared-memory
          // loads filled.  Arriving right after the loads were issued was measured to be too early:
          // with two slots the refill landed while loads were still queued (wrong results).
          tmem_wait_st();
          mbar_arrive_warp(&empty_a[sa]);
        }
        ok = mbar_wait(&full_b[s], (it / B_SLOTS) & 1, 7, a.dev_status, abort_flag);
        if (!ok) break;
        // B: lo = tf32(v - trunc(v)) into the second buffer, same (swizzled) layout; raw B is hi.
        {
          const float4* bh = reinterpret_cast<const float4*>(smem + B_RING + s * B_BYTES);
          float4* bl = reinterpret_cast<float4*>(smem + LO_RING + sp * B_BYTES);
#pragma unroll 4
          for (int i = tt; i < B_BYTES / 16; i += 128) {
            const float4 v = bh[i];
            float4 l;
            l.x = tf32_lo(v.x); l.y = tf32_lo(v.y);
            l.z = tf32_lo(v.z); l.w = tf32_lo(v.w);
            bl[i] = l;
          }
        }
        tmem_wait_st();
        tc_fence_before();
        // make the generic-proxy writes visible to the tensor core (async proxy)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive_warp(&ready[sp]);
      }
    }
  } else {
    // ------------------------------------------------ drain + epilogue
    // Two warps per TMEM lane quarter: the first takes columns [0, FIRST), the second [FIRST, BN),
    // both in pieces of 16 columns (FIRST is a multiple of 16, so BN = 112 splits into 64 + 48).
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const int col0 = second_half ? FIRST : 0;
    const int mycols = second_half ? BN - FIRST : FIRST;
    const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
    uint32_t it0 = 0, dc[2] = {0, 0};  // running k-block number of the tile; chunks drained per issuer
    bool ok = true;
    for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, it0 += (uint32_t)num_kb) {
      int m0, n0, bz;
      tile_coords(t, &m0, &n0, &bz);
      const int row = m0 + q * 32 + lane;
      float* crow = a.C + (int64_t)bz * a.stride_c + (int64_t)row * a.ldc;
      const float bias_m = (has_bias && a.bias_on_m && row < a.M) ? __ldg(a.bias + row) : 0.f;
      // Per-column bias of this warp's columns, fetched now: lane l keeps columns col0 + 2l and
      // col0 + 2l + 1 and the epilogue gets them by shuffle.  Loading them in the epilogue, between
      // the output stores, serialised sixteen global-load latencies per thread (the compiler may not
      // move a load across a store that could alias it): ~9000 cycles per tile, measured, during
      // which the drain warps could not serve the next tile's first chunks.
      float2 bias_n = make_float2(0.f, 0.f);
      if (has_bias && !a.bias_on_m && 2 * lane < mycols) {
        const int c = n0 + col0 + 2 * lane;
        if (c < a.N) bias_n.x = __ldg(a.bias + c);
        if (c + 1 < a.N) bias_n.y = __ldg(a.bias + c + 1);
      }

      auto store16 = [&](const float* v, int c0) {
        const int nb = n0 + c0;
        float bb[16];  // bias of columns c0 .. c0 + 15 (every lane takes part in the shuffles)
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const int src = (c0 - col0 + j) >> 1;
          bb[j] = a.bias_on_m ? bias_m : __shfl_sync(0xffffffffu, bias_n.x, src);
          bb[j + 1] = a.bias_on_m ? bias_m : __shfl_sync(0xffffffffu, bias_n.y, src);
        }
        if (row >= a.M || nb >= a.N) return;
        if (a.c_vec && nb + 16 <= a.N) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 b4 = make_float4(bb[j], bb[j + 1], bb[j + 2], bb[j + 3]);
            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            float4* dst = reinterpret_cast<float4*>(crow + nb + j);
            if (a.accumulate) {
              const float4 old = *dst;
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            o.x = apply_epilogue_rt(a.epi, o.x, b4.x);
            o.y = apply_epilogue_rt(a.epi, o.y, b4.y);
            o.z = apply_epilogue_rt(a.epi, o.z, b4.z);
            o.w = apply_epilogue_rt(a.epi, o.w, b4.w);
            *dst = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int n = nb + j;
            if (n < a.N) {
              float o = v[j];
              if (a.accumulate) o += crow[n];
              crow[n] = apply_epilogue_rt(a.epi, o, bb[j]);
            }
          }
        }
      };

      float acc[PIECES][16];
#pragma unroll
      for (int g = 0; g < PIECES; ++g)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[g][j] = 0.f;
      // Chunks of both issuers in the order of the k-block that closes them (the same order on
      // every run; the two can never tie because their k-blocks differ in parity).
      const int first0 = own_first(it0, 0), first1 = own_first(it0, 1);
      const int count0 = own_count(it0, 0), count1 = own_count(it0, 1);
      int j0 = 0, j1 = 0;  // own k-block index from which the next chunk of each issuer is searched
      while (j0 < count0 || j1 < count1) {
        int e0 = j0, e1 = j1;  // own index that closes the next chunk
        while (e0 < count0 && !closes_chunk(e0, count0, 0)) ++e0;
        while (e1 < count1 && !closes_chunk(e1, count1, 1)) ++e1;
        const bool take1 = j0 >= count0 || (j1 < count1 && first1 + 2 * e1 < first0 + 2 * e0);
        const int i = take1 ? 1 : 0;
        if (take1) j1 = e1 + 1; else j0 = e0 + 1;
        ok = mbar_wait(&acc_full[i], dc[i] & 1, 4, a.dev_status, abort_flag);
        if (!ok) break;
        ++dc[i];
        tc_fence_after();
#pragma unroll
        for (int g = 0; g < PIECES; ++g) {
          if (g * 16 < mycols) {  // the same for the whole warp
            float v[16];
            tmem_ld16(tmem_base + i * ACC_STRIDE + lane_base + col0 + g * 16, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[g][j] += v[j];
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[i]);  // issuer i may overwrite its accumulator
      }
      if (!ok) break;
#pragma unroll
      for (int g = 0; g < PIECES; ++g)
        if (g * 16 < mycols) store16(acc[g], col0 + g * 16);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------- kernel (TS, CTA pair)
// The same kernel on a CTA PAIR (cluster of two, tcgen05 cta_group::2): one 256 x 128 output tile per
// pair.  Each CTA loads and splits its own 128 rows of A into its own tensor memory and HALF of the B
// tile (64 rows) into its own shared memory; the leader's MMAs (M = 256) read both halves, so per
// k-block a CTA moves 80 KB through shared memory instead of 128 KB (TMA 16 + 8 in, split 24 out +
// 8 in, MMA operand reads 24), which is what bounds the single-CTA kernel.  Barriers: everything a CTA's
// own warps produce and consume stays local; the peer's split and drain warps arrive on the LEADER's
// `ready` / `acc_empty`, and the leader's commits arrive on `empty_b`, `pfree`, `acc_full` in both CTAs.
// Epilogue: a thread owns a row of the output tile, so storing straight from registers makes every
// warp store touch 32 different rows (32 sectors per instruction): ~7500 cycles per tile, measured,
// during which the drain warps cannot serve the next tile's first chunks.  The CTA's 128 x 128 tile
// is therefore staged in shared memory (128-byte swizzle, conflict-free 128-bit stores) and written
// by four tiled TMA stores that clip at the tensor's edge; `accumulate` and unaligned outputs keep
// the direct path.
constexpr int kPairBN = 128;
constexpr int kPairBSlots = 8;
constexpr int kPairOutBytes = BM * kPairBN * 4;  // staging tile of the epilogue
__host__ __device__ constexpr int ts_pair_rings_bytes() {
  return kTsASlots * BM * BK * 4 + (kPairBSlots + kTsPSlots) * (kPairBN / 2) * BK * 4 + kTsBarrierBytes;
}
__host__ __device__ constexpr int ts_pair_out_offset() { return (ts_pair_rings_bytes() + 1023) / 1024 * 1024; }
__host__ __device__ constexpr int ts_pair_smem_bytes() { return ts_pair_out_offset() + kPairOutBytes + 1024; }
static_assert(ts_pair_smem_bytes() <= kTsSmemLimit, "rings + output staging tile exceed shared memory");

// TAIL: the launch ends with split tail units (a compile-time switch: carried as run-time state the unit
// bookkeeping cost the kernel 2 % on launches that have no tail).
template <int CHUNK, bool TAIL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kTsThreads, 1)
contraction_ts_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                           const __grid_constant__ CUtensorMap tmB,
                           const __grid_constant__ CUtensorMap tmC,
                           const __grid_constant__ CUtensorMap tmP, TcArgs a) {
  constexpr int BN = kPairBN;
  constexpr int A_SLOTS = kTsASlots, P_SLOTS = kTsPSlots, B_SLOTS = kPairBSlots;
  constexpr int A_BYTES = BM * BK * 4;
  constexpr int B_BYTES = (BN / 2) * BK * 4;  // this CTA's half of the B tile
  constexpr int B_RING = A_SLOTS * A_BYTES;          // byte offset of the raw B ring
  constexpr int LO_RING = B_RING + B_SLOTS * B_BYTES;  // byte offset of the B lo ring
  constexpr uint32_t A_RING = 256;         // first TMEM column of the A ring
  constexpr uint32_t ACC_STRIDE = 128;     // TMEM columns between the two accumulators
  static_assert(BN <= 128 && BN % 16 == 0, "two accumulators and the A ring share 512 TMEM columns");
  constexpr uint32_t IDESC = make_idesc_tf32(2 * BM, BN);  // M = 256 over the pair
  constexpr int SPLIT_WARP0 = 3;  // after the TMA warp and the two MMA issuer warps
  constexpr int SPLIT_WARPS = 8;
  constexpr int DRAIN_WARP0 = SPLIT_WARP0 + SPLIT_WARPS;  // 8 warps from here cover every TMEM lane quarter twice
  constexpr int FIRST = ((BN / 2 + 15) / 16) * 16;         // columns of the first drain warp of a quarter
  constexpr int PIECES = FIRST / 16;
  constexpr uint32_t TMEM_COLS = 512;
  static_assert(B_SLOTS >= 2 && B_SLOTS <= 8 && A_SLOTS <= 4 && P_SLOTS == 4, "barrier arrays / TMEM ring sizes");
  static_assert(A_SLOTS % 2 == 0 && B_SLOTS % 2 == 0 && P_SLOTS % 2 == 0, "a slot must stay with one set");
  static_assert(B_BYTES % 1024 == 0, "128-byte swizzle atoms must stay 1024-byte aligned");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_a = reinterpret_cast<uint64_t*>(smem + LO_RING + P_SLOTS * B_BYTES);  // [4]
  uint64_t* empty_a = full_a + 4;        // [4] raw A slot read by the split warps
  uint64_t* pfree = empty_a + 4;         // [4] processed slot (A hi/lo, B lo) read by its MMAs
  uint64_t* ready = pfree + 4;           // [4] processed slot filled
  uint64_t* full_b = ready + 4;          // [8]
  uint64_t* empty_b = full_b + 8;        // [8] raw B slot read by its MMAs
  uint64_t* acc_full = empty_b + 8;      // [2]
  uint64_t* acc_empty = acc_full + 2;    // [2]
  uint64_t* out_ready = acc_empty + 2;   // staging tile written by the eight drain warps
  uint64_t* out_free = out_ready + 1;    // staging tile read by the TMA stores of the previous tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(out_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: leader (issues the MMAs), 1: peer
  const int64_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  // split-K: every split runs the same number of k-blocks; those past the end of K read zeros (TMA fill)
  const int num_kb = a.ksplit_kb > 0 ? a.ksplit_kb : (a.K + BK - 1) / BK;
  const int tiles_n = (a.N + BN - 1) / BN, tiles_m = (a.M + 2 * BM - 1) / (2 * BM);
  // Work units, one per pair at a time.  Units [0, main_units) are whole tiles (in a split-K launch: (tile, split)
  // pairs, the split being the "batch" index).  A launch whose tiles do not fill its last wave ends with a TAIL:
  // the last tail_tiles tiles have their reduction split tail_S ways, unit main_units + s * tail_tiles + j being
  // split s of tail tile j.  A tail unit runs tail_kb k-blocks and leaves a raw partial tile in scratch memory
  // (tile number = its index in the tail, through the map tmP); a second kernel adds the splits and applies the
  // epilogue.  256 tiles on 74 pairs are then 3 rounds of whole tiles and one round of half-length units
  // instead of 4 rounds.
  const int64_t all_tiles = (int64_t)tiles_n * tiles_m * a.batch;  // tiles of 256 x BN
  const int64_t main_units = TAIL ? all_tiles - a.tail_tiles : all_tiles;
  const int64_t num_tiles = main_units + (TAIL ? (int64_t)a.tail_tiles * a.tail_S : 0);  // units
  auto unit_kb = [&](int64_t t) { return !TAIL || t < main_units ? num_kb : a.tail_kb; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < 4; ++s) {
      mbar_init(&full_a[s], 1);
      mbar_init(&empty_a[s], 4);  // one elected arrival per warp of the split set
      mbar_init(&pfree[s], 1);
      mbar_init(&ready[s], 8);    // used in the leader only: four split warps of each CTA
    }
    for (int s = 0; s < 8; ++s) {
      mbar_init(&full_b[s], 1);
      mbar_init(&empty_b[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 16);  // used in the leader only: eight drain warps of each CTA
    }
    mbar_init(out_ready, 8);
    mbar_init(out_free, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);  // collective over the pair
  tc_fence_before();
  cluster_sync_all();  // both CTAs' barriers exist before anything arrives on them from the other CTA
  tc_fence_after();
  pdl_sync();  // nothing above touches global memory
  const uint32_t tmem_base = *tmem_slot;
  const bool second_half = warp >= DRAIN_WARP0 + 4;  // drain warps: which column range of the quarter

  // Issuer i takes the k-blocks whose running number (counted over all tiles of this CTA) has
  // parity i.  Within a tile that starts at running number it0 these are kb = first + 2j,
  // j = 0 .. count-1; own k-block j closes a chunk when (j + 1 + skew) % kPairChunkKB == 0 (skew 0 for
  // issuer 0, kPairChunkKB / 2 for issuer 1) or when it is the issuer's last k-block of the tile.
  auto own_first = [](uint32_t it0, int i) { return (int)((it0 ^ (uint32_t)i) & 1u); };
  auto own_count = [&](uint32_t it0, int i, int nkb) {
    const int f = own_first(it0, i);
    return nkb > f ? (nkb - f + 1) / 2 : 0;
  };
  // chunk length CHUNK: kPairChunkKB, or 1 for the strict-accumulation tiles (a compile-time constant: the test
  // sits on the single issuing thread's critical path)
  auto closes_chunk = [](int j, int count, int i) {
    return j == count - 1 || (j + 1 + (i ? CHUNK / 2 : 0)) % CHUNK == 0;
  };

  // Static persistent schedule: tile t -> (batch, m-tile, n-tile) with n fastest, so the CTAs that
  // run at the same time share rows of A (L2 hits) while B tiles differ.
  // slot: -1 for a unit that writes the output, else the number of the partial tile a tail unit writes;
  // k0: first k of the unit
  auto tile_coords = [&](int64_t t, int* m0, int* n0, int* bz, int* k0, int* slot) {
    int64_t tile = t;
    *slot = -1;
    *k0 = 0;
    if (TAIL && t >= main_units) {
      const int64_t r = t - main_units;
      tile = main_units + r % a.tail_tiles;
      *k0 = (int)(r / a.tail_tiles) * a.tail_kb * BK;
      *slot = (int)r;
    }
    *n0 = (int)(tile % tiles_n) * BN;
    *m0 = (int)((tile / tiles_n) % tiles_m) * (2 * BM) + (int)rank * BM;  // this CTA's 128 rows
    *bz = (int)(tile / ((int64_t)tiles_n * tiles_m));
    if (*slot < 0 && a.ksplit_kb > 0) *k0 = *bz * a.ksplit_kb * BK;  // split-K launch: the batch index is the split
  };

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      for (int64_t t = pair; t < num_tiles; t += num_pairs) {
        int m0, n0, bz, k0, slot;
        tile_coords(t, &m0, &n0, &bz, &k0, &slot);
        const int za = a.a_batched ? bz : 0, zb = a.b_batched ? bz : 0;
        const int nkb = unit_kb(t);
        bool ok = true;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int sa = it % A_SLOTS, sb = it % B_SLOTS;
          ok = mbar_wait(&empty_a[sa], ((it / A_SLOTS) & 1) ^ 1, 1, a.dev_status, abort_flag);
          if (!ok) break;
          mbar_expect_tx(&full_a[sa], A_BYTES);
          tma_load_3d(smem + sa * A_BYTES, &tmA, k0 + kb * BK, m0, za, &full_a[sa]);
          ok = mbar_wait(&empty_b[sb], ((it / B_SLOTS) & 1) ^ 1, 1, a.dev_status, abort_flag);
          if (!ok) break;
          mbar_expect_tx(&full_b[sb], B_BYTES);
          tma_load_3d(smem + B_RING + sb * B_BYTES, &tmB, k0 + kb * BK, n0 + (int)rank * (BN / 2), zb, &full_b[sb]);
        }
        if (!ok) break;
      }
    }
  } else if (warp < SPLIT_WARP0) {
    // ------------------------------------------------ MMA issuers
    const int issuer = warp - 1;
    if (lane == 0 && rank == 0) {  // the leader's two issuers drive both CTAs' tensor cores
      uint32_t it0 = 0, cc = 0;  // running k-block number at the start of the tile; chunks of this issuer
      bool ok = true;
      const uint32_t tmem_d = tmem_base + issuer * ACC_STRIDE;
      int nkb = 0;
      for (int64_t t = pair; t < num_tiles && ok; t += num_pairs, it0 += (uint32_t)nkb) {
        nkb = unit_kb(t);
        const int first = own_first(it0, issuer), count = own_count(it0, issuer, nkb);
        bool opens = true;
        for (int j = 0; j < count; ++j) {
          const uint32_t it = it0 + (uint32_t)(first + 2 * j);
          uint32_t accumulate = 1;
          if (opens) {  // the drain warps have read the previous chunk out of this accumulator
            ok = mbar_wait(&acc_empty[issuer], (cc & 1) ^ 1, 5, a.dev_status, abort_flag);
            if (!ok) break;
            accumulate = 0;
            opens = false;
          }
          const int s = it % B_SLOTS, sp = it % P_SLOTS;
          ok = mbar_wait(&ready[sp], (it / P_SLOTS) & 1, 2, a.dev_status, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sb = smem_u32(smem + B_RING + s * B_BYTES);
          const uint32_t sl = smem_u32(smem + LO_RING + sp * B_BYTES);
          const uint32_t ta_hi = tmem_base + A_RING + sp * 64, ta_lo = ta_hi + 32;
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            const uint32_t koff = ks * UMMA_K * 4;
            const uint64_t b_hi = make_desc(sb + koff), b_lo = make_desc(sl + koff);
            umma_tf32_ts_pair(tmem_d, ta_lo + ks * UMMA_K, b_hi, IDESC, accumulate);
            umma_tf32_ts_pair(tmem_d, ta_hi + ks * UMMA_K, b_lo, IDESC, 1);
            umma_tf32_ts_pair(tmem_d, ta_hi + ks * UMMA_K, b_hi, IDESC, 1);
            accumulate = 1;
          }
          umma_commit_pair(&empty_b[s]);  // both fire, in both CTAs, once the MMAs above have read their operands
          umma_commit_pair(&pfree[sp]);
          if (closes_chunk(j, count, issuer)) {
            umma_commit_pair(&acc_full[issuer]);
            ++cc;
            opens = true;
          }
        }
      }
    }
  } else if (warp < DRAIN_WARP0) {
    // ------------------------------------------------ 3xTF32 split: A -> TMEM, B lo -> smem
    const int set = (warp - SPLIT_WARP0) >> 2;             // which of the two alternating sets
    const int tt = (threadIdx.x - SPLIT_WARP0 * 32) & 127;  // 0..127 within the set
    const int arow = (warp & 3) * 32 + lane;          // TMEM lane quarter of this warp
    uint32_t it = 0;
    bool ok = true;
    for (int64_t t = pair; t < num_tiles && ok; t += num_pairs) {
      const int nkb = unit_kb(t);
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        if ((int)(it & 1) != set) continue;
        const int sa = it % A_SLOTS, sp = it % P_SLOTS, s = it % B_SLOTS;
        ok = mbar_wait(&pfree[sp], ((it / P_SLOTS) & 1) ^ 1, 6, a.dev_status, abort_flag) &&
             mbar_wait(&full_a[sa], (it / A_SLOTS) & 1, 3, a.dev_status, abort_flag);
        if (!ok) break;
        tc_fence_after();
        // A: this thread owns row `arow` of the 128 x 32 tile (TMEM lane = row).  The tile sits in
        // shared memory with the 128-byte swizzle: 16-byte chunk c of row r is stored at c ^ (r & 7).
        {
          const float4* arow_p = reinterpret_cast<const float4*>(smem + sa * A_BYTES + arow * 128);
          float hi[32], lo[32];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const float4 v = arow_p[c ^ (arow & 7)];
            hi[4 * c + 0] = v.x; hi[4 * c + 1] = v.y; hi[4 * c + 2] = v.z; hi[4 * c + 3] = v.w;
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) lo[j] = tf32_lo(hi[j]);
          const uint32_t ta = tmem_base + A_RING + sp * 64 + ((uint32_t)(arow & ~31) << 16);
          tmem_st32(ta, hi);        // the tensor core truncates the fp32 words itself
          tmem_st32(ta + 32, lo);
          // Free the raw A slot only once the stores have consumed the registers the shared-memory
          // loads filled.  Arriving right after the loads were issued was measured to be too early:
          // with two slots the refill landed while loads were still queued (wrong results).
          tmem_wait_st();
          mbar_arrive_warp(&empty_a[sa]);
        }
        ok = mbar_wait(&full_b[s], (it / B_SLOTS) & 1, 7, a.dev_status, abort_flag);
        if (!ok) break;
        // B: lo = tf32(v - trunc(v)) into the second buffer, same (swizzled) layout; raw B is hi.
        {
          const float4* bh = reinterpret_cast<const float4*>(smem + B_RING + s * B_BYTES);
          float4* bl = reinterpret_cast<float4*>(smem + LO_RING + sp * B_BYTES);
#pragma unroll 4
          for (int i = tt; i < B_BYTES / 16; i += 128) {
            const float4 v = bh[i];
            float4 l;
            l.x = tf32_lo(v.x); l.y = tf32_lo(v.y);
            l.z = tf32_lo(v.z); l.w = tf32_lo(v.w);
            bl[i] = l;
          }
        }
        tmem_wait_st();
        tc_fence_before();
        // make the generic-proxy writes visible to the tensor core (async proxy)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive_warp_remote(&ready[sp], 0);  // the leader's barrier counts both CTAs' split warps
      }
    }
  } else {
    // ------------------------------------------------ drain + epilogue
    // Two warps per TMEM lane quarter: the first takes columns [0, FIRST), the second [FIRST, BN),
    // both in pieces of 16 columns (FIRST is a multiple of 16, so BN = 112 splits into 64 + 48).
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const int col0 = second_half ? FIRST : 0;
    const int mycols = second_half ? BN - FIRST : FIRST;
    const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
    uint32_t it0 = 0, dc[2] = {0, 0};  // running k-block number of the tile; chunks drained per issuer
    uint32_t staged = 0;               // tiles that went through the staging tile
    bool ok = true;
    int nkb = 0;
    for (int64_t t = pair; t < num_tiles && ok; t += num_pairs, it0 += (uint32_t)nkb) {
      nkb = unit_kb(t);
      int m0, n0, bz, k0, slot;
      tile_coords(t, &m0, &n0, &bz, &k0, &slot);
      const bool tail = TAIL && slot >= 0;       // raw partial tile to scratch, no epilogue
      const int epi = tail ? (int)TCB200_EPI_NONE : a.epi;
      const int row = m0 + q * 32 + lane;
      float* crow = a.C + (int64_t)bz * a.stride_c + (int64_t)row * a.ldc;
      const float bias_m = (has_bias && a.bias_on_m && row < a.M) ? __ldg(a.bias + row) : 0.f;
      // Per-column bias of this warp's columns, fetched now: lane l keeps columns col0 + 2l and
      // col0 + 2l + 1 and the epilogue gets them by shuffle.  Loading them in the epilogue, between
      // the output stores, serialised sixteen global-load latencies per thread (the compiler may not
      // move a load across a store that could alias it): ~9000 cycles per tile, measured, during
      // which the drain warps could not serve the next tile's first chunks.
      float2 bias_n = make_float2(0.f, 0.f);
      if (has_bias && !tail && !a.bias_on_m && 2 * lane < mycols) {
        const int c = n0 + col0 + 2 * lane;
        if (c < a.N) bias_n.x = __ldg(a.bias + c);
        if (c + 1 < a.N) bias_n.y = __ldg(a.bias + c + 1);
      }

      auto store16 = [&](const float* v, int c0) {
        const int nb = n0 + c0;
        float bb[16];  // bias of columns c0 .. c0 + 15 (every lane takes part in the shuffles)
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const int src = (c0 - col0 + j) >> 1;
          bb[j] = a.bias_on_m ? bias_m : __shfl_sync(0xffffffffu, bias_n.x, src);
          bb[j + 1] = a.bias_on_m ? bias_m : __shfl_sync(0xffffffffu, bias_n.y, src);
        }
        if (row >= a.M || nb >= a.N) return;
        if (a.c_transposed) {   // (only when the staged path is not available: strided 4-byte stores)
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (nb + j < a.N) a.C[(int64_t)bz * a.stride_c + (int64_t)(nb + j) * a.ldc + row] = v[j];
          return;
        }
        if (a.c_vec && nb + 16 <= a.N) {
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 b4 = make_float4(bb[j], bb[j + 1], bb[j + 2], bb[j + 3]);
            float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            float4* dst = reinterpret_cast<float4*>(crow + nb + j);
            if (a.accumulate) {
              const float4 old = *dst;
              o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
            }
            o.x = apply_epilogue_rt(a.epi, o.x, b4.x);
            o.y = apply_epilogue_rt(a.epi, o.y, b4.y);
            o.z = apply_epilogue_rt(a.epi, o.z, b4.z);
            o.w = apply_epilogue_rt(a.epi, o.w, b4.w);
            *dst = o;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int n = nb + j;
            if (n < a.N) {
              float o = v[j];
              if (a.accumulate) o += crow[n];
              crow[n] = apply_epilogue_rt(a.epi, o, bb[j]);
            }
          }
        }
      };

      float acc[PIECES][16];
#pragma unroll
      for (int g = 0; g < PIECES; ++g)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[g][j] = 0.f;
      // Chunks of both issuers in the order of the k-block that closes them (the same order on
      // every run; the two can never tie because their k-blocks differ in parity).
      const int first0 = own_first(it0, 0), first1 = own_first(it0, 1);
      const int count0 = own_count(it0, 0, nkb), count1 = own_count(it0, 1, nkb);
      int j0 = 0, j1 = 0;  // own k-block index from which the next chunk of each issuer is searched
      while (j0 < count0 || j1 < count1) {
        int e0 = j0, e1 = j1;  // own index that closes the next chunk
        while (e0 < count0 && !closes_chunk(e0, count0, 0)) ++e0;
        while (e1 < count1 && !closes_chunk(e1, count1, 1)) ++e1;
        const bool take1 = j0 >= count0 || (j1 < count1 && first1 + 2 * e1 < first0 + 2 * e0);
        const int i = take1 ? 1 : 0;
        if (take1) j1 = e1 + 1; else j0 = e0 + 1;
        ok = mbar_wait(&acc_full[i], dc[i] & 1, 4, a.dev_status, abort_flag);
        if (!ok) break;
        ++dc[i];
        tc_fence_after();
        // Two pieces per round trip to tensor memory; the accumulator is handed back as soon as the last
        // pieces sit in registers, before they are added.
#pragma unroll
        for (int g = 0; g < PIECES; g += 2) {
          float v0[16], v1[16];
          const bool has0 = g * 16 < mycols, has1 = g + 1 < PIECES && (g + 1) * 16 < mycols;  // warp-uniform
          if (has0) tmem_ld16_nowait(tmem_base + i * ACC_STRIDE + lane_base + col0 + g * 16, v0);
          if (has1) tmem_ld16_nowait(tmem_base + i * ACC_STRIDE + lane_base + col0 + (g + 1) * 16, v1);
          tmem_wait_ld();
          if (g + 2 >= PIECES) {
            tc_fence_before();
            mbar_arrive_warp_remote(&acc_empty[i], 0);  // issuer i (in the leader) may overwrite its accumulator
          }
          if (has0) {
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[g][j] += v0[j];
          }
          if (has1) {
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[g + 1][j] += v1[j];
          }
        }
      }
      if (!ok) break;
      if (!a.tma_store && !tail) {
#pragma unroll
        for (int g = 0; g < PIECES; ++g)
          if (g * 16 < mycols) store16(acc[g], col0 + g * 16);
        continue;
      }
      // staged epilogue: the previous tile's TMA stores must have read the staging tile
      ok = mbar_wait(out_free, (staged & 1) ^ 1, 10, a.dev_status, abort_flag);
      if (!ok) break;
      {
        const int r = q * 32 + lane;  // row of the CTA's tile
        uint8_t* out_tile = smem + ts_pair_out_offset();
        if (a.c_transposed) {
          // The tile leaves transposed: box q holds my warp's 32 rows as its 32 columns, my column c is its row
          // c.  For one c the 32 lanes write the 32 words of one 128-byte row (its 16-byte chunks permuted by the
          // swizzle): conflict-free 4-byte stores.
#pragma unroll
          for (int g = 0; g < PIECES; ++g) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int c = col0 + g * 16 + j;
              *reinterpret_cast<float*>(out_tile + q * (BM * 128) + c * 128 + ((((lane >> 2) ^ (c & 7)) << 4) | ((lane & 3) << 2))) =
                  acc[g][j];
            }
          }
        } else
#pragma unroll
        for (int g = 0; g < PIECES; ++g) {
          const int c0 = col0 + g * 16;  // 16 columns = 4 chunks of one 32-column box
          uint8_t* box_row = out_tile + (c0 >> 5) * (BM * 128) + r * 128;
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const int src = (c0 - col0 + j) >> 1;
            float4 b4;
            b4.x = a.bias_on_m ? bias_m : __shfl_sync(0xffffffffu, bias_n.x, src);
            b4.y = a.bias_on_m ? bias_m : __shfl_sync(0xffffffffu, bias_n.y, src);
            b4.z = a.bias_on_m ? bias_m : __shfl_sync(0xffffffffu, bias_n.x, src + 1);
            b4.w = a.bias_on_m ? bias_m : __shfl_sync(0xffffffffu, bias_n.y, src + 1);
            float4 o;
            o.x = apply_epilogue_rt(epi, acc[g][j + 0], b4.x);
            o.y = apply_epilogue_rt(epi, acc[g][j + 1], b4.y);
            o.z = apply_epilogue_rt(epi, acc[g][j + 2], b4.z);
            o.w = apply_epilogue_rt(epi, acc[g][j + 3], b4.w);
            const int chunk = ((c0 & 31) + j) >> 2;
            *reinterpret_cast<float4*>(box_row + ((chunk ^ (r & 7)) << 4)) = o;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      mbar_arrive_warp(out_ready);
      if (warp == DRAIN_WARP0 && lane == 0) {
        ok = mbar_wait(out_ready, staged & 1, 11, a.dev_status, abort_flag);
        if (ok) {
          const uint8_t* out_tile = smem + ts_pair_out_offset();
#pragma unroll
          for (int bx = 0; bx < BN / 32; ++bx) {
            if (tail)  // partial tile `slot`, this CTA's 128 rows of it: a dense [tiles * 256][128] matrix
              tma_store_3d(&tmP, out_tile + bx * (BM * 128), bx * 32, slot * (2 * BM) + (int)rank * BM, 0);
            else if (a.c_transposed) {
              if (m0 + bx * 32 < a.M && n0 < a.N) tma_store_3d(&tmC, out_tile + bx * (BM * 128), m0 + bx * 32, n0, bz);
            } else if (n0 + bx * 32 < a.N && m0 < a.M)
              tma_store_3d(&tmC, out_tile + bx * (BM * 128), n0 + bx * 32, m0, bz);
          }
          tma_store_commit();
          tma_store_wait_read();  // the stores have read the tile: it may be overwritten
          mbar_arrive(out_free);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      ++staged;
    }
    if (warp == DRAIN_WARP0 && lane == 0) tma_store_wait_all();  // global writes done before the kernel ends
  }

  tc_fence_before();
  __syncwarp();
  cluster_sync_all();  // no CTA leaves (or frees tensor memory) while its peer may still use it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      (void)cudaGetLastError();
  }
  return fn;
}

// {k, rows, batch} fp32 tensor, box {32, box_rows, 1}, 128-byte swizzle, zero fill out of bounds.
int make_operand_map(CUtensorMap* tm, const float* base, int64_t K, int64_t rows, int64_t ld,
                     int64_t batch, int64_t stride, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return TCB200_ERR_CUDA;
  const bool batched = batch > 1 && stride > 0;
  cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)(batched ? batch : 1)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)(batched ? stride : rows * ld) * 4};
  cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TCB200_OK : TCB200_ERR_CUDA;
}

bool shape_ok(const tcb200_problem_t& p) {
  return p.a_k_major && p.b_k_major && p.batch > 0 && p.batch <= 65535 && p.M > 0 && p.N > 0 &&
         p.K > 0 && p.M < (1ll << 31) && p.N < (1ll << 31) && p.K < (1ll << 31) &&
         p.lda % 4 == 0 && p.ldb % 4 == 0 && p.lda >= p.K && p.ldb >= p.K && p.ldc >= p.N &&
         p.stride_a % 4 == 0 && p.stride_b % 4 == 0 && p.stride_a >= 0 && p.stride_b >= 0 &&
         ceil_div(p.M, BM) <= 65535;
}

// "Large enough to be a real dense contraction": at least four 32-wide k-blocks and one full tile
// of rows; everything smaller is bandwidth/latency bound and is not offered the tensor-core tiles.
bool worth_it(const tcb200_problem_t& p) { return p.K >= 128 && p.M >= 64 && p.N >= 64; }

template <int BN, int SPLIT>
int launch_inst(const Plan& plan, const CUtensorMap& ta, const CUtensorMap& tb, const TcArgs& args,
                cudaStream_t s) {
  static std::atomic<uint64_t> configured{0};  // bit per device
  const uint64_t bit = 1ull << (plan.device & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    TCB200_CUDA_TRY(cudaFuncSetAttribute(contraction_tc_kernel<BN, SPLIT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         smem_bytes(BN, SPLIT)));
    configured.fetch_or(bit, std::memory_order_release);
  }
  contraction_tc_kernel<BN, SPLIT>
      <<<plan.launch.grid, plan.launch.block, smem_bytes(BN, SPLIT), s>>>(ta, tb, args);
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}

template <int BN, int CHUNK>
int launch_ts(const Plan& plan, const CUtensorMap& ta, const CUtensorMap& tb, const TcArgs& args,
              cudaStream_t s) {
  static std::atomic<uint64_t> configured{0};  // bit per device
  const uint64_t bit = 1ull << (plan.device & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    TCB200_CUDA_TRY(cudaFuncSetAttribute(contraction_ts_kernel<BN, CHUNK>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         ts_smem_bytes(BN)));
    configured.fetch_or(bit, std::memory_order_release);
  }
  TCB200_CUDA_TRY(launch_pdl(contraction_ts_kernel<BN, CHUNK>, plan.launch.grid, dim3(kTsThreads, 1, 1),
                             (size_t)ts_smem_bytes(BN), s, ta, tb, args));
  return TCB200_OK;
}
// strict: the accumulators are drained after every k-block (tile.split_tf32 == 4)
template <int BN>
int launch_ts(const Plan& plan, const CUtensorMap& ta, const CUtensorMap& tb, const TcArgs& args, cudaStream_t s) {
  return plan.tile.split_tf32 == 4 ? launch_ts<BN, 1>(plan, ta, tb, args, s)
                                   : launch_ts<BN, kTsChunkKB>(plan, ta, tb, args, s);
}

template <int CHUNK, bool TAIL>
int launch_pair_inst(const Plan& plan, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                     const CUtensorMap& tp, const TcArgs& args, cudaStream_t s) {
  static std::atomic<uint64_t> configured{0};  // bit per device
  const uint64_t bit = 1ull << (plan.device & 63);
  if (!(configured.load(std::memory_order_acquire) & bit)) {
    TCB200_CUDA_TRY(cudaFuncSetAttribute(contraction_ts_pair_kernel<CHUNK, TAIL>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, ts_pair_smem_bytes()));
    configured.fetch_or(bit, std::memory_order_release);
  }
  // the kernel carries its cluster shape (2 CTAs); the grid is a multiple of 2
  TCB200_CUDA_TRY(launch_pdl(contraction_ts_pair_kernel<CHUNK, TAIL>, plan.launch.grid, dim3(kTsThreads, 1, 1),
                             (size_t)ts_pair_smem_bytes(), s, ta, tb, tc, tp, args));
  return TCB200_OK;
}
int launch_pair(const Plan& plan, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
                const CUtensorMap& tp, const TcArgs& args, cudaStream_t s) {
  const bool strict = plan.tile.split_tf32 == 4, tail = args.tail_S > 0;
  if (strict) return tail ? launch_pair_inst<1, true>(plan, ta, tb, tc, tp, args, s)
                          : launch_pair_inst<1, false>(plan, ta, tb, tc, tp, args, s);
  return tail ? launch_pair_inst<kPairChunkKB, true>(plan, ta, tb, tc, tp, args, s)
              : launch_pair_inst<kPairChunkKB, false>(plan, ta, tb, tc, tp, args, s);
}

}  // namespace

// Below 2^24 multiply-adds the launch dominates either way and the family default is a SIMT kernel,
// whose round-to-nearest fp32 FMAs also keep all-positive sums (the reference's U[0,1) test data)
// within its 3e-7 * L bound, which the truncating tensor-core accumulation does not at small L; the
// tensor-core tiles stay in the sweep.
bool contraction_tc_preferred(const tcb200_problem_t& p) {
  return shape_ok(p) && worth_it(p) && (double)p.batch * p.M * p.N * p.K >= (double)(1 << 24);
}

// Split-K choice.  Estimated time of a tile shape with the reduction split S ways, in microseconds, from the
// measured cost of one 32-wide k-block of a tile (single CTA 128 x 128: 0.62 us, CTA pair 256 x 128: 0.56 us; a
// narrower tile is not proportionally cheaper), ~3 us per tile for pipeline fill, drain and epilogue, and for
// S > 1 the second pass (launch + S partial planes through L2 at ~5 TB/s).  waves = units / slots rounded up.
constexpr int kMaxSplitK = 32;
double tc_time_estimate(const tcb200_problem_t& p, int64_t tiles, int slots, double kb_us, int S) {
  const int64_t kbs = ceil_div(p.K, BK);
  const int64_t waves = ceil_div(tiles * S, slots);
  double t = (double)waves * ((double)ceil_div(kbs, S) * kb_us + 3.0);
  if (S > 1) t += 2.0 + (double)(S + 1) * p.M * p.N * 4.0 / 5.0e6;
  return t;
}
// Best S for a tile shape: 1 unless the problem is a single (unbatched) contraction whose tiles leave SMs idle.
int pick_split_k(const tcb200_problem_t& p, int64_t tiles, int slots, double kb_us, double* est) {
  int best = 1;
  double best_t = tc_time_estimate(p, tiles, slots, kb_us, 1);
  const int64_t kbs = ceil_div(p.K, BK);
  if (p.batch == 1 && tiles < slots) {
    for (int S = 2; S <= kMaxSplitK && kbs / S >= 4; ++S) {
      const double t = tc_time_estimate(p, tiles, slots, kb_us, S);
      if (t < best_t * 0.97) { best_t = t; best = S; }  // a split has to pay for itself
    }
  }
  if (est) *est = best_t;
  return best;
}

// Tail split of the CTA-pair tiles (tile.split_k = kTailSplitBase + S).  When the tiles do not fill the last round
// of the persistent pairs (256 tiles on 74 pairs: three full rounds and 34 tiles), the last r = tiles % pairs
// tiles have their reduction split S ways so that the last round lasts 1 / S of a round.  S is the largest
// split, up to 4, whose r * S units still fit one round and leave every unit at least 8 k-blocks.
// Offered only when a round is long (K >= 1792): the second pass and the extra launch cost ~3 us, and the board
// runs these kernels at its power limit, so SMs that idle at the end of a launch are partly paid back in clock
// to the busy ones.  Measured with the plain tile beside it: 8192 x 1024 x 2048 146.1 -> 141.8 us, but
// 16384 x 512 x 1024 (K = 1024) 77.4 -> 79.8 us.
constexpr int kTailSplitBase = 100;
constexpr int64_t kTailSplitMinKB = 56;
int tail_split_factor(const tcb200_problem_t& p, int64_t tiles, int pairs) {
  if (p.batch != 1 || tiles <= pairs) return 0;
  const int64_t r = tiles % pairs;
  if (r == 0) return 0;
  const int64_t kbs = ceil_div(p.K, BK);
  if (kbs < kTailSplitMinKB) return 0;
  int64_t S = std::min<int64_t>({(int64_t)pairs / r, 4, kbs / 8});
  return S >= 2 ? (int)S : 0;
}

// A contraction of at most 128 rows has no two row tiles to pair, but C^T = B A^T has: the CTA-pair kernel then
// runs with the operands swapped and writes its tile transposed (transposed matmul 128 x 16384 x 4096: 64 pair
// tiles of 256 x 128; per k-block a CTA moves 80 KB through shared memory instead of the 116 KB of the 128 x 112
// single-CTA tile).  Plain "=" outputs without an epilogue only.
bool pair_transposable(const tcb200_problem_t& p) {
  return p.batch == 1 && p.M <= BM && p.N >= 2 * BM && p.epilogue == TCB200_EPI_NONE && !p.accumulate;
}

int contraction_tc_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n) {
  *n = 0;
  if (!shape_ok(p) || !worth_it(p)) return TCB200_OK;
  const int sms = sm_count(-1);
  int cnt = 0;
  auto push = [&](int bn, int split) {
    if (cnt < max && out)
      out[cnt] = tcb200_tile_t{TCB200_VARIANT_TCGEN05, BM, bn, BK, num_stages(bn, split), split == 3 ? 448 : 320, split, 1};
    ++cnt;
  };
  // Candidates in the order of their estimated time: the tensor-memory tiles of three widths and, where there are
  // two 128-row tiles to pair up, the CTA-pair tile, each with the split of the reduction that suits it.
  // N = 16384 with M = 128 gives 128 tiles at BN = 128 but 147 at BN = 112, which fills 147 of the 148 SMs in the
  // same single wave; a 2048-column shard of it has 16 tiles and splits its K = 4096 nine ways.
  struct Cand { int variant, bm, bn, stages, split_k; double t; };
  Cand cands[4];
  int nc = 0;
  const int ts_bn[3] = {128, 112, 64};
  const double ts_kb_us[3] = {0.62, 0.60, 0.40};
  for (int i = 0; i < 3; ++i) {
    if (p.N < ts_bn[i]) continue;
    const int64_t tiles = ceil_div(p.N, ts_bn[i]) * ceil_div(p.M, BM) * p.batch;
    Cand c{TCB200_VARIANT_TCGEN05_TS, BM, ts_bn[i], ts_b_slots(ts_bn[i]), 1, 0.0};
    c.split_k = pick_split_k(p, tiles, sms, ts_kb_us[i], &c.t);
    cands[nc++] = c;
  }
  if (p.M > BM && p.N >= kPairBN) {
    const int64_t tiles = ceil_div(p.N, kPairBN) * ceil_div(p.M, 2 * BM) * p.batch;
    Cand c{TCB200_VARIANT_TCGEN05_PAIR, 2 * BM, kPairBN, kPairBSlots, 1, 0.0};
    const int pairs = std::max(1, sms / 2);
    c.split_k = pick_split_k(p, tiles, pairs, 0.56, &c.t);
    const int tailS = c.split_k == 1 ? tail_split_factor(p, tiles, pairs) : 0;
    if (tailS) {
      // full rounds + a round of 1 / S length + the second pass over the tail tiles
      const int64_t kbs = ceil_div(p.K, BK);
      const double t = (double)(tiles / pairs) * ((double)kbs * 0.56 + 3.0) + ((double)ceil_div(kbs, tailS) * 0.56 + 3.0) + 3.0;
      if (t < c.t * 0.98) { c.t = t; c.split_k = kTailSplitBase + tailS; }
    }
    c.t *= 0.999;  // ties go to the pair tile
    cands[nc++] = c;
  }
  if (pair_transposable(p)) {
    const int pairs = std::max(1, sms / 2);
    const int64_t tiles = ceil_div(p.N, 2 * BM);
    Cand c{TCB200_VARIANT_TCGEN05_PAIR, 2 * BM, kPairBN, kPairBSlots, 1, 0.0};
    c.split_k = pick_split_k(p, tiles, pairs, 0.56, &c.t);   // the shards of a multi-GPU run: 8-32 tiles for 74 pairs
    cands[nc++] = c;
  }
  for (int i = 0; i < nc; ++i)
    for (int j = i + 1; j < nc; ++j)
      if (cands[j].t < cands[i].t) std::swap(cands[i], cands[j]);
  for (int i = 0; i < nc; ++i) {
    if (cnt < max && out)
      out[cnt] = tcb200_tile_t{cands[i].variant, cands[i].bm, cands[i].bn, BK, cands[i].stages, kTsThreads, 3,
                               cands[i].split_k};
    ++cnt;
  }
  for (int i = 0; i < nc; ++i) {  // the unsplit forms of the split candidates stay in the sweep
    if (cands[i].split_k == 1) continue;
    if (cnt < max && out)
      out[cnt] = tcb200_tile_t{cands[i].variant, cands[i].bm, cands[i].bn, BK, cands[i].stages, kTsThreads, 3, 1};
    ++cnt;
  }
  // strict accumulation (split_tf32 = 4): the 3xTF32 tiles with every accumulator drained after each of its
  // k-blocks.  The tensor core adds into its fp32 accumulator with truncation; on all-positive operands (the
  // reference's own rand() benchmark data) that bias grows with the number of additions between two drains, and
  // only this form meets the reference's 3e-7 * K bound there (K = 4096: 1.2e-3).  Slower; never the default.
  for (int i = 0; i < nc; ++i) {
    if (cnt < max && out)
      out[cnt] = tcb200_tile_t{cands[i].variant, cands[i].bm, cands[i].bn, BK, cands[i].stages, kTsThreads, 4,
                               cands[i].split_k};
    ++cnt;
  }
  // both operands in shared memory.  The 256-wide form of this kernel keeps one accumulation over the whole K
  // per tile and does not meet the reference's own precision bound at K = 4096: it is not listed (a plan
  // still takes it, as a one-pass TF32 tile only, when asked for by name).
  const int bns[] = {128, 64};
  for (int bn : bns)
    if (p.N >= bn) push(bn, 3);
  *n = cnt;
  return TCB200_OK;
}

int contraction_tc_plan(Plan& plan) {
  const tcb200_problem_t& p = plan.p;
  if (!shape_ok(p)) return TCB200_ERR_UNSUPPORTED;
  tcb200_tile_t& t = plan.tile;
  if (t.split_k <= 0) t.split_k = 1;
  const bool tail_split = t.split_k > kTailSplitBase;
  if (tail_split) {
    // tail split: CTA-pair tiles only; the factor must be the one this problem and device call for
    const int64_t tiles = ceil_div(p.N, kPairBN) * ceil_div(p.M, 2 * BM) * p.batch;
    const int S = t.split_k - kTailSplitBase;
    if (t.variant != TCB200_VARIANT_TCGEN05_PAIR || S != tail_split_factor(p, tiles, std::max(1, plan.sms / 2)))
      return TCB200_ERR_UNSUPPORTED;
    plan.scratch_floats = (size_t)S * (size_t)(tiles % std::max(1, plan.sms / 2)) * 2 * BM * kPairBN;
  } else if (t.split_k > 1) {
    // split-K: tensor-memory tiles only, one unbatched contraction, every split at least one k-block
    if (t.variant == TCB200_VARIANT_TCGEN05 || p.batch != 1 || t.split_k > kMaxSplitK ||
        ceil_div(p.K, BK) < t.split_k || p.M * p.N > (1ll << 40))
      return TCB200_ERR_UNSUPPORTED;
    plan.scratch_floats = (size_t)t.split_k * (size_t)p.M * (size_t)p.N;
  }
  if (t.variant == TCB200_VARIANT_TCGEN05_PAIR) {
    if (t.bn == 0) t.bn = kPairBN;
    if (t.split_tf32 == 0) t.split_tf32 = 3;
    if (t.bn != kPairBN || (t.split_tf32 != 3 && t.split_tf32 != 4)) return TCB200_ERR_UNSUPPORTED;
    if (ceil_div(p.M, 2 * BM) > 65535) return TCB200_ERR_UNSUPPORTED;
    t.bm = 2 * BM; t.bk = BK; t.stages = kPairBSlots; t.threads = kTsThreads;
    if (pair_transposable(p) && !tail_split) {   // operands swapped, tile written transposed
      const int64_t tiles = ceil_div(p.N, 2 * BM) * ceil_div(p.M, kPairBN) * t.split_k;
      plan.launch.grid = dim3(2u * (unsigned)std::min<int64_t>(tiles, std::max(1, plan.sms / 2)), 1, 1);
      plan.launch.block = dim3(kTsThreads, 1, 1);
      plan.launch.smem = ts_pair_smem_bytes();
      plan.kernel_id = 301284;
      return TCB200_OK;
    }
    const int64_t tiles = ceil_div(p.N, kPairBN) * ceil_div(p.M, 2 * BM) * p.batch * (tail_split ? 1 : t.split_k);
    plan.launch.grid = dim3(2u * (unsigned)std::min<int64_t>(tiles, std::max(1, plan.sms / 2)), 1, 1);
    plan.launch.block = dim3(kTsThreads, 1, 1);
    plan.launch.smem = ts_pair_smem_bytes();
    plan.kernel_id = 301283;
    return TCB200_OK;
  }
  if (t.bn == 0) t.bn = 128;
  if (t.split_tf32 == 0) t.split_tf32 = t.bn == 256 ? 1 : 3;
  if (t.bn != 64 && t.bn != 128 && t.bn != 256 && !(t.bn == 112 && t.variant == TCB200_VARIANT_TCGEN05_TS))
    return TCB200_ERR_UNSUPPORTED;
  if (t.split_tf32 != 1 && t.split_tf32 != 3 && !(t.split_tf32 == 4 && t.variant == TCB200_VARIANT_TCGEN05_TS))
    return TCB200_ERR_UNSUPPORTED;
  // the 256-wide tile accumulates the whole K in tensor memory: with the 3xTF32 split it would claim fp32
  // accuracy that its truncating accumulation does not deliver at large K
  if (t.bn == 256 && t.split_tf32 == 3) return TCB200_ERR_UNSUPPORTED;
  t.bm = BM;
  t.bk = BK;
  const bool ts_mode = t.variant == TCB200_VARIANT_TCGEN05_TS;
  if (ts_mode && (t.bn > 128 || t.split_tf32 < 3)) return TCB200_ERR_UNSUPPORTED;
  t.stages = ts_mode ? ts_b_slots(t.bn) : num_stages(t.bn, t.split_tf32);
  t.threads = ts_mode ? kTsThreads : (t.split_tf32 == 3 ? 448 : 320);
  // persistent CTAs, one per SM, walking the tiles with a static stride
  const int64_t tiles = ceil_div(p.N, t.bn) * ceil_div(p.M, BM) * p.batch * t.split_k;
  plan.launch.grid = dim3((unsigned)std::min<int64_t>(tiles, plan.sms), 1, 1);
  plan.launch.block = dim3(t.threads, 1, 1);
  plan.launch.smem = ts_mode ? ts_smem_bytes(t.bn) : smem_bytes(t.bn, t.split_tf32);
  plan.kernel_id = t.bn * 10 + (t.split_tf32 == 4 ? 3 : t.split_tf32) + (ts_mode ? 100000 : 0);
  return TCB200_OK;
}

// Tensor maps of one set of base pointers.  Encoding a map is host work of the order of a microsecond; a plan
// that is launched again and again on the same few buffers (an executor in a loop, a benchmark rotating
// over buffer sets) takes them from this small per-plan cache instead.
struct TcMaps {
  const void* key[3] = {nullptr, nullptr, nullptr};
  CUtensorMap ta, tb, tc, tp;
  bool valid = false, has_tc = false;
};
struct TcMapCache {
  std::mutex mu;
  TcMaps slot[kTcMapSlots];
  int next = 0;
};

void* tc_map_cache_new() { return new (std::nothrow) TcMapCache(); }
void tc_map_cache_delete(void* c) { delete static_cast<TcMapCache*>(c); }

int contraction_tc_launch(const Plan& plan, const float* A, const float* B, const float* bias,
                          float* C, cudaStream_t s, int* dev_status, float* scratch, void* map_cache) {
  const tcb200_problem_t& po = plan.p;                  // the problem as the caller states it (C's layout)
  if (((uintptr_t)A | (uintptr_t)B) & 15) return TCB200_ERR_ALIGNMENT;
  const bool transposed = plan.kernel_id == 301284;     // C^T = B A^T on the pair kernel
  tcb200_problem_t p = po;                              // the problem as the kernel runs it
  if (transposed) {
    std::swap(p.M, p.N);
    std::swap(p.lda, p.ldb);
    std::swap(p.stride_a, p.stride_b);
    std::swap(A, B);
  }
  const bool pair = plan.kernel_id == 301283 || transposed;
  const int tailS = plan.tile.split_k > kTailSplitBase ? plan.tile.split_k - kTailSplitBase : 0;
  const int S = !tailS && plan.tile.split_k > 1 ? plan.tile.split_k : 1;
  if ((S > 1 || tailS) && !scratch) return TCB200_ERR_INVALID_ARGUMENT;
  const int64_t pair_tiles = ceil_div(p.N, kPairBN) * ceil_div(p.M, 2 * BM) * p.batch;
  const int tail_tiles = tailS ? (int)(pair_tiles % std::max(1, plan.sms / 2)) : 0;
  // where the tensor-core kernel writes: the output, or the partial planes [S][M][N] of a split-K launch
  float* Ck = S > 1 ? scratch : C;
  // (the partial planes of a split-K launch are dense [S][M][N] in the caller's orientation)
  const int64_t ldck = S > 1 ? po.N : po.ldc, stride_ck = S > 1 ? po.M * po.N : po.stride_c;
  const int64_t batch_k = S > 1 ? S : p.batch;

  TcArgs a;
  a.C = Ck; a.bias = S > 1 ? nullptr : bias;
  a.M = (int)p.M; a.N = (int)p.N; a.K = (int)p.K; a.batch = (int)batch_k;
  a.ldc = ldck; a.stride_c = stride_ck;
  a.epi = S > 1 ? TCB200_EPI_NONE : p.epilogue; a.bias_on_m = p.bias_on_m; a.accumulate = S > 1 ? 0 : p.accumulate;
  a.a_batched = S == 1 && p.batch > 1 && p.stride_a > 0;
  a.b_batched = S == 1 && p.batch > 1 && p.stride_b > 0;
  a.ksplit_kb = S > 1 ? (int)ceil_div(ceil_div(p.K, BK), S) : 0;
  a.tail_S = tailS;
  a.tail_tiles = tail_tiles;
  a.tail_kb = tailS ? (int)ceil_div(ceil_div(p.K, BK), tailS) : 0;
  const bool bias_vec = !a.bias || p.bias_on_m || ((uintptr_t)a.bias & 15) == 0;
  a.c_vec = ((uintptr_t)Ck & 15) == 0 && ldck % 4 == 0 && stride_ck % 4 == 0 && bias_vec;
  a.dev_status = dev_status;
  a.tma_store = pair && a.c_vec && !a.accumulate;
  a.c_transposed = transposed;

  TcMaps local;
  TcMaps* m = &local;
  TcMapCache* cache = static_cast<TcMapCache*>(map_cache);
  std::unique_lock<std::mutex> lock;
  if (cache) {
    lock = std::unique_lock<std::mutex>(cache->mu);
    m = nullptr;
    for (int i = 0; i < kTcMapSlots; ++i)
      if (cache->slot[i].valid && cache->slot[i].key[0] == A && cache->slot[i].key[1] == B && cache->slot[i].key[2] == Ck)
        m = &cache->slot[i];
    if (!m) {
      m = &cache->slot[cache->next];
      cache->next = (cache->next + 1) % kTcMapSlots;
      m->valid = false;
    }
  }
  if (!m->valid) {
    // split-K: the operands are not batched (the split index selects a k range inside the kernel)
    int st = make_operand_map(&m->ta, A, p.K, p.M, p.lda, S > 1 ? 1 : p.batch, p.stride_a, BM);
    if (st != TCB200_OK) return st;
    st = make_operand_map(&m->tb, B, p.K, p.N, p.ldb, S > 1 ? 1 : p.batch, p.stride_b, pair ? kPairBN / 2 : plan.tile.bn);
    if (st != TCB200_OK) return st;
    m->tc = m->tb;  // unused by the kernel unless the staged epilogue is on
    // output map for the staged epilogue: {N, M, batch}, boxes of 32 columns x 128 rows
    // (C as the caller lays it out: in a transposed launch its rows are the kernel's columns)
    m->has_tc = a.tma_store &&
                make_operand_map(&m->tc, Ck, po.N, po.M, ldck, batch_k, stride_ck, BM) == TCB200_OK;
    m->tp = m->tb;  // unused by the kernel unless the launch has a split tail
    if (tailS) {
      // the partial tiles of the tail: a dense matrix of [tailS * tail_tiles * 256] rows of 128 floats
      st = make_operand_map(&m->tp, scratch, kPairBN, (int64_t)tailS * tail_tiles * 2 * BM, kPairBN, 1, 0, BM);
      if (st != TCB200_OK) return st;
    }
    m->key[0] = A; m->key[1] = B; m->key[2] = Ck;
    m->valid = true;
  }
  a.tma_store = a.tma_store && m->has_tc;
  const CUtensorMap ta = m->ta, tb = m->tb, tc = m->tc, tp = m->tp;
  if (cache) lock.unlock();

  int st;
  switch (plan.kernel_id) {
    case 301283:
    case 301284: st = launch_pair(plan, ta, tb, tc, tp, a, s); break;
    case 100643: st = launch_ts<64>(plan, ta, tb, a, s); break;
    case 101283: st = launch_ts<128>(plan, ta, tb, a, s); break;
    case 101123: st = launch_ts<112>(plan, ta, tb, a, s); break;
    case 643: st = launch_inst<64, 3>(plan, ta, tb, a, s); break;
    case 641: st = launch_inst<64, 1>(plan, ta, tb, a, s); break;
    case 1283: st = launch_inst<128, 3>(plan, ta, tb, a, s); break;
    case 1281: st = launch_inst<128, 1>(plan, ta, tb, a, s); break;
    case 2561: st = launch_inst<256, 1>(plan, ta, tb, a, s); break;
    default: st = TCB200_ERR_UNSUPPORTED; break;
  }
  if (st != TCB200_OK) return st;
  if (tailS)  // second pass over the tail tiles only: C = epilogue([C +] sum of their tailS partial tiles)
    return tail_tiles_reduce(scratch, C, bias, (int)p.M, (int)p.N, tailS, tail_tiles, (int)(pair_tiles - tail_tiles),
                             p.ldc, p.epilogue, p.bias_on_m, p.accumulate, s);
  if (S == 1) return st;

  // second pass: C = epilogue([C +] sum_s P[s])
  return partial_planes_reduce(scratch, C, bias, (int)po.M, (int)po.N, S, po.ldc, po.epilogue, po.bias_on_m, po.accumulate,
                               plan.sms, s);
}

}  // namespace tcb200
