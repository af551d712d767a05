// K3 (tensor-core variant, filter rows) — grouped valid convolution on tcgen05 with the FILTERS as the
// stationary operand and the filter rows (kh) as rows of the accumulator, 3xTF32.
//
//   O(n,g,f,oh,ow) = sum_{c,kh,kw} I(n,g,c,oh+kh,ow+kw) * W(g,f,c,kh,kw)  [+ B(g,f)]
//
// With C = F = 16 an implicit GEMM whose accumulator is (pixels x F) issues MMAs of N = 16: an eighth of
// the tensor pipe, two hundred of them per item.  Here the roles are turned round.  Per work item (n, g)
//
//   D[(kh, f), p] = sum_{kw, c}  A[(kh, f), (kw, c)] * B[p + kw, c]        p = flat pixel h * W + w
//   A[(kh, f), (kw, c)] = W(g, f, c, kh, kw)          48 x 48, in TENSOR MEMORY, loaded once per group
//   B[p, c]             = I(n, g, c, p)               the item's own 16 KB slab, never replicated
//   O(f, oh, ow)        = D[(0,f), oh*W+ow] + D[(1,f), (oh+1)*W+ow] + D[(2,f), (oh+2)*W+ow]
//
// so an MMA is 128 x 128 x 8 (N = 128 pixels), 36 of them per item, and the only im2col left is the sum
// over the three filter rows, done on the accumulator rows after the MMAs.
//   * kw is a shift of B by kw pixels.  B sits in shared memory k-major WITHOUT swizzle as
//     [chunk of 4 channels][pixel][4 floats]: pixel p of a chunk is 16 bytes at p * 16, i.e. the 8-row core
//     matrices follow each other at 128 bytes and a descriptor may start at ANY pixel.  The shift is the
//     descriptor's start address; nothing is copied per tap.
//   * kh is a shift by W = 16 accumulator columns, i.e. a sum over accumulator ROWS at shifted columns.  It is
//     done through shared memory: eight warps copy the 48 live rows of a finished accumulator to shared memory
//     (one 32-column load and eight 128-bit stores per warp and unit: the accumulator is free again a few
//     hundred cycles after its last MMA), then every thread forms four adjacent outputs from three 128-bit
//     loads, always as (kh0 + kh1) + kh2, adds the bias and stores them (8-byte stores; a warp covers 448
//     contiguous bytes of one output channel).
// The slab arrives by one bulk copy (cp.async.bulk + mbarrier, 3 stages), a group's filters by another; four warps re-lay it into the
// chunked layout and produce the low half of the 3xTF32 split (the tensor core truncates the raw fp32 to
// its high half itself); three threads in different warps issue the MMAs, each into its own accumulator (one
// thread gets an MMA out every ~100 cycles, the pipe takes one every ~60).  A warp reads only the 32 tensor-memory lanes of its position in its warp
// quad, so the filter rows are written twice, into lanes 0-63 and 64-127 (the MMA computes 128 rows whatever
// it is given): the warps at positions 0/1 copy the first 64 columns of a unit, those at 2/3 the other 64.
// CTAs are persistent (one per SM) over a contiguous run of items in group-major order, so the filters change
// at most once or twice per CTA.
// All mbarrier waits are bounded; on expiry a code is written to *dev_status and every role leaves its loop.
#include <atomic>

#include "async.cuh"
#include "common.cuh"
#include "tcgen05.cuh"

namespace tcb200 {
namespace {

// Out of line: the waits sit in loops whose bodies should stay small in the instruction cache.
static __device__ __noinline__ bool wait_bar_poll(uint64_t* bar, uint32_t parity, unsigned ns, int code,
                                                  int* dev_status, volatile int* abort_flag) {
  return mbar_wait_relaxed(bar, parity, ns, code, dev_status, abort_flag);
}
// ... but a wait that is already over must not pay for a call (measured: ~230 cycles each)
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, unsigned ns, int code, int* dev_status,
                                         volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  return wait_bar_poll(bar, parity, ns, code, dev_status, abort_flag);
}

constexpr int kThreads = 512;
constexpr int kW = 16;              // input row pitch = accumulator columns per input row
constexpr int kRawStages = 3;
constexpr int kAccRing = 3;         // 128-column accumulators, one per unit of 8 input rows
constexpr int kDrainWarps = 8;
constexpr int kDumpPitch = 260;     // floats per accumulator row in shared memory: 128-bit stores of 32 rows hit all banks
// Barriers of the accumulator hand-off, indexed by unit mod 6 although there are three accumulators.  A parity
// wait only tells two phases apart, so every waiter must see each phase of its barrier: every drain warp waits
// for every unit, and issuer u mod 3 owns barriers u mod 3 and u mod 3 + 3.  6 is also a multiple of the ring length,
// so the next unit on a barrier reuses the same accumulator and cannot complete a phase before the waiters of
// the previous one have been through.
constexpr int kAccBars = 6;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kACol = 128 * kAccRing;   // filters: hi at [384, 384 + KW*C), lo right behind
constexpr int kPadPixels = 8;       // zeroed pixels behind the plane: the shifted reads of the last unit

struct TapRowsArgs {
  const float* I;
  const float* W;
  const float* bias;
  float* O;
  int N, G, F, H, KH, KW, OH, OW;
  int items;
  int units;            // 128-pixel units per item
  int n_last;           // pixels of the last unit
  int epi;
  uint32_t in_bytes;    // one item's slab
  uint32_t pitch_b;     // bytes between channel chunks of the re-laid operand
  uint32_t w_bytes;     // one group's filters
  int* dev_status;
};

// shared-memory map (offsets are multiples of 128):
//   kRawStages x in_bytes                     raw slabs (c, h, w)
//   2 x 2 x (C/4) x pitch_b                   re-laid operand, [buffer][hi | lo][chunk][pixel][4]
//   w_bytes                                   raw filters of the current group (f, c, kh, kw)
//   2 x 3 x 16 x kDumpPitch floats            accumulator rows (kh, f) of the items being copied / reduced
//   barriers
template <int C>
__global__ void __launch_bounds__(kThreads, 1) group_conv_tap_rows_kernel(TapRowsArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int PL = a.H * kW;
  const int KC = a.KW * C;                        // reduction length of one accumulator row
  const uint32_t b_half = (uint32_t)(C / 4) * a.pitch_b;
  uint8_t* raw = smem;
  uint8_t* bop = raw + (size_t)kRawStages * a.in_bytes;
  const float* wraw = reinterpret_cast<const float*>(bop + (size_t)4 * b_half);
  float* dump = reinterpret_cast<float*>(bop + (size_t)4 * b_half + a.w_bytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(dump + 2 * 48 * kDumpPitch);
  uint64_t* raw_full = bars;                      // [kRawStages]
  uint64_t* raw_empty = raw_full + kRawStages;    // [kRawStages]
  uint64_t* b_ready = raw_empty + kRawStages;     // [2]
  uint64_t* b_free = b_ready + 2;                 // [2]
  uint64_t* acc_full = b_free + 2;                // [kAccBars]
  uint64_t* acc_empty = acc_full + kAccBars;      // [kAccBars]
  uint64_t* a_ready = acc_empty + kAccBars;       // [1]
  uint64_t* a_free = a_ready + 1;                 // [1]
  uint64_t* w_full = a_free + 1;                  // [1] a group's raw filters have landed
  uint64_t* w_free = w_full + 1;                  // [1] ... and have been read into registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 4);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&b_ready[b], 4);
      mbar_init(&b_free[b], a.units >= 2 ? 2 : 1);
    }
    for (int k = 0; k < kAccBars; ++k) {
      mbar_init(&acc_full[k], 1);
      mbar_init(&acc_empty[k], kDrainWarps);
    }
    mbar_init(a_ready, 4);
    mbar_init(a_free, 3);
    mbar_init(w_full, 1);
    mbar_init(w_free, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 12) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // contiguous run of work indices w = g * N + n for this CTA; the slab index of I and O is n * G + g
  const int begin = (int)((int64_t)a.items * blockIdx.x / gridDim.x);
  const int end = (int)((int64_t)a.items * (blockIdx.x + 1) / gridDim.x);
  const int nitems = end - begin;
  const int U = a.units;

  // The first slab and the first group's filters are asked into L2 before the wait for the preceding kernel:
  // a prefetch uses no value, and L2 is where that kernel's writes land, so a line fetched early is still the
  // line the later bulk copy reads.  It takes the first DRAM round trip off the start of the CTA.
  if (threadIdx.x == 64 && nitems > 0) {
    const int g = begin / a.N, n = begin - g * a.N;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<const uint8_t*>(a.I) +
                                                                     ((size_t)n * a.G + g) * a.in_bytes),
                 "r"(a.in_bytes)
                 : "memory");
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<const uint8_t*>(a.W) +
                                                                     (size_t)g * a.w_bytes),
                 "r"(a.w_bytes)
                 : "memory");
  }
  pdl_sync();  // nothing above uses a value from global memory

  // Filters of a group into tensor memory, by the four warps of one quad (every position writes its 32 lanes):
  // lane 8 kh + j of position q holds filter row kh of output channel 8 (q mod 2) + j, columns (kw, c).  They are
  // read from the staged block before the wait for the MMAs of the previous group (which still read the old
  // ones) and written after it.  `epoch` = groups loaded before this one.
  auto load_filters = [&](const uint32_t epoch) -> bool {
    const int wkh = lane >> 3, wf = (warp & 1) * 8 + (lane & 7);
    const bool wlive = wkh < a.KH && wf < a.F;
    const uint32_t ta = tmem_base + kACol + ((uint32_t)((warp & 3) * 32) << 16);
    if (!wait_bar(w_full, epoch & 1, 32, 35, a.dev_status, abort_flag)) return false;
    const float* wg = wraw + (size_t)wf * C * a.KH * a.KW + wkh * a.KW;
    float wv[3 * C];
#pragma unroll
    for (int col = 0; col < 3 * C; ++col) {
      const int kw = col / C, c = col - kw * C;
      wv[col] = wlive && kw < a.KW ? wg[c * a.KH * a.KW + kw] : 0.f;
    }
    mbar_arrive_warp(w_free);   // the values are in registers: the next group's block may land
    if (epoch > 0) {
      if (!wait_bar(a_free, (epoch - 1) & 1, 64, 21, a.dev_status, abort_flag)) return false;
      tc_fence_after();
    }
#pragma unroll
    for (int k8 = 0; k8 < 3 * C / 8; ++k8) {
      if (k8 * 8 < KC) {
        float lo[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) lo[i] = tf32_lo(wv[k8 * 8 + i]);
        tmem_st8(ta + k8 * 8, &wv[k8 * 8]);
        tmem_st8(ta + KC + k8 * 8, lo);
      }
    }
    tmem_wait_st();
    tc_fence_before();
    mbar_arrive_warp(a_ready);
    return true;
  };

  if (warp == 12) {
    // ------------------------------------------------ producer: one bulk copy per item
    if (lane == 0) {
      int cur_g = -1;
      uint32_t epoch = 0;
      for (int j = 0; j < nitems; ++j) {
        const int st = j % kRawStages;
        const uint32_t ph = (uint32_t)(j / kRawStages) & 1;
        const int w = begin + j, g = w / a.N, n = w - g * a.N;
        if (g != cur_g) {   // first item of a group: its filters, one contiguous block, ahead of the slab
          if (epoch > 0 && !wait_bar(w_free, (epoch - 1) & 1, 32, 34, a.dev_status, abort_flag)) break;
          mbar_expect_tx(w_full, a.w_bytes);
          bulk_load(const_cast<float*>(wraw), reinterpret_cast<const uint8_t*>(a.W) + (size_t)g * a.w_bytes, a.w_bytes,
                    w_full);
          cur_g = g;
          ++epoch;
        }
        if (!wait_bar(&raw_empty[st], ph ^ 1, 32, 22, a.dev_status, abort_flag)) break;
        mbar_expect_tx(&raw_full[st], a.in_bytes);
        bulk_load(raw + (size_t)st * a.in_bytes,
                  reinterpret_cast<const uint8_t*>(a.I) + ((size_t)n * a.G + g) * a.in_bytes, a.in_bytes,
                  &raw_full[st]);
      }
    }
  } else if (warp >= 13) {
    // ------------------------------------------------ MMA issuers: issuer q owns accumulator q (units u = q mod 3)
    // One thread feeds the tensor pipe an MMA every ~100 cycles, the pipe takes one every ~60: with three
    // issuers, one per accumulator, two or three units are in flight whenever the accumulators allow it.
    if (lane == 0) {
      const uint32_t q = (uint32_t)(warp - 13);
      int cur_g = -1;
      uint32_t epoch = 0;
      bool ok = true;
      for (int j = 0; j < nitems && ok; ++j) {
        const int g = (begin + j) / a.N;
        if (g != cur_g) {
          if (cur_g >= 0) umma_commit(a_free);   // my MMAs on the old filters are done when this arrives
          ok = wait_bar(a_ready, epoch & 1, 32, 23, a.dev_status, abort_flag);
          if (!ok) break;
          tc_fence_after();
          ++epoch;
          cur_g = g;
        }
        const uint32_t b = (uint32_t)j & 1, bph = ((uint32_t)j >> 1) & 1;
        const uint32_t bhi = smem_u32(bop + (size_t)(b * 2 + 0) * b_half);
        const uint32_t blo = smem_u32(bop + (size_t)(b * 2 + 1) * b_half);
        // every issuer sees every phase of the barrier, also for an item in which it has no unit
        ok = wait_bar(&b_ready[b], bph, 32, 24, a.dev_status, abort_flag);
        if (!ok) break;
        bool mine = false;
        for (int h = 0; h < U && ok; ++h) {
          const uint32_t u = (uint32_t)(j * U + h);
          if (u % kAccRing != q) continue;
          mine = true;
          const uint32_t k = u % kAccRing;
          if (u >= kAccRing) {   // the accumulator's previous unit has been drained
            const uint32_t v = u - kAccRing;
            ok = wait_bar(&acc_empty[v % kAccBars], (v / kAccBars) & 1, 32, 25, a.dev_status, abort_flag);
            if (!ok) break;
            tc_fence_after();
          }
          const uint32_t idesc = make_idesc_tf32(128, h == U - 1 ? a.n_last : 128);
          const uint32_t acc = tmem_base + k * 128;
          uint32_t accumulate = 0;
          for (int kw = 0; kw < a.KW; ++kw) {
#pragma unroll
            for (int c8 = 0; c8 < C / 8; ++c8) {
              const uint32_t boff = (uint32_t)(2 * c8) * a.pitch_b + (uint32_t)(h * 128 + kw) * 16;
              const uint64_t d_hi = make_desc_noswizzle(bhi + boff, a.pitch_b, 128);
              const uint64_t d_lo = make_desc_noswizzle(blo + boff, a.pitch_b, 128);
              const uint32_t a_hi = tmem_base + kACol + kw * C + c8 * 8, a_lo = a_hi + KC;
              umma_tf32_ts(acc, a_lo, d_hi, idesc, accumulate);   // small terms first
              umma_tf32_ts(acc, a_hi, d_lo, idesc, 1u);
              umma_tf32_ts(acc, a_hi, d_hi, idesc, 1u);
              accumulate = 1u;
            }
          }
          umma_commit(&acc_full[u % kAccBars]);
        }
        if (ok && mine) umma_commit(&b_free[b]);
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------ re-lay + split (and the filters, once per group): warps 0-3
    const int t = threadIdx.x;   // 0..127
    // the first group's filters are loaded by the drain warps 4-7, which have nothing else to do yet; later
    // groups here, after their first item's operand has been handed over (the MMAs of that item wait for both)
    int cur_g = nitems > 0 ? begin / a.N : -1;
    uint32_t epoch = 1;
    // pixels behind the plane, read by the shifted descriptors of the last unit: zero, once
    for (int e = t; e < 4 * (C / 4) * kPadPixels; e += 128) {
      const int buf = e / ((C / 4) * kPadPixels), r = e - buf * (C / 4) * kPadPixels;
      const int ch = r / kPadPixels, px = r - ch * kPadPixels;
      *reinterpret_cast<float4*>(bop + (size_t)buf * b_half + (size_t)ch * a.pitch_b + (size_t)(PL + px) * 16) =
          make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int j = 0; j < nitems; ++j) {
      const int st = j % kRawStages;
      const uint32_t ph = (uint32_t)(j / kRawStages) & 1;
      const uint32_t b = (uint32_t)j & 1, bph = ((uint32_t)j >> 1) & 1;
      if (!wait_bar(&raw_full[st], ph, 64, 26, a.dev_status, abort_flag)) break;
      if (!wait_bar(&b_free[b], bph ^ 1, 64, 27, a.dev_status, abort_flag)) break;
      const float* src = reinterpret_cast<const float*>(raw + (size_t)st * a.in_bytes);
      uint8_t* hi = bop + (size_t)(b * 2 + 0) * b_half;
      uint8_t* lo = bop + (size_t)(b * 2 + 1) * b_half;
      for (int p = t; p < PL; p += 128) {
#pragma unroll
        for (int ch = 0; ch < C / 4; ++ch) {
          float4 v;
          v.x = src[(ch * 4 + 0) * PL + p];
          v.y = src[(ch * 4 + 1) * PL + p];
          v.z = src[(ch * 4 + 2) * PL + p];
          v.w = src[(ch * 4 + 3) * PL + p];
          *reinterpret_cast<float4*>(hi + (size_t)ch * a.pitch_b + (size_t)p * 16) = v;
          *reinterpret_cast<float4*>(lo + (size_t)ch * a.pitch_b + (size_t)p * 16) =
              make_float4(tf32_lo(v.x), tf32_lo(v.y), tf32_lo(v.z), tf32_lo(v.w));
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive_warp(&raw_empty[st]);
      mbar_arrive_warp(&b_ready[b]);
      const int g = (begin + j) / a.N;
      if (g != cur_g) {
        if (!load_filters(epoch)) break;
        cur_g = g;
        ++epoch;
      }
    }
  } else if (warp < 12) {
    // ------------------------------------------------ drain: warps 4-11, all of them on every item
    // Copy: position in the quad = 2 * (column half of the unit) + (half of the output channels); the two
    // warps of a position take 32 columns each.  Lane 8 kh + j holds filter row kh of channel 8 q + j.
    const int q = warp & 1;
    const int col0 = (warp & 2) * 32 + (warp >= 8 ? 32 : 0);            // first of my 32 columns of a unit
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int kh = lane >> 3, f_mine = q * 8 + (lane & 7);
    const bool live_row = kh < 3 && f_mine < a.F;
    const int my_row = (kh * 16 + f_mine) * kDumpPitch;
    // Reduce: a warp task = one output channel x eight output rows; lane = (row, group of four columns).
    const int dw = warp - 4;
    const int orow = lane >> 2, oc4 = (lane & 3) * 4;
    const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
    const bool relu = a.epi == TCB200_EPI_BIAS_RELU;
    const int plane_out = a.OH * a.OW;
    const bool even_ow = (a.OW & 1) == 0;
    const int row_blocks = (a.OH + 7) >> 3;
    const int ntasks = a.F * row_blocks;               // at most 32: four per warp
    int tf[4], toh[4];                                 // my tasks: channel and output row of this lane
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int task = dw + k * kDrainWarps;
      tf[k] = task / row_blocks;
      toh[k] = (task - tf[k] * row_blocks) * 8 + orow;
      if (task >= ntasks || toh[k] >= a.OH) tf[k] = -1;
    }
    // The eight warps meet once per item on a hardware barrier: the copy is complete.  Items alternate between
    // two copy areas, so the barrier of item j + 1 (which a warp reaches after its reduction of item j) is also
    // what lets the copy of item j + 2 overwrite item j.  A warp whose wait ran out keeps meeting the others
    // there and skips the work in between, so that nobody is left waiting at a barrier.
    bool ok = true;
    if (warp < 8 && nitems > 0) ok = load_filters(0);   // while the first slab is re-laid by warps 0-3
    for (int j = 0; j < nitems; ++j) {
      const int g = (begin + j) / a.N;
      const int w = begin + j, n = w - g * a.N;
      float* out = a.O + ((size_t)n * a.G + g) * (size_t)a.F * plane_out;
      float* area = dump + (size_t)(j & 1) * 48 * kDumpPitch;
      float bias[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) bias[k] = has_bias && tf[k] >= 0 ? __ldg(a.bias + g * a.F + tf[k]) : 0.f;
      for (int h = 0; h < U && ok; ++h) {
        const uint32_t u = (uint32_t)(j * U + h);
        ok = wait_bar(&acc_full[u % kAccBars], (u / kAccBars) & 1, 20, 28, a.dev_status, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const int ncols = h == U - 1 ? a.n_last : 128;
        float v[32];
        const uint32_t ta = tmem_base + (u % kAccRing) * 128 + (uint32_t)col0 + lane_addr;
        if (col0 < ncols) tmem_ld16_nowait(ta, v);
        if (col0 + 16 < ncols) tmem_ld16_nowait(ta + 16, v + 16);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive_warp(&acc_empty[u % kAccBars]);          // the accumulator goes back to the issuers
        if (live_row) {
          float4* dst = reinterpret_cast<float4*>(area + my_row + h * 128 + col0);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (col0 + 4 * i < ncols) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");           // all 48 rows of the item are in shared memory
      if (ok) {
        float4 x[4][3];   // the loads of all four tasks in flight together
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (tf[k] >= 0) {
            const float* src = area + (size_t)tf[k] * kDumpPitch + toh[k] * kW + oc4;
            x[k][0] = *reinterpret_cast<const float4*>(src);
            x[k][1] = *reinterpret_cast<const float4*>(src + 16 * kDumpPitch + kW);
            x[k][2] = *reinterpret_cast<const float4*>(src + 32 * kDumpPitch + 2 * kW);
          }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (tf[k] >= 0) {
            float r[4] = {((x[k][0].x + x[k][1].x) + x[k][2].x) + bias[k], ((x[k][0].y + x[k][1].y) + x[k][2].y) + bias[k],
                          ((x[k][0].z + x[k][1].z) + x[k][2].z) + bias[k], ((x[k][0].w + x[k][1].w) + x[k][2].w) + bias[k]};
            if (relu) {
#pragma unroll
              for (int i = 0; i < 4; ++i) r[i] = fmaxf(r[i], 0.f);
            }
            float* dst = out + (size_t)tf[k] * plane_out + toh[k] * a.OW + oc4;
            if (even_ow) {   // rows of an even length start on 8-byte boundaries
              if (oc4 < a.OW) *reinterpret_cast<float2*>(dst) = make_float2(r[0], r[1]);
              if (oc4 + 2 < a.OW) *reinterpret_cast<float2*>(dst + 2) = make_float2(r[2], r[3]);
            } else {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (oc4 + i < a.OW) dst[i] = r[i];
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 12) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

struct Geometry {
  int units, n_last;
  uint32_t in_bytes, pitch_b, w_bytes;
  size_t smem;
};

bool geometry(const tcb200_problem_t& p, Geometry* g) {
  if (conv_sh(p) != 1 || conv_sw(p) != 1) return false;
  const int64_t C = p.conv[2], F = p.conv[3], H = p.conv[4], W = p.conv[5], KH = p.conv[6], KW = p.conv[7];
  if (W != kW || H < 3 || H > 16) return false;
  if (KH != 3 || KW < 1 || KW > 3) return false;
  if (!(C == 8 || C == 16) || !(F == 8 || F == 16)) return false;
  const int64_t PL = H * W;
  g->units = (int)ceil_div(PL, 128);
  g->n_last = (int)(PL - 128 * (g->units - 1));
  g->in_bytes = (uint32_t)(C * PL * 4);
  g->pitch_b = (uint32_t)((PL + kPadPixels) * 16);
  g->w_bytes = (uint32_t)(F * C * KH * KW * 4);
  g->smem = (size_t)kRawStages * g->in_bytes + (size_t)4 * (C / 4) * g->pitch_b +
            g->w_bytes + (size_t)2 * 48 * kDumpPitch * 4 + 512;   // barriers, tensor-memory slot, abort flag
  return g->in_bytes % 128 == 0 && g->w_bytes % 128 == 0 && g->smem <= 226 * 1024;
}

}  // namespace

bool group_conv_tap_rows_ok(const tcb200_problem_t& p) {
  Geometry g;
  return geometry(p, &g) && p.epilogue != TCB200_EPI_RELU && !p.accumulate;
}

int group_conv_tap_rows_plan(Plan& plan) {
  Geometry g;
  if (!group_conv_tap_rows_ok(plan.p) || !geometry(plan.p, &g)) return TCB200_ERR_UNSUPPORTED;
  tcb200_tile_t& t = plan.tile;
  t.variant = TCB200_VARIANT_TCGEN05_TS;
  t.bm = 128; t.bn = 128; t.bk = 8; t.stages = kAccRing; t.threads = kThreads; t.split_tf32 = 3;
  const int64_t items = plan.p.conv[0] * plan.p.conv[1];
  if (items > 0x7fffffffll) return TCB200_ERR_TOO_LARGE;
  plan.launch.grid = dim3((unsigned)std::min<int64_t>(items, plan.sms), 1, 1);
  plan.launch.block = dim3(kThreads, 1, 1);
  plan.launch.smem = g.smem;
  plan.kernel_id = 201;
  return TCB200_OK;
}

// false: the pointers do not allow the bulk copies (16-byte alignment); the caller takes another kernel
bool group_conv_tap_rows_aligned(const float* I, const float* W, const float* O) {
  return ((((uintptr_t)I) | ((uintptr_t)W)) & 15) == 0 && (((uintptr_t)O) & 7) == 0;   // bulk copies in, 8-byte stores out
}

int group_conv_tap_rows_launch(const Plan& plan, const float* I, const float* W, const float* bias, float* O,
                               cudaStream_t s, int* dev_status) {
  const tcb200_problem_t& p = plan.p;
  Geometry g;
  if (!geometry(p, &g)) return TCB200_ERR_UNSUPPORTED;
  if (!group_conv_tap_rows_aligned(I, W, O)) return TCB200_ERR_ALIGNMENT;
  TapRowsArgs a;
  a.I = I; a.W = W; a.bias = bias; a.O = O;
  a.N = (int)p.conv[0]; a.G = (int)p.conv[1]; a.F = (int)p.conv[3];
  a.H = (int)p.conv[4]; a.KH = (int)p.conv[6]; a.KW = (int)p.conv[7];
  a.OH = a.H - a.KH + 1; a.OW = kW - a.KW + 1;
  a.items = a.N * a.G;
  a.units = g.units; a.n_last = g.n_last;
  a.epi = p.epilogue;
  a.in_bytes = g.in_bytes; a.pitch_b = g.pitch_b; a.w_bytes = g.w_bytes;
  a.dev_status = dev_status;
  const bool c16 = p.conv[2] == 16;
  auto fn = c16 ? group_conv_tap_rows_kernel<16> : group_conv_tap_rows_kernel<8>;
  static std::atomic<uint64_t> configured[2];
  TCB200_CUDA_TRY(ensure_dynamic_smem(fn, 226 * 1024, plan.device, configured[c16]));
  TCB200_CUDA_TRY(launch_pdl(fn, plan.launch.grid, plan.launch.block, g.smem, s, a));
  return TCB200_OK;
}

}  // namespace tcb200
