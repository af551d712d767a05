// K3 (tensor-core variant) — grouped valid convolution as an implicit GEMM on tcgen05, 3xTF32.
//
//   O(n,g,f,oh,ow) = sum_{c,kh,kw} I(n,g,c,oh+kh,ow+kw) * W(g,f,c,kh,kw)  [+ B(g,f)]
//
// Per work item (n, g):  D[m, f] = sum over shifts s=(kh,kw) of  A_s[m, c] * B_s[f, c]^T
//   m   = oh * W + ow          flat pixel index WITH the input row pitch (the KW-1 right-most
//                              columns of every row are garbage outputs that are never stored)
//   A_s[m, c] = I[c][m + kh*W + kw]   a pure flat shift inside channel plane c
//   B_s[f, c] = W[f][c][kh][kw]
// so the whole halo tile of the item (C planes of H*W floats, one contiguous 16 KB slab) is staged
// once by a bulk copy and every shift re-reads it from shared memory.
//
// Blackwell mapping (one persistent CTA per SM, 448 threads):
//   warp 0      producer: one bulk copy (cp.async.bulk + mbarrier) of the item's input slab and of
//               its group's filter slab into a double-buffered shared-memory stage
//   warps 2-9   operand builders, two sets of four warps alternating (m-tile, shift) steps: a thread
//               owns pixel row m of the 128-row tile (= its TMEM lane), reads its C channel values
//               for the shift (bank-conflict free: consecutive lanes, consecutive addresses), splits
//               them into hi = v (the tensor core truncates fp32 to TF32 itself) and
//               lo = tf32(v - trunc(v)) and writes both into a TMEM ring slot with tcgen05.st.
//               Once per item they also re-lay the filters into the no-swizzle k-major core-matrix
//               layout the MMA reads (hi and lo copies).
//   warp 1      issues tcgen05.mma.kind::tf32 (M=128, N=F, K=8), A from TMEM, B from shared memory:
//               lo*hi, hi*lo, hi*hi per 8-channel slice, each into its own TMEM accumulator that
//               sums over the shifts
//   warps 10-13 epilogue: tcgen05.ld of the partial accumulators, fp32 sum, + bias, scatter to O
//               (ow < OW only)
// Measured on B200 (N=32, G=32, C=F=16, 16x16, 3x3): 70 us, i.e. slower than the SIMT rows kernel
// (~50 us), so the family lists this variant AFTER the SIMT ones.  Ablation (no loads, no TMEM
// traffic, no MMAs) shows ~0.22 us per (pixel tile, tap) hand-off of pure mbarrier round trip
// with the 4-slot ring: 18 hand-offs per item dominate the 108 tiny (N = 16) MMAs.
// All mbarrier waits are bounded; on expiry a code is written to *dev_status and every role exits.
#include <atomic>

#include "async.cuh"
#include "common.cuh"
#include "tcgen05.cuh"

namespace tcb200 {
namespace {

constexpr int kThreads = 448;
constexpr int kSlots = 4;          // TMEM ring slots for the A operand
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kAccPerBuf = 192;            // accumulator columns of one item buffer
constexpr uint32_t kAccCols = 2 * kAccPerBuf;   // [0, 384): 2 item buffers x (MT x 3 x C/8) accumulators x F
                                                // [384, 512): A ring, kSlots x 2*C columns (C <= 16)
// Every (pixel tile, split term, 8-channel slice) has its OWN accumulator: an MMA with N = F = 16 is
// far shorter than the tensor pipe's latency, so MMAs chained on one accumulator would run at the
// pipe's latency; with 12 independent chains consecutive MMAs overlap.  The short chains (one MMA
// per filter tap) also keep the accumulator's truncating adds from drifting; the epilogue sums the
// partial accumulators with round-to-nearest adds.

struct ConvTcArgs {
  const float* I;
  const float* W;
  const float* bias;
  float* O;
  int N, G, F, H, Wd, KH, KW, OH, OW;
  int MT;          // 128-row pixel tiles per item
  int items;       // N * G
  int epi, accumulate;
  uint32_t in_bytes, w_bytes;     // per item
  uint32_t in_stride;             // bytes between the two input stages (in_bytes + pad)
  int* dev_status;
};

// shared-memory map (all offsets multiples of 128):
//   [0)                2 x in_stride            input stages
//   [+)                2 x w_bytes              raw filter slabs (f, c, kh, kw)
//   [+)                2 x 2 x w_bytes          canonical filters: [buf][hi|lo][shift][core matrices]
//   [+)                barriers
template <int C>
__global__ void __launch_bounds__(kThreads, 1) group_conv_tc_kernel(ConvTcArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int TAPS = a.KH * a.KW;
  const int PL = a.H * a.Wd;
  const int F = a.F;
  uint8_t* in_st = smem;
  uint8_t* wraw = in_st + 2 * a.in_stride;
  uint8_t* wcan = wraw + 2 * a.w_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(wcan + 4 * a.w_bytes);
  uint64_t* in_full = bars;            // [2]
  uint64_t* in_empty = bars + 2;       // [2]
  uint64_t* w_free = bars + 4;         // [2]
  uint64_t* w_ready = bars + 6;        // [2]
  uint64_t* acc_full = bars + 8;       // [2]
  uint64_t* acc_empty = bars + 10;     // [2]
  uint64_t* slot_ready = bars + 12;    // [kSlots]
  uint64_t* slot_empty = bars + 12 + kSlots;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12 + 2 * kSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&in_full[b], 1);
      mbar_init(&in_empty[b], 8);
      mbar_init(&w_free[b], 1);
      mbar_init(&w_ready[b], 8);
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(&slot_ready[s], 4);
      mbar_init(&slot_empty[s], 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // contiguous range of items for this CTA; item = n * G + g is also the slab index of I and O
  const int64_t begin = (int64_t)a.items * blockIdx.x / gridDim.x;
  const int64_t end = (int64_t)a.items * (blockIdx.x + 1) / gridDim.x;
  const uint32_t shift_bytes = (uint32_t)F * C * 4;   // one shift's B matrix
  const uint32_t lbo = (uint32_t)(F / 8) * 128;       // bytes between 16-byte chunks along k
  const uint32_t idesc = make_idesc_tf32(128, F);

  if (warp == 0) {
    // ------------------------------------------------ producer
    if (lane == 0) {
      uint32_t j = 0;
      for (int64_t item = begin; item < end; ++item, ++j) {
        const uint32_t buf = j & 1, ph = (j >> 1) & 1;
        if (!mbar_wait(&in_empty[buf], ph ^ 1, 1, a.dev_status, abort_flag)) break;
        const int g = (int)(item % a.G);
        mbar_expect_tx(&in_full[buf], a.in_bytes + a.w_bytes);
        bulk_load(in_st + buf * a.in_stride, reinterpret_cast<const uint8_t*>(a.I) + (size_t)item * a.in_bytes,
                  a.in_bytes, &in_full[buf]);
        bulk_load(wraw + buf * a.w_bytes, reinterpret_cast<const uint8_t*>(a.W) + (size_t)g * a.w_bytes,
                  a.w_bytes, &in_full[buf]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t j = 0, q = 0;
      bool ok = true;
      for (int64_t item = begin; item < end && ok; ++item, ++j) {
        const uint32_t buf = j & 1, ph = (j >> 1) & 1;
        ok = mbar_wait(&w_ready[buf], ph, 2, a.dev_status, abort_flag) &&
             mbar_wait(&acc_empty[buf], ph ^ 1, 3, a.dev_status, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t bhi = smem_u32(wcan + (size_t)(buf * 2 + 0) * a.w_bytes);
        const uint32_t blo = smem_u32(wcan + (size_t)(buf * 2 + 1) * a.w_bytes);
        for (int s = 0; s < TAPS && ok; ++s) {
          for (int mt = 0; mt < a.MT; ++mt, ++q) {
            const uint32_t slot = q % kSlots, sph = (q / kSlots) & 1;
            ok = mbar_wait(&slot_ready[slot], sph, 4, a.dev_status, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const uint32_t ta_hi = tmem_base + kAccCols + slot * (2 * C), ta_lo = ta_hi + C;
            const uint32_t acc0 = tmem_base + buf * kAccPerBuf + (uint32_t)(mt * 3 * (C / 8)) * F;
            const uint32_t accumulate = s == 0 ? 0u : 1u;
#pragma unroll
            for (int k8 = 0; k8 < C / 8; ++k8) {
              const uint32_t boff = s * shift_bytes + (k8 * 2) * lbo;
              const uint64_t d_hi = make_desc_noswizzle(bhi + boff, lbo, 128);
              const uint64_t d_lo = make_desc_noswizzle(blo + boff, lbo, 128);
              umma_tf32_ts(acc0 + (0 * (C / 8) + k8) * F, ta_lo + k8 * 8, d_hi, idesc, accumulate);
              umma_tf32_ts(acc0 + (1 * (C / 8) + k8) * F, ta_hi + k8 * 8, d_lo, idesc, accumulate);
              umma_tf32_ts(acc0 + (2 * (C / 8) + k8) * F, ta_hi + k8 * 8, d_hi, idesc, accumulate);
            }
            umma_commit(&slot_empty[slot]);
          }
        }
        if (ok) {
          umma_commit(&acc_full[buf]);  // accumulators of the item complete
          umma_commit(&w_free[buf]);    // ... and its canonical filters no longer read
        }
      }
    }
  } else if (warp < 10) {
    // ------------------------------------------------ operand builders
    const int set = (warp - 2) >> 2;
    const int bt = threadIdx.x - 64;                 // 0..255 among all builders
    const int row = (warp & 3) * 32 + lane;          // TMEM lane of this thread
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t j = 0, q = 0;
    bool ok = true;
    for (int64_t item = begin; item < end && ok; ++item, ++j) {
      const uint32_t buf = j & 1, ph = (j >> 1) & 1;
      ok = mbar_wait(&in_full[buf], ph, 5, a.dev_status, abort_flag) &&
           mbar_wait(&w_free[buf], ph ^ 1, 6, a.dev_status, abort_flag);
      if (!ok) break;
      // filters: raw (f, c, tap) -> per tap the k-major core-matrix layout, hi and lo copies
      {
        const float* raw = reinterpret_cast<const float*>(wraw + buf * a.w_bytes);
        uint8_t* chi = wcan + (size_t)(buf * 2 + 0) * a.w_bytes;
        uint8_t* clo = wcan + (size_t)(buf * 2 + 1) * a.w_bytes;
        const int total = F * C * TAPS;
        for (int e = bt; e < total; e += 256) {
          const int fc = e / TAPS, s = e - fc * TAPS;
          const int f = fc / C, c = fc - f * C;
          const float v = raw[e];
          const uint32_t off = s * shift_bytes + (c >> 2) * lbo + (f >> 3) * 128 + (f & 7) * 16 + (c & 3) * 4;
          *reinterpret_cast<float*>(chi + off) = v;
          *reinterpret_cast<float*>(clo + off) = tf32_lo(v);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive_warp(&w_ready[buf]);
      }
      const float* in = reinterpret_cast<const float*>(in_st + buf * a.in_stride);
      for (int kh = 0; kh < a.KH && ok; ++kh)
        for (int kw = 0; kw < a.KW && ok; ++kw)
          for (int mt = 0; mt < a.MT; ++mt, ++q) {
            if ((int)(q & 1) != set) continue;
            const uint32_t slot = q % kSlots, sph = (q / kSlots) & 1;
            ok = mbar_wait(&slot_empty[slot], sph ^ 1, 7, a.dev_status, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const float* src = in + mt * 128 + row + kh * a.Wd + kw;
            float hi[C], lo[C];
#pragma unroll
            for (int c = 0; c < C; ++c) hi[c] = src[(size_t)c * PL];
#pragma unroll
            for (int c = 0; c < C; ++c) lo[c] = tf32_lo(hi[c]);
            const uint32_t ta = tmem_base + kAccCols + slot * (2 * C) + lane_addr;
            if (C == 16) {
              tmem_st16(ta, hi);
              tmem_st16(ta + C, lo);
            } else {
              tmem_st8(ta, hi);
              tmem_st8(ta + C, lo);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive_warp(&slot_ready[slot]);
          }
      if (ok) mbar_arrive_warp(&in_empty[buf]);  // this warp is done with the item's input slab
    }
  } else {
    // ------------------------------------------------ epilogue
    const int qd = warp & 3;
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
    const int plane_out = a.OH * a.OW;
    uint32_t j = 0;
    bool ok = true;
    for (int64_t item = begin; item < end && ok; ++item, ++j) {
      const uint32_t buf = j & 1, ph = (j >> 1) & 1;
      ok = mbar_wait(&acc_full[buf], ph, 8, a.dev_status, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int g = (int)(item % a.G);
      float* Oi = a.O + (size_t)item * F * plane_out;
      for (int mt = 0; mt < a.MT; ++mt) {
        const int m = mt * 128 + qd * 32 + lane;
        const int oh = m / a.Wd, ow = m - oh * a.Wd;
        const bool valid = oh < a.OH && ow < a.OW;
        const uint32_t acc0 = tmem_base + buf * kAccPerBuf + (uint32_t)(mt * 3 * (C / 8)) * F + lane_addr;
        for (int f0 = 0; f0 < F; f0 += 16) {
          // all partial accumulators of the tile are requested before the single wait, so the TMEM
          // read latencies overlap; summed small terms first, then the hi*hi partials
          float v[3 * (C / 8)][16];
#pragma unroll
#pragma unroll
          for (int p = 0; p < 3 * (C / 8); ++p) tmem_ld16_nowait(acc0 + p * F + f0, v[p]);
          tmem_wait_ld();
          float sum[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            sum[i] = v[0][i];
#pragma unroll
            for (int p = 1; p < 3 * (C / 8); ++p) sum[i] += v[p][i];
          }
          if (valid) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int f = f0 + i;
              float* o = Oi + (size_t)f * plane_out + oh * a.OW + ow;
              float r = sum[i];
              if (a.accumulate) r += *o;
              *o = apply_epilogue_rt(a.epi, r, has_bias ? __ldg(a.bias + g * F + f) : 0.f);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive_warp(&acc_empty[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

struct Geometry {
  int MT;
  uint32_t in_bytes, in_stride, w_bytes;
  size_t smem;
};

bool geometry(const tcb200_problem_t& p, Geometry* g) {
  if (conv_sh(p) != 1 || conv_sw(p) != 1) return false;
  const int64_t C = p.conv[2], F = p.conv[3], H = p.conv[4], W = p.conv[5], KH = p.conv[6], KW = p.conv[7];
  const int64_t OH = H - KH + 1;
  if (!(C == 8 || C == 16)) return false;
  if (F % 16 != 0 || F > 128) return false;
  if ((H * W) % 4 != 0 || KH * KW > 64) return false;
  const int64_t MT = ceil_div(OH * W, 128);
  if (MT * 3 * (C / 8) * F > (int64_t)kAccPerBuf) return false;
  const int64_t in_bytes = C * H * W * 4, w_bytes = F * C * KH * KW * 4;
  if (w_bytes % 16 != 0) return false;
  // rows of the last tile read up to (MT*128 - 1) + (KH-1)*W + KW - 1 inside the LAST channel plane
  const int64_t overrun = std::max<int64_t>(0, MT * 128 + (KH - 1) * W + KW - H * W) * 4;
  const int64_t in_stride = round_up(in_bytes + overrun, 128);
  const size_t smem = (size_t)(2 * in_stride + 6 * round_up(w_bytes, 128) + 512);
  if (smem > 200 * 1024) return false;
  g->MT = (int)MT;
  g->in_bytes = (uint32_t)in_bytes;
  g->in_stride = (uint32_t)in_stride;
  g->w_bytes = (uint32_t)w_bytes;
  g->smem = smem;
  return w_bytes % 128 == 0;  // keeps every filter area 128-byte aligned
}

}  // namespace

bool group_conv_tc_ok(const tcb200_problem_t& p) {
  Geometry g;
  return geometry(p, &g) && p.epilogue != TCB200_EPI_RELU;
}

int group_conv_tc_plan(Plan& plan) {
  Geometry g;
  if (!geometry(plan.p, &g) || plan.p.epilogue == TCB200_EPI_RELU) return TCB200_ERR_UNSUPPORTED;
  tcb200_tile_t& t = plan.tile;
  t.variant = TCB200_VARIANT_TCGEN05_TS;
  t.bm = 128; t.bn = (int)plan.p.conv[3]; t.bk = 8; t.stages = kSlots; t.threads = kThreads; t.split_tf32 = 3;
  const int64_t items = plan.p.conv[0] * plan.p.conv[1];
  plan.launch.grid = dim3((unsigned)std::min<int64_t>(items, plan.sms), 1, 1);
  plan.launch.block = dim3(kThreads, 1, 1);
  plan.launch.smem = g.smem;
  plan.kernel_id = 200;
  return TCB200_OK;
}

int group_conv_tc_launch(const Plan& plan, const float* I, const float* W, const float* bias, float* O,
                         cudaStream_t s, int* dev_status) {
  const tcb200_problem_t& p = plan.p;
  Geometry g;
  if (!geometry(p, &g)) return TCB200_ERR_UNSUPPORTED;
  if (((uintptr_t)I | (uintptr_t)W) & 15) return TCB200_ERR_ALIGNMENT;
  ConvTcArgs a;
  a.I = I; a.W = W; a.bias = bias; a.O = O;
  a.N = (int)p.conv[0]; a.G = (int)p.conv[1]; a.F = (int)p.conv[3];
  a.H = (int)p.conv[4]; a.Wd = (int)p.conv[5]; a.KH = (int)p.conv[6]; a.KW = (int)p.conv[7];
  a.OH = a.H - a.KH + 1; a.OW = a.Wd - a.KW + 1;
  a.MT = g.MT;
  a.items = a.N * a.G;
  a.epi = p.epilogue; a.accumulate = p.accumulate;
  a.in_bytes = g.in_bytes; a.in_stride = g.in_stride; a.w_bytes = g.w_bytes;
  a.dev_status = dev_status;
  auto fn = p.conv[2] == 16 ? group_conv_tc_kernel<16> : group_conv_tc_kernel<8>;
  static std::atomic<uint64_t> configured[2];
  // the attribute is the largest size any shape of this kernel may ask for
  TCB200_CUDA_TRY(ensure_dynamic_smem(fn, 200 * 1024, plan.device, configured[p.conv[2] == 16]));
  fn<<<plan.launch.grid, plan.launch.block, g.smem, s>>>(a);
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}

}  // namespace tcb200
