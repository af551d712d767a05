// K3 — grouped 2-D valid convolution, fused bias:
//   O(n,g,f,h,w)  = sum_{c,kh,kw} I(n,g,c,SH*h+kh,SW*w+kw) * W1(g,f,c,kh,kw)
//   O(n,g,f,h,w) += B(g,f)
// Replaces the kernel the reference generates for tc/benchmarks/group_convolution.cc:124-132
// (library twins tc/library/group_convolution.h:26-44 and tc/library/convolution.h:26-31, whose
// strides are template parameters; strides other than 1 run on the band kernel only).
//
// SIMT kernels (the tensor-core forms live in group_conv_tap_rows.cu, the default where it applies, and group_conv_tcgen05.cu):
//  * rows kernel (default when W <= 16 and F % 4 == 0): one CTA per (g, pair of n).  A thread owns
//    one output row h of four output channels: 4 x OW accumulators in registers.  Per (c, kh) it
//    reads one input row (four 128-bit shared loads, row pitch padded to 20 floats so the eight
//    rows a quarter-warp touches fall into distinct banks) and three 128-bit filter vectors, and
//    issues 4 * OW * KW FMAs: ~24 FMAs per shared load, so the kernel is bound by the fp32 pipe,
//    not by shared memory.
//  * band kernel (any size): one CTA per (n, g, band of output rows), one pixel x four channels
//    per thread.
// Band kernel: one CTA per (n, g, band of output rows).  The band's input halo
// (C x (rows+KH-1) x W) and the group's filters are staged in shared memory once; the
// filters are re-laid out as Ws[c][kh][kw][f] so one 128-bit shared load feeds four
// output channels.  Consecutive threads take consecutive output pixels, so the halo
// reads are bank-conflict free and the output stores are coalesced along w.
#include "async.cuh"
#include "common.cuh"

namespace tcb200 {
namespace {

struct ConvArgs {
  const float* I;
  const float* W;
  const float* bias;
  float* O;
  int G, C, F, H, Wd, KH, KW, OH, OW;
  int band;     // output rows per CTA
  int SH, SW;   // strides (band kernel; the other kernels take unit strides only)
  int epi, accumulate;
};

template <int FT>
__global__ void __launch_bounds__(256) group_conv_simt_kernel(ConvArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int ng = blockIdx.x;  // n * G + g
  const int g = ng % a.G;
  const int h0 = blockIdx.y * a.band;
  const int rows = min(a.band, a.OH - h0);
  const int in_rows = (rows - 1) * a.SH + a.KH;
  const int h0_in = h0 * a.SH;
  const int taps = a.C * a.KH * a.KW;
  const int Fp = (a.F + FT - 1) / FT * FT;

  float* Ws = smem;                       // [taps][Fp]
  float* Is = smem + (size_t)taps * Fp;   // [C][in_rows][W]
  const int tid = threadIdx.x, nt = blockDim.x;

  // Filters of this group: global (f, c, kh, kw) -> shared (c, kh, kw, f).
  const float* Wg = a.W + (size_t)g * a.F * taps;
  for (int i = tid; i < taps * Fp; i += nt) {
    const int t = i / Fp, f = i - t * Fp;
    Ws[i] = f < a.F ? __ldg(Wg + (size_t)f * taps + t) : 0.f;
  }
  // Input halo of the band: rows [h0, h0 + in_rows) of every channel, full width.
  const float* Ig = a.I + (size_t)ng * a.C * a.H * a.Wd;
  const int row_elems = in_rows * a.Wd;
  for (int i = tid; i < a.C * row_elems; i += nt) {
    const int c = i / row_elems, r = i - c * row_elems;
    Is[i] = __ldg(Ig + ((size_t)c * a.H + h0_in) * a.Wd + r);
  }
  __syncthreads();

  const int pix = rows * a.OW;
  const int items = (Fp / FT) * pix;
  float* Og = a.O + (size_t)ng * a.F * a.OH * a.OW;
  for (int it = tid; it < items; it += nt) {
    const int fg = it / pix, p = it - fg * pix;
    const int h = p / a.OW, w = p - h * a.OW;
    float acc[FT];
#pragma unroll
    for (int j = 0; j < FT; ++j) acc[j] = 0.f;
    int t = 0;
    for (int c = 0; c < a.C; ++c)
      for (int kh = 0; kh < a.KH; ++kh) {
        const float* irow = Is + ((size_t)c * in_rows + h * a.SH + kh) * a.Wd + w * a.SW;
        for (int kw = 0; kw < a.KW; ++kw, ++t) {
          const float x = irow[kw];
          const float* wv = Ws + (size_t)t * Fp + fg * FT;
          if constexpr (FT == 4) {
            const float4 q = *reinterpret_cast<const float4*>(wv);
            acc[0] = fmaf(x, q.x, acc[0]);
            acc[1] = fmaf(x, q.y, acc[1]);
            acc[2] = fmaf(x, q.z, acc[2]);
            acc[3] = fmaf(x, q.w, acc[3]);
          } else {
#pragma unroll
            for (int j = 0; j < FT; ++j) acc[j] = fmaf(x, wv[j], acc[j]);
          }
        }
      }
#pragma unroll
    for (int j = 0; j < FT; ++j) {
      const int f = fg * FT + j;
      if (f >= a.F) break;
      float bias = 0.f;
      if (a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU)
        bias = __ldg(a.bias + g * a.F + f);
      float* o = Og + ((size_t)f * a.OH + h0 + h) * a.OW + w;
      float v = acc[j];
      if (a.accumulate) v += *o;
      *o = apply_epilogue_rt(a.epi, v, bias);
    }
  }
}


// ------------------------------------------------------------------------------------------------
// rows kernel
// ------------------------------------------------------------------------------------------------
constexpr int kRowsMaxW = 16;   // input width held in registers
constexpr int kRowsPitch = 20;  // shared-memory row pitch in floats (80 B)

__global__ void __launch_bounds__(256) group_conv_rows_kernel(ConvArgs a, int n_per_cta, int N) {
  extern __shared__ __align__(16) float smem[];
  const int g = blockIdx.x;
  const int n0 = blockIdx.y * n_per_cta;
  const int nn = min(n_per_cta, N - n0);
  const int taps = a.C * a.KH * a.KW;
  const int Fp = a.F;  // multiple of 4 (checked by the plan)
  float* Ws = smem;                        // [taps][F]
  float* Is = smem + (size_t)taps * Fp;    // [nn][C][H][kRowsPitch]
  const int tid = threadIdx.x, nt = blockDim.x;

  // Staging uses asynchronous copies so every thread has all of its loads in flight at once.
  // Filters: read in global order (f, tap) and scattered to the transposed layout [tap][f].
  const float* Wg = a.W + (size_t)g * a.F * taps;
  for (int i = tid; i < taps * Fp; i += nt) {
    const int f = i / taps, t = i - f * taps;
    cp_async_4(Ws + (size_t)t * Fp + f, Wg + i);
  }
  const int plane = a.C * a.H;  // rows per n
  const float* Ig = a.I + ((size_t)n0 * a.G + g) * plane * a.Wd;
  const size_t n_stride = (size_t)a.G * plane * a.Wd;
  if ((a.Wd & 3) == 0 && (((uintptr_t)a.I) & 15) == 0) {
    const int w4 = a.Wd >> 2;
    for (int i = tid; i < nn * plane * w4; i += nt) {
      const int q = i % w4, r = i / w4;  // r = ni * plane + c * H + h
      const int ni = r / plane, ch = r - ni * plane;
      cp_async_16(Is + (size_t)r * kRowsPitch + 4 * q, Ig + ni * n_stride + (size_t)ch * a.Wd + 4 * q);
    }
  } else {
    for (int i = tid; i < nn * plane * a.Wd; i += nt) {
      const int w = i % a.Wd, r = i / a.Wd;
      const int ni = r / plane, ch = r - ni * plane;
      cp_async_4(Is + (size_t)r * kRowsPitch + w, Ig + ni * n_stride + (size_t)ch * a.Wd + w);
    }
  }
  cp_async_wait_all();
  __syncthreads();

  const int FQ = a.F / 4;
  const int per_n = FQ * a.OH;
  if (tid >= nn * per_n) return;
  const int ni = tid / per_n, rem = tid - ni * per_n;
  const int fq = rem / a.OH, h = rem - fq * a.OH;

  float acc[4][kRowsMaxW];
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int w = 0; w < kRowsMaxW; ++w) acc[j][w] = 0.f;

  const float* in = Is + (size_t)ni * plane * kRowsPitch;
  for (int c = 0; c < a.C; ++c) {
    for (int kh = 0; kh < a.KH; ++kh) {
      const float4* row = reinterpret_cast<const float4*>(in + (size_t)(c * a.H + h + kh) * kRowsPitch);
      float x[kRowsMaxW + 4];
#pragma unroll
      for (int q = 0; q < kRowsMaxW / 4; ++q) {
        const float4 v = row[q];
        x[4 * q] = v.x; x[4 * q + 1] = v.y; x[4 * q + 2] = v.z; x[4 * q + 3] = v.w;
      }
#pragma unroll
      for (int q = kRowsMaxW; q < kRowsMaxW + 4; ++q) x[q] = 0.f;
      const float* wrow = Ws + (size_t)((c * a.KH + kh) * a.KW) * Fp + fq * 4;
#pragma unroll
      for (int kw = 0; kw < 4; ++kw) {  // KW <= 4 (checked by the plan)
        if (kw < a.KW) {
          const float4 wv = *reinterpret_cast<const float4*>(wrow + (size_t)kw * Fp);
#pragma unroll
          for (int w = 0; w < kRowsMaxW; ++w) {
            const float xv = x[w + kw];
            acc[0][w] = fmaf(xv, wv.x, acc[0][w]);
            acc[1][w] = fmaf(xv, wv.y, acc[1][w]);
            acc[2][w] = fmaf(xv, wv.z, acc[2][w]);
            acc[3][w] = fmaf(xv, wv.w, acc[3][w]);
          }
        }
      }
    }
  }
  const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int f = fq * 4 + j;
    const float bias = has_bias ? __ldg(a.bias + g * a.F + f) : 0.f;
    float* o = a.O + ((((size_t)(n0 + ni) * a.G + g) * a.F + f) * a.OH + h) * a.OW;
#pragma unroll
    for (int w = 0; w < kRowsMaxW; ++w) {
      if (w < a.OW) {
        float v = acc[j][w];
        if (a.accumulate) v += o[w];
        o[w] = apply_epilogue_rt(a.epi, v, bias);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// item kernel: one CTA of 64 threads per (n, g), W = 16 in registers, OW <= 14, KW <= 3
// ------------------------------------------------------------------------------------------------
// Same thread tile as the rows kernel (one output row x four output channels) with three changes
// that the rows kernel's profile asked for (FMA pipe 44 % busy, a third of the warp time waiting
// for the staging copies, SMs idle 18 % of the kernel because 512 CTAs do not divide over 148 SMs):
//  * one item per CTA: 1024 CTAs of 30 KB, seven resident per SM, all in one balanced wave;
//  * the input planes arrive in four cp.async groups of C/4 channels and the loop over channels
//    starts as soon as the first group (and the filters) has landed;
//  * exactly OW accumulators per channel (no padded columns, no zero fill of the row registers)
//    and the output tile goes through shared memory so that it leaves in 128-bit coalesced stores.
constexpr int kItemOW = 14;
constexpr int kItemKW = 3;
constexpr int kItemThreads = 64;  // default form: four output channels per thread
// KHT > 0: filter height known at compile time (rows and taps fully unrolled); 0: read from the arguments.
// FPT: output channels per thread (4: 64 threads per item; 2: 128 threads, twice the warps in flight
// at twice the input-row loads).
template <int KHT, int FPT>
__global__ void __launch_bounds__(256 / FPT) group_conv_item_kernel(ConvArgs a) {
  constexpr int kItemThreads = 256 / FPT;
  extern __shared__ __align__(16) float smem[];
  pdl_sync();  // launched as a programmatic dependent: wait for the preceding kernel before any global access
  const int item = blockIdx.x;  // n * G + g
  const int g = item % a.G;
  const int taps = a.C * a.KH * a.KW;
  const int F = a.F;
  // Filters stay in their global order (f, tap), rows padded to `wp` floats: 16-byte copies in, and the
  // FPT rows a thread reads at one tap fall into distinct banks (wp = taps + 4: 2 * wp = 8 mod 32 for the
  // benchmark's 144 taps).  Transposing them to [tap][f] on the way in took 2304 four-byte cp.async per
  // item whose shared-memory writes conflict 16 ways: 4.7 us of the kernel, measured by leaving it out.
  const int wp = taps + 4;
  float* Ws = smem;                       // [F][wp]
  float* Is = smem + (size_t)F * wp;      // [C][H][kRowsPitch]
  const int tid = threadIdx.x;

  // group 0: filters + first quarter of the channels
  const float* Wg = a.W + (size_t)g * F * taps;
  const int tq = taps >> 2;  // 16-byte pieces per filter (taps % 4 == 0 because C % 4 == 0)
  for (int i = tid; i < F * tq; i += kItemThreads) {
    const int f = i / tq, piece = i - f * tq;
    cp_async_16(Ws + (size_t)f * wp + 4 * piece, Wg + (size_t)f * taps + 4 * piece);
  }
  const float* Ig = a.I + (size_t)item * a.C * a.H * a.Wd;
  const int rows_q = (a.C / 4) * a.H;  // rows per quarter (C % 4 == 0 checked by the plan)
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    for (int i = tid; i < rows_q * 4; i += kItemThreads) {  // four 16-byte pieces per row of 16 floats
      const int r = q * rows_q + (i >> 2), piece = i & 3;
      cp_async_16(Is + (size_t)r * kRowsPitch + 4 * piece, Ig + (size_t)r * 16 + 4 * piece);
    }
    cp_async_commit();
  }

  // Thread -> (channel quad, output row) with the rows of a quad padded to a multiple of 8 lanes: a
  // 128-bit shared load is served a quarter-warp at a time, and eight consecutive rows (pitch 80 B)
  // fall into distinct banks, which rows of two different quads in one quarter-warp would not.
  const int FQ = F / FPT;
  const int hslots = (a.OH + 7) & ~7;
  const int fq_t = tid / hslots, h_t = tid - fq_t * hslots;
  const bool active = fq_t < FQ && h_t < a.OH;
  const int fq = active ? fq_t : 0, h = active ? h_t : 0;

  // accumulators as pairs of output channels: the packed fp32 FMA of sm_100 (two independent,
  // individually rounded fused multiply-adds per instruction) halves the FMA instruction count
  float2 acc[FPT / 2][kItemOW];
#pragma unroll
  for (int j = 0; j < FPT / 2; ++j)
#pragma unroll
    for (int w = 0; w < kItemOW; ++w) acc[j][w] = make_float2(0.f, 0.f);

  const int KH = KHT > 0 ? KHT : a.KH;
  const int KW = KHT > 0 ? kItemKW : a.KW;  // the compile-time form is the square 3x3 filter
  const int plane_step = (a.H - KH) * kRowsPitch;  // from the last filter row of a channel to the next channel
  auto channels = [&](int c0, int c1) {
    // running pointers: input row (c, h + kh) and the taps (c, kh, kw = 0) of filter FPT * fq
    const float* rp = Is + (c0 * a.H + h) * kRowsPitch;
    const float* wrow = Ws + (size_t)(fq * FPT) * wp + c0 * KH * KW;
    for (int c = c0; c < c1; ++c, rp += plane_step) {
#pragma unroll
      for (int kh = 0; kh < KH; ++kh, rp += kRowsPitch, wrow += KW) {
        const float4* row = reinterpret_cast<const float4*>(rp);
        float x[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 v = row[q];
          x[4 * q] = v.x; x[4 * q + 1] = v.y; x[4 * q + 2] = v.z; x[4 * q + 3] = v.w;
        }
#pragma unroll
        for (int kw = 0; kw < kItemKW; ++kw) {
          if (kw < KW) {
            float2 wv[FPT / 2];
#pragma unroll
            for (int j = 0; j < FPT / 2; ++j) wv[j] = make_float2(wrow[(2 * j) * wp + kw], wrow[(2 * j + 1) * wp + kw]);
#pragma unroll
            for (int w = 0; w < kItemOW; ++w) {
              const float2 xx = make_float2(x[w + kw], x[w + kw]);
#pragma unroll
              for (int j = 0; j < FPT / 2; ++j) acc[j][w] = __ffma2_rn(xx, wv[j], acc[j][w]);
            }
          }
        }
      }
    }
  };
  const int cq = a.C / 4;
  cp_async_wait_group<3>(); __syncthreads(); if (active) channels(0, cq);
  cp_async_wait_group<2>(); __syncthreads(); if (active) channels(cq, 2 * cq);
  cp_async_wait_group<1>(); __syncthreads(); if (active) channels(2 * cq, 3 * cq);
  cp_async_wait_group<0>(); __syncthreads(); if (active) channels(3 * cq, a.C);
  __syncthreads();  // every thread is done with the input planes: reuse them for the output tile

  // output tile of the item, dense (f, oh, ow): F * OH * OW floats (<= C * H * kRowsPitch)
  float* Os = Is;
  const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
  if (active) {
#pragma unroll
    for (int j = 0; j < FPT; ++j) {
      const int f = fq * FPT + j;
      const float bias = has_bias ? __ldg(a.bias + g * F + f) : 0.f;
      float* o = Os + ((size_t)f * a.OH + h) * a.OW;
#pragma unroll
      for (int w = 0; w < kItemOW; ++w) {
        const float v = (j & 1) ? acc[j >> 1][w].y : acc[j >> 1][w].x;
        if (w < a.OW) o[w] = a.accumulate ? v : apply_epilogue_rt(a.epi, v, bias);
      }
    }
  }
  __syncthreads();
  const int out_elems = F * a.OH * a.OW;
  float* Og = a.O + (size_t)item * out_elems;
  if (!a.accumulate && (out_elems & 3) == 0 && (((uintptr_t)a.O) & 15) == 0) {
    for (int i = tid; i < out_elems / 4; i += kItemThreads)
      reinterpret_cast<float4*>(Og)[i] = reinterpret_cast<const float4*>(Os)[i];
  } else if (!a.accumulate) {
    for (int i = tid; i < out_elems; i += kItemThreads) Og[i] = Os[i];
  } else {
    // O = epilogue(O + conv): the bias index needs f again
    const int per_f = a.OH * a.OW;
    for (int i = tid; i < out_elems; i += kItemThreads) {
      const float bias = has_bias ? __ldg(a.bias + g * F + i / per_f) : 0.f;
      Og[i] = apply_epilogue_rt(a.epi, Os[i] + Og[i], bias);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// item kernel, channels split over four thread groups: for launches with about one item per SM or fewer
// ------------------------------------------------------------------------------------------------
// With few items (the 4-image shard of an 8-GPU run has 128) every SM holds one CTA of the item kernel: four
// warps that each run the 48 (channel, filter row) steps of their thread tile one after the other, with nothing
// to hide the shared-memory latency of a step behind: 12.9 us for 128 items, against 26 us for 1024.  Here an
// item gets 512 threads: four groups of 128 with the item kernel's thread tile (one output row x two output
// channels), group q taking channels [q C/4, (q+1) C/4) -- exactly the quarter of the input planes that the q-th
// cp.async group brings in.  The four partial tiles are added through shared memory in the fixed order
// q = 0, 1, 2, 3 (the same bits on every run), with bias, and leave in 128-bit coalesced stores.
constexpr int kSplitGroups = 4;
template <int KHT>
__global__ void __launch_bounds__(128 * kSplitGroups) group_conv_item_split_kernel(ConvArgs a) {
  extern __shared__ __align__(16) float smem[];
  pdl_sync();  // launched as a programmatic dependent: wait for the preceding kernel before any global access
  const int item = blockIdx.x;  // n * G + g
  const int g = item % a.G;
  const int taps = a.C * a.KH * a.KW;
  const int F = a.F;
  const int wp = taps + 4;                // filters in their global (f, tap) order, rows padded (see the item kernel)
  float* Ws = smem;                       // [F][wp]
  float* Is = smem + (size_t)F * wp;      // [C][H][kRowsPitch]
  const int out_elems = F * a.OH * a.OW;
  float* Ps = Is + (size_t)a.C * a.H * kRowsPitch;  // [kSplitGroups][out_elems] partial tiles
  const int tid = threadIdx.x, nt = 128 * kSplitGroups;
  const int q = tid >> 7, t = tid & 127;  // channel quarter of this thread's group, thread within the group

  const float* Wg = a.W + (size_t)g * F * taps;
  const int tq = taps >> 2;
  for (int i = tid; i < F * tq; i += nt) {
    const int f = i / tq, piece = i - f * tq;
    cp_async_16(Ws + (size_t)f * wp + 4 * piece, Wg + (size_t)f * taps + 4 * piece);
  }
  const float* Ig = a.I + (size_t)item * a.C * a.H * a.Wd;
  const int rows = a.C * a.H;
  for (int i = tid; i < rows * 4; i += nt)  // four 16-byte pieces per row of 16 floats
    cp_async_16(Is + (size_t)(i >> 2) * kRowsPitch + 4 * (i & 3), Ig + (size_t)(i >> 2) * 16 + 4 * (i & 3));

  const int FQ = F / 2;
  const int hslots = (a.OH + 7) & ~7;
  const int fq_t = t / hslots, h_t = t - fq_t * hslots;
  const bool active = fq_t < FQ && h_t < a.OH;
  const int fq = active ? fq_t : 0, h = active ? h_t : 0;
  float2 acc[kItemOW];
#pragma unroll
  for (int w = 0; w < kItemOW; ++w) acc[w] = make_float2(0.f, 0.f);
  const int KH = KHT > 0 ? KHT : a.KH;
  const int KW = KHT > 0 ? kItemKW : a.KW;
  const int plane_step = (a.H - KH) * kRowsPitch;
  cp_async_wait_all();
  __syncthreads();
  if (active) {
    const int cq = a.C / kSplitGroups, c0 = q * cq;
    const float* rp = Is + (c0 * a.H + h) * kRowsPitch;
    const float* wrow = Ws + (size_t)(fq * 2) * wp + c0 * KH * KW;
    for (int c = c0; c < c0 + cq; ++c, rp += plane_step) {
#pragma unroll
      for (int kh = 0; kh < KH; ++kh, rp += kRowsPitch, wrow += KW) {
        const float4* row = reinterpret_cast<const float4*>(rp);
        float x[16];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float4 v = row[k];
          x[4 * k] = v.x; x[4 * k + 1] = v.y; x[4 * k + 2] = v.z; x[4 * k + 3] = v.w;
        }
#pragma unroll
        for (int kw = 0; kw < kItemKW; ++kw) {
          if (kw < KW) {
            const float2 wv = make_float2(wrow[kw], wrow[wp + kw]);
#pragma unroll
            for (int w = 0; w < kItemOW; ++w) acc[w] = __ffma2_rn(make_float2(x[w + kw], x[w + kw]), wv, acc[w]);
          }
        }
      }
    }
    // this group's partial tile, dense (f, oh, ow)
    float* o0 = Ps + (size_t)q * out_elems + ((size_t)(fq * 2) * a.OH + h) * a.OW;
    float* o1 = o0 + (size_t)a.OH * a.OW;
#pragma unroll
    for (int w = 0; w < kItemOW; ++w)
      if (w < a.OW) { o0[w] = acc[w].x; o1[w] = acc[w].y; }
  }
  __syncthreads();
  const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
  const int per_f = a.OH * a.OW;
  float* Og = a.O + (size_t)item * out_elems;
  if ((out_elems & 3) == 0 && (per_f & 3) == 0 && (((uintptr_t)a.O) & 15) == 0) {
    for (int i = tid; i < out_elems / 4; i += nt) {
      float4 v = reinterpret_cast<const float4*>(Ps)[i];
#pragma unroll
      for (int k = 1; k < kSplitGroups; ++k) {
        const float4 u = reinterpret_cast<const float4*>(Ps + (size_t)k * out_elems)[i];
        v.x += u.x; v.y += u.y; v.z += u.z; v.w += u.w;
      }
      const float bias = has_bias ? __ldg(a.bias + g * F + (4 * i) / per_f) : 0.f;  // four outputs of one channel
      float4* dst = reinterpret_cast<float4*>(Og) + i;
      if (a.accumulate) {
        const float4 old = *dst;
        v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
      }
      v.x = apply_epilogue_rt(a.epi, v.x, bias); v.y = apply_epilogue_rt(a.epi, v.y, bias);
      v.z = apply_epilogue_rt(a.epi, v.z, bias); v.w = apply_epilogue_rt(a.epi, v.w, bias);
      *dst = v;
    }
  } else {
    for (int i = tid; i < out_elems; i += nt) {
      float v = Ps[i];
#pragma unroll
      for (int k = 1; k < kSplitGroups; ++k) v += Ps[(size_t)k * out_elems + i];
      const float bias = has_bias ? __ldg(a.bias + g * F + i / per_f) : 0.f;
      if (a.accumulate) v += Og[i];
      Og[i] = apply_epilogue_rt(a.epi, v, bias);
    }
  }
}

size_t item_split_smem(const tcb200_problem_t& p) {
  const int64_t C = p.conv[2], F = p.conv[3], H = p.conv[4], KH = p.conv[6], KW = p.conv[7];
  const int64_t OH = H - KH + 1, OW = p.conv[5] - KW + 1;
  return sizeof(float) * (size_t)((C * KH * KW + 4) * F + C * H * kRowsPitch + kSplitGroups * F * OH * OW);
}

// ------------------------------------------------------------------------------------------------
// multi-item kernel: one CTA per SM-sized run of items, W = 16 in registers, OW <= 14, KW <= 3
// ------------------------------------------------------------------------------------------------
// What the item kernel's profile asked for (FMA pipe 63 % busy; shared memory at 60 % of its wavefront rate, i.e.
// the two co-limit; two of sixteen lanes idle because 14 output rows are padded to 16 thread slots; a single
// wave of 1024 small CTAs that loads, computes and stores in lock-step):
//  * a thread owns one output row of FOUR output channels (56 accumulators as 28 packed pairs): per input
//    row it loads 16 + 12 words from shared memory for 168 multiply-adds, half the words per multiply-add of
//    the two-channel tile, so the FMA pipe, not shared memory, is the limit;
//  * a CTA owns `ipc` consecutive items of the (g, n) order (1024 items / 148 SMs -> 7): every SM gets the same
//    amount of work in ONE CTA, threads are numbered densely over (item, channel quad, row) so that no lane
//    idles, and the filters of the (at most two) groups the run touches are staged once per CTA, transposed
//    to [tap][f] so that a thread's four channels are one 128-bit load;
//  * the input planes of all items arrive in four cp.async groups of C/4 channels; the channel loop starts
//    when the first has landed, the other three land under the multiply-adds;
//  * the output tiles go back through shared memory (each item's own input slab) and leave as one bulk copy
//    per item (cp.async.bulk shared -> global), issued by one thread.
constexpr int kMultiMaxThreads = 512;
constexpr int kMultiWPitch = 20;  // floats per tap row of the transposed filters: F <= 16, conflict-free writes

// PACKED: accumulate pairs of output channels with the packed fp32x2 FMA (half the FMA instructions, one
// register move per input word to duplicate it); else plain FMAs (no moves, twice the FMA instructions).
template <int KHT, bool PACKED>
__global__ void __launch_bounds__(kMultiMaxThreads, 1) group_conv_multi_kernel(ConvArgs a, int ipc, int N, int total) {
  extern __shared__ __align__(16) float smem[];
  pdl_sync();  // launched as a programmatic dependent: wait for the preceding kernel before any global access
  const int tid = threadIdx.x, nt = blockDim.x;
  const int taps = a.C * a.KH * a.KW;
  const int F = a.F;
  const int w0 = blockIdx.x * ipc;                 // first work index of this CTA; work w -> (g = w / N, n = w % N)
  const int mine = min(ipc, total - w0);           // items of this CTA
  const int g0 = w0 / N;                           // first group the run touches (it touches g0 and maybe g0 + 1)
  const int groups = (w0 + mine - 1) / N - g0 + 1; // 1 or 2 (ipc <= N, checked by the plan)
  float* Ws = smem;                                // [2][taps][kMultiWPitch]
  float* Is = smem + 2 * (size_t)taps * kMultiWPitch;  // [ipc][C][H][kRowsPitch]
  const int slab = a.C * a.H * kRowsPitch;         // floats per item in shared memory
  const int in_elems = a.C * a.H * 16;             // floats per item in global memory
  auto item_of = [&](int j) { const int w = w0 + j; return (w % N) * a.G + w / N; };

  // input planes: quarter q of every item, 16-byte pieces, one commit group per quarter
  const int rows_q = (a.C / 4) * a.H;
#pragma unroll 1
  for (int q = 0; q < 4; ++q) {
    const int pieces = mine * rows_q * 4;
    for (int i = tid; i < pieces; i += nt) {
      const int j = i / (rows_q * 4), rem = i - j * rows_q * 4;
      const int r = q * rows_q + (rem >> 2), piece = rem & 3;
      cp_async_16(Is + (size_t)j * slab + (size_t)r * kRowsPitch + 4 * piece,
                  a.I + (size_t)item_of(j) * in_elems + (size_t)r * 16 + 4 * piece);
    }
    cp_async_commit();
  }
  // filters of the run's groups, transposed on the way: thread -> (f = i % F, four consecutive taps).  The
  // 16 threads of one piece index write 16 consecutive words of a tap row, the next piece index lands 80
  // words further: no bank is hit twice.
  {
    const int tq = taps >> 2;  // taps % 4 == 0 because C % 4 == 0
    for (int i = tid; i < groups * F * tq; i += nt) {
      const int s = i / (F * tq), rem = i - s * F * tq;
      const int piece = rem / F, f = rem - piece * F;
      const float4 v = __ldg(reinterpret_cast<const float4*>(a.W + ((size_t)(g0 + s) * F + f) * taps) + piece);
      float* dst = Ws + ((size_t)s * taps + 4 * piece) * kMultiWPitch + f;
      dst[0] = v.x; dst[kMultiWPitch] = v.y; dst[2 * kMultiWPitch] = v.z; dst[3 * kMultiWPitch] = v.w;
    }
  }

  // thread -> (item j, channel quad fq, output row h), densely numbered
  const int FQ = F >> 2;
  const int tpi = FQ * a.OH;  // threads per item
  const int j = tid / tpi, rem = tid - j * tpi;
  const bool active = j < mine;
  const int fq = active ? rem / a.OH : 0, h = active ? rem - (rem / a.OH) * a.OH : 0;
  const int jj = active ? j : 0;
  const int gslot = (w0 + jj) / N - g0;

  float2 acc[2][kItemOW];
#pragma unroll
  for (int p = 0; p < 2; ++p)
#pragma unroll
    for (int w = 0; w < kItemOW; ++w) acc[p][w] = make_float2(0.f, 0.f);

  const int KH = KHT > 0 ? KHT : a.KH;
  const int KW = KHT > 0 ? kItemKW : a.KW;
  const int plane_step = (a.H - KH) * kRowsPitch;
  const float* in = Is + (size_t)jj * slab;
  const float* wt = Ws + (size_t)gslot * taps * kMultiWPitch + 4 * fq;
  auto channels = [&](int c0, int c1) {
    const float* rp = in + (c0 * a.H + h) * kRowsPitch;
    const float* wrow = wt + (size_t)(c0 * KH * KW) * kMultiWPitch;
    for (int c = c0; c < c1; ++c, rp += plane_step) {
#pragma unroll
      for (int kh = 0; kh < KH; ++kh, rp += kRowsPitch) {
        const float4* row = reinterpret_cast<const float4*>(rp);
        float x[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 v = row[q];
          x[4 * q] = v.x; x[4 * q + 1] = v.y; x[4 * q + 2] = v.z; x[4 * q + 3] = v.w;
        }
#pragma unroll
        for (int kw = 0; kw < kItemKW; ++kw) {
          if (kw < KW) {
            const float4 wv = *reinterpret_cast<const float4*>(wrow);
            wrow += kMultiWPitch;
            const float2 w01 = make_float2(wv.x, wv.y), w23 = make_float2(wv.z, wv.w);
#pragma unroll
            for (int w = 0; w < kItemOW; ++w) {
              if (PACKED) {
                const float2 xx = make_float2(x[w + kw], x[w + kw]);
                acc[0][w] = __ffma2_rn(xx, w01, acc[0][w]);
                acc[1][w] = __ffma2_rn(xx, w23, acc[1][w]);
              } else {
                const float xv = x[w + kw];
                acc[0][w].x = fmaf(xv, wv.x, acc[0][w].x);
                acc[0][w].y = fmaf(xv, wv.y, acc[0][w].y);
                acc[1][w].x = fmaf(xv, wv.z, acc[1][w].x);
                acc[1][w].y = fmaf(xv, wv.w, acc[1][w].y);
              }
            }
          }
        }
      }
    }
  };
  const int cq = a.C / 4;
  cp_async_wait_group<3>(); __syncthreads(); if (active) channels(0, cq);   // (the sync also publishes the filters)
  cp_async_wait_group<2>(); __syncthreads(); if (active) channels(cq, 2 * cq);
  cp_async_wait_group<1>(); __syncthreads(); if (active) channels(2 * cq, 3 * cq);
  cp_async_wait_group<0>(); __syncthreads(); if (active) channels(3 * cq, a.C);
  __syncthreads();  // every thread is done with the input planes: each item's slab now takes its output tile

  const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
  const int out_elems = F * a.OH * a.OW;
  if (active) {
    float* Os = Is + (size_t)j * slab;
    const int g = (w0 + j) / N;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int f = fq * 4 + k;
      const float bias = has_bias ? __ldg(a.bias + g * F + f) : 0.f;
      float* o = Os + ((size_t)f * a.OH + h) * a.OW;
#pragma unroll
      for (int w = 0; w < kItemOW; ++w) {
        const float v = (k & 1) ? acc[k >> 1][w].y : acc[k >> 1][w].x;
        if (w < a.OW) o[w] = apply_epilogue_rt(a.epi, v, bias);
      }
    }
  }
  // the output tiles are read by the bulk copies (async proxy): order the generic writes before them
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if ((out_elems & 3) == 0 && (((uintptr_t)a.O) & 15) == 0) {
    if (tid == 0) {
      for (int k = 0; k < mine; ++k)
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                         a.O + (size_t)item_of(k) * out_elems),
                     "r"(smem_u32(Is + (size_t)k * slab)), "r"((uint32_t)out_elems * 4)
                     : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // written before the CTA (and its memory) goes away
    }
  } else {
    for (int i = tid; i < mine * out_elems; i += nt) {
      const int k = i / out_elems, e = i - k * out_elems;
      a.O[(size_t)item_of(k) * out_elems + e] = Is[(size_t)k * slab + e];
    }
  }
}

// Items per CTA of the multi-item kernel for this problem on `sms` multiprocessors (0: the kernel does not apply).
int multi_ipc(const tcb200_problem_t& p, int sms);

// Threads the two-channels-per-thread form of the item kernel would use (it takes up to 128).
int item_two_threads(const tcb200_problem_t& p) {
  return (int)((p.conv[3] / 2) * ((p.conv[4] - p.conv[6] + 1 + 7) / 8 * 8));
}

bool unit_stride(const tcb200_problem_t& p) { return conv_sh(p) == 1 && conv_sw(p) == 1; }

bool item_ok(const tcb200_problem_t& p) {
  if (!unit_stride(p)) return false;
  const int64_t C = p.conv[2], F = p.conv[3], H = p.conv[4], W = p.conv[5], KH = p.conv[6], KW = p.conv[7];
  const int64_t OH = H - KH + 1, OW = W - KW + 1;
  return W == 16 && OW <= kItemOW && KW <= kItemKW && F % 4 == 0 && C % 4 == 0 &&
         (F / 4) * ((OH + 7) / 8 * 8) <= kItemThreads &&
         F * OH * OW <= C * H * kRowsPitch &&
         sizeof(float) * (size_t)((C * KH * KW + 4) * F + C * H * kRowsPitch) <= 48 * 1024;
}

// the channel-split form of the item kernel: the item kernel's two-channel tile must fit 128 threads
bool item_split_ok(const tcb200_problem_t& p) {
  return item_ok(p) && item_two_threads(p) <= 128 && p.conv[2] % (4 * kSplitGroups) == 0 &&
         item_split_smem(p) <= 160 * 1024;
}

int multi_threads(const tcb200_problem_t& p, int ipc) {
  return (int)round_up((int64_t)ipc * (p.conv[3] / 4) * (p.conv[4] - p.conv[6] + 1), 32);
}
size_t multi_smem(const tcb200_problem_t& p, int ipc) {
  return sizeof(float) * (2 * (size_t)(p.conv[2] * p.conv[6] * p.conv[7]) * kMultiWPitch +
                          (size_t)ipc * p.conv[2] * p.conv[4] * kRowsPitch);
}
int multi_ipc(const tcb200_problem_t& p, int sms) {
  if (!item_ok(p) || p.accumulate || p.conv[3] > 16) return 0;
  const int64_t items = p.conv[0] * p.conv[1];
  // worth it from about four items per SM on; below that the one-item CTAs fill the SMs better
  if (items < 4 * (int64_t)sms) return 0;
  int ipc = (int)ceil_div(items, sms);
  while (ipc > 1 && (ipc > p.conv[0] || multi_threads(p, ipc) > kMultiMaxThreads || multi_smem(p, ipc) > 200 * 1024)) --ipc;
  return ipc >= 2 ? ipc : 0;
}

bool rows_ok(const tcb200_problem_t& p) {
  if (!unit_stride(p)) return false;
  const int64_t C = p.conv[2], F = p.conv[3], H = p.conv[4], W = p.conv[5], KH = p.conv[6], KW = p.conv[7];
  const int64_t OH = H - KH + 1;
  return W <= kRowsMaxW && KW <= 4 && F % 4 == 0 && (F / 4) * OH <= 256 &&
         sizeof(float) * (size_t)(C * KH * KW * F + C * H * kRowsPitch) <= 96 * 1024;
}

// n per CTA: as many as fit 256 threads and the shared-memory budget
int rows_n_per_cta(const tcb200_problem_t& p, int want, size_t* bytes) {
  const int64_t C = p.conv[2], F = p.conv[3], H = p.conv[4], KH = p.conv[6], KW = p.conv[7];
  const int64_t per_n = (F / 4) * (H - KH + 1);
  int64_t n = want > 0 ? want : 2;
  n = std::max<int64_t>(1, std::min<int64_t>(n, std::min<int64_t>(256 / per_n, p.conv[0])));
  auto need = [&](int64_t k) { return sizeof(float) * (size_t)(C * KH * KW * F + k * C * H * kRowsPitch); };
  while (n > 1 && need(n) > 96 * 1024) --n;
  if (bytes) *bytes = need(n);
  return (int)n;
}

bool valid(const tcb200_problem_t& p) {
  for (int i = 0; i < 8; ++i)
    if (p.conv[i] <= 0 || p.conv[i] > (1 << 24)) return false;
  if (p.conv_stride[0] < 0 || p.conv_stride[1] < 0 || p.conv_stride[0] > (1 << 16) || p.conv_stride[1] > (1 << 16))
    return false;
  return p.conv[4] >= p.conv[6] && p.conv[5] >= p.conv[7] &&
         p.conv[0] * p.conv[1] < (1ll << 31);
}

constexpr size_t kSmemBudget = 96 * 1024;

// Largest band of output rows whose halo + filters fit the shared-memory budget.
int pick_band(const tcb200_problem_t& p, int ft, size_t* bytes) {
  const int64_t C = p.conv[2], F = p.conv[3], H = p.conv[4], W = p.conv[5], KH = p.conv[6],
                KW = p.conv[7];
  const int64_t OH = conv_oh(p), SH = conv_sh(p);
  const int64_t Fp = round_up(F, ft);
  const size_t wbytes = sizeof(float) * (size_t)(C * KH * KW * Fp);
  for (int64_t band = OH; band >= 1; band = (band == 1 ? 0 : (band + 1) / 2)) {
    const size_t b = wbytes + sizeof(float) * (size_t)(C * ((band - 1) * SH + KH) * W);
    if (b <= kSmemBudget) {
      if (bytes) *bytes = b;
      return (int)band;
    }
  }
  return 0;
}

}  // namespace

int group_conv_query(const tcb200_problem_t& p, tcb200_tile_t* out, int max, int* n) {
  if (!valid(p)) return TCB200_ERR_INVALID_ARGUMENT;
  int cnt = 0;
  // tensor-core form with the filters stationary in tensor memory (stages = 3: its accumulator ring)
  if (group_conv_tap_rows_ok(p)) {
    if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_TCGEN05_TS, 128, 128, 8, 3, 512, 3};
    ++cnt;
  }
  if (item_ok(p)) {  // stages = 4: one item per CTA, input staged in four cp.async groups
    if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_SIMT, 0, 4, 1, 4, kItemThreads, 0};
    ++cnt;
    if (item_two_threads(p) <= 128) {
      if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_SIMT, 0, 2, 1, 4, 128, 0};
      ++cnt;
    }
  }
  // stages = 5: a run of items per CTA (bk = items per CTA, chosen by the plan; bm = 1: plain FMAs).  Measured
  // on the benchmark shape: 29.9 us (packed FMAs) / 32.7 us (plain) against 26.0 us for the one-item CTAs: its
  // 13 warps per SM run in lock-step between CTA-wide barriers, where seven independent small CTAs drift apart.
  if (multi_ipc(p, sm_count(-1)) > 0) {
    if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_SIMT, 0, 4, 0, 5, 0, 0};
    ++cnt;
    if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_SIMT, 1, 4, 0, 5, 0, 0};
    ++cnt;
  }
  // stages = 6: one item per CTA of 512 threads, the channels split over four thread groups (few items)
  if (item_split_ok(p)) {
    if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_SIMT, 0, 2, 1, 6, 128 * kSplitGroups, 0};
    ++cnt;
  }
  if (rows_ok(p)) {
    // bk = n per CTA of the rows kernel
    const int ns[] = {2, 1, 4};
    for (int k : ns) {
      if (k > p.conv[0] || k * (p.conv[3] / 4) * (p.conv[4] - p.conv[6] + 1) > 256) continue;
      if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_SIMT, 0, 0, k, 0, 0, 0};
      ++cnt;
    }
  }
  // tensor-core implicit GEMM: correct and fp32-accurate, but hand-off latency bound on small
  // problems (see group_conv_tcgen05.cu); the sweep can still pick it where it wins
  if (group_conv_tc_ok(p)) {
    if (cnt < max && out)
      out[cnt] = tcb200_tile_t{TCB200_VARIANT_TCGEN05_TS, 128, (int)p.conv[3], 8, 4, 448, 3};
    ++cnt;
  }
  const int threads[] = {256, 224, 128};
  for (int t : threads) {
    if (cnt < max && out) out[cnt] = tcb200_tile_t{TCB200_VARIANT_SIMT, 0, 0, 0, 0, t, 0};
    ++cnt;
  }
  *n = cnt;
  return TCB200_OK;
}

int group_conv_plan(Plan& plan) {
  const tcb200_problem_t& p = plan.p;
  if (!valid(p)) return TCB200_ERR_INVALID_ARGUMENT;
  if (p.epilogue == TCB200_EPI_RELU) return TCB200_ERR_UNSUPPORTED;
  tcb200_tile_t& t = plan.tile;
  // default where it applies: the tensor-core kernel with the filters stationary in tensor memory (measured
  // against the one-item SIMT kernels on 1024 / 512 / 256 / 128 items: 18.35 / 12.25 / 8.3 / 6.06 us against
  // 26.1 / 16.8 / 10.6 / 9.9 us)
  if (t.variant == TCB200_VARIANT_AUTO && group_conv_tap_rows_ok(p)) { t.variant = TCB200_VARIANT_TCGEN05_TS; t.stages = 3; }
  if (t.variant == TCB200_VARIANT_AUTO && !rows_ok(p) && group_conv_tc_ok(p)) t.variant = TCB200_VARIANT_TCGEN05_TS;
  if (t.variant == TCB200_VARIANT_TCGEN05_TS && t.stages == 3) return group_conv_tap_rows_plan(plan);
  if (t.variant == TCB200_VARIANT_TCGEN05_TS) return group_conv_tc_plan(plan);
  if (t.variant == TCB200_VARIANT_AUTO) {
    t.variant = TCB200_VARIANT_SIMT;
    t.threads = 256;
    t.bk = rows_ok(p) ? 2 : 0;
    if (item_ok(p)) {
      t.bk = 1; t.stages = 4;
      // more warps in flight per item when the item has the work for them
      t.threads = item_two_threads(p) > kItemThreads && item_two_threads(p) <= 128 ? 128 : kItemThreads;
      // about one item per SM or fewer: more threads per item (channel split) instead of more items per SM
      if (item_split_ok(p) && p.conv[0] * p.conv[1] <= 2 * (int64_t)plan.sms) { t.stages = 6; t.threads = 128 * kSplitGroups; }
    }
  }
  if (t.variant != TCB200_VARIANT_SIMT) return TCB200_ERR_UNSUPPORTED;
  if (t.stages == 6) {  // item kernel, channels split over four thread groups
    if (!item_split_ok(p)) return TCB200_ERR_UNSUPPORTED;
    t.bm = 0; t.bn = 2; t.bk = 1; t.threads = 128 * kSplitGroups;
    plan.launch.grid = dim3((unsigned)(p.conv[0] * p.conv[1]), 1, 1);
    plan.launch.block = dim3(t.threads, 1, 1);
    plan.launch.smem = item_split_smem(p);
    plan.kernel_id = 105;
    return TCB200_OK;
  }
  if (t.stages == 5) {  // multi-item kernel
    const int ipc = multi_ipc(p, plan.sms);
    if (ipc == 0) return TCB200_ERR_UNSUPPORTED;
    t.bm = t.bm ? 1 : 0; t.bn = 4; t.bk = ipc;
    t.threads = multi_threads(p, ipc);
    plan.launch.grid = dim3((unsigned)ceil_div(p.conv[0] * p.conv[1], ipc), 1, 1);
    plan.launch.block = dim3(t.threads, 1, 1);
    plan.launch.smem = multi_smem(p, ipc);
    plan.kernel_id = t.bm ? 104 : 103;
    return TCB200_OK;
  }
  if (t.bk == 1 && t.stages == 4) {  // item kernel
    if (!item_ok(p)) return TCB200_ERR_UNSUPPORTED;
    if (p.conv[0] * p.conv[1] > 0x7fffffffll) return TCB200_ERR_TOO_LARGE;
    // threads = 128: two output channels per thread (bn = 2), else four
    const bool two = t.threads == 128 && item_two_threads(p) <= 128;
    t.bm = 0; t.bn = two ? 2 : 4;
    t.threads = two ? 128 : kItemThreads;
    plan.launch.grid = dim3((unsigned)(p.conv[0] * p.conv[1]), 1, 1);
    plan.launch.block = dim3(t.threads, 1, 1);
    plan.launch.smem = sizeof(float) * (size_t)((p.conv[2] * p.conv[6] * p.conv[7] + 4) * p.conv[3] +
                                                 p.conv[2] * p.conv[4] * kRowsPitch);
    plan.kernel_id = two ? 102 : 101;
    return TCB200_OK;
  }
  t.stages = 0;
  if (t.bk > 0) {  // rows kernel
    if (!rows_ok(p)) return TCB200_ERR_UNSUPPORTED;
    size_t bytes = 0;
    const int npc = rows_n_per_cta(p, t.bk, &bytes);
    const int per_n = (int)((p.conv[3] / 4) * (p.conv[4] - p.conv[6] + 1));
    t.bk = npc;
    t.bm = 0; t.bn = 4;
    t.threads = (int)round_up((int64_t)npc * per_n, 32);
    if (ceil_div(p.conv[0], npc) > 65535) return TCB200_ERR_TOO_LARGE;
    plan.launch.grid = dim3((unsigned)p.conv[1], (unsigned)ceil_div(p.conv[0], npc), 1);
    plan.launch.block = dim3(t.threads, 1, 1);
    plan.launch.smem = bytes;
    plan.kernel_id = 100;
    return TCB200_OK;
  }
  if (t.threads <= 0) t.threads = 256;
  if (t.threads > 256 || t.threads % 32) return TCB200_ERR_INVALID_ARGUMENT;
  const int ft = p.conv[3] % 4 == 0 ? 4 : 1;
  size_t bytes = 0;
  const int band = pick_band(p, ft, &bytes);
  if (band == 0) return TCB200_ERR_TOO_LARGE;
  const int64_t OH = conv_oh(p);
  if (ceil_div(OH, band) > 65535) return TCB200_ERR_TOO_LARGE;
  t.bm = band;
  t.bn = ft;
  plan.launch.grid = dim3((unsigned)(p.conv[0] * p.conv[1]), (unsigned)ceil_div(OH, band), 1);
  plan.launch.block = dim3(t.threads, 1, 1);
  plan.launch.smem = bytes;
  plan.kernel_id = ft;
  return TCB200_OK;
}

int group_conv_launch(const Plan& plan, const float* I, const float* W, const float* bias,
                      float* O, cudaStream_t s, int* dev_status) {
  if (plan.kernel_id == 200) return group_conv_tc_launch(plan, I, W, bias, O, s, dev_status);
  const tcb200_problem_t& p = plan.p;
  ConvArgs a;
  a.I = I; a.W = W; a.bias = bias; a.O = O;
  a.G = (int)p.conv[1]; a.C = (int)p.conv[2]; a.F = (int)p.conv[3];
  a.H = (int)p.conv[4]; a.Wd = (int)p.conv[5]; a.KH = (int)p.conv[6]; a.KW = (int)p.conv[7];
  a.SH = (int)conv_sh(p); a.SW = (int)conv_sw(p);
  a.OH = (int)conv_oh(p); a.OW = (int)conv_ow(p);
  a.band = plan.tile.bm;
  a.epi = p.epilogue; a.accumulate = p.accumulate;
  // The item kernel stages I and W with 16-byte asynchronous copies.  A dense tensor may still start at any
  // 4-byte offset of a larger buffer (a view): such a launch runs on the band kernel, which uses 4-byte loads.
  const bool multi = plan.kernel_id == 103 || plan.kernel_id == 104;
  const bool item_misaligned = ((plan.kernel_id == 101 || plan.kernel_id == 102 || plan.kernel_id == 105 || multi) &&
                                ((((uintptr_t)I) | ((uintptr_t)W)) & 15) != 0) ||
                               (plan.kernel_id == 201 && !group_conv_tap_rows_aligned(I, W, O));
  if (plan.kernel_id == 201 && !item_misaligned) return group_conv_tap_rows_launch(plan, I, W, bias, O, s, dev_status);
  if (plan.kernel_id == 105 && !item_misaligned) {
    const bool k33 = a.KH == 3 && a.KW == 3;
    auto fn = k33 ? group_conv_item_split_kernel<3> : group_conv_item_split_kernel<0>;
    static std::atomic<uint64_t> split_configured[2];
    TCB200_CUDA_TRY(ensure_dynamic_smem(fn, 160 * 1024, plan.device, split_configured[k33]));
    TCB200_CUDA_TRY(launch_pdl(fn, plan.launch.grid, plan.launch.block, plan.launch.smem, s, a));
    return TCB200_OK;
  }
  if (multi && !item_misaligned) {
    const bool k33 = a.KH == 3 && a.KW == 3, packed = plan.kernel_id == 103;
    auto fn = k33 ? (packed ? group_conv_multi_kernel<3, true> : group_conv_multi_kernel<3, false>)
                  : (packed ? group_conv_multi_kernel<0, true> : group_conv_multi_kernel<0, false>);
    static std::atomic<uint64_t> multi_configured[4];
    TCB200_CUDA_TRY(ensure_dynamic_smem(fn, 200 * 1024, plan.device, multi_configured[(k33 ? 2 : 0) + (packed ? 1 : 0)]));
    TCB200_CUDA_TRY(launch_pdl(fn, plan.launch.grid, plan.launch.block, plan.launch.smem, s, a, plan.tile.bk,
                               (int)p.conv[0], (int)(p.conv[0] * p.conv[1])));
    return TCB200_OK;
  }
  if ((plan.kernel_id == 101 || plan.kernel_id == 102) && !item_misaligned) {
    const bool k33 = a.KH == 3 && a.KW == 3;
    if (plan.kernel_id == 102) {
      if (k33) TCB200_CUDA_TRY(launch_pdl(group_conv_item_kernel<3, 2>, plan.launch.grid, plan.launch.block, plan.launch.smem, s, a));
      else TCB200_CUDA_TRY(launch_pdl(group_conv_item_kernel<0, 2>, plan.launch.grid, plan.launch.block, plan.launch.smem, s, a));
    } else {
      if (k33) TCB200_CUDA_TRY(launch_pdl(group_conv_item_kernel<3, 4>, plan.launch.grid, plan.launch.block, plan.launch.smem, s, a));
      else TCB200_CUDA_TRY(launch_pdl(group_conv_item_kernel<0, 4>, plan.launch.grid, plan.launch.block, plan.launch.smem, s, a));
    }
    TCB200_CUDA_TRY(cudaGetLastError());
    return TCB200_OK;
  }
  if (plan.kernel_id == 100) {
    static std::atomic<uint64_t> rows_configured{0};
    TCB200_CUDA_TRY(ensure_dynamic_smem(group_conv_rows_kernel, (int)kSmemBudget, plan.device, rows_configured));
    group_conv_rows_kernel<<<plan.launch.grid, plan.launch.block, plan.launch.smem, s>>>(
        a, plan.tile.bk, (int)p.conv[0]);
    TCB200_CUDA_TRY(cudaGetLastError());
    return TCB200_OK;
  }
  int ft = plan.kernel_id;
  dim3 grid = plan.launch.grid, block = plan.launch.block;
  size_t smem = plan.launch.smem;
  if (item_misaligned) {  // geometry of the band kernel for this problem, worked out here
    ft = p.conv[3] % 4 == 0 ? 4 : 1;
    const int band = pick_band(p, ft, &smem);
    if (band == 0 || ceil_div((int64_t)a.OH, band) > 65535) return TCB200_ERR_ALIGNMENT;
    a.band = band;
    grid = dim3((unsigned)(p.conv[0] * p.conv[1]), (unsigned)ceil_div((int64_t)a.OH, band), 1);
    block = dim3(256, 1, 1);
  }
  auto fn = ft == 4 ? group_conv_simt_kernel<4> : group_conv_simt_kernel<1>;
  static std::atomic<uint64_t> band_configured[2];
  TCB200_CUDA_TRY(ensure_dynamic_smem(fn, (int)kSmemBudget, plan.device, band_configured[ft == 4]));
  fn<<<grid, block, smem, s>>>(a);
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}

}  // namespace tcb200
