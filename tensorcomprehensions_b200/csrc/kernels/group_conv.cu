// K3 — grouped 2-D valid convolution, unit stride, fused bias:
//   O(n,g,f,h,w)  = sum_{c,kh,kw} I(n,g,c,h+kh,w+kw) * W1(g,f,c,kh,kw)
//   O(n,g,f,h,w) += B(g,f)
// Replaces the kernel the reference generates for tc/benchmarks/group_convolution.cc:124-132
// (library twin tc/library/group_convolution.h:26-44 with stride 1).
//
// SIMT variant: one CTA per (n, g, band of output rows).  The band's input halo
// (C x (rows+KH-1) x W) and the group's filters are staged in shared memory once; the
// filters are re-laid out as Ws[c][kh][kw][f] so one 128-bit shared load feeds four
// output channels.  Consecutive threads take consecutive output pixels, so the halo
// reads are bank-conflict free and the output stores are coalesced along w.
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
  int epi, accumulate;
};

template <int FT>
__global__ void __launch_bounds__(256) group_conv_simt_kernel(ConvArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int ng = blockIdx.x;  // n * G + g
  const int g = ng % a.G;
  const int h0 = blockIdx.y * a.band;
  const int rows = min(a.band, a.OH - h0);
  const int in_rows = rows + a.KH - 1;
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
    Is[i] = __ldg(Ig + ((size_t)c * a.H + h0) * a.Wd + r);
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
        const float* irow = Is + ((size_t)c * in_rows + h + kh) * a.Wd + w;
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

bool valid(const tcb200_problem_t& p) {
  for (int i = 0; i < 8; ++i)
    if (p.conv[i] <= 0 || p.conv[i] > (1 << 24)) return false;
  return p.conv[4] >= p.conv[6] && p.conv[5] >= p.conv[7] &&
         p.conv[0] * p.conv[1] < (1ll << 31);
}

constexpr size_t kSmemBudget = 96 * 1024;

// Largest band of output rows whose halo + filters fit the shared-memory budget.
int pick_band(const tcb200_problem_t& p, int ft, size_t* bytes) {
  const int64_t C = p.conv[2], F = p.conv[3], H = p.conv[4], W = p.conv[5], KH = p.conv[6],
                KW = p.conv[7];
  const int64_t OH = H - KH + 1;
  const int64_t Fp = round_up(F, ft);
  const size_t wbytes = sizeof(float) * (size_t)(C * KH * KW * Fp);
  for (int64_t band = OH; band >= 1; band = (band == 1 ? 0 : (band + 1) / 2)) {
    const size_t b = wbytes + sizeof(float) * (size_t)(C * (band + KH - 1) * W);
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
  if (t.variant == TCB200_VARIANT_AUTO) {
    t.variant = TCB200_VARIANT_SIMT;
    t.threads = 256;
  }
  if (t.variant != TCB200_VARIANT_SIMT) return TCB200_ERR_UNSUPPORTED;
  if (t.threads <= 0) t.threads = 256;
  if (t.threads > 256 || t.threads % 32) return TCB200_ERR_INVALID_ARGUMENT;
  const int ft = p.conv[3] % 4 == 0 ? 4 : 1;
  size_t bytes = 0;
  const int band = pick_band(p, ft, &bytes);
  if (band == 0) return TCB200_ERR_TOO_LARGE;
  const int64_t OH = p.conv[4] - p.conv[6] + 1;
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
                      float* O, cudaStream_t s) {
  const tcb200_problem_t& p = plan.p;
  ConvArgs a;
  a.I = I; a.W = W; a.bias = bias; a.O = O;
  a.G = (int)p.conv[1]; a.C = (int)p.conv[2]; a.F = (int)p.conv[3];
  a.H = (int)p.conv[4]; a.Wd = (int)p.conv[5]; a.KH = (int)p.conv[6]; a.KW = (int)p.conv[7];
  a.OH = a.H - a.KH + 1; a.OW = a.Wd - a.KW + 1;
  a.band = plan.tile.bm;
  a.epi = p.epilogue; a.accumulate = p.accumulate;
  auto fn = plan.kernel_id == 4 ? group_conv_simt_kernel<4> : group_conv_simt_kernel<1>;
  if (plan.launch.smem > 48 * 1024)
    TCB200_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kSmemBudget));
  fn<<<plan.launch.grid, plan.launch.block, plan.launch.smem, s>>>(a);
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}

}  // namespace tcb200
