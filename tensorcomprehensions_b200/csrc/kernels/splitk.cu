// Second pass of a contraction whose reduction was computed in pieces: adds S planes of partial sums in a
// fixed order and applies the epilogue.  Two producers write such planes into scratch memory owned by the plan:
//  * a tensor-core contraction whose output has too few tiles for the SMs (a 128 x 2048 x 4096 shard of the
//    transposed matmul: 16 tiles for 148 SMs) splits its reduction over S CTAs per tile (tile.split_k);
//  * a contraction that also reduces over its batch index (C(m,n) = sum_b sum_k A(b,m,k) B(b,n,k): the weight
//    gradient of a convolution, tensor_comprehensions/__init__.py:570-574) runs as a batched contraction into
//    one plane per batch entry.
#include "common.cuh"

namespace tcb200 {
namespace {

// P[s][m][n] dense planes; the S partials of every element are added in the order s = 0 .. S-1 (the same
// bits on every run), then the old output for "+=", bias and ReLU are applied as the single-pass kernels do.
struct SplitKArgs {
  const float* P;
  float* C;
  const float* bias;
  int M, N, S;
  int64_t ldc;
  int epi, bias_on_m, accumulate;
};

template <bool VEC>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(SplitKArgs a) {
  pdl_sync();  // the partial sums come from the kernel launched just before this one
  const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
  const int64_t plane = (int64_t)a.M * a.N;
  if (VEC) {
    const int n4 = a.N >> 2;
    const int64_t total = (int64_t)a.M * n4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
      const int m = (int)(i / n4), n = (int)(i - (int64_t)m * n4) * 4;
      const float4* src = reinterpret_cast<const float4*>(a.P + (int64_t)m * a.N + n);
      float4 acc = src[0];
      for (int s = 1; s < a.S; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) + s * plane);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      float4* dst = reinterpret_cast<float4*>(a.C + (int64_t)m * a.ldc + n);
      if (a.accumulate) {
        const float4 old = *dst;
        acc.x += old.x; acc.y += old.y; acc.z += old.z; acc.w += old.w;
      }
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (has_bias) {
        if (a.bias_on_m) b.x = b.y = b.z = b.w = __ldg(a.bias + m);
        else b = make_float4(__ldg(a.bias + n), __ldg(a.bias + n + 1), __ldg(a.bias + n + 2), __ldg(a.bias + n + 3));
      }
      acc.x = apply_epilogue_rt(a.epi, acc.x, b.x);
      acc.y = apply_epilogue_rt(a.epi, acc.y, b.y);
      acc.z = apply_epilogue_rt(a.epi, acc.z, b.z);
      acc.w = apply_epilogue_rt(a.epi, acc.w, b.w);
      *dst = acc;
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < plane; i += (int64_t)gridDim.x * blockDim.x) {
      const int m = (int)(i / a.N), n = (int)(i - (int64_t)m * a.N);
      float acc = a.P[i];
      for (int s = 1; s < a.S; ++s) acc += a.P[i + s * plane];
      float* dst = a.C + (int64_t)m * a.ldc + n;
      if (a.accumulate) acc += *dst;
      const float b = has_bias ? __ldg(a.bias + (a.bias_on_m ? m : n)) : 0.f;
      *dst = apply_epilogue_rt(a.epi, acc, b);
    }
  }
}

// Tail tiles of a CTA-pair launch: partial tile (s * tail_tiles + j) is a dense 256 x 128 block; output tile
// tile0 + j covers rows ((tile0 + j) / tiles_n) * 256 .. and columns ((tile0 + j) % tiles_n) * 128 ..
struct TailArgs {
  const float* P;
  float* C;
  const float* bias;
  int M, N, S, tail_tiles, tile0, tiles_n;
  int64_t ldc;
  int epi, bias_on_m, accumulate, vec;
};

__global__ void __launch_bounds__(256) tail_tiles_reduce_kernel(TailArgs a) {
  pdl_sync();  // the partial tiles come from the kernel launched just before this one
  const bool has_bias = a.epi == TCB200_EPI_BIAS || a.epi == TCB200_EPI_BIAS_RELU;
  const int j = blockIdx.y, tile = a.tile0 + j;
  const int m0 = (tile / a.tiles_n) * 256, n0 = (tile % a.tiles_n) * 128;
  const int64_t tile_elems = 256 * 128;
  const float* P0 = a.P + (int64_t)j * tile_elems;
  const int64_t split_stride = (int64_t)a.tail_tiles * tile_elems;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < 256 * 32; i += gridDim.x * blockDim.x) {
    const int r = i >> 5, c = (i & 31) << 2;
    const int m = m0 + r, n = n0 + c;
    if (m >= a.M || n >= a.N) continue;
    float4 acc = *reinterpret_cast<const float4*>(P0 + r * 128 + c);
    for (int s = 1; s < a.S; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(P0 + s * split_stride + r * 128 + c);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    float v[4] = {acc.x, acc.y, acc.z, acc.w};
    float* dst = a.C + (int64_t)m * a.ldc + n;
    if (a.vec && n + 3 < a.N) {
      float4 o = make_float4(v[0], v[1], v[2], v[3]);
      if (a.accumulate) {
        const float4 old = *reinterpret_cast<const float4*>(dst);
        o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
      }
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (has_bias) {
        if (a.bias_on_m) b.x = b.y = b.z = b.w = __ldg(a.bias + m);
        else b = make_float4(__ldg(a.bias + n), __ldg(a.bias + n + 1), __ldg(a.bias + n + 2), __ldg(a.bias + n + 3));
      }
      o.x = apply_epilogue_rt(a.epi, o.x, b.x); o.y = apply_epilogue_rt(a.epi, o.y, b.y);
      o.z = apply_epilogue_rt(a.epi, o.z, b.z); o.w = apply_epilogue_rt(a.epi, o.w, b.w);
      *reinterpret_cast<float4*>(dst) = o;
    } else {
      for (int k = 0; k < 4 && n + k < a.N; ++k) {
        float o = v[k];
        if (a.accumulate) o += dst[k];
        const float b = has_bias ? __ldg(a.bias + (a.bias_on_m ? m : n + k)) : 0.f;
        dst[k] = apply_epilogue_rt(a.epi, o, b);
      }
    }
  }
}

}  // namespace

int tail_tiles_reduce(const float* P, float* C, const float* bias, int M, int N, int S, int tail_tiles, int tile0,
                      int64_t ldc, int epi, int bias_on_m, int accumulate, cudaStream_t s) {
  TailArgs a;
  a.P = P; a.C = C; a.bias = bias;
  a.M = M; a.N = N; a.S = S; a.tail_tiles = tail_tiles; a.tile0 = tile0;
  a.tiles_n = (int)ceil_div(N, 128);
  a.ldc = ldc;
  a.epi = epi; a.bias_on_m = bias_on_m; a.accumulate = accumulate;
  a.vec = ldc % 4 == 0 && (((uintptr_t)C) & 15) == 0;
  const dim3 grid(8, (unsigned)tail_tiles, 1);
  TCB200_CUDA_TRY(launch_pdl(tail_tiles_reduce_kernel, grid, dim3(256, 1, 1), (size_t)0, s, a));
  return TCB200_OK;
}

int partial_planes_reduce(const float* P, float* C, const float* bias, int M, int N, int S, int64_t ldc, int epi,
                          int bias_on_m, int accumulate, int sms, cudaStream_t s) {
  SplitKArgs r;
  r.P = P; r.C = C; r.bias = bias;
  r.M = M; r.N = N; r.S = S;
  r.ldc = ldc;
  r.epi = epi; r.bias_on_m = bias_on_m; r.accumulate = accumulate;
  const bool vec = N % 4 == 0 && ldc % 4 == 0 && (((uintptr_t)C | (uintptr_t)P) & 15) == 0;
  const int64_t work = vec ? (int64_t)M * N / 4 : (int64_t)M * N;
  const dim3 grid((unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(work, 256), (int64_t)sms * 8)), 1, 1);
  if (vec) TCB200_CUDA_TRY(launch_pdl(splitk_reduce_kernel<true>, grid, dim3(256, 1, 1), (size_t)0, s, r));
  else TCB200_CUDA_TRY(launch_pdl(splitk_reduce_kernel<false>, grid, dim3(256, 1, 1), (size_t)0, s, r));
  return TCB200_OK;
}

}  // namespace tcb200
