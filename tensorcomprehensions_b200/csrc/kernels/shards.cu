// Assembly of an all-gathered output: the one device-side step of the opt-in exchange that follows a
// sharded run.  The all-gather (NCCL) leaves the shards of all ranks one after the other, each padded to
// the largest shard: G[k][r][j] with k = rank, r = the `rows` in front of the sharded dimension,
// j < max_count * inner.  The caller wants the unsharded row-major tensor O[r][start_k * inner + j],
// j < count_k * inner.  For a dimension-0 shard rows = 1 and this trims the padding; for the transposed
// matmul (C's columns are sharded) rows = M and this is the [g][M][N/g] -> [M][N] permutation.
// One CTA column per (k, r) run, 128-bit copies when every run is 16-byte aligned.
#include "common.cuh"

namespace tcb200 {
namespace {

struct AssembleArgs {
  const float* G;
  float* O;
  int world;
  int64_t rows, base, rem, inner, max_run, total_run;  // runs in elements: count * inner
};

template <bool VEC>
__global__ void __launch_bounds__(256) assemble_shards_kernel(AssembleArgs a) {
  const int64_t run = blockIdx.y;  // k * rows + r
  const int k = (int)(run / a.rows);
  const int64_t r = run - (int64_t)k * a.rows;
  const int64_t count = a.base + (k < a.rem ? 1 : 0);
  const int64_t start = (int64_t)k * a.base + (k < a.rem ? k : a.rem);
  const int64_t len = count * a.inner;
  const float* src = a.G + run * a.max_run;
  float* dst = a.O + r * a.total_run + start * a.inner;
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, step = (int64_t)gridDim.x * blockDim.x;
  if (VEC) {
    const float4* s4 = reinterpret_cast<const float4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
    for (int64_t i = i0; i < len / 4; i += step) stg_stream4(d4 + i, ldg_stream4(s4 + i));
  } else {
    for (int64_t i = i0; i < len; i += step) dst[i] = __ldg(src + i);
  }
}

}  // namespace
}  // namespace tcb200

using namespace tcb200;

extern "C" int tcb200_assemble_shards(const void* gathered, void* out, int world, int64_t rows, int64_t total,
                                      int64_t inner, tcb200_stream_t stream) {
  if (!gathered || !out || world <= 0 || rows <= 0 || total <= 0 || inner <= 0) return TCB200_ERR_INVALID_ARGUMENT;
  if ((int64_t)world * rows > 65535) return TCB200_ERR_TOO_LARGE;
  AssembleArgs a;
  a.G = static_cast<const float*>(gathered);
  a.O = static_cast<float*>(out);
  a.world = world;
  a.rows = rows;
  a.base = total / world;
  a.rem = total % world;
  a.inner = inner;
  const int64_t max_count = a.base + (a.rem ? 1 : 0);
  a.max_run = max_count * inner;
  a.total_run = total * inner;
  // every run starts on a 16-byte boundary and has a length that is a multiple of 16 bytes
  const bool vec = (((uintptr_t)gathered | (uintptr_t)out) & 15) == 0 && inner % 4 == 0;
  const int64_t per_run = vec ? a.max_run / 4 : a.max_run;
  const unsigned gx = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(per_run, 256 * 4), 64));
  const dim3 grid(gx, (unsigned)(world * rows), 1);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (vec) assemble_shards_kernel<true><<<grid, 256, 0, s>>>(a);
  else assemble_shards_kernel<false><<<grid, 256, 0, s>>>(a);
  TCB200_CUDA_TRY(cudaGetLastError());
  return TCB200_OK;
}
