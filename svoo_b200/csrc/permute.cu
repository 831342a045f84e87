// Cluster-order gather (permute) and scatter (inverse permute) of [BH, N, 128] bf16 rows.
// One 256-byte row is moved by 16 lanes with one 128-bit access each; every row is a
// whole number of 32-byte sectors, so neither side of the copy wastes DRAM bytes.
// Reference: svoo/kernels/triton/permute.py:10-65.
#include "common.cuh"

namespace svoo {

constexpr int kPermRowsPerCta = 64;     // 256 threads = 16 rows per pass, 4 passes

template <bool kInverse>
__global__ void __launch_bounds__(256) permute_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ idx,
                                                      uint4* __restrict__ y, int N, int64_t x_head_rows, int64_t y_head_rows) {
  const int bh = blockIdx.y;
  const int lane = threadIdx.x % 16, sub = threadIdx.x / 16;
  const int s_base = blockIdx.x * kPermRowsPerCta + sub;
  const int32_t* ib = idx + (int64_t)bh * N;
  const uint4* xb = x + (int64_t)bh * x_head_rows * 16;
  uint4* yb = y + (int64_t)bh * y_head_rows * 16;
  int other[4];
  uint4 v[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int s = s_base + u * 16;
    other[u] = (s < N) ? ib[s] : -1;
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int s = s_base + u * 16;
    if (other[u] >= 0 && other[u] < N) {
      const int src = kInverse ? s : other[u];
      v[u] = __ldg(xb + (int64_t)src * 16 + lane);
    }
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int s = s_base + u * 16;
    if (other[u] >= 0 && other[u] < N) {
      const int dst = kInverse ? other[u] : s;
      yb[(int64_t)dst * 16 + lane] = v[u];
    }
  }
}

cudaError_t launch_permute(const void* x, const int32_t* idx, void* y, int64_t BH, int64_t N, int64_t x_head_rows,
                           int64_t y_head_rows, bool inverse, cudaStream_t st) {
  dim3 grid((unsigned)ceil_div64(N, kPermRowsPerCta), (unsigned)BH);
  if (inverse)
    permute_kernel<true><<<grid, 256, 0, st>>>((const uint4*)x, idx, (uint4*)y, (int)N, x_head_rows, y_head_rows);
  else
    permute_kernel<false><<<grid, 256, 0, st>>>((const uint4*)x, idx, (uint4*)y, (int)N, x_head_rows, y_head_rows);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo
