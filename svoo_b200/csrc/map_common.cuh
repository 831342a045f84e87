// Pieces shared by the two cluster-block map kernels (the probability map of blockmap.cu and the
// error-aware one of ear.cu): fixed-order fp32 exp, per-head limits, the warp-wide bitonic sort.
#pragma once

#include "common.cuh"

namespace svoo {

__device__ __forceinline__ float exp_f32_fixed(float x) {
  // exp(x), x <= 0, from fp32 mul/add only; mirrored operation by operation on the CPU side
  if (x < -87.0f) return 0.0f;
  const float n = rintf(__fmul_rn(x, (float)1.4426950408889634));
  float r = __fsub_rn(x, __fmul_rn(n, 0.693145751953125f));
  r = __fsub_rn(r, __fmul_rn(n, (float)1.428606765330187e-06));
  float p = (float)(1.0 / 720);
  p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 120));
  p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 24));
  p = __fadd_rn(__fmul_rn(p, r), (float)(1.0 / 6));
  p = __fadd_rn(__fmul_rn(p, r), 0.5f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f);
  int ni = (int)n;
  ni = ni < -126 ? -126 : ni;
  return __fmul_rn(p, __int_as_float((ni + 127) << 23));
}

struct HeadLimits {
  int32_t preserve[SVOO_MAX_HEADS];
  int32_t cap[SVOO_MAX_HEADS];
};

// Bitonic sort (descending) of 32 * M keys held by one warp, element t in register t / 32 of lane
// t % 32: partners at distance >= 32 are other registers of the same lane, closer ones come by
// shuffle.  Keys are unique (the cluster index is part of the key) except for the zero padding.
template <int M, typename Key = uint32_t>
__device__ __forceinline__ void warp_sort_desc(Key (&v)[M], int lane) {
#pragma unroll
  for (int k = 2; k <= 32 * M; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      if (j >= 32) {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const int pm = m ^ (j >> 5);
          if (pm > m) {
            const bool desc = ((lane + 32 * m) & k) == 0;
            const Key a = v[m], b = v[pm];
            if (desc ? (a < b) : (a > b)) { v[m] = b; v[pm] = a; }
          }
        }
      } else {
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const Key a = v[m];
          const Key b = __shfl_xor_sync(0xffffffffu, a, j);
          const bool lower = (lane & j) == 0;                      // this lane holds the smaller index of the pair
          const bool desc = ((lane + 32 * m) & k) == 0;
          v[m] = (lower == desc) ? max(a, b) : min(a, b);
        }
      }
    }
  }
}

}  // namespace svoo
