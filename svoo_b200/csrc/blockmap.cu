// Cluster-block map (which key clusters each query cluster attends), and the two small
// index builders the attention kernel consumes: merged key-row runs per query cluster and
// the list of 128-row query tiles.
//
// The map follows identify_dynamic_map (svoo/co_clustering.py:556-633) for bf16
// centroids.  Its arithmetic is fixed to IEEE fp32 add/mul/div in a fixed order (no
// fma, sequential sums), so the result is reproducible bit for bit:
//   score  = sum_d q_d*k_d (d ascending, fp32) -> bf16 -> / fp32(sqrt(D)) -> bf16
//   prob   = size_j * exp(score - max) / max(sum_j, 1e-12)  (sum j ascending) -> bf16
//   order  = descending prob, ties by lower cluster index
//   cumsum = running fp32 sum of sorted probs, each prefix rounded to bf16, vs bf16(top_p)
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

__global__ void __launch_bounds__(256) block_map_kernel(const bf16* __restrict__ qc, const bf16* __restrict__ kc,
                                                        const int32_t* __restrict__ ksizes, uint8_t* __restrict__ map,
                                                        int QC, int KC, int KCpad, float sqrt_d, float top_p,
                                                        const __grid_constant__ HeadLimits lim) {
  __shared__ float q_s[kHeadDim];
  __shared__ float val[SVOO_MAX_CLUSTERS];        // scores, then weighted exps, then bf16 prefix sums
  __shared__ uint32_t key[SVOO_MAX_CLUSTERS];
  __shared__ float red[8];
  __shared__ float bcast;
  const int i = blockIdx.x, bh = blockIdx.y, tid = threadIdx.x;
  uint8_t* out = map + ((int64_t)bh * QC + i) * KC;
  if (top_p >= 1.0f) {
    for (int j = tid; j < KC; j += 256) out[j] = 1;
    return;
  }
  if (tid < kHeadDim) q_s[tid] = __bfloat162float(qc[((int64_t)bh * QC + i) * kHeadDim + tid]);
  __syncthreads();

  float lmax = -INFINITY;
  for (int j = tid; j < KC; j += 256) {
    const uint4* row = reinterpret_cast<const uint4*>(kc + ((int64_t)bh * KC + j) * kHeadDim);
    float acc = 0.f;
#pragma unroll 4
    for (int c = 0; c < 16; ++c) {
      const uint4 v = __ldg(row + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc = __fadd_rn(acc, __fmul_rn(q_s[c * 8 + 2 * e], __low2float(h[e])));
        acc = __fadd_rn(acc, __fmul_rn(q_s[c * 8 + 2 * e + 1], __high2float(h[e])));
      }
    }
    float s = bf16_round(acc);
    s = bf16_round(__fdiv_rn(s, sqrt_d));
    val[j] = s;
    lmax = fmaxf(lmax, s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
  if (tid % 32 == 0) red[tid / 32] = lmax;
  __syncthreads();
  float mx = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
  for (int j = tid; j < KC; j += 256) {
    const float e = exp_f32_fixed(__fsub_rn(val[j], mx));
    val[j] = __fmul_rn((float)ksizes[(int64_t)bh * KC + j], e);
  }
  __syncthreads();
  if (tid == 0) {
    float tot = 0.f;
    for (int j = 0; j < KC; ++j) tot = __fadd_rn(tot, val[j]);
    bcast = fmaxf(tot, 1e-12f);
  }
  __syncthreads();
  const float tot = bcast;
  for (int j = tid; j < KCpad; j += 256) {
    uint32_t kk = 0;
    if (j < KC) {
      const bf16 pb = __float2bfloat16_rn(__fdiv_rn(val[j], tot));
      kk = ((uint32_t)__bfloat16_as_ushort(pb) << 16) | (uint32_t)(0xFFFF - j);
    }
    key[j] = kk;
  }
  __syncthreads();
  // bitonic sort, descending
  for (int k = 2; k <= KCpad; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int t = tid; t < KCpad; t += 256) {
        const int u = t ^ j;
        if (u > t) {
          const uint32_t a = key[t], b = key[u];
          const bool desc = (t & k) == 0;
          if (desc ? (a < b) : (a > b)) { key[t] = b; key[u] = a; }
        }
      }
      __syncthreads();
    }
  }
  if (tid == 0) {
    float run = 0.f;
    for (int r = 0; r < KC; ++r) {
      run = __fadd_rn(run, __bfloat162float(__ushort_as_bfloat16((unsigned short)(key[r] >> 16))));
      val[r] = bf16_round(run);
    }
  }
  __syncthreads();
  const float p_b = bf16_round(top_p);
  const int preserve = lim.preserve[bh], cap = lim.cap[bh];
  for (int r = tid; r < KC; r += 256) {
    bool remove = (r >= 1) && (val[r - 1] > p_b);
    if (r < preserve) remove = false;
    if (r >= cap) remove = true;
    out[0xFFFF - (key[r] & 0xFFFFu)] = remove ? 0 : 1;
  }
}

// One warp per (head, query cluster): maximal stretches of consecutive selected, non-empty
// key clusters become runs of the cluster-ordered K/V.  Run r is stored as
// (first_row, virtual_begin): virtual_begin is the number of selected key rows before it, so
// the concatenation of all runs is addressed by one "virtual" row index; entry [nruns] is a
// sentinel (0, total selected rows).
__global__ void __launch_bounds__(256) build_runs_kernel(const uint8_t* __restrict__ map,
                                                         const int32_t* __restrict__ k_offsets, int2* __restrict__ runs,
                                                         int32_t* __restrict__ nruns, int QC, int KC, int max_runs,
                                                         int rows_total) {
  const int row = blockIdx.x * 8 + threadIdx.x / 32;
  if (row >= rows_total) return;
  const int lane = threadIdx.x % 32;
  const int bh = row / QC;
  const uint8_t* m = map + (int64_t)row * KC;
  const int32_t* off = k_offsets + (int64_t)bh * (KC + 1);
  int2* out = runs + (int64_t)row * max_runs;
  bool carry = false;
  int n_start = 0, n_end = 0;
  for (int base = 0; base <= KC; base += 32) {
    const int j = base + lane;
    int o0 = 0;
    bool act = false;
    if (j <= KC) o0 = off[j];
    if (j < KC) act = m[j] != 0 && off[j + 1] > o0;
    const unsigned bal = __ballot_sync(0xffffffffu, act);
    const bool prev = lane > 0 ? ((bal >> (lane - 1)) & 1u) : carry;
    const bool is_start = act && !prev;
    const bool is_end = (j <= KC) && !act && prev;
    const unsigned sb = __ballot_sync(0xffffffffu, is_start);
    const unsigned eb = __ballot_sync(0xffffffffu, is_end);
    const unsigned lt = (1u << lane) - 1u;
    if (is_start) { const int r = n_start + __popc(sb & lt); if (r < max_runs) out[r].x = o0; }
    if (is_end) { const int r = n_end + __popc(eb & lt); if (r < max_runs) out[r].y = o0; }
    n_start += __popc(sb);
    n_end += __popc(eb);
    carry = (bal >> 31) & 1u;
  }
  const int n = n_start < max_runs - 1 ? n_start : max_runs - 1;
  __syncwarp();
  if (lane == 0) {
    int vbeg = 0;
    for (int r = 0; r < n; ++r) {
      const int2 se = out[r];
      out[r] = make_int2(se.x, vbeg);
      vbeg += se.y - se.x;
    }
    out[n] = make_int2(0, vbeg);
    nruns[row] = n;
  }
}

// One CTA per head: the 128-row query tiles of every non-empty query cluster.
__global__ void __launch_bounds__(1024) build_qtiles_kernel(const int32_t* __restrict__ q_offsets,
                                                            int4* __restrict__ qtiles, int32_t* __restrict__ nqtiles,
                                                            int QC, int max_tiles, int tile_rows) {
  __shared__ int warp_tot[32];
  const int bh = blockIdx.x, i = threadIdx.x, lane = i % 32, warp = i / 32;
  int begin = 0, end = 0;
  if (i < QC) {
    begin = q_offsets[(int64_t)bh * (QC + 1) + i];
    end = q_offsets[(int64_t)bh * (QC + 1) + i + 1];
  }
  const int nt = (end - begin + tile_rows - 1) / tile_rows;
  int incl = nt;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, s);
    if (lane >= s) incl += o;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int t = warp_tot[lane];
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, t, s);
      if (lane >= s) t += o;
    }
    warp_tot[lane] = t;
  }
  __syncthreads();
  int pos = incl - nt + (warp ? warp_tot[warp - 1] : 0);
  int4* out = qtiles + (int64_t)bh * max_tiles;
  for (int r = begin; r < end; r += tile_rows, ++pos)
    if (pos < max_tiles) out[pos] = make_int4(i, r, min(r + tile_rows, end), 0);
  if (i == 1023) nqtiles[bh] = min(warp_tot[31], max_tiles);
}

cudaError_t launch_block_map(const void* qc, const void* kc, const int32_t* ksizes, uint8_t* map, int64_t BH,
                             int64_t QC, int64_t KC, float top_p, const int32_t* preserve_host,
                             const int32_t* cap_host, cudaStream_t st) {
  HeadLimits lim;
  for (int h = 0; h < SVOO_MAX_HEADS; ++h) {
    lim.preserve[h] = h < BH ? preserve_host[h] : 0;
    lim.cap[h] = h < BH ? cap_host[h] : (int32_t)KC;
  }
  int KCpad = 2;
  while (KCpad < KC) KCpad <<= 1;
  dim3 grid((unsigned)QC, (unsigned)BH);
  block_map_kernel<<<grid, 256, 0, st>>>((const bf16*)qc, (const bf16*)kc, ksizes, map, (int)QC, (int)KC, KCpad,
                                         (float)sqrt((double)kHeadDim), top_p, lim);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t launch_build_runs(const uint8_t* map, const int32_t* k_offsets, int2* runs, int32_t* nruns, int64_t BH,
                              int64_t QC, int64_t KC, cudaStream_t st) {
  const int rows = (int)(BH * QC);
  build_runs_kernel<<<(unsigned)ceil_div(rows, 8), 256, 0, st>>>(map, k_offsets, runs, nruns, (int)QC, (int)KC,
                                                                 max_runs(KC), rows);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t launch_build_qtiles(const int32_t* q_offsets, int4* qtiles, int32_t* nqtiles, int64_t BH, int64_t N,
                                int64_t QC, int tile_rows, cudaStream_t st) {
  build_qtiles_kernel<<<(unsigned)BH, 1024, 0, st>>>(q_offsets, qtiles, nqtiles, (int)QC, max_qtiles(N, QC), tile_rows);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo
