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
#include "map_common.cuh"

namespace svoo {

// Keys of one query cluster: (bf16 probability << 16) | (0xFFFF - cluster index), sorted descending
// into kw[0 .. KCpad).
template <int M>
__device__ __forceinline__ void make_sorted_keys(const float* vw, uint32_t* kw, float tot, int KC, int KCpad, int lane) {
  uint32_t v[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const int j = lane + 32 * m;
    uint32_t kk = 0;
    if (j < KC) {
      const bf16 pb = __float2bfloat16_rn(__fdiv_rn(vw[j], tot));
      kk = ((uint32_t)__bfloat16_as_ushort(pb) << 16) | (uint32_t)(0xFFFF - j);
    }
    v[m] = kk;
  }
  warp_sort_desc<M>(v, lane);
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const int t = lane + 32 * m;
    if (t < KCpad) kw[t] = v[m];
  }
}

// One CTA = 8 consecutive query clusters of one head, one warp each.  The score phase is shared:
// a thread reads a key centroid once and accumulates its product with all 8 query centroids
// (each (query, key) sum still runs over d in ascending order).  Everything after it -- exp,
// the sequential sum, the sort, the sequential bf16 prefix sum -- is per query cluster and runs in
// the 8 warps side by side, which is what the fixed summation orders leave to parallelise.
constexpr int kMapRows = 8;

__global__ void __launch_bounds__(256, 2) block_map_kernel(const bf16* __restrict__ qc, const bf16* __restrict__ kc,
                                                        const int32_t* __restrict__ ksizes, uint8_t* __restrict__ map,
                                                        int QC, int KC, int KCpad, float sqrt_d, float top_p,
                                                        const __grid_constant__ HeadLimits lim) {
  extern __shared__ __align__(16) unsigned char map_sm[];
  float* q_s = reinterpret_cast<float*>(map_sm);                       // [8][128]
  float* val = q_s + kMapRows * kHeadDim;                              // [8][KCpad]: scores, weighted exps, prefix sums
  uint32_t* key = reinterpret_cast<uint32_t*>(val + kMapRows * KCpad); // [8][KCpad]
  __shared__ float red[8][kMapRows];
  const int i0 = blockIdx.x * kMapRows, bh = blockIdx.y, tid = threadIdx.x;
  const int lane = tid % 32, warp = tid / 32;
  if (top_p >= 1.0f) {
    for (int r = 0; r < kMapRows && i0 + r < QC; ++r)
      for (int j = tid; j < KC; j += 256) map[((int64_t)bh * QC + i0 + r) * KC + j] = 1;
    return;
  }
  for (int t = tid; t < kMapRows * kHeadDim; t += 256) {
    const int r = t / kHeadDim, d = t % kHeadDim;
    q_s[t] = i0 + r < QC ? __bfloat162float(qc[((int64_t)bh * QC + i0 + r) * kHeadDim + d]) : 0.f;
  }
  __syncthreads();

  float lmax[kMapRows];
#pragma unroll
  for (int r = 0; r < kMapRows; ++r) lmax[r] = -INFINITY;
  for (int j = tid; j < KC; j += 256) {
    const uint4* row = reinterpret_cast<const uint4*>(kc + ((int64_t)bh * KC + j) * kHeadDim);
    float acc[kMapRows];
#pragma unroll
    for (int r = 0; r < kMapRows; ++r) acc[r] = 0.f;
#pragma unroll 2
    for (int c = 0; c < 16; ++c) {
      const uint4 v = __ldg(row + c);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
      float kv[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        kv[2 * e] = __low2float(h[e]);
        kv[2 * e + 1] = __high2float(h[e]);
      }
#pragma unroll
      for (int r = 0; r < kMapRows; ++r) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[r] = __fadd_rn(acc[r], __fmul_rn(q_s[r * kHeadDim + c * 8 + e], kv[e]));
      }
    }
#pragma unroll
    for (int r = 0; r < kMapRows; ++r) {
      float sc = bf16_round(acc[r]);
      sc = bf16_round(__fdiv_rn(sc, sqrt_d));
      val[r * KCpad + j] = sc;
      lmax[r] = fmaxf(lmax[r], sc);
    }
  }
#pragma unroll
  for (int r = 0; r < kMapRows; ++r) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lmax[r] = fmaxf(lmax[r], __shfl_xor_sync(0xffffffffu, lmax[r], o));
    if (lane == 0) red[warp][r] = lmax[r];
  }
  __syncthreads();

  // ---- from here on: warp w works on query cluster i0 + w
  const int i = i0 + warp;
  if (i >= QC) return;
  float* vw = val + warp * KCpad;
  uint32_t* kw = key + warp * KCpad;
  float mx = red[0][warp];
#pragma unroll
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w][warp]);
  for (int j = lane; j < KC; j += 32) {
    const float e = exp_f32_fixed(__fsub_rn(vw[j], mx));
    vw[j] = __fmul_rn((float)ksizes[(int64_t)bh * KC + j], e);
  }
  __syncwarp();
  float tot = 0.f;
  if (lane == 0) {                                   // j ascending; four values per shared-memory read
    int j = 0;
    if (KCpad >= 4)
      for (; j + 4 <= KC; j += 4) {
        const float4 t4 = *reinterpret_cast<const float4*>(vw + j);
        tot = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(tot, t4.x), t4.y), t4.z), t4.w);
      }
    for (; j < KC; ++j) tot = __fadd_rn(tot, vw[j]);
    tot = fmaxf(tot, 1e-12f);
  }
  tot = __shfl_sync(0xffffffffu, tot, 0);
  switch (KCpad <= 32 ? 1 : KCpad / 32) {           // registers per lane
    case 1: make_sorted_keys<1>(vw, kw, tot, KC, KCpad, lane); break;
    case 2: make_sorted_keys<2>(vw, kw, tot, KC, KCpad, lane); break;
    case 4: make_sorted_keys<4>(vw, kw, tot, KC, KCpad, lane); break;
    case 8: make_sorted_keys<8>(vw, kw, tot, KC, KCpad, lane); break;
    case 16: make_sorted_keys<16>(vw, kw, tot, KC, KCpad, lane); break;
    default: make_sorted_keys<32>(vw, kw, tot, KC, KCpad, lane); break;
  }
  __syncwarp();
  if (lane == 0) {                                   // r ascending; padding keys are zero probabilities
    float run = 0.f;
    int r = 0;
    if (KCpad >= 4)
      for (; r + 4 <= KCpad; r += 4) {
        const uint4 k4 = *reinterpret_cast<const uint4*>(kw + r);
        float4 o;
        run = __fadd_rn(run, __uint_as_float(k4.x & 0xFFFF0000u)); o.x = bf16_round(run);
        run = __fadd_rn(run, __uint_as_float(k4.y & 0xFFFF0000u)); o.y = bf16_round(run);
        run = __fadd_rn(run, __uint_as_float(k4.z & 0xFFFF0000u)); o.z = bf16_round(run);
        run = __fadd_rn(run, __uint_as_float(k4.w & 0xFFFF0000u)); o.w = bf16_round(run);
        *reinterpret_cast<float4*>(vw + r) = o;
      }
    for (; r < KC; ++r) {
      run = __fadd_rn(run, __uint_as_float(kw[r] & 0xFFFF0000u));
      vw[r] = bf16_round(run);
    }
  }
  __syncwarp();
  const float p_b = bf16_round(top_p);
  const int preserve = lim.preserve[bh], cap = lim.cap[bh];
  uint8_t* out = map + ((int64_t)bh * QC + i) * KC;
  for (int r = lane; r < KC; r += 32) {
    bool remove = (r >= 1) && (vw[r - 1] > p_b);
    if (r < preserve) remove = false;
    if (r >= cap) remove = true;
    out[0xFFFF - (kw[r] & 0xFFFFu)] = remove ? 0 : 1;
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

// One CTA per head: the query tiles (`tile_rows` rows each) of every non-empty query cluster, in
// cluster order.  Thread i owns clusters 2i and 2i + 1, so up to 2048 clusters fit one CTA.
__global__ void __launch_bounds__(1024) build_qtiles_kernel(const int32_t* __restrict__ q_offsets,
                                                            int4* __restrict__ qtiles, int32_t* __restrict__ nqtiles,
                                                            int QC, int max_tiles, int tile_rows) {
  __shared__ int warp_tot[32];
  const int bh = blockIdx.x, i = threadIdx.x, lane = i % 32, warp = i / 32;
  const int32_t* off = q_offsets + (int64_t)bh * (QC + 1);
  int b[3] = {0, 0, 0};
#pragma unroll
  for (int u = 0; u < 3; ++u)
    if (2 * i + u <= QC) b[u] = off[2 * i + u];
  const int nt0 = 2 * i < QC ? (b[1] - b[0] + tile_rows - 1) / tile_rows : 0;
  const int nt1 = 2 * i + 1 < QC ? (b[2] - b[1] + tile_rows - 1) / tile_rows : 0;
  const int nt = nt0 + nt1;
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
  if (nt0)
    for (int r = b[0]; r < b[1]; r += tile_rows, ++pos)
      if (pos < max_tiles) out[pos] = make_int4(2 * i, r, min(r + tile_rows, b[1]), 0);
  if (nt1)
    for (int r = b[1]; r < b[2]; r += tile_rows, ++pos)
      if (pos < max_tiles) out[pos] = make_int4(2 * i + 1, r, min(r + tile_rows, b[2]), 0);
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
  const size_t smem = (size_t)kMapRows * (kHeadDim + 2 * KCpad) * 4;           // at most 68 KB (1024 clusters)
  cudaError_t e = cudaFuncSetAttribute(block_map_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)ceil_div64(QC, kMapRows), (unsigned)BH);
  block_map_kernel<<<grid, 256, smem, st>>>((const bf16*)qc, (const bf16*)kc, ksizes, map, (int)QC, (int)KC, KCpad,
                                            (float)sqrt((double)kHeadDim), top_p, lim);
  count_launches(1);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Text tokens of a joint-attention layer (svoo/models/hunyuan10/attention.py:999-1019): the
// `text` rows that follow the N clustered video rows of every head become two more blocks,
// "prompt" (the first `prompt` text rows) and "unused prompt" (the rest).
//   map  [BH, QC, KC]   -> [BH, QC+2, KC+2]: prompt queries see every video and prompt key, every
//                          query but the unused prompt sees the prompt keys, the unused prompt sees itself
//   offsets [BH, K+1]   -> [BH, K+3]  (block sizes `prompt`, `text - prompt` appended)
//   sorted_idx [BH, N]  -> [BH, N+text]  (identity on the text rows)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) append_text_blocks_kernel(
    const uint8_t* __restrict__ map, const int32_t* __restrict__ q_off, const int32_t* __restrict__ k_off,
    const int32_t* __restrict__ q_idx, const int32_t* __restrict__ k_idx, uint8_t* __restrict__ map_out,
    int32_t* __restrict__ q_off_out, int32_t* __restrict__ k_off_out, int32_t* __restrict__ q_idx_out,
    int32_t* __restrict__ k_idx_out, int N, int QC, int KC, int text, int prompt) {
  const int bh = blockIdx.y;
  const int S = N + text, QC2 = QC + 2, KC2 = KC + 2;
  const int stride = gridDim.x * 256;
  for (int t = blockIdx.x * 256 + threadIdx.x; t < QC2 * KC2; t += stride) {
    const int i = t / KC2, j = t - i * KC2;
    uint8_t v;
    if (i < QC) v = j < KC ? (uint8_t)(map[((int64_t)bh * QC + i) * KC + j] != 0) : (uint8_t)(j == KC);
    else if (i == QC) v = (uint8_t)(j <= KC);
    else v = (uint8_t)(j == KC + 1);
    map_out[(int64_t)bh * QC2 * KC2 + t] = v;
  }
  for (int t = blockIdx.x * 256 + threadIdx.x; t < S; t += stride) {
    q_idx_out[(int64_t)bh * S + t] = t < N ? q_idx[(int64_t)bh * N + t] : t;
    k_idx_out[(int64_t)bh * S + t] = t < N ? k_idx[(int64_t)bh * N + t] : t;
  }
  for (int t = blockIdx.x * 256 + threadIdx.x; t <= QC2; t += stride)
    q_off_out[(int64_t)bh * (QC2 + 1) + t] = t <= QC ? q_off[(int64_t)bh * (QC + 1) + t] : (t == QC + 1 ? N + prompt : S);
  for (int t = blockIdx.x * 256 + threadIdx.x; t <= KC2; t += stride)
    k_off_out[(int64_t)bh * (KC2 + 1) + t] = t <= KC ? k_off[(int64_t)bh * (KC + 1) + t] : (t == KC + 1 ? N + prompt : S);
}

cudaError_t launch_append_text_blocks(const uint8_t* map, const int32_t* q_off, const int32_t* k_off, const int32_t* q_idx,
                                      const int32_t* k_idx, uint8_t* map_out, int32_t* q_off_out, int32_t* k_off_out,
                                      int32_t* q_idx_out, int32_t* k_idx_out, int64_t BH, int64_t N, int64_t QC, int64_t KC,
                                      int64_t text, int64_t prompt, cudaStream_t st) {
  const int64_t work = (QC + 2) * (KC + 2) > N + text ? (QC + 2) * (KC + 2) : N + text;
  int64_t blocks = ceil_div64(work, 256 * 4);
  blocks = blocks < 1 ? 1 : (blocks > 1024 ? 1024 : blocks);
  append_text_blocks_kernel<<<dim3((unsigned)blocks, (unsigned)BH), 256, 0, st>>>(
      map, q_off, k_off, q_idx, k_idx, map_out, q_off_out, k_off_out, q_idx_out, k_idx_out, (int)N, (int)QC, (int)KC,
      (int)text, (int)prompt);
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
