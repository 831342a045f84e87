// Block-sparse attention over cluster-ordered Q/K/V, warp-level MMA version.
//
// One CTA = one 128-row tile of one query cluster.  It walks the merged key-row runs
// that the cluster's map row selects, 64 key rows at a time, with an online softmax;
// key tiles never cross a run end (the tail columns are masked to -inf).  Rows of the
// tile past the cluster end are computed on zero queries and not stored.
// Semantics: svoo/co_clustering.py:949-1108 (scale D^-0.5, zero output without keys).
#include "common.cuh"

namespace svoo {

constexpr int kBM = kAttnBM;     // 128 query rows, 8 warps x 16
constexpr int kBN = 64;          // key rows per step
constexpr int kAttnSmem = kBM * kRowBytes + 2 * 2 * kBN * kRowBytes;   // Q 32 KB + K,V double buffered 64 KB

__device__ __forceinline__ void load_kv_tile(uint32_t k_dst, uint32_t v_dst, const bf16* kb, const bf16* vb,
                                             int row0, int row_end, int tid) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = tid + i * 256, row = c >> 4, chunk = c & 15;
    const bool ok = row0 + row < row_end;
    const int64_t off = (int64_t)(ok ? row0 + row : row0) * kHeadDim + chunk * 8;
    cp_async16(k_dst + swz(row, chunk), kb + off, ok);
    cp_async16(v_dst + swz(row, chunk), vb + off, ok);
  }
}

__global__ void __launch_bounds__(256, 1) sparse_attn_mma_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, bf16* __restrict__ out,
    const int32_t* __restrict__ out_row_idx, const int4* __restrict__ qtiles, const int32_t* __restrict__ nqtiles,
    const int2* __restrict__ runs, const int32_t* __restrict__ nruns, int S, int QC, int max_tiles, int max_runs,
    float scale_log2) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int bh = blockIdx.y;
  if ((int)blockIdx.x >= nqtiles[bh]) return;
  const int4 tile = qtiles[(int64_t)bh * max_tiles + blockIdx.x];
  const int qi = tile.x, row0 = tile.y, row1 = tile.z;
  const int nr = nruns[(int64_t)bh * QC + qi];
  const int2* rl = runs + ((int64_t)bh * QC + qi) * max_runs;

  const uint32_t q_s = smem_u32(smem_raw);
  const uint32_t kv_s = q_s + kBM * kRowBytes;            // stage s: K at kv_s + s*32K, V at +16K
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const bf16* qb = q + (int64_t)bh * S * kHeadDim;
  const bf16* kb = k + (int64_t)bh * S * kHeadDim;
  const bf16* vb = v + (int64_t)bh * S * kHeadDim;

#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = tid + i * 256, row = c >> 4, chunk = c & 15;
    const bool ok = row0 + row < row1;
    cp_async16(q_s + swz(row, chunk), qb + (int64_t)(ok ? row0 + row : row0) * kHeadDim + chunk * 8, ok);
  }
  // key-tile cursor: run index and first row of the tile inside that run
  int r_cur = 0, p_cur = 0, e_cur = 0;
  if (nr > 0) { const int2 r = rl[0]; p_cur = max(r.x, 0); e_cur = min(r.x + rl[1].y - r.y, S); }
  if (nr > 0) load_kv_tile(kv_s, kv_s + kBN * kRowBytes, kb, vb, p_cur, e_cur, tid);
  cp_async_commit();

  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  uint32_t qa[8][4];
  bool q_loaded = false;
  int stage = 0;

  while (r_cur < nr) {
    // next tile
    int r_nxt = r_cur, p_nxt = p_cur + kBN, e_nxt = e_cur;
    if (p_nxt >= e_cur) {
      r_nxt = r_cur + 1;
      if (r_nxt < nr) { const int2 r = rl[r_nxt]; p_nxt = max(r.x, 0); e_nxt = min(r.x + rl[r_nxt + 1].y - r.y, S); }
    }
    if (r_nxt < nr) {
      const uint32_t dst = kv_s + (stage ^ 1) * (2 * kBN * kRowBytes);
      load_kv_tile(dst, dst + kBN * kRowBytes, kb, vb, p_nxt, e_nxt, tid);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (!q_loaded) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int row = warp * 16 + (lane % 8) + ((lane / 8) % 2) * 8;
        ldmatrix_x4(qa[ks], q_s + swz(row, ks * 2 + lane / 16));
      }
      q_loaded = true;
    }
    const uint32_t k_t = kv_s + stage * (2 * kBN * kRowBytes), v_t = k_t + kBN * kRowBytes;

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        const int row = np * 16 + (lane % 8) + (lane / 16) * 8;
        uint32_t b[4];
        ldmatrix_x4(b, k_t + swz(row, ks * 2 + ((lane / 8) % 2)));
        mma_bf16(s[np * 2], qa[ks], b[0], b[1]);
        mma_bf16(s[np * 2 + 1], qa[ks], b[2], b[3]);
      }
    }
    const int valid = e_cur - p_cur;        // >= 1; columns >= valid are past the run end
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int col = nt * 8 + 2 * (lane % 4) + (c & 1);
        const float val = col < valid ? s[nt][c] * scale_log2 : -INFINITY;
        s[nt][c] = val;
        mx[c >> 1] = fmaxf(mx[c >> 1], val);
      }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      alpha[h] = exp2f(m_run[h] - m_new);      // m_new is finite: every tile has a valid column
      m_run[h] = m_new;
      l_run[h] *= alpha[h];
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = exp2f(s[nt][c] - m_run[c >> 1]);
        s[nt][c] = p;
        l_run[c >> 1] += p;
      }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0];
      o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        const int row = kk * 16 + (lane % 8) + ((lane / 8) % 2) * 8;
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_t + swz(row, dp * 2 + lane / 16));
        mma_bf16(o[dp * 2], pa, b[0], b[1]);
        mma_bf16(o[dp * 2 + 1], pa, b[2], b[3]);
      }
    }
    __syncthreads();
    r_cur = r_nxt; p_cur = p_nxt; e_cur = e_nxt;
    stage ^= 1;
  }
  cp_async_wait<0>();
  __syncthreads();

  // normalise, stage through shared memory (the Q tile is dead), store whole 256-byte rows
  float inv[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = l_run[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    inv[h] = l > 0.f ? 1.f / l : 0.f;
  }
  unsigned char* stage_o = smem_raw;
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    const int col = nt * 8 + 2 * (lane % 4);
    const int r_a = warp * 16 + lane / 4, r_b = r_a + 8;
    *reinterpret_cast<uint32_t*>(stage_o + swz(r_a, col >> 3) + (col & 7) * 2) =
        pack_bf16x2(o[nt][0] * inv[0], o[nt][1] * inv[0]);
    *reinterpret_cast<uint32_t*>(stage_o + swz(r_b, col >> 3) + (col & 7) * 2) =
        pack_bf16x2(o[nt][2] * inv[1], o[nt][3] * inv[1]);
  }
  __syncwarp();
  bf16* ob = out + (int64_t)bh * S * kHeadDim;
  const int32_t* ridx = out_row_idx ? out_row_idx + (int64_t)bh * S : nullptr;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int lr = warp * 16 + it * 2 + lane / 16, chunk = lane % 16;
    const int row = row0 + lr;
    if (row < row1) {
      const int dst = ridx ? ridx[row] : row;
      if (dst >= 0 && dst < S)
        *reinterpret_cast<uint4*>(ob + (int64_t)dst * kHeadDim + chunk * 8) =
            *reinterpret_cast<const uint4*>(stage_o + swz(lr, chunk));
    }
  }
}

cudaError_t launch_sparse_attn_mma(const void* q, const void* k, const void* v, void* out, const int32_t* out_row_idx,
                                   const int4* qtiles, const int32_t* nqtiles, const int2* runs, const int32_t* nruns,
                                   int64_t BH, int64_t S, int64_t QC, int64_t KC, float sm_scale, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(sparse_attn_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)max_qtiles(S, QC), (unsigned)BH);
  sparse_attn_mma_kernel<<<grid, 256, kAttnSmem, st>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, (bf16*)out,
                                                       out_row_idx, qtiles, nqtiles, runs, nruns, (int)S, (int)QC,
                                                       max_qtiles(S, QC), max_runs(KC),
                                                       sm_scale * 1.4426950408889634f);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo
