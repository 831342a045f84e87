// Block-sparse attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One CTA owns up to two 128-row query tiles of one query cluster.  The key rows that the
// cluster's map row selects form a list of runs of the cluster-ordered K/V; the CTA walks
// their concatenation 128 keys at a time, so key tiles are always full except the last one
// (tiles are packed across run boundaries by gathering rows, which a TMA box cannot do).
//
//   warps 0-3   softmax of query tile 0: thread r owns row r (TMEM lane r): running max and
//   warps 4-7   sum, P written back over S as packed bf16; same for tile 1
//   warps 8-11  K loader (and Q, once): cp.async 16-byte gathers into the 128-byte-swizzled
//               K-major layout the MMA descriptors expect, fence.proxy.async, mbarrier arrive
//   warps 12-15 V loader, same, two-stage rings for K and for V
//   warp 16     MMA issuer (one elected thread): S_w = Q_w K^T into TMEM (tcgen05.mma, both
//               operands from shared memory), then O_w += P_w V with P_w read from TMEM
//
// Rows can be fetched through index vectors (q_row_idx / kv_row_idx): the cluster-order
// permutation of Q, K and V is then fused into the loads and no permuted copy exists.
//
// The two query tiles ping-pong: while one tile's rows are in the softmax, the tensor
// core works on the other tile's products.  O stays in TMEM; it is rescaled by the owning
// softmax thread only when a row maximum grows by more than 2^8 (the running sum uses the
// same stale maximum, so the final normalisation is exact).  Every mbarrier wait is bounded;
// on expiry the CTA raises an abort flag, sets the status word and leaves through the
// normal teardown.
//
// TMEM columns (512 allocated): S0 [0,128)  S1 [128,256)  O0 [256,384)  O1 [384,512).
// Semantics: svoo/co_clustering.py:949-1108 (scale D^-0.5, zero output without keys).
#include "tc_common.cuh"

namespace svoo {
namespace tc {

constexpr int kBM = 128;                 // query rows per softmax warpgroup
constexpr int kBN = 128;                 // key rows per step
constexpr int kTile = 128 * kRowBytes;   // 32 KB: one [128 x 128] bf16 tile = two 16 KB boxes
constexpr int kBox = 128 * 128;          // 16 KB: 128 rows x 64 columns
constexpr int kSmemTiles = 6 * kTile;    // Q0 Q1 | K0 K1 | V0 V1
constexpr int kMaxRunsSmem = SVOO_MAX_CLUSTERS / 2 + 2;
constexpr int kRunTableBytes = (kMaxRunsSmem * 8 + 255) / 256 * 256;
constexpr int kSmemBytes = kSmemTiles + 256 + kRunTableBytes + 2048 + 1024;   // + barriers, run table, row maps, slack
constexpr int kThreads = 544;            // 8 softmax + 4 K-loader + 4 V-loader + 1 MMA warps
constexpr int kLoaderThreads = 128;      // per tensor (K, V): one thread per key row of a tile
constexpr float kRescaleThreshold = 8.0f;

enum Bar { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, P_READY = 11, O_DONE = 13, NUM_BARS = 15 };

__device__ __forceinline__ void row_max(const uint32_t (&r)[32], float& m) {
#pragma unroll
  for (int i = 0; i < 32; i += 2) m = fmaxf(m, fmaxf(__uint_as_float(r[i]), __uint_as_float(r[i + 1])));
}
// Only the first `valid` of the 32 columns count (valid may be <= 0 or >= 32).
__device__ __forceinline__ void row_max_masked(const uint32_t (&r)[32], float& m, int valid) {
#pragma unroll
  for (int i = 0; i < 32; ++i) m = fmaxf(m, i < valid ? __uint_as_float(r[i]) : -INFINITY);
}
// p = exp2(s * scale + neg_m) for 32 columns -> 16 packed bf16 pairs; columns >= valid give 0.
__device__ __forceinline__ void exp_pack(const uint32_t (&r)[32], uint32_t (&pk)[16], float scale, float neg_m,
                                         float& l0, float& l1, int valid) {
  if (valid >= 32) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float p0 = fast_exp2(fmaf(__uint_as_float(r[2 * i]), scale, neg_m));
      const float p1 = fast_exp2(fmaf(__uint_as_float(r[2 * i + 1]), scale, neg_m));
      l0 += p0;
      l1 += p1;
      pk[i] = pack_bf16x2(p0, p1);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float p0 = fast_exp2(fmaf(__uint_as_float(r[2 * i]), scale, neg_m));
      float p1 = fast_exp2(fmaf(__uint_as_float(r[2 * i + 1]), scale, neg_m));
      p0 = (2 * i < valid) ? p0 : 0.f;
      p1 = (2 * i + 1 < valid) ? p1 : 0.f;
      l0 += p0;
      l1 += p1;
      pk[i] = pack_bf16x2(p0, p1);
    }
  }
}

// Shared-memory matrix descriptors, 128-byte swizzle, descriptor version 1 (sm_100).
//   K-major  (Q, K: rows = M/N index, 64 contiguous elements of the reduction dim per 128-byte row):
//            8-row groups 1024 B apart (SBO); LBO unused.
//   MN-major (V: rows = reduction index (key), 64 contiguous head-dim elements per 128-byte row):
//            8-key groups 1024 B apart (SBO); the next 64 head-dim columns are one 16 KB box further (LBO).
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(kBox >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor: D fp32, A/B bf16, M = 128, N = 128; bit 16 = B is MN-major.
constexpr uint32_t kIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescPV = kIdescQK | (1u << 16);

// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` (0..127) inside a [128 x 128] bf16
// tile stored as two [128 rows x 128 B] halves with the 128-byte swizzle (chunk ^= row % 8).
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)((chunk >> 3) * kBox + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

// Gathers the 128 key rows of packed tile j (virtual rows [128 j, 128 j + 128) of the
// concatenated runs) into one swizzled tile; rows past the end are zero-filled.  Thread tl
// (0..127) first resolves the source row of virtual row 128 j + tl into `rowmap` (shared
// memory), then the 128 threads copy the tile with 16 lanes per 256-byte row.
__device__ __forceinline__ void gather_tile(uint32_t dst, const bf16* __restrict__ base, const int32_t* __restrict__ row_idx,
                                            const int2* runs_s, int nr, int& r_cur, int* rowmap, int bar_id, int j,
                                            int L, int tl) {
  const int v = j * kBN + tl;
  int p = -1;
  if (v < L) {
    while (r_cur + 1 < nr && v >= runs_s[r_cur + 1].y) ++r_cur;
    p = runs_s[r_cur].x + (v - runs_s[r_cur].y);
    if (row_idx) p = __ldg(row_idx + p);
  }
  rowmap[tl] = p;
  asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(kLoaderThreads) : "memory");
#pragma unroll 4
  for (int it = 0; it < 16; ++it) {
    const int row = it * 8 + (tl >> 4), chunk = tl & 15;
    const int src = rowmap[row];
    cp_async16(dst + tile_off(row, chunk), base + (int64_t)(src < 0 ? 0 : src) * kHeadDim + chunk * 8, src >= 0);
  }
}

__global__ void __launch_bounds__(kThreads, 1) sparse_attn_tc_kernel(
    const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, bf16* __restrict__ out,
    const int32_t* __restrict__ q_row_idx, const int32_t* __restrict__ kv_row_idx,
    const int32_t* __restrict__ out_row_idx, const int4* __restrict__ qtiles, const int32_t* __restrict__ nqtiles,
    const int2* __restrict__ runs, const int32_t* __restrict__ nruns, int S, int QC, int max_tiles, int max_runs,
    float scale_log2, int32_t* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  const int bh = blockIdx.y;
  if ((int)blockIdx.x >= nqtiles[bh]) return;
  const int4 tile = qtiles[(int64_t)bh * max_tiles + blockIdx.x];
  const int qi = tile.x, row0 = tile.y, row1 = tile.z;
  const int nr = min(nruns[(int64_t)bh * QC + qi], kMaxRunsSmem - 1);
  const int2* rl = runs + ((int64_t)bh * QC + qi) * max_runs;
  const int nq = (row1 - row0 > kBM) ? 2 : 1;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base, k_s = base + 2 * kTile, v_s = base + 4 * kTile;
  const uint32_t bars = base + kSmemTiles;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + kSmemTiles + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + kSmemTiles + NUM_BARS * 8 + 8);
  int2* runs_s = reinterpret_cast<int2*>(gen_base + kSmemTiles + 256);
  int* rowmaps = reinterpret_cast<int*>(gen_base + kSmemTiles + 256 + kRunTableBytes);   // [K,V][stage][128]
  auto bar = [&](int i) { return bars + 8u * i; };

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  if (tid == 0) {
    for (int i = 0; i < NUM_BARS; ++i) {
      int count = 1;
      if (i == P_READY || i == P_READY + 1) count = kBM;
      if (i == Q_FULL || i == K_FULL || i == K_FULL + 1 || i == V_FULL || i == V_FULL + 1) count = kLoaderThreads;
      mbar_init(bar(i), count);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i <= nr; i += kThreads) runs_s[i] = rl[i];
  if (warp == 16) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int L = runs_s[nr].y;                      // selected key rows in total
  const int T = (L + kBN - 1) / kBN;               // packed key tiles

  if (warp >= 8 && warp < 12) {
    // ---------------------------------------------------------------- Q and K loader
    const int tl = tid - 8 * 32;
    if (T > 0) {
      const bf16* qb = q + (int64_t)bh * S * kHeadDim;
      const int32_t* qidx = q_row_idx ? q_row_idx + (int64_t)bh * S : nullptr;
      for (int it = 0; it < nq * 16; ++it) {
        const int row = it * 8 + (tl >> 4), chunk = tl & 15;
        const int grow = row0 + row;
        const bool ok = grow < row1;
        int p = ok ? grow : row0;
        if (ok && qidx) p = __ldg(qidx + p);
        cp_async16(q_s + (row >> 7) * kTile + tile_off(row & 127, chunk), qb + (int64_t)p * kHeadDim + chunk * 8, ok);
      }
      const bf16* kb = k + (int64_t)bh * S * kHeadDim;
      const int32_t* kidx = kv_row_idx ? kv_row_idx + (int64_t)bh * S : nullptr;
      int r_cur = 0;
      bool ok = true;
      for (int j = 0; j < T && ok; ++j) {
        const int s = j & 1;
        ok = mbar_wait(bar(K_EMPTY + s), ((j >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        gather_tile(k_s + s * kTile, kb, kidx, runs_s, nr, r_cur, rowmaps + s * 128, 1, j, L, tl);
        cp_async_commit();
        if (j >= 1) {
          cp_async_wait<1>();
          fence_async_proxy();
          if (j == 1) mbar_arrive(bar(Q_FULL));
          mbar_arrive(bar(K_FULL + (s ^ 1)));
        }
      }
      cp_async_wait<0>();
      fence_async_proxy();
      if (ok) {
        if (T == 1) mbar_arrive(bar(Q_FULL));
        mbar_arrive(bar(K_FULL + ((T - 1) & 1)));
      }
    }
  } else if (warp >= 12 && warp < 16) {
    // ---------------------------------------------------------------- V loader
    const int tl = tid - 12 * 32;
    const bf16* vb = v + (int64_t)bh * S * kHeadDim;
    const int32_t* kidx = kv_row_idx ? kv_row_idx + (int64_t)bh * S : nullptr;
    int r_cur = 0;
    bool ok = true;
    for (int j = 0; j < T && ok; ++j) {
      const int s = j & 1;
      ok = mbar_wait(bar(V_EMPTY + s), ((j >> 1) & 1) ^ 1, abort_flag);
      if (!ok) break;
      gather_tile(v_s + s * kTile, vb, kidx, runs_s, nr, r_cur, rowmaps + 256 + s * 128, 2, j, L, tl);
      cp_async_commit();
      if (j >= 1) {
        cp_async_wait<1>();
        fence_async_proxy();
        mbar_arrive(bar(V_FULL + (s ^ 1)));
      }
    }
    cp_async_wait<0>();
    fence_async_proxy();
    if (ok && T > 0) mbar_arrive(bar(V_FULL + ((T - 1) & 1)));
  } else if (warp == 16) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && T > 0) {
      auto issue_qk = [&](int w, int s) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * kBox + (ks & 3) * 32;
          umma_ss(tmem + w * 128, desc_kmajor(q_s + w * kTile + off), desc_kmajor(k_s + s * kTile + off), kIdescQK, ks > 0);
        }
      };
      auto issue_pv = [&](int w, int s, bool accumulate) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts(tmem + 256 + w * 128, tmem + w * 128 + ks * 8, desc_mnmajor(v_s + s * kTile + ks * 2048), kIdescPV,
                  (accumulate || ks > 0) ? 1u : 0u);
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag) && mbar_wait(bar(K_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        for (int w = 0; w < nq; ++w) { issue_qk(w, 0); tc_commit(bar(S_FULL + w)); }
        tc_commit(bar(K_EMPTY));
      }
      for (int j = 0; ok && j < T; ++j) {
        const int s = j & 1, sn = s ^ 1;
        const bool has_next = j + 1 < T;
        if (!mbar_wait(bar(V_FULL + s), (j >> 1) & 1, abort_flag)) break;
        for (int w = 0; w < nq && ok; ++w) {
          ok = mbar_wait(bar(P_READY + w), j & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          issue_pv(w, s, j > 0);
          tc_commit(bar(O_DONE + w));
          if (has_next) {
            if (w == 0) {
              ok = mbar_wait(bar(K_FULL + sn), ((j + 1) >> 1) & 1, abort_flag);
              if (!ok) break;
              tc_fence_after();
            }
            issue_qk(w, sn);
            tc_commit(bar(S_FULL + w));
          }
        }
        if (!ok) break;
        tc_commit(bar(V_EMPTY + s));
        if (has_next) tc_commit(bar(K_EMPTY + sn));
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue
    const int w = warp >> 2;
    if (w < nq) {
      const int quad = warp & 3;
      const int r_local = quad * 32 + lane;                       // row of the query tile == TMEM lane
      const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
      const uint32_t s_t = tmem + lane_addr + w * 128;            // S (and P) columns
      const uint32_t o_t = tmem + lane_addr + 256 + w * 128;      // O columns
      float m_used = -INFINITY, l_sum = 0.f;
      bool ok = true;
      uint32_t ra[32], rb[32];
      for (int j = 0; j < T; ++j) {
        const int valid = min(L - j * kBN, kBN);
        ok = __all_sync(0xffffffffu, mbar_wait(bar(S_FULL + w), j & 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
        // pass 1: row maximum of the raw scores (the scale is positive), two loads in flight
        float m_raw = -INFINITY;
        tmem_ld32_nowait(s_t, ra);
        tmem_ld32_nowait(s_t + 32, rb);
        tmem_wait_ld();
        if (valid >= kBN) {
          row_max(ra, m_raw);
          row_max(rb, m_raw);
          tmem_ld32_nowait(s_t + 64, ra);
          tmem_ld32_nowait(s_t + 96, rb);
          tmem_wait_ld();
          row_max(ra, m_raw);
          row_max(rb, m_raw);
        } else {
          row_max_masked(ra, m_raw, valid);
          row_max_masked(rb, m_raw, valid - 32);
          tmem_ld32_nowait(s_t + 64, ra);
          tmem_ld32_nowait(s_t + 96, rb);
          tmem_wait_ld();
          row_max_masked(ra, m_raw, valid - 64);
          row_max_masked(rb, m_raw, valid - 96);
        }
        const float m_tile = m_raw * scale_log2;
        if (j == 0) {
          m_used = m_tile;
        } else {
          const bool need = m_tile > m_used + kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar(O_DONE + w), (j - 1) & 1, abort_flag));
            if (!ok) break;
            tc_fence_after();
            const float alpha = need ? fast_exp2(m_used - m_tile) : 1.0f;
#pragma unroll 1
            for (int ch = 0; ch < 4; ++ch) {
              tmem_ld32(o_t + ch * 32, ra);
#pragma unroll
              for (int i = 0; i < 32; ++i) ra[i] = __float_as_uint(__uint_as_float(ra[i]) * alpha);
              tmem_st32(o_t + ch * 32, ra);
            }
            tmem_wait_st();
            l_sum *= alpha;
            if (need) m_used = m_tile;
          }
        }
        // pass 2: P = exp2(s * scale - m) as packed bf16 over the first 64 columns of S; the
        // load of the next 32 columns is in flight while the current 32 are processed
        const float neg_m = -m_used;
        float l0 = 0.f, l1 = 0.f;
        uint32_t pk[16];
        tmem_ld32_nowait(s_t, ra);
        tmem_wait_ld();
        tmem_ld32_nowait(s_t + 32, rb);
        exp_pack(ra, pk, scale_log2, neg_m, l0, l1, valid);
        tmem_st16(s_t, pk);
        tmem_wait_ld();
        tmem_ld32_nowait(s_t + 64, ra);
        exp_pack(rb, pk, scale_log2, neg_m, l0, l1, valid - 32);
        tmem_st16(s_t + 16, pk);
        tmem_wait_ld();
        tmem_ld32_nowait(s_t + 96, rb);
        exp_pack(ra, pk, scale_log2, neg_m, l0, l1, valid - 64);
        tmem_st16(s_t + 32, pk);
        tmem_wait_ld();
        exp_pack(rb, pk, scale_log2, neg_m, l0, l1, valid - 96);
        tmem_st16(s_t + 48, pk);
        l_sum += l0 + l1;
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar(P_READY + w));
      }
      // epilogue: O / l -> bf16 rows
      const int row = row0 + w * kBM + r_local;
      const bool store = row < row1;
      int dst = row;
      if (store && out_row_idx) dst = out_row_idx[(int64_t)bh * S + row];
      bf16* orow = out + ((int64_t)bh * S + (store ? min(max(dst, 0), S - 1) : 0)) * kHeadDim;
      if (T == 0) {
        if (store) {
#pragma unroll
          for (int ch = 0; ch < 16; ++ch) reinterpret_cast<uint4*>(orow)[ch] = make_uint4(0, 0, 0, 0);
        }
      } else if (ok && __all_sync(0xffffffffu, mbar_wait(bar(O_DONE + w), (T - 1) & 1, abort_flag))) {
        tc_fence_after();
        const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(o_t + ch * 32, ra);
          if (store) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 val;
              val.x = pack_bf16x2(__uint_as_float(ra[8 * g + 0]) * inv, __uint_as_float(ra[8 * g + 1]) * inv);
              val.y = pack_bf16x2(__uint_as_float(ra[8 * g + 2]) * inv, __uint_as_float(ra[8 * g + 3]) * inv);
              val.z = pack_bf16x2(__uint_as_float(ra[8 * g + 4]) * inv, __uint_as_float(ra[8 * g + 5]) * inv);
              val.w = pack_bf16x2(__uint_as_float(ra[8 * g + 6]) * inv, __uint_as_float(ra[8 * g + 7]) * inv);
              reinterpret_cast<uint4*>(orow)[ch * 4 + g] = val;
            }
          }
        }
      }
    }
  }
  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(status, 1);
  if (warp == 16) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

}  // namespace tc

cudaError_t launch_sparse_attn_tc(const void* q, const void* k, const void* v, void* out, const int32_t* q_row_idx,
                                  const int32_t* kv_row_idx, const int32_t* out_row_idx, const int4* qtiles,
                                  const int32_t* nqtiles, const int2* runs, const int32_t* nruns, int32_t* status,
                                  int64_t BH, int64_t S, int64_t QC, int64_t KC, float sm_scale, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(tc::sparse_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       tc::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)max_qtiles(S, QC), (unsigned)BH);
  tc::sparse_attn_tc_kernel<<<grid, tc::kThreads, tc::kSmemBytes, st>>>(
      (const bf16*)q, (const bf16*)k, (const bf16*)v, (bf16*)out, q_row_idx, kv_row_idx, out_row_idx, qtiles, nqtiles,
      runs, nruns, (int)S, (int)QC, max_qtiles(S, QC), max_runs(KC), sm_scale * 1.4426950408889634f, status);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo
