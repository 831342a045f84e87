// Block-sparse attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One CTA owns up to two 128-row query tiles of one query cluster.  The key rows that the
// cluster's map row selects form a list of runs of the cluster-ordered K/V; the CTA walks
// their concatenation 128 keys at a time, so key tiles are always full except the last one
// (a tile is packed across run boundaries from several TMA boxes of power-of-two heights).  A
// query tile with at most 64 rows (the tail of a cluster) runs M = 64 MMAs.
//
//   warps 0-3   softmax of query tile 0: thread r owns row r (TMEM lane r).  The 128 scores of the
//   warps 4-7   row are copied to registers and S is handed back at once; row max, exp2, row sum,
//               P packed to bf16 into the tile's own TMEM columns; same for query tile 1
//   warp 8      TMA producer for Q (once) and K, warp 9 for V: cp.async.bulk.tensor 2-D boxes of
//               64 columns with the 128-byte swizzle, no multicast; two-stage rings for K and V
//   warp 10     MMA issuer (one elected thread): S = Q_w K^T into TMEM (tcgen05.mma, both
//               operands from shared memory), then O_w += P_w V with P_w read from TMEM
//   warp 11     idle; it completes the service warpgroup, which gives registers to the softmax
//               warpgroups (setmaxnreg)
//
// The softmax jobs alternate between the two query tiles and share ONE S accumulator: because a
// job frees S as soon as its scores are in registers, the tensor core computes the next score
// tile while the previous one is still in its exponentials.  O stays in TMEM; it is rescaled by
// the owning softmax thread only when a row maximum grows by more than 2^8 (the running sum uses
// the same stale maximum, so the final normalisation is exact).  Every mbarrier wait is bounded;
// on expiry the CTA raises an abort flag, sets the status word and leaves through the
// normal teardown.
//
// TMEM columns (512 allocated): S [0,128)  P0 [128,192)  P1 [192,256)  O0 [256,384)  O1 [384,512).
// Semantics: svoo/co_clustering.py:949-1108 (scale D^-0.5, zero output without keys).
#include <type_traits>
#include "tc_common.cuh"

namespace svoo {
namespace tc {

constexpr int kBM = 128;                 // query rows per softmax warpgroup
constexpr int kBN = 128;                 // key rows per step
constexpr int kTile = 128 * kRowBytes;   // 32 KB: one [128 x 128] bf16 tile = two 16 KB boxes
constexpr int kBox = 128 * 128;          // 16 KB: 128 rows x 64 columns
constexpr int kSmemTiles = 6 * kTile;    // Q0 Q1 | K0 K1 | V0 V1
// Run table in shared memory: runs of selected clusters alternate with gaps, at most KC / 2 + 1 of
// them.  EAR mode (see ear.cu) appends one run, the centroid rows of the head; its bias table holds
// one value per key of the tiles that contain centroid keys.
template <bool kEar>
struct AttnSmem {
  static constexpr int kMaxRuns = SVOO_MAX_ATTN_CLUSTERS / 2 + (kEar ? 4 : 2);
  static constexpr int kRunTableBytes = (kMaxRuns * 8 + 255) / 256 * 256;
  static constexpr int kBiasFloats = kEar ? SVOO_MAX_ATTN_CLUSTERS + 128 + 6 : 0;
  static constexpr int kBiasBytes = (kBiasFloats * 4 + 255) / 256 * 256;
  static constexpr int kBytes = kSmemTiles + 256 + kRunTableBytes + kBiasBytes + 1024;   // + barriers, tables, slack
};
constexpr int kKWarp = 8, kVWarp = 9, kMmaWarp = 10;     // after the 8 softmax warps
// 12 warps; 65536 / (12 * 32) leaves 168 registers per thread at launch.
constexpr int kThreads = 12 * 32;       // warp 11 only completes the service warpgroup (register hand-over below)
#ifndef SVOO_REGS_SERVICE
#define SVOO_REGS_SERVICE 104        // 128 * 104 + 256 * 200 = 64512 = the 12 warps' launch allotment
#endif
constexpr int kRegsService = SVOO_REGS_SERVICE, kRegsSoftmax = 200;
constexpr int kBoxHeights = 8;                           // TMA boxes of 1, 2, 4, ..., 128 rows

// Tensor maps of one launch: Q with 128-row boxes; K and V with one map per box height, so a
// run segment of any length is fetched as a few power-of-two pieces.
struct AttnMaps {
  CUtensorMap q;
  CUtensorMap k[kBoxHeights];
  CUtensorMap v[kBoxHeights];
};
// Optional destination of the output rows on other GPUs: row n of local head bh goes to rank
// n / n_loc, row n % n_loc, head head[bh] of that rank's [n_loc, H, 128] array.  n_loc == 0: the
// rows go to `out` of this GPU.
struct OutPeers {
  bf16* dst[16];
  int n_loc;
  int H;
  int16_t head[128];
};
constexpr float kRescaleThreshold = 8.0f;

enum Bar { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, P_READY = 11, P_FREE = 13, S_FREE = 15, NUM_BARS = 17 };
// TMEM columns: one S accumulator shared by the two query tiles, then P0, P1 (packed bf16), O0, O1.
constexpr uint32_t kColS = 0, kColP = 128, kColO = 256;

// Packed fp32 pairs (one instruction for two lanes of data): x = s * scale + neg_m and the
// running pair of row sums.
__device__ __forceinline__ void fma2(float& x0, float& x1, uint32_t a0, uint32_t a1, uint64_t scale2, uint64_t negm2) {
  asm("{\n\t.reg .b64 a, x;\n\t"
      "mov.b64 a, {%2, %3};\n\t"
      "fma.rn.f32x2 x, a, %4, %5;\n\t"
      "mov.b64 {%0, %1}, x;\n\t}\n"
      : "=f"(x0), "=f"(x1) : "r"(a0), "r"(a1), "l"(scale2), "l"(negm2));
}
__device__ __forceinline__ void add2(uint64_t& acc, float p0, float p1) {
  asm("{\n\t.reg .b64 p;\n\t"
      "mov.b64 p, {%1, %2};\n\t"
      "add.rn.f32x2 %0, %0, p;\n\t}\n"
      : "+l"(acc) : "f"(p0), "f"(p1));
}
__device__ __forceinline__ uint64_t pair2(float v) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float pair_sum(uint64_t acc) {
  float a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(acc));
  return a + b;
}
// 16 columns: p = exp2(s * scale + neg_m) -> 8 packed bf16 pairs, row sums into `acc`.
__device__ __forceinline__ void exp_pack16(const uint32_t (&r)[16], uint32_t* pk, uint64_t scale2, uint64_t negm2,
                                           uint64_t& acc) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float x0, x1;
    fma2(x0, x1, r[2 * i], r[2 * i + 1], scale2, negm2);
    const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
    add2(acc, p0, p1);
    pk[i] = pack_bf16x2(p0, p1);
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
// M = 64 forms for a query tile with at most 64 rows (the last tile of a cluster): half the rows of
// every MMA.  Row i of such a tile lives in TMEM lane (i % 16) + 32 * (i / 16) -- sixteen rows per
// warp quadrant -- for the accumulators S and O and for the A operand P alike, so the softmax thread
// of that lane serves it and the other lanes of the quadrant idle.
constexpr uint32_t kIdescM64 = (128u >> 4) << 24 ^ (64u >> 4) << 24;      // xor turns the M = 128 field into M = 64

// Packed key tile j = virtual rows [128 j, 128 j + 128) of the concatenated runs.  Every run
// segment inside it is contiguous in the cluster-ordered tensor and is fetched by TMA as
// power-of-two pieces (two boxes of 64 columns each) placed at its row offset of the swizzled
// tile; rows past the last selected key are fetched from beyond the end of the tensor, which
// TMA fills with zeros.  Always 32 KB of transactions per tile.
__device__ __forceinline__ void tma_gather_tile(uint32_t dst, const CUtensorMap* maps, const int2* runs_s, int nr,
                                                int& r_cur, int j, int L, int head_row0, int rows_total, uint32_t bar) {
  int row = 0;
  while (row < kBN) {
    const int v = j * kBN + row;
    int len, y;
    if (v < L) {
      while (r_cur + 1 < nr && v >= runs_s[r_cur + 1].y) ++r_cur;
      len = min(runs_s[r_cur + 1].y - v, kBN - row);
      y = head_row0 + runs_s[r_cur].x + (v - runs_s[r_cur].y);
    } else {
      len = kBN - row;
      y = rows_total;                                   // out of range: zero fill
    }
    while (len > 0) {
      const int lg = 31 - __clz(len);                   // largest power of two <= len (<= 128)
      const int h = 1 << lg;
      tma_load_2d(dst + row * 128, maps + lg, 0, y, bar);
      tma_load_2d(dst + kBox + row * 128, maps + lg, 64, y, bar);
      row += h;
      len -= h;
      if (y < rows_total) y += h;
    }
  }
}

// kEar: the key list of a query cluster ends with the KC centroid rows of its head (read from the rows
// that follow the tokens of all heads in K and V).  Centroid j is a virtual key standing for the whole
// cluster j: it carries the additive bias log(|K_j| + 1e-6) (svoo/co_clustering.py:1873-1876) when the
// cluster was pruned and -inf when its tokens are in the list themselves.
template <bool kEar>
__global__ void __launch_bounds__(kThreads, 1) sparse_attn_tc_kernel(
    const __grid_constant__ AttnMaps maps, const __grid_constant__ OutPeers peers, bf16* __restrict__ out,
    const int32_t* __restrict__ out_row_idx, const int4* __restrict__ qtiles, const int32_t* __restrict__ nqtiles,
    const int2* __restrict__ runs, const int32_t* __restrict__ nruns, int S, int QC, int max_tiles, int max_runs,
    float scale_log2, int32_t* __restrict__ status, float* __restrict__ lse, const uint8_t* __restrict__ map,
    const int32_t* __restrict__ k_offsets, int KC, int rows_total) {
  constexpr int kMaxRunsSmem = AttnSmem<kEar>::kMaxRuns;
  extern __shared__ unsigned char smem_raw[];
  const int bh = blockIdx.y;
  if ((int)blockIdx.x >= nqtiles[bh]) return;
  const int4 tile = qtiles[(int64_t)bh * max_tiles + blockIdx.x];
  const int qi = tile.x, row0 = tile.y, row1 = tile.z;
  const int nr = min(nruns[(int64_t)bh * QC + qi], kMaxRunsSmem - 1);
  const int2* rl = runs + ((int64_t)bh * QC + qi) * max_runs;
  const int nq = (row1 - row0 > kBM) ? 2 : 1;
  const int rows_w[2] = {min(row1 - row0, kBM), max(row1 - row0 - kBM, 0)};      // rows of the CTA's query tiles

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base, k_s = base + 2 * kTile, v_s = base + 4 * kTile;
  const uint32_t bars = base + kSmemTiles;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + kSmemTiles + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + kSmemTiles + NUM_BARS * 8 + 8);
  int2* runs_s = reinterpret_cast<int2*>(gen_base + kSmemTiles + 256);
  float* bias_s = reinterpret_cast<float*>(gen_base + kSmemTiles + 256 + AttnSmem<kEar>::kRunTableBytes);
  auto bar = [&](int i) { return bars + 8u * i; };

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  if (tid == 0) {
    for (int i = 0; i < NUM_BARS; ++i) {
      int count = 1;
      if (i == P_READY || i == P_READY + 1 || i == S_FREE || i == S_FREE + 1) count = 4;   // one arrival per softmax warp
      mbar_init(bar(i), count);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i <= nr; i += kThreads) runs_s[i] = rl[i];
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int L = runs_s[nr].y;                      // selected key rows in total
  const int T = (L + kBN - 1) / kBN;               // packed key tiles
  // EAR: keys [l_tok, L) are the head's KC centroid rows (the last run); bias_s[v - bias0] (bias0 = first
  // key of the first tile that holds one) is the logit bias of key v divided by the softmax scale, so
  // that adding it to the raw score leaves the rest of the softmax unchanged: zero for the token keys
  // of that tile, -inf for the centroid of a selected cluster.
  int l_tok = L, bias0 = L;
  if (kEar) {
    l_tok = nr > 0 ? runs_s[nr - 1].y : L;
    bias0 = l_tok / kBN * kBN;
    const int32_t* ko = k_offsets + (int64_t)bh * (KC + 1);
    const uint8_t* mrow = map + ((int64_t)bh * QC + qi) * KC;
    for (int v = bias0 + tid; v < L; v += kThreads) {
      float b = 0.f;
      if (v >= l_tok) {
        const int j = min(v - l_tok, KC - 1);
        b = mrow[j] ? -INFINITY : __log2f((float)(ko[j + 1] - ko[j]) + 1e-6f) / scale_log2;
      }
      bias_s[v - bias0] = b;
    }
    __syncthreads();
  }

  // Registers move from the service warpgroup (TMA producers, MMA issuer, one idle warp) to the
  // two softmax warpgroups: 12 warps leave 168 registers per thread at launch; the softmax keeps
  // a whole tile of exponentials in registers and needs about 190.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsService));
  if (warp == kKWarp || warp == kVWarp) {
    // ---------------------------------------------------------------- TMA producers (K + Q, V)
    if (lane == 0 && T > 0) {
      const int is_v = warp == kVWarp;
      if (!is_v) {
        mbar_expect_tx(bar(Q_FULL), nq * kTile);
        for (int w = 0; w < nq; ++w)
          for (int h = 0; h < 2; ++h)
            tma_load_2d(q_s + w * kTile + h * kBox, &maps.q, h * 64, bh * S + row0 + w * kBM, bar(Q_FULL));
      }
      const CUtensorMap* tm = is_v ? maps.v : maps.k;
      const uint32_t stage0 = is_v ? v_s : k_s;
      const int full = is_v ? V_FULL : K_FULL, empty = is_v ? V_EMPTY : K_EMPTY;
      int r_cur = 0;
      for (int j = 0; j < T; ++j) {
        const int s = j & 1;
        if (!mbar_wait(bar(empty + s), ((j >> 1) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(bar(full + s), kTile);
        tma_gather_tile(stage0 + s * kTile, tm, runs_s, nr, r_cur, j, L, bh * S, rows_total, bar(full + s));
      }
    }
  } else if (warp == kMmaWarp) {
    // ---------------------------------------------------------------- MMA issuer
    // One thread issues every tcgen05.mma of the CTA, sharing its scheduler with two softmax
    // warps, so each instruction it executes between two MMAs is tensor-pipe idle time.  All 48
    // shared-memory descriptors are therefore built once (only their low words differ) and the
    // tile loop is specialised on the ring stage, which leaves a register move and the MMA per step.
    if (lane == 0 && T > 0) {
      constexpr uint32_t kDescHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
      // low descriptor words of the first Q / K / V tile; every other operand is a compile-time
      // offset (in 16-byte units) from these
      const uint32_t q_lo = ((q_s & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t k_lo = ((k_s & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t v_lo = ((v_s & 0x3FFFFu) >> 4) | ((uint32_t)(kBox >> 4) << 16);
      const uint32_t m64x[2] = {rows_w[0] <= 64 ? kIdescM64 : 0u, rows_w[1] <= 64 ? kIdescM64 : 0u};
      auto issue_qk = [&](auto wc, auto sc) {
        constexpr int w = decltype(wc)::value, st = decltype(sc)::value;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * kBox + (ks & 3) * 32) >> 4;
          umma_ss_lo(tmem + kColS, q_lo + ((w * kTile) >> 4) + off, k_lo + ((st * kTile) >> 4) + off, kDescHi,
                     kIdescQK ^ m64x[w], ks > 0);
        }
      };
      auto issue_pv = [&](auto wc, auto sc, bool accumulate) {
        constexpr int w = decltype(wc)::value, st = decltype(sc)::value;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts_lo(tmem + kColO + w * 128, tmem + kColP + w * 64 + ks * 8, v_lo + ((st * kTile + ks * 2048) >> 4), kDescHi,
                     kIdescPV ^ m64x[w], (accumulate || ks > 0) ? 1u : 0u);
      };
      using I0 = std::integral_constant<int, 0>;
      using I1 = std::integral_constant<int, 1>;
      // The softmax jobs run in the order (tile 0, query tile 0), (0, 1), (1, 0), (1, 1), ...  Job n
      // copies S into registers and frees it at once (S_FREE), so the QK of job n + 1 is issued
      // while job n is still computing; the PV of job n - 1 follows when its P is complete.
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag) && mbar_wait(bar(K_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_qk(I0{}, I0{});
        tc_commit(bar(S_FULL));
        if (nq == 1) tc_commit(bar(K_EMPTY));
      }
      // PV of (query tile w, key tile j) on V stage `st`
      auto pv = [&](auto wc, auto sc, int j) -> bool {
        constexpr int w = decltype(wc)::value, st = decltype(sc)::value;
        if (w == 0 && !mbar_wait(bar(V_FULL + st), (j >> 1) & 1, abort_flag)) return false;
        if (!mbar_wait(bar(P_READY + w), j & 1, abort_flag)) return false;
        tc_fence_after();
        issue_pv(wc, sc, j > 0);
        tc_commit(bar(P_FREE + w));
        if (w == nq - 1) tc_commit(bar(V_EMPTY + st));
        return true;
      };
      if (nq == 2) {
        auto tile2 = [&](auto sc, int j) -> bool {
          constexpr int st = decltype(sc)::value, sn = st ^ 1;
          using SN = std::integral_constant<int, sn>;
          // job (j, 0) has taken its S: QK of (j, 1); then PV of (j - 1, 1)
          if (!mbar_wait(bar(S_FREE), j & 1, abort_flag)) return false;
          tc_fence_after();
          issue_qk(I1{}, sc);
          tc_commit(bar(S_FULL + 1));
          tc_commit(bar(K_EMPTY + st));
          if (j > 0 && !pv(I1{}, SN{}, j - 1)) return false;
          // job (j, 1) has taken its S: QK of (j + 1, 0); then PV of (j, 0)
          if (j + 1 < T) {
            if (!mbar_wait(bar(S_FREE + 1), j & 1, abort_flag)) return false;
            if (!mbar_wait(bar(K_FULL + sn), ((j + 1) >> 1) & 1, abort_flag)) return false;
            tc_fence_after();
            issue_qk(I0{}, SN{});
            tc_commit(bar(S_FULL));
          }
          return pv(I0{}, sc, j);
        };
        for (int j = 0; ok && j < T; j += 2) {
          ok = tile2(I0{}, j);
          if (ok && j + 1 < T) ok = tile2(I1{}, j + 1);
        }
        if (ok) ok = ((T - 1) & 1) ? pv(I1{}, I1{}, T - 1) : pv(I1{}, I0{}, T - 1);
      } else {
        auto tile1 = [&](auto sc, int j) -> bool {
          constexpr int st = decltype(sc)::value, sn = st ^ 1;
          using SN = std::integral_constant<int, sn>;
          if (j + 1 < T) {
            if (!mbar_wait(bar(S_FREE), j & 1, abort_flag)) return false;
            if (!mbar_wait(bar(K_FULL + sn), ((j + 1) >> 1) & 1, abort_flag)) return false;
            tc_fence_after();
            issue_qk(I0{}, SN{});
            tc_commit(bar(S_FULL));
            tc_commit(bar(K_EMPTY + sn));
          }
          return j > 0 ? pv(I0{}, SN{}, j - 1) : true;
        };
        for (int j = 0; ok && j < T; j += 2) {
          ok = tile1(I0{}, j);
          if (ok && j + 1 < T) ok = tile1(I1{}, j + 1);
        }
        if (ok) ok = ((T - 1) & 1) ? pv(I0{}, I1{}, T - 1) : pv(I0{}, I0{}, T - 1);
      }
    }
  }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int w = warp >> 2;
    if (w < nq) {
      const int quad = warp & 3;
      const bool m64 = rows_w[w] <= 64;                           // M = 64 tile: sixteen rows per quadrant
      const int r_local = m64 ? quad * 16 + (lane & 15) : quad * 32 + lane;   // row of the query tile served by this TMEM lane
      const bool lane_has_row = !m64 || lane < 16;
      const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
      const uint32_t s_t = tmem + lane_addr + kColS;              // S, shared with the other query tile
      const uint32_t p_t = tmem + lane_addr + kColP + w * 64;     // P of this query tile (packed bf16)
      const uint32_t o_t = tmem + lane_addr + kColO + w * 128;    // O of this query tile
      float m_used = -INFINITY, l_sum = 0.f;
      bool ok = true;
      const uint64_t scale2 = pair2(scale_log2);
      for (int j = 0; j < T; ++j) {
        const int valid = min(L - j * kBN, kBN);
        ok = __all_sync(0xffffffffu, mbar_wait(bar(S_FULL + w), j & 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
        // the whole score row goes to registers; S is handed back at once so that the tensor pipe
        // can compute the next score tile (of the other query tile) while this one is processed
        uint32_t sc[128];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32_nowait(s_t + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sc[c * 32]));
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(S_FREE + w));
        if (kEar && (j + 1) * kBN > l_tok) {                      // a tile with centroid keys
          const float* bj = bias_s + (j * kBN - bias0);
#pragma unroll
          for (int i = 0; i < 128; ++i) sc[i] = __float_as_uint(__uint_as_float(sc[i]) + bj[i]);
        }
        if (valid < kBN) {                                        // last tile only: columns past the last key
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i >= valid) sc[i] = 0xff800000u;
        }
        float mr[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 128; i += 8) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mr[u] = fmaxf(mr[u], fmaxf(__uint_as_float(sc[i + 2 * u]), __uint_as_float(sc[i + 2 * u + 1])));
        }
        const float m_tile = fmaxf(fmaxf(mr[0], mr[1]), fmaxf(mr[2], mr[3])) * scale_log2;   // the scale is positive
        bool pv_done = (j == 0);                                  // PV of the previous tile complete (O and P free)
        if (j == 0) {
          m_used = kEar ? fmaxf(m_tile, -1e30f) : m_tile;           // EAR: a first tile of masked centroids only
        } else {
          // O is rescaled only when a row maximum grows by more than 2^8; the running sum keeps
          // the same stale maximum, so O / l stays exact
          const bool need = lane_has_row && m_tile > m_used + kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar(P_FREE + w), (j - 1) & 1, abort_flag));
            if (!ok) break;
            tc_fence_after();
            pv_done = true;
            const float alpha = need ? fast_exp2(m_used - m_tile) : 1.0f;
#pragma unroll 1
            for (int ch = 0; ch < 8; ++ch) {
              uint32_t t[16];
              tmem_ld16_nowait(o_t + ch * 16, t);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
              tmem_st16(o_t + ch * 16, t);
            }
            tmem_wait_st();
            l_sum *= alpha;
            if (need) m_used = m_tile;
          }
        }
        // P = exp2(s * scale - m) as packed bf16.  The first half is kept in registers until the PV
        // of the previous tile (which reads the same P columns) is known to be complete.
        const uint64_t negm2 = pair2(-m_used);
        uint64_t acc = 0;                                         // two fp32 zeros
        uint32_t pkh[32];
#pragma unroll
        for (int c = 0; c < 4; ++c)
          exp_pack16(*reinterpret_cast<const uint32_t(*)[16]>(&sc[c * 16]), &pkh[c * 8], scale2, negm2, acc);
        if (!pv_done) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar(P_FREE + w), (j - 1) & 1, abort_flag));
          if (!ok) break;
          tc_fence_after();
        }
        tmem_st16(p_t, *reinterpret_cast<uint32_t(*)[16]>(&pkh[0]));
        tmem_st16(p_t + 16, *reinterpret_cast<uint32_t(*)[16]>(&pkh[16]));
#pragma unroll
        for (int c = 4; c < 8; c += 2) {
          uint32_t pk[16];
          exp_pack16(*reinterpret_cast<const uint32_t(*)[16]>(&sc[c * 16]), &pk[0], scale2, negm2, acc);
          exp_pack16(*reinterpret_cast<const uint32_t(*)[16]>(&sc[(c + 1) * 16]), &pk[8], scale2, negm2, acc);
          tmem_st16(p_t + c * 8, pk);
        }
        l_sum += pair_sum(acc);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_READY + w));
      }
      uint32_t ra[32];
      // epilogue: O / l -> bf16 rows
      const int row = row0 + w * kBM + r_local;
      const bool store = lane_has_row && row < row1;
      int dst = row;
      if (store && out_row_idx) dst = out_row_idx[(int64_t)bh * S + row];
      dst = store ? min(max(dst, 0), S - 1) : 0;
      bf16* orow;
      if (peers.n_loc == 0) {
        orow = out + ((int64_t)bh * S + dst) * kHeadDim;
      } else {                                           // store straight into the owning rank's sequence shard
        const int p = dst / peers.n_loc;
        orow = peers.dst[p] + ((int64_t)(dst - p * peers.n_loc) * peers.H + peers.head[bh]) * kHeadDim;
      }
      // log2 of the softmax denominator, sum_j 2^(s_j * scale * log2 e); -inf for a row without keys
      if (lse && store && (T == 0 || ok))
        lse[(int64_t)bh * S + dst] = (T == 0 || !(l_sum > 0.f)) ? -INFINITY : m_used + __log2f(l_sum);
      if (T == 0) {
        if (store) {
#pragma unroll
          for (int ch = 0; ch < 16; ++ch) reinterpret_cast<uint4*>(orow)[ch] = make_uint4(0, 0, 0, 0);
        }
      } else if (ok && __all_sync(0xffffffffu, mbar_wait(bar(P_FREE + w), (T - 1) & 1, abort_flag))) {
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
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

}  // namespace tc


cudaError_t launch_sparse_attn_tc(const void* q, const void* k, const void* v, void* out, const int32_t* out_row_idx,
                                  const int4* qtiles, const int32_t* nqtiles, const int2* runs, const int32_t* nruns,
                                  int32_t* status, int64_t BH, int64_t S, int64_t QC, int64_t KC, float sm_scale,
                                  void* const* peer_dst, const int32_t* my_heads, int world, int64_t n_loc, int H,
                                  float* lse, cudaStream_t st, const uint8_t* ear_map, const int32_t* ear_k_offsets,
                                  int ear_max_runs) {
  // a build whose register hand-over does not add up (the spill-check build) must never launch:
  // its softmax warps would wait for registers that nobody frees
  if (128 * tc::kRegsService + 256 * tc::kRegsSoftmax > 168 * tc::kThreads) return cudaErrorInvalidConfiguration;
  tc::OutPeers peers{};
  if (peer_dst) {
    for (int p = 0; p < world; ++p) peers.dst[p] = (bf16*)peer_dst[p];
    for (int64_t i = 0; i < BH; ++i) peers.head[i] = (int16_t)my_heads[i];
    peers.n_loc = (int)n_loc;
    peers.H = H;
  }
  // EAR: K and V hold the centroid rows of all heads after the token rows of all heads
  const bool ear = ear_map != nullptr;
  const int64_t kv_rows = BH * S + (ear ? BH * KC : 0);
  alignas(64) tc::AttnMaps maps;
  bool ok = tc::make_row_tensor_map(&maps.q, q, BH * S, 128);
  for (int i = 0; i < tc::kBoxHeights && ok; ++i)
    ok = tc::make_row_tensor_map(&maps.k[i], k, kv_rows, 1 << i) && tc::make_row_tensor_map(&maps.v[i], v, kv_rows, 1 << i);
  if (!ok) return cudaErrorInvalidValue;
  dim3 grid((unsigned)max_qtiles(S, QC), (unsigned)BH);
  const float scale_log2 = sm_scale * 1.4426950408889634f;
  cudaError_t e;
  if (ear) {
    e = cudaFuncSetAttribute(tc::sparse_attn_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             tc::AttnSmem<true>::kBytes);
    if (e != cudaSuccess) return e;
    tc::sparse_attn_tc_kernel<true><<<grid, tc::kThreads, tc::AttnSmem<true>::kBytes, st>>>(
        maps, peers, (bf16*)out, out_row_idx, qtiles, nqtiles, runs, nruns, (int)S, (int)QC, max_qtiles(S, QC), ear_max_runs,
        scale_log2, status, peer_dst ? nullptr : lse, ear_map, ear_k_offsets, (int)KC, (int)kv_rows);
  } else {
    e = cudaFuncSetAttribute(tc::sparse_attn_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             tc::AttnSmem<false>::kBytes);
    if (e != cudaSuccess) return e;
    tc::sparse_attn_tc_kernel<false><<<grid, tc::kThreads, tc::AttnSmem<false>::kBytes, st>>>(
        maps, peers, (bf16*)out, out_row_idx, qtiles, nqtiles, runs, nruns, (int)S, (int)QC, max_qtiles(S, QC), max_runs(KC),
        scale_log2, status, peer_dst ? nullptr : lse, nullptr, nullptr, (int)KC, (int)kv_rows);
  }
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo
