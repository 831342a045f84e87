// Block-sparse attention on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One CTA owns up to two 128-row query tiles of one query cluster.  The key rows that the
// cluster's map row selects form a list of runs of the cluster-ordered K/V; the CTA walks
// their concatenation 128 keys at a time, so key tiles are always full except the last one
// (a tile is packed across run boundaries from several TMA boxes of power-of-two heights).
//
//   warps 0-3   softmax of query tile 0: thread r owns row r (TMEM lane r): running max and
//   warps 4-7   sum, P written back over S as packed bf16; same for tile 1
//   warp 8      TMA producer for Q (once) and K, warp 9 for V: cp.async.bulk.tensor 2-D boxes of
//               64 columns with the 128-byte swizzle, no multicast; two-stage rings for K and V
//   warp 10     MMA issuer (one elected thread): S_w = Q_w K^T into TMEM (tcgen05.mma, both
//               operands from shared memory), then O_w += P_w V with P_w read from TMEM
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
#include <type_traits>
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
constexpr int kSmemBytes = kSmemTiles + 256 + kRunTableBytes + 1024;   // + barriers, run table, slack
#ifndef SVOO_SINGLE_PASS
#define SVOO_SINGLE_PASS 1
#endif
constexpr int kKWarp = 8, kVWarp = 9, kMmaWarp = 10;     // after the 8 softmax warps
// 11 warps; registers are allotted to a CTA in groups of four warps: 65536 / (12 * 32) = 170.
constexpr int kThreads = 12 * 32;       // warp 11 only completes the service warpgroup (register hand-over below)
constexpr int kRegsService = 104, kRegsSoftmax = 200;
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
#ifndef SVOO_EXP_BF16X2
#define SVOO_EXP_BF16X2 0
#endif
// Two exponentials per special-function instruction: the arguments are rounded to bf16 first,
// the results are the bf16 pair that P needs anyway.  An argument x <= 0 carries an absolute error
// of at most |x| 2^-9, so p is off by at most p |x| ln2 2^-9 <= 7e-4 of the row maximum -- the
// size of P's own bf16 rounding.  The row sum adds the rounded values, i.e. exactly the weights
// the PV product uses.
__device__ __forceinline__ uint32_t ex2_bf16x2(uint32_t x) {
  uint32_t y;
  asm("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
// p = exp2(s * scale + neg_m) for 32 columns -> 16 packed bf16 pairs; columns >= valid give 0.
__device__ __forceinline__ void exp_pack(const uint32_t (&r)[32], uint32_t (&pk)[16], float scale, float neg_m,
                                         float& l0, float& l1, int valid) {
#if SVOO_EXP_BF16X2
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float x0 = fmaf(__uint_as_float(r[2 * i]), scale, neg_m);
    const float x1 = fmaf(__uint_as_float(r[2 * i + 1]), scale, neg_m);
    uint32_t e = ex2_bf16x2(pack_bf16x2(x0, x1));
    if (valid < 32) e &= (2 * i < valid ? 0x0000ffffu : 0u) | (2 * i + 1 < valid ? 0xffff0000u : 0u);
    l0 += __uint_as_float(e << 16);
    l1 += __uint_as_float(e & 0xffff0000u);
    pk[i] = e;
  }
#else
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
#endif
}

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
#ifndef SVOO_POLY_PAIRS
#define SVOO_POLY_PAIRS 2
#endif
// exp2 of a pair on the FMA pipe instead of the special-function unit (which is the scarcer
// resource of this kernel): x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a cubic with
// relative error 7.5e-5 (P is rounded to bf16, 4e-3, afterwards); n goes into the exponent field
// with one shift-add.  Arguments below -126 are clamped (their result flushes to zero either way).
struct PolyConst {
  uint64_t magic, neg_magic, c0, c1, c2, c3;
};
__device__ __forceinline__ PolyConst poly_const() {
  PolyConst k;
  k.magic = pair2(12582912.0f);
  k.neg_magic = pair2(-12582912.0f);
  k.c0 = pair2(0.9999280571937561f);
  k.c1 = pair2(0.6932609677314758f);
  k.c2 = pair2(0.2426111251115799f);
  k.c3 = pair2(0.0551716685295105f);
  return k;
}
__device__ __forceinline__ void exp2_poly2(float x0, float x1, const PolyConst& k, float& p0, float& p1) {
  x0 = fmaxf(x0, -126.0f);
  x1 = fmaxf(x1, -126.0f);
  uint32_t t0, t1, q0, q1;
  asm("{\n\t.reg .b64 x, t, n, f, p;\n\t"
      "mov.b64 x, {%4, %5};\n\t"
      "add.rn.f32x2 t, x, %6;\n\t"
      "add.rn.f32x2 n, t, %7;\n\t"
      "sub.rn.f32x2 f, x, n;\n\t"
      "fma.rn.f32x2 p, %11, f, %10;\n\t"
      "fma.rn.f32x2 p, p, f, %9;\n\t"
      "fma.rn.f32x2 p, p, f, %8;\n\t"
      "mov.b64 {%0, %1}, t;\n\t"
      "mov.b64 {%2, %3}, p;\n\t}\n"
      : "=r"(t0), "=r"(t1), "=r"(q0), "=r"(q1)
      : "f"(x0), "f"(x1), "l"(k.magic), "l"(k.neg_magic), "l"(k.c0), "l"(k.c1), "l"(k.c2), "l"(k.c3));
  p0 = __uint_as_float((t0 << 23) + q0);
  p1 = __uint_as_float((t1 << 23) + q1);
}
// 16 columns: p = exp2(s * scale + neg_m) -> 8 packed bf16 pairs, row sums into `acc`.  The first
// SVOO_POLY_PAIRS of the 8 pairs take the polynomial, the others ex2.approx.
__device__ __forceinline__ void exp_pack16(const uint32_t (&r)[16], uint32_t* pk, uint64_t scale2, uint64_t negm2,
                                           const PolyConst& k, uint64_t& acc) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float x0, x1, p0, p1;
    fma2(x0, x1, r[2 * i], r[2 * i + 1], scale2, negm2);
    if (i < SVOO_POLY_PAIRS) {
      exp2_poly2(x0, x1, k, p0, p1);
    } else {
      p0 = fast_exp2(x0);
      p1 = fast_exp2(x1);
    }
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

#ifdef SVOO_TRACE
// Debug builds only: clock64 stamps of pipeline events of one CTA, [role][tile][slot].
__device__ long long g_trace[8 * 64 * 4];
#define TRACE(role, tile, slot) do { if (blockIdx.x == SVOO_TRACE && blockIdx.y == 0 && (tile) < 64) g_trace[((role) * 64 + (tile)) * 4 + (slot)] = clock64(); } while (0)
#else
#define TRACE(role, tile, slot) do { } while (0)
#endif

__global__ void __launch_bounds__(kThreads, 1) sparse_attn_tc_kernel(
    const __grid_constant__ AttnMaps maps, const __grid_constant__ OutPeers peers, bf16* __restrict__ out,
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
  auto bar = [&](int i) { return bars + 8u * i; };

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  if (tid == 0) {
    for (int i = 0; i < NUM_BARS; ++i) {
      int count = 1;
      if (i == P_READY || i == P_READY + 1) count = 4;       // one arrival per softmax warp
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

  // Registers move from the service warpgroup (TMA producers, MMA issuer, one idle warp) to the
  // two softmax warpgroups: 12 warps leave 168 registers per thread at launch; the softmax keeps
  // a whole tile of exponentials in registers and needs about 190.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsService));
  if (warp == kKWarp || warp == kVWarp) {
    // ---------------------------------------------------------------- TMA producers (K + Q, V)
    if (lane == 0 && T > 0) {
      const int is_v = warp == kVWarp;
      const int rows_total = (int)gridDim.y * S;
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
        TRACE(3 + is_v, j, 0);
        mbar_expect_tx(bar(full + s), kTile);
        tma_gather_tile(stage0 + s * kTile, tm, runs_s, nr, r_cur, j, L, bh * S, rows_total, bar(full + s));
        TRACE(3 + is_v, j, 1);
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
      auto issue_qk = [&](auto wc, auto sc) {
        constexpr int w = decltype(wc)::value, st = decltype(sc)::value;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * kBox + (ks & 3) * 32) >> 4;
          umma_ss_lo(tmem + w * 128, q_lo + ((w * kTile) >> 4) + off, k_lo + ((st * kTile) >> 4) + off, kDescHi, kIdescQK,
                     ks > 0);
        }
      };
      auto issue_pv = [&](auto wc, auto sc, bool accumulate) {
        constexpr int w = decltype(wc)::value, st = decltype(sc)::value;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts_lo(tmem + 256 + w * 128, tmem + w * 128 + ks * 8, v_lo + ((st * kTile + ks * 2048) >> 4), kDescHi, kIdescPV,
                     (accumulate || ks > 0) ? 1u : 0u);
      };
      using I0 = std::integral_constant<int, 0>;
      using I1 = std::integral_constant<int, 1>;
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag) && mbar_wait(bar(K_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_qk(I0{}, I0{});
        tc_commit(bar(S_FULL));
        if (nq > 1) { issue_qk(I1{}, I0{}); tc_commit(bar(S_FULL + 1)); }
        tc_commit(bar(K_EMPTY));
      }
      // one key tile: PV of both query tiles on stage `st`, QK of the next tile on the other stage
      auto tile = [&](auto sc, int j) -> bool {
        constexpr int st = decltype(sc)::value, sn = st ^ 1;
        using SN = std::integral_constant<int, sn>;
        const bool has_next = j + 1 < T;
        const uint32_t ph = (j >> 1) & 1, phn = ((j + 1) >> 1) & 1;
        TRACE(7, j, 0);
        if (!mbar_wait(bar(V_FULL + st), ph, abort_flag)) return false;
        TRACE(7, j, 1);
        if (!mbar_wait(bar(P_READY), j & 1, abort_flag)) return false;
        TRACE(2, j, 0);
        tc_fence_after();
        issue_pv(I0{}, sc, j > 0);
        if (!has_next) tc_commit(bar(O_DONE));          // only the last PV needs its own signal (see the rescale path)
        if (has_next) {
          TRACE(7, j, 2);
          if (!mbar_wait(bar(K_FULL + sn), phn, abort_flag)) return false;
          TRACE(7, j, 3);
          tc_fence_after();
          issue_qk(I0{}, SN{});
          tc_commit(bar(S_FULL));
          TRACE(2, j, 2);
        }
        if (nq > 1) {
          if (!mbar_wait(bar(P_READY + 1), j & 1, abort_flag)) return false;
          TRACE(2, j, 1);
          tc_fence_after();
          issue_pv(I1{}, sc, j > 0);
          if (!has_next) tc_commit(bar(O_DONE + 1));
          if (has_next) {
            issue_qk(I1{}, SN{});
            tc_commit(bar(S_FULL + 1));
            TRACE(2, j, 3);
          }
        }
        tc_commit(bar(V_EMPTY + st));
        if (has_next) tc_commit(bar(K_EMPTY + sn));
        return true;
      };
      for (int j = 0; ok && j < T; j += 2) {
        ok = tile(I0{}, j);
        if (ok && j + 1 < T) ok = tile(I1{}, j + 1);
      }
    }
  }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int w = warp >> 2;
    if (w < nq) {
      const int quad = warp & 3;
      const int r_local = quad * 32 + lane;                       // row of the query tile == TMEM lane
      const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
      const uint32_t s_t = tmem + lane_addr + w * 128;            // S (and P) columns
      const uint32_t o_t = tmem + lane_addr + 256 + w * 128;      // O columns
      float m_used = -INFINITY, l_sum = 0.f;
      bool ok = true;
      const PolyConst pc = poly_const();
      uint32_t ra[32], rb[32];
      for (int j = 0; j < T; ++j) {
        const int valid = min(L - j * kBN, kBN);
        ok = __all_sync(0xffffffffu, mbar_wait(bar(S_FULL + w), j & 1, abort_flag));
        if (lane == 0) TRACE(5 + w, j, warp & 3);
        if (!ok) break;
        tc_fence_after();
        if (SVOO_SINGLE_PASS && j > 0 && valid >= kBN) {
          // Common case, one TMEM pass: exponentials are taken against the running maximum of
          // the previous tiles and kept in registers; they are stored only if no row of the
          // warp outgrew that maximum by more than 2^8, otherwise the two-pass path redoes the tile.
          // Scale-and-subtract and the row sums run as packed fp32 pairs, so the special-function
          // unit (two ex2 per pair), not instruction issue, bounds the tile.
          const uint64_t scale2 = pair2(scale_log2), negm2 = pair2(-m_used);
          uint64_t acc = 0;                                // two fp32 zeros
          uint32_t pk[64];
          uint32_t xa[16], xb[16];
          tmem_ld16_nowait(s_t, xa);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 8; c += 2) {
            tmem_ld16_nowait(s_t + (c + 1) * 16, xb);
            exp_pack16(xa, &pk[c * 8], scale2, negm2, pc, acc);
            tmem_wait_ld();
            if (c + 2 < 8) tmem_ld16_nowait(s_t + (c + 2) * 16, xa);
            exp_pack16(xb, &pk[(c + 1) * 8], scale2, negm2, pc, acc);
            tmem_wait_ld();
          }
          // every p is at most the tile's row sum: a sum within 2^8 means no score outgrew the
          // running maximum by more than 8 (an overflow to inf or a NaN fails the test as well)
          const float tile_sum = pair_sum(acc);
          if (__all_sync(0xffffffffu, tile_sum <= 256.0f)) {
#pragma unroll
            for (int c = 0; c < 4; ++c) tmem_st16(s_t + c * 16, *reinterpret_cast<uint32_t(*)[16]>(&pk[c * 16]));
            l_sum += tile_sum;
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(P_READY + w));
            if (lane == 0) TRACE(w, j, warp & 3);
            continue;
          }
        }
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
            // S_FULL of this tile was committed after the PV of the previous tile by the same thread,
            // and a commit tracks every earlier tcgen05 operation of that thread: O is complete here.
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
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_READY + w));
        if (lane == 0) TRACE(w, j, warp & 3);
      }
      // epilogue: O / l -> bf16 rows
      const int row = row0 + w * kBM + r_local;
      const bool store = row < row1;
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
      if (T == 0) {
        if (store) {
#pragma unroll
          for (int ch = 0; ch < 16; ++ch) reinterpret_cast<uint4*>(orow)[ch] = make_uint4(0, 0, 0, 0);
        }
      } else if (ok && __all_sync(0xffffffffu, mbar_wait(bar(O_DONE + w), 0, abort_flag))) {
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

#ifdef SVOO_TRACE
extern "C" int svoo_b200_debug_trace(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, tc::g_trace, sizeof(tc::g_trace));
}
#endif

cudaError_t launch_sparse_attn_tc(const void* q, const void* k, const void* v, void* out, const int32_t* out_row_idx,
                                  const int4* qtiles, const int32_t* nqtiles, const int2* runs, const int32_t* nruns,
                                  int32_t* status, int64_t BH, int64_t S, int64_t QC, int64_t KC, float sm_scale,
                                  void* const* peer_dst, const int32_t* my_heads, int world, int64_t n_loc, int H,
                                  cudaStream_t st) {
  tc::OutPeers peers{};
  if (peer_dst) {
    for (int p = 0; p < world; ++p) peers.dst[p] = (bf16*)peer_dst[p];
    for (int64_t i = 0; i < BH; ++i) peers.head[i] = (int16_t)my_heads[i];
    peers.n_loc = (int)n_loc;
    peers.H = H;
  }
  alignas(64) tc::AttnMaps maps;
  bool ok = tc::make_row_tensor_map(&maps.q, q, BH * S, 128);
  for (int i = 0; i < tc::kBoxHeights && ok; ++i)
    ok = tc::make_row_tensor_map(&maps.k[i], k, BH * S, 1 << i) && tc::make_row_tensor_map(&maps.v[i], v, BH * S, 1 << i);
  if (!ok) return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(tc::sparse_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       tc::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)max_qtiles(S, QC), (unsigned)BH);
  tc::sparse_attn_tc_kernel<<<grid, tc::kThreads, tc::kSmemBytes, st>>>(
      maps, peers, (bf16*)out, out_row_idx, qtiles, nqtiles, runs, nruns, (int)S, (int)QC, max_qtiles(S, QC), max_runs(KC),
      sm_scale * 1.4426950408889634f, status);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo
