// Block-sparse attention over cluster-ordered Q/K/V on the 5th-generation tensor cores.
//
// One CTA owns up to two 128-row query tiles of one query cluster (they share the key
// runs the cluster's map row selects) and walks those runs 128 key rows at a time:
//
//   warp 0      TMA producer: Q tiles once, then K and V tiles through two 2-stage rings
//               (cp.async.bulk.tensor 2-D boxes of 64 columns x 128 rows, 128-byte swizzle)
//   warp 1      MMA issuer (one elected thread): S_w = Q_w K^T into TMEM (tcgen05.mma, both
//               operands from shared memory), then O_w += P_w V with P_w read from TMEM
//   warps 4-7   softmax of query tile 0: thread r owns row r (TMEM lane r): running max and
//   warps 8-11  sum, P written back over S as packed bf16; same for tile 1
//
// The two query tiles ping-pong: while one tile's rows are in the softmax, the tensor
// core works on the other tile's products.  O stays in TMEM; it is rescaled by the owning
// softmax thread only when a row maximum grows by more than 2^8 (the running sum uses the
// same stale maximum, so the final normalisation is exact).  Key tiles never cross a run
// end: columns past it are masked to -inf.  Every mbarrier wait is bounded; on expiry the
// CTA raises an abort flag, sets the status word and leaves through the normal teardown.
//
// TMEM columns (512 allocated): S0 [0,128)  S1 [128,256)  O0 [256,384)  O1 [384,512).
// Semantics: svoo/co_clustering.py:949-1108 (scale D^-0.5, zero output without keys).
#include <cuda.h>

#include "common.cuh"

namespace svoo {
namespace tc {

constexpr int kBM = 128;                 // query rows per softmax warpgroup
constexpr int kBN = 128;                 // key rows per step
constexpr int kTile = 128 * kRowBytes;   // 32 KB: one [128 x 128] bf16 tile = two 16 KB boxes
constexpr int kBox = 128 * 128;          // 16 KB: 128 rows x 64 columns
constexpr int kSmemTiles = 6 * kTile;    // Q0 Q1 | K0 K1 | V0 V1
constexpr int kSmemBytes = kSmemTiles + 256 + 1024;   // + barriers + alignment slack
constexpr int kThreads = 384;
constexpr float kRescaleThreshold = 8.0f;
constexpr long long kWaitCycles = 2000000000LL;       // ~1 s

enum Bar { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, P_READY = 11, O_DONE = 13, NUM_BARS = 15 };

// ------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}\n"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false when the wait expired or another thread of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) { *abort_flag = 1; return false; }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
      ::"r"(d), "r"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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

// Cursor over the 128-row key tiles of a run list.
struct TileCursor {
  const int2* runs;
  int nr, S, r, p, e;
  __device__ __forceinline__ void load_run() {
    if (r < nr) { const int2 x = runs[r]; p = max(x.x, 0); e = min(x.y, S); }
  }
  __device__ __forceinline__ TileCursor(const int2* runs_, int nr_, int S_) : runs(runs_), nr(nr_), S(S_), r(0), p(0), e(0) {
    load_run();
    skip_empty();
  }
  __device__ __forceinline__ void skip_empty() { while (r < nr && p >= e) { ++r; load_run(); } }
  __device__ __forceinline__ bool done() const { return r >= nr; }
  __device__ __forceinline__ int valid() const { return min(e - p, kBN); }
  __device__ __forceinline__ void next() {
    p += kBN;
    if (p >= e) { ++r; load_run(); skip_empty(); }
  }
};

__global__ void __launch_bounds__(kThreads, 1) sparse_attn_tc_kernel(
    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
    const __grid_constant__ CUtensorMap tm_v, bf16* __restrict__ out, const int32_t* __restrict__ out_row_idx,
    const int4* __restrict__ qtiles, const int32_t* __restrict__ nqtiles, const int2* __restrict__ runs,
    const int32_t* __restrict__ nruns, int S, int QC, int max_tiles, int max_runs, float scale_log2,
    int32_t* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  const int bh = blockIdx.y;
  if ((int)blockIdx.x >= nqtiles[bh]) return;
  const int4 tile = qtiles[(int64_t)bh * max_tiles + blockIdx.x];
  const int qi = tile.x, row0 = tile.y, row1 = tile.z;
  const int nr = nruns[(int64_t)bh * QC + qi];
  const int2* rl = runs + ((int64_t)bh * QC + qi) * max_runs;
  const int nq = (row1 - row0 > kBM) ? 2 : 1;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_s = base, k_s = base + 2 * kTile, v_s = base + 4 * kTile;
  const uint32_t bars = base + kSmemTiles;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + kSmemTiles + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + kSmemTiles + NUM_BARS * 8 + 8);
  auto bar = [&](int i) { return bars + 8u * i; };

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  if (tid == 0) {
    for (int i = 0; i < NUM_BARS; ++i) mbar_init(bar(i), (i == P_READY || i == P_READY + 1) ? kBM : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(bar(Q_FULL), nq * kTile);
      for (int w = 0; w < nq; ++w)
        for (int h = 0; h < 2; ++h)
          tma_load_2d(q_s + w * kTile + h * kBox, &tm_q, h * 64, bh * S + row0 + w * kBM, bar(Q_FULL));
      int j = 0;
      for (TileCursor c(rl, nr, S); !c.done(); c.next(), ++j) {
        const int s = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(bar(K_EMPTY + s), ph, abort_flag)) break;
        mbar_expect_tx(bar(K_FULL + s), kTile);
        for (int h = 0; h < 2; ++h) tma_load_2d(k_s + s * kTile + h * kBox, &tm_k, h * 64, bh * S + c.p, bar(K_FULL + s));
        if (!mbar_wait(bar(V_EMPTY + s), ph, abort_flag)) break;
        mbar_expect_tx(bar(V_FULL + s), kTile);
        for (int h = 0; h < 2; ++h) tma_load_2d(v_s + s * kTile + h * kBox, &tm_v, h * 64, bh * S + c.p, bar(V_FULL + s));
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
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
      TileCursor c(rl, nr, S);
      bool ok = !c.done() && mbar_wait(bar(Q_FULL), 0, abort_flag) && mbar_wait(bar(K_FULL), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        for (int w = 0; w < nq; ++w) { issue_qk(w, 0); tc_commit(bar(S_FULL + w)); }
        tc_commit(bar(K_EMPTY));
      }
      for (int j = 0; ok && !c.done(); ++j) {
        const int s = j & 1, sn = s ^ 1;
        c.next();
        const bool has_next = !c.done();
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
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax + epilogue
    const int w = (warp - 4) >> 2;
    if (w < nq) {
      const int quad = warp & 3;
      const int r_local = quad * 32 + lane;                       // row of the query tile == TMEM lane
      const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
      const uint32_t s_t = tmem + lane_addr + w * 128;            // S (and P) columns
      const uint32_t o_t = tmem + lane_addr + 256 + w * 128;      // O columns
      float m_used = -INFINITY, l_sum = 0.f;
      bool ok = true;
      int j = 0;
      uint32_t r[32];
      for (TileCursor c(rl, nr, S); !c.done(); c.next(), ++j) {
        const int valid = c.valid();
        ok = mbar_wait(bar(S_FULL + w), j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        // pass 1: row maximum of the scaled scores
        float m_tile = -INFINITY;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(s_t + ch * 32, r);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float v = __uint_as_float(r[i]) * scale_log2;
            m_tile = fmaxf(m_tile, (ch * 32 + i < valid) ? v : -INFINITY);
          }
        }
        if (j == 0) {
          m_used = m_tile;
        } else {
          const bool need = m_tile > m_used + kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            ok = mbar_wait(bar(O_DONE + w), (j - 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            const float alpha = need ? fast_exp2(m_used - m_tile) : 1.0f;
#pragma unroll 1
            for (int ch = 0; ch < 4; ++ch) {
              tmem_ld32(o_t + ch * 32, r);
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st32(o_t + ch * 32, r);
            }
            tmem_wait_st();
            l_sum *= alpha;
            if (need) m_used = m_tile;
          }
        }
        // pass 2: P = exp2(s - m), packed bf16 written over the first 64 columns of S
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(s_t + ch * 32, r);
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int c0 = ch * 32 + 2 * i;
            float p0 = fast_exp2(__uint_as_float(r[2 * i]) * scale_log2 - m_used);
            float p1 = fast_exp2(__uint_as_float(r[2 * i + 1]) * scale_log2 - m_used);
            p0 = (c0 < valid) ? p0 : 0.f;
            p1 = (c0 + 1 < valid) ? p1 : 0.f;
            l_sum += p0 + p1;
            pk[i] = pack_bf16x2(p0, p1);
          }
          tmem_st16(s_t + ch * 16, pk);
        }
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
      if (j == 0 || !ok) {
        if (store && ok) {
#pragma unroll
          for (int ch = 0; ch < 16; ++ch) reinterpret_cast<uint4*>(orow)[ch] = make_uint4(0, 0, 0, 0);
        }
      } else if (mbar_wait(bar(O_DONE + w), (j - 1) & 1, abort_flag)) {
        tc_fence_after();
        const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(o_t + ch * 32, r);
          if (store) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[8 * g + 0]) * inv, __uint_as_float(r[8 * g + 1]) * inv);
              v.y = pack_bf16x2(__uint_as_float(r[8 * g + 2]) * inv, __uint_as_float(r[8 * g + 3]) * inv);
              v.z = pack_bf16x2(__uint_as_float(r[8 * g + 4]) * inv, __uint_as_float(r[8 * g + 5]) * inv);
              v.w = pack_bf16x2(__uint_as_float(r[8 * g + 6]) * inv, __uint_as_float(r[8 * g + 7]) * inv);
              reinterpret_cast<uint4*>(orow)[ch * 4 + g] = v;
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
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [rows, 128] bf16 row-major tensor, boxes of 64 columns x 128 rows, 128-byte swizzle, zero fill.
static bool make_row_map(CUtensorMap* map, const void* ptr, int64_t rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)kHeadDim, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)kRowBytes};
  const cuuint32_t box[2] = {64, 128};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc

cudaError_t launch_sparse_attn_tc(const void* q, const void* k, const void* v, void* out, const int32_t* out_row_idx,
                                  const int4* qtiles, const int32_t* nqtiles, const int2* runs, const int32_t* nruns,
                                  int32_t* status, int64_t BH, int64_t S, int64_t QC, int64_t KC, float sm_scale,
                                  cudaStream_t st) {
  alignas(64) CUtensorMap mq, mk, mv;
  if (!tc::make_row_map(&mq, q, BH * S) || !tc::make_row_map(&mk, k, BH * S) || !tc::make_row_map(&mv, v, BH * S))
    return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(tc::sparse_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       tc::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)max_qtiles(S, QC), (unsigned)BH);
  tc::sparse_attn_tc_kernel<<<grid, tc::kThreads, tc::kSmemBytes, st>>>(
      mq, mk, mv, (bf16*)out, out_row_idx, qtiles, nqtiles, runs, nruns, (int)S, (int)QC, max_qtiles(S, QC),
      max_runs(KC), sm_scale * 1.4426950408889634f, status);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo
