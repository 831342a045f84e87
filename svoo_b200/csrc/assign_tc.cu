// Co-clustering assignment on the 5th-generation tensor cores:
//     label[n] = first argmax_j  x_n . (W_hi[j] + W_lo[j]),   j < J
// (see cluster.cu for how W = Phat . C replaces the reference's two chained GEMMs,
// svoo/co_clustering.py:2148-2255).
//
// W-stationary, persistent.  The job list is (head, block of 256 W rows, tile of 128 tokens),
// token tile fastest; each CTA (one per SM) takes a contiguous slice of it.  A block of W
// (hi and lo, 128 KB) stays in shared memory while the token tiles of that head stream
// through a three-stage ring (32 KB each), so shared memory is filled at 16 B per MMA clock
// instead of re-reading W for every token tile.
//
//   warp 0      TMA producer (cp.async.bulk.tensor 2-D boxes, 128-byte swizzle, no multicast)
//   warp 1      MMA issuer: D[128 x 256] (+)= X[128 x 16] . W^T[16 x 256], 8 k-steps for hi and
//               8 for lo into one of two TMEM accumulators (tcgen05.mma kind::f16, M128 N256)
//   warps 4-11  epilogue: thread r of each group of four warps owns token row r (TMEM lane r)
//               and one half of the accumulator columns: running first-argmax, one (score, j)
//               pair per token and column group written to scratch
//
// A small second kernel reduces the per-block pairs to labels (lower block wins ties).
// Every mbarrier wait is bounded; on expiry the CTA sets the status word and leaves.
#include "tc_common.cuh"

namespace svoo {
namespace tc {

constexpr int kAsgXT = 128;                       // tokens per tile
constexpr int kAsgXBytes = kAsgXT * kRowBytes;    // 32 KB
constexpr int kAsgXHalf = kAsgXT * 128;           // 16 KB: 128 rows x 64 columns
constexpr int kAsgThreads = 384;                  // producer, MMA, 2 idle, 8 epilogue warps

// JB = W rows per block (256, or 128 when there are at most 128 clusters to assign to).
template <int JB>
struct AsgCfg {
  static constexpr int kWHalf = JB * 128;                       // JB rows x 64 columns
  static constexpr int kWBytes = 2 * kWHalf;                    // per hi / lo
  static constexpr int kXStages = JB == 256 ? 3 : 4;
  static constexpr int kSmemData = 2 * kWBytes + kXStages * kAsgXBytes;
  static constexpr int kSmemBytes = kSmemData + 256 + 1024;
  // barrier indices
  static constexpr int W_FULL = 0, W_EMPTY = 1, X_FULL = 2, X_EMPTY = X_FULL + kXStages,
                       ACC_FULL = X_EMPTY + kXStages, ACC_EMPTY = ACC_FULL + 2, NUM = ACC_EMPTY + 2;
};

struct AsgJob {
  int bh, jb, t;
};
__device__ __forceinline__ AsgJob asg_job(int64_t g, int n_jb, int n_xt) {
  AsgJob j;
  j.t = (int)(g % n_xt);
  const int64_t r = g / n_xt;
  j.jb = (int)(r % n_jb);
  j.bh = (int)(r / n_jb);
  return j;
}

// Running first-argmax over 32 accumulator columns starting at column c0; with kBias the
// per-column bias (shared memory, indexed like the columns) is added to the score first.
template <bool kBias>
__device__ __forceinline__ void argmax32(const uint32_t (&r)[32], int c0, int jlim, const float* bias, float& best,
                                         int& best_c) {
  if (c0 + 32 <= jlim) {
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      float val = __uint_as_float(r[c]);
      if (kBias) val += bias[c0 + c];
      if (val > best) { best = val; best_c = c0 + c; }
    }
  } else {
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      float val = __uint_as_float(r[c]);
      if (kBias) val += bias[c0 + c];
      if (c0 + c < jlim && val > best) { best = val; best_c = c0 + c; }
    }
  }
}

// kEuclid = false: scores x . (W_hi + W_lo), W rows of head bh at [bh * w_head_rows, +J).
// kEuclid = true:  nearest centroid in Euclidean distance, argmax_j x . c_j + bias[bh, j] with
//                  bias = -|c_j|^2 / 2 (one product per k-step: the centroids are bf16 already);
//                  tm_hi then maps the centroid tensor itself, tm_lo is unused.
template <int JB, bool kEuclid>
__global__ void __launch_bounds__(kAsgThreads, 1) assign_tc_kernel(
    const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_hi,
    const __grid_constant__ CUtensorMap tm_lo, int2* __restrict__ partial, int BH, int N, int J, int w_head_rows,
    const float* __restrict__ bias, int32_t* __restrict__ status) {
  using C = AsgCfg<JB>;
  constexpr int NS = C::kXStages;
  constexpr uint32_t kIdesc = idesc_bf16(128, JB, false);
  // At most 128 clusters: W_hi and W_lo are stacked as ONE 256-row operand (per 64-column half: the
  // 128 hi rows, then the 128 lo rows), so that one M128 x N256 MMA per k-step computes both
  // products, into accumulator columns j and j + 128, which the epilogue adds.
  constexpr bool kStack = JB == 128 && !kEuclid;
  constexpr uint32_t kIdescStack = idesc_bf16(128, 256, false);
  extern __shared__ unsigned char smem_raw[];
  const int n_jb = (J + JB - 1) / JB, n_xt = (N + kAsgXT - 1) / kAsgXT;
  const int64_t total = (int64_t)BH * n_jb * n_xt;
  const int64_t per = (total + gridDim.x - 1) / gridDim.x;
  const int64_t g0 = (int64_t)blockIdx.x * per;
  const int64_t g1 = g0 + per < total ? g0 + per : total;
  if (g0 >= g1) return;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t whi_s = base, wlo_s = base + C::kWBytes, x_s = base + 2 * C::kWBytes;
  const uint32_t bars = base + C::kSmemData;
  unsigned char* gen_base = smem_raw + (base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + C::kSmemData + C::NUM * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + C::kSmemData + C::NUM * 8 + 8);
  auto bar = [&](int i) { return bars + 8u * i; };

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  if (tid == 0) {
    for (int i = 0; i < C::NUM; ++i) mbar_init(bar(i), (i >= C::ACC_EMPTY) ? 256 : 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_trigger();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();                                             // W (and the centroids before it) come from the previous kernels

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int wq = 0, prev_block = -1, i = 0;
      for (int64_t g = g0; g < g1; ++g, ++i) {
        const AsgJob job = asg_job(g, n_jb, n_xt);
        const int block = job.bh * n_jb + job.jb;
        if (block != prev_block) {
          if (!mbar_wait(bar(C::W_EMPTY), (wq & 1) ^ 1, abort_flag)) break;
          mbar_expect_tx(bar(C::W_FULL), (kEuclid ? 1 : 2) * C::kWBytes);
          const int y = job.bh * w_head_rows + job.jb * JB;
          for (int h = 0; h < 2; ++h) {
            if (kStack) {
              tma_load_2d(whi_s + h * 2 * C::kWHalf, &tm_hi, h * 64, y, bar(C::W_FULL));
              tma_load_2d(whi_s + h * 2 * C::kWHalf + C::kWHalf, &tm_lo, h * 64, y, bar(C::W_FULL));
            } else {
              tma_load_2d(whi_s + h * C::kWHalf, &tm_hi, h * 64, y, bar(C::W_FULL));
              if (!kEuclid) tma_load_2d(wlo_s + h * C::kWHalf, &tm_lo, h * 64, y, bar(C::W_FULL));
            }
          }
          prev_block = block;
          ++wq;
        }
        const int s = i % NS;
        if (!mbar_wait(bar(C::X_EMPTY + s), ((i / NS) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(bar(C::X_FULL + s), kAsgXBytes);
        for (int h = 0; h < 2; ++h)
          tma_load_2d(x_s + s * kAsgXBytes + h * kAsgXHalf, &tm_x, h * 64, job.bh * N + job.t * kAsgXT, bar(C::X_FULL + s));
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int wq = 0, prev_block = -1, i = 0;
      for (int64_t g = g0; g < g1; ++g, ++i) {
        const AsgJob job = asg_job(g, n_jb, n_xt);
        const int block = job.bh * n_jb + job.jb;
        if (block != prev_block) {
          if (!mbar_wait(bar(C::W_FULL), wq & 1, abort_flag)) break;
          prev_block = block;
          ++wq;
        }
        const int s = i % NS, b = i & 1;
        if (!mbar_wait(bar(C::X_FULL + s), (i / NS) & 1, abort_flag)) break;
        if (!mbar_wait(bar(C::ACC_EMPTY + b), ((i >> 1) & 1) ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d = tmem + b * 256;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t a = smem_desc_sw128(x_s + s * kAsgXBytes + (ks >> 2) * kAsgXHalf + (ks & 3) * 32, 16, 1024);
          if (kStack) {
            umma_ss(d, a, smem_desc_sw128(whi_s + (ks >> 2) * 2 * C::kWHalf + (ks & 3) * 32, 16, 1024), kIdescStack, ks > 0);
          } else {
            const uint32_t woff = (ks >> 2) * C::kWHalf + (ks & 3) * 32;
            umma_ss(d, a, smem_desc_sw128(whi_s + woff, 16, 1024), kIdesc, ks > 0);
            if (!kEuclid) umma_ss(d, a, smem_desc_sw128(wlo_s + woff, 16, 1024), kIdesc, 1);
          }
        }
        tc_commit(bar(C::X_EMPTY + s));
        tc_commit(bar(C::ACC_FULL + b));
        bool last_of_block = g + 1 >= g1;
        if (!last_of_block) {
          const AsgJob nxt = asg_job(g + 1, n_jb, n_xt);
          last_of_block = nxt.bh * n_jb + nxt.jb != block;
        }
        if (last_of_block) tc_commit(bar(C::W_EMPTY));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------- epilogue: running argmax, half of the columns per warp
    const int quad = warp & 3, half = (warp - 4) >> 2;
    const int r_local = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    constexpr int HC = JB / 2;                               // columns per half
    uint32_t ra[32], rb[32];
    int i = 0;
    bool ok = true;
    // Euclidean mode: the bias of the current W block, one private copy per epilogue warp in the
    // shared memory that the (absent) W_lo operand would occupy
    float* bias_s = reinterpret_cast<float*>(gen_base + C::kWBytes) + (warp - 4) * HC;
    int bias_block = -1;
    for (int64_t g = g0; g < g1 && ok; ++g, ++i) {
      const AsgJob job = asg_job(g, n_jb, n_xt);
      const int b = i & 1;
      if (kEuclid && job.bh * n_jb + job.jb != bias_block) {
        bias_block = job.bh * n_jb + job.jb;
        __syncwarp();
        for (int c = lane; c < HC; c += 32) {
          const int j = job.jb * JB + half * HC + c;
          bias_s[c] = j < J ? bias[(int64_t)job.bh * J + j] : 0.f;
        }
        __syncwarp();
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar(C::ACC_FULL + b), (i >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem + lane_addr + b * 256 + half * HC;
      const int jlim = J - job.jb * JB - half * HC;            // valid columns of this half (may be <= 0)
      float best = -INFINITY;
      int best_c = 0;
      if (kStack) {
#pragma unroll
        for (int ch = 0; ch < HC / 32; ++ch) {
          tmem_ld32_nowait(acc + ch * 32, ra);
          tmem_ld32_nowait(acc + 128 + ch * 32, rb);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) ra[c] = __float_as_uint(__uint_as_float(ra[c]) + __uint_as_float(rb[c]));
          argmax32<false>(ra, ch * 32, jlim, bias_s, best, best_c);
        }
      } else {
      tmem_ld32_nowait(acc, ra);
      tmem_wait_ld();
#pragma unroll
      for (int ch = 0; ch < HC / 32; ch += 2) {
        tmem_ld32_nowait(acc + (ch + 1) * 32, rb);
        argmax32<kEuclid>(ra, ch * 32, jlim, bias_s, best, best_c);
        tmem_wait_ld();
        if (ch + 2 < HC / 32) tmem_ld32_nowait(acc + (ch + 2) * 32, ra);
        argmax32<kEuclid>(rb, (ch + 1) * 32, jlim, bias_s, best, best_c);
        tmem_wait_ld();
      }
      }
      tc_fence_before();
      mbar_arrive(bar(C::ACC_EMPTY + b));
      const int n = job.t * kAsgXT + r_local;
      if (n < N)
        partial[((int64_t)(job.jb * 2 + half) * BH + job.bh) * N + n] =
            make_int2(__float_as_int(best), job.jb * JB + half * HC + best_c);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicExch(status, 2);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// labels[bh, n] = j of the best (score, j) pair over the column groups; the lower group wins ties.
__global__ void __launch_bounds__(256) assign_reduce_kernel(const int2* __restrict__ partial, int32_t* __restrict__ labels,
                                                            int64_t BHN, int groups) {
  pdl_trigger();
  pdl_wait();
  const int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (i >= BHN) return;
  int2 b = partial[i];
  for (int g = 1; g < groups; ++g) {
    const int2 c = partial[(int64_t)g * BHN + i];
    if (__int_as_float(c.x) > __int_as_float(b.x)) b = c;
  }
  labels[i] = b.y;
}

// The same reduction fused with the first pass of the label sort: one CTA per (2048-token chunk,
// head) also leaves the chunk's label histogram, which saves a kernel and a second read of the labels.
__global__ void __launch_bounds__(256) assign_reduce_hist_kernel(const int2* __restrict__ partial,
                                                                 int32_t* __restrict__ labels,
                                                                 int32_t* __restrict__ chunk_hist, int BH, int N, int K,
                                                                 int groups, int nchunks) {
  __shared__ int hist[SVOO_MAX_CLUSTERS];
  pdl_trigger();
  const int bh = blockIdx.y, chunk = blockIdx.x;
  for (int k = threadIdx.x; k < K; k += 256) hist[k] = 0;
  __syncthreads();
  pdl_wait();
  const int64_t BHN = (int64_t)BH * N;
  const int base = chunk * kSortChunk;
  for (int t = threadIdx.x; t < kSortChunk; t += 256) {
    const int n = base + t;
    if (n < N) {
      const int64_t i = (int64_t)bh * N + n;
      int2 b = partial[i];
      for (int g = 1; g < groups; ++g) {
        const int2 c = partial[(int64_t)g * BHN + i];
        if (__int_as_float(c.x) > __int_as_float(b.x)) b = c;
      }
      labels[i] = b.y;
      if (b.y >= 0 && b.y < K) atomicAdd(&hist[b.y], 1);
    }
  }
  __syncthreads();
  int32_t* out = chunk_hist + ((int64_t)bh * nchunks + chunk) * K;
  for (int k = threadIdx.x; k < K; k += 256) out[k] = hist[k];
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

bool make_row_tensor_map(CUtensorMap* map, const void* ptr, int64_t rows, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)kHeadDim, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)kRowBytes};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace tc

template <int JB, bool kEuclid>
static cudaError_t launch_assign_tc_jb(const void* x, const void* w_hi, const void* w_lo, const float* bias, int2* partial,
                                       int32_t* status, int64_t BH, int64_t N, int64_t J, int w_head_rows,
                                       cudaStream_t st) {
  using C = tc::AsgCfg<JB>;
  alignas(64) CUtensorMap mx, mh, ml;
  if (!tc::make_row_tensor_map(&mx, x, BH * N, tc::kAsgXT) || !tc::make_row_tensor_map(&mh, w_hi, BH * w_head_rows, JB) ||
      !tc::make_row_tensor_map(&ml, w_lo, BH * w_head_rows, JB))
    return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(tc::assign_tc_kernel<JB, kEuclid>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       C::kSmemBytes);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t total = BH * ceil_div64(J, JB) * ceil_div64(N, tc::kAsgXT);
  const unsigned grid = (unsigned)(total < sms ? total : sms);
  return launch_pdl(tc::assign_tc_kernel<JB, kEuclid>, dim3(grid), dim3(tc::kAsgThreads), (size_t)C::kSmemBytes, st, mx, mh, ml,
                    partial, (int)BH, (int)N, (int)J, w_head_rows, bias, status);
}

static cudaError_t launch_assign_reduce(const int2* partial, int32_t* labels, int64_t BH, int64_t N, int64_t J, int jb,
                                        int32_t* chunk_hist, cudaStream_t st) {
  const int groups = 2 * (int)ceil_div64(J, jb);
  if (chunk_hist) {
    const int nchunks = sort_chunks(N);
    count_launches(2);
    return launch_pdl(tc::assign_reduce_hist_kernel, dim3((unsigned)nchunks, (unsigned)BH), dim3(256), 0, st,
                      (const int2*)partial, labels, chunk_hist, (int)BH, (int)N, (int)J, groups, nchunks);
  }
  count_launches(2);
  return launch_pdl(tc::assign_reduce_kernel, dim3((unsigned)ceil_div64(BH * N, 256)), dim3(256), 0, st, (const int2*)partial,
                    labels, BH * N, groups);
}

// chunk_hist != nullptr: also write the per-chunk label histograms of the sort (its first pass).
cudaError_t launch_assign_tc(const void* x, const void* w_hi, const void* w_lo, int32_t* labels, int2* partial,
                             int32_t* status, int64_t BH, int64_t N, int64_t J, int32_t* chunk_hist, cudaStream_t st) {
  const int Jpad = pad_clusters(J);
  const int jb = J <= 128 ? 128 : 256;
  cudaError_t e = jb == 128 ? launch_assign_tc_jb<128, false>(x, w_hi, w_lo, nullptr, partial, status, BH, N, J, Jpad, st)
                            : launch_assign_tc_jb<256, false>(x, w_hi, w_lo, nullptr, partial, status, BH, N, J, Jpad, st);
  if (e != cudaSuccess) return e;
  return launch_assign_reduce(partial, labels, BH, N, J, jb, chunk_hist, st);
}

// bias[bh, j] = -sum_d bf16(c_d * c_d) / 2: the centroid term of the squared distance with the
// products rounded to the input type before the fp32 sum (svoo/co_clustering.py:389-390).
__global__ void __launch_bounds__(256) euclid_bias_kernel(const bf16* __restrict__ c, float* __restrict__ bias, int64_t rows) {
  pdl_trigger();
  pdl_wait();
  const int64_t row = (int64_t)blockIdx.x * 16 + threadIdx.x / 16;
  const int lane = threadIdx.x % 16;
  if (row >= rows) return;
  const uint4 v = reinterpret_cast<const uint4*>(c + row * kHeadDim)[lane];
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = __low2float(h[i]), b = __high2float(h[i]);
    s += bf16_round(a * a);
    s += bf16_round(b * b);
  }
#pragma unroll
  for (int o = 8; o >= 1; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o, 16);
  if (lane == 0) bias[row] = -0.5f * s;
}

// labels[bh, n] = first argmin_j |x_n - c_j|^2 (svoo/co_clustering.py:335-416): the assignment GEMM with
// the centroids themselves as the stationary operand and -|c_j|^2 / 2 added in the epilogue.
cudaError_t launch_euclid_assign_tc(const void* x, const void* centroids, float* bias, int32_t* labels, int2* partial,
                                    int32_t* status, int64_t BH, int64_t N, int64_t K, int32_t* chunk_hist, cudaStream_t st) {
  cudaError_t eb = launch_pdl(euclid_bias_kernel, dim3((unsigned)ceil_div64(BH * K, 16)), dim3(256), 0, st,
                              (const bf16*)centroids, bias, BH * K);
  if (eb != cudaSuccess) return eb;
  count_launches(1);
  const int jb = K <= 128 ? 128 : 256;
  cudaError_t e = jb == 128
      ? launch_assign_tc_jb<128, true>(x, centroids, centroids, bias, partial, status, BH, N, K, (int)K, st)
      : launch_assign_tc_jb<256, true>(x, centroids, centroids, bias, partial, status, BH, N, K, (int)K, st);
  if (e != cudaSuccess) return e;
  return launch_assign_reduce(partial, labels, BH, N, K, jb, chunk_hist, st);
}

}  // namespace svoo
