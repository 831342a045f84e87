// QK co-clustering kernels: profile prologue (builds the W operand of the assignment GEMM,
// which lives in assign_tc.cu), stable counting sort of labels, deterministic centroid update.
//
// Algebra used by the assignment.  The reference (svoo/co_clustering.py:2148-2255)
// computes, for token x and own-centroid j,
//     score_j = sum_k ((x . c_k) / norm(x)) * Phat[j,k],   label = first argmax_j score_j
// with c_k the profile-forming centroids and Phat the row-normalised centroid-centroid
// profile.  norm(x) > 0 does not depend on j and the double sum is linear in x, so
//     label = first argmax_j  x . W_j,     W_j = sum_k Phat[j,k] c_k      (W is [J,128])
// One GEMM [N,128] x [128,J] per side and iteration replaces the two chained GEMMs and
// the separate norm pass.  W is carried as a bf16 pair (hi, lo = bf16(W - hi)) so the
// products keep ~16 mantissa bits, more than the TF32 operands of the reference.
#include "common.cuh"

namespace svoo {

// ---------------------------------------------------------------------------------------
// centroids[bh,c,:] = x[bh, idx[bh,c], :]     (svoo/co_clustering.py:2417-2421)
// ---------------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const bf16* __restrict__ x, const int32_t* __restrict__ idx,
                                   bf16* __restrict__ out, int N, int K) {
  pdl_trigger();
  pdl_wait();
  const int bh = blockIdx.y;
  const int c = blockIdx.x * (blockDim.x / 16) + threadIdx.x / 16;
  if (c >= K) return;
  const int lane = threadIdx.x % 16;
  int src = idx[(int64_t)bh * K + c];
  src = min(max(src, 0), N - 1);
  const uint4* s = reinterpret_cast<const uint4*>(x + ((int64_t)bh * N + src) * kHeadDim);
  uint4* d = reinterpret_cast<uint4*>(out + ((int64_t)bh * K + c) * kHeadDim);
  d[lane] = s[lane];
}

// ---------------------------------------------------------------------------------------
// Prologue: P = bf16(own . form^T), Phat = P / sqrt(sum P^2 + 1e-8) (fp32),
//           W = Phat . form (fp32) -> (hi, lo) bf16.     One CTA = 16 rows j of one head.
// Both products run on mma.sync (m16n8k16, fp32 accumulation): the problem is a few MFLOP
// per head and latency-bound, so the point is the short dependency chain, not throughput.
// `form` is streamed twice through a double-buffered shared-memory ring of 64-row chunks
// (cp.async).  Phat (fp32) enters the second product as three bf16 terms hi + mid + lo,
// which carries 24 mantissa bits, so W matches an fp32 product to rounding.
// (svoo/co_clustering.py:2427-2428 and svoo/kernels/triton/l2norm.py:36-41)
// ---------------------------------------------------------------------------------------
constexpr int kProR = 16;            // own rows per CTA
constexpr int kProC = 64;            // form rows per chunk

__host__ __device__ inline int pro_kround(int K) { return (K + kProC - 1) / kProC * kProC; }
__host__ __device__ inline int pro_p_stride(int K) { return pro_kround(K) + 4; }       // floats
__host__ __device__ inline int pro_hat_stride(int K) { return pro_kround(K) + 8; }     // bf16: 16 bytes past a multiple of 128
inline size_t pro_smem_bytes(int K) {
  return (size_t)kProR * kRowBytes + 2 * (size_t)kProC * kRowBytes + (size_t)kProR * pro_p_stride(K) * 4 +
         3 * (size_t)kProR * pro_hat_stride(K) * 2;
}

__global__ void __launch_bounds__(256) profile_prologue_kernel(
    const bf16* __restrict__ own, const bf16* __restrict__ form, bf16* __restrict__ w_hi,
    bf16* __restrict__ w_lo, int J, int K, int Jpad) {
  extern __shared__ __align__(128) unsigned char pro_sm[];
  pdl_trigger();
  pdl_wait();                                           // the centroids come from the previous kernel
  const int bh = blockIdx.y, j0 = blockIdx.x * kProR;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (j0 >= J) {                                        // padding rows of W: zeros
    const int d = tid & 127, rg = tid >> 7;
    for (int r = rg * 8; r < rg * 8 + 8; ++r)
      if (j0 + r < Jpad) {
        w_hi[((int64_t)bh * Jpad + j0 + r) * kHeadDim + d] = __float2bfloat16_rn(0.f);
        w_lo[((int64_t)bh * Jpad + j0 + r) * kHeadDim + d] = __float2bfloat16_rn(0.f);
      }
    return;
  }
  const int pstride = pro_p_stride(K), hstride = pro_hat_stride(K);
  unsigned char* own_p = pro_sm;                                    // [16][128] bf16, swizzled
  unsigned char* form_p = own_p + kProR * kRowBytes;                // 2 x [64][128] bf16, swizzled
  float* p_s = reinterpret_cast<float*>(form_p + 2 * kProC * kRowBytes);       // [16][pstride]
  bf16* hat = reinterpret_cast<bf16*>(p_s + kProR * pstride);                  // 3 x [16][hstride]
  const uint32_t own_s = smem_u32(own_p), form_s = smem_u32(form_p), hat_s = smem_u32(hat);
  const bf16* form_b = form + (int64_t)bh * K * kHeadDim;
  const int nch = (K + kProC - 1) / kProC;

  auto load_chunk = [&](int c, int buf) {               // rows past K arrive as zeros
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      const int i = tid + pass * 256, row = i >> 4, ch = i & 15;
      const int k = c * kProC + row;
      cp_async16(form_s + buf * (kProC * kRowBytes) + swz(row, ch),
                 form_b + (int64_t)min(k, K - 1) * kHeadDim + ch * 8, k < K);
    }
  };
  {
    const int row = tid >> 4, ch = tid & 15;
    const int j = j0 + row;
    cp_async16(own_s + swz(row, ch), own + ((int64_t)bh * J + min(j, J - 1)) * kHeadDim + ch * 8, j < J);
  }
  load_chunk(0, 0);
  cp_async_commit();

  // ---- sweep 1: P[16][K]; warps 0..3 take 16 form rows of the chunk each
  uint32_t qa[8][4];
  for (int c = 0; c < nch; ++c) {
    if (c + 1 < nch) load_chunk(c + 1, (c + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (warp < 4) {
      if (c == 0) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          ldmatrix_x4(qa[ks], own_s + swz((lane % 8) + ((lane / 8) % 2) * 8, ks * 2 + lane / 16));
      }
      const uint32_t f = form_s + (c & 1) * (kProC * kRowBytes);
      float acc[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t b[4];
        ldmatrix_x4(b, f + swz(warp * 16 + (lane % 8) + (lane / 16) * 8, ks * 2 + ((lane / 8) % 2)));
        mma_bf16(acc[0], qa[ks], b[0], b[1]);
        mma_bf16(acc[1], qa[ks], b[2], b[3]);
      }
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {                   // torch.matmul of bf16 tensors returns bf16
          const int row = lane / 4 + (e >> 1) * 8;
          const int k = c * kProC + warp * 16 + nt * 8 + 2 * (lane % 4) + (e & 1);
          p_s[row * pstride + k] = bf16_round(acc[nt][e]);
        }
    }
    __syncthreads();
  }
  load_chunk(0, 0);                                     // first chunk of sweep 2, in flight during the norms
  cp_async_commit();

  // ---- row norms (16 threads per row, fixed order), Phat = P / norm split into three bf16 terms
  {
    const int row = tid >> 4, sub = tid & 15;
    const int kr = pro_kround(K);
    float ss = 0.f;
    for (int k = sub; k < kr; k += 16) { const float x = p_s[row * pstride + k]; ss = fmaf(x, x, ss); }
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float nr = sqrtf(ss + 1e-8f);
    for (int k = sub; k < kr; k += 16) {
      const float x = p_s[row * pstride + k] / nr;
      const bf16 h = __float2bfloat16_rn(x);
      const float r1 = x - __bfloat162float(h);
      const bf16 m = __float2bfloat16_rn(r1);
      const bf16 l = __float2bfloat16_rn(r1 - __bfloat162float(m));
      hat[(0 * kProR + row) * hstride + k] = h;
      hat[(1 * kProR + row) * hstride + k] = m;
      hat[(2 * kProR + row) * hstride + k] = l;
    }
  }

  // ---- sweep 2: W[16][128] = sum_k Phat[r][k] form[k][d]; warp w owns dims 16w .. 16w+15
  float wacc[3][2][4];
#pragma unroll
  for (int t = 0; t < 3; ++t)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int e = 0; e < 4; ++e) wacc[t][i][e] = 0.f;
  for (int c = 0; c < nch; ++c) {
    if (c + 1 < nch) load_chunk(c + 1, (c + 1) & 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint32_t f = form_s + (c & 1) * (kProC * kRowBytes);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, f + swz(kk * 16 + (lane % 8) + ((lane / 8) % 2) * 8, warp * 2 + lane / 16));
#pragma unroll
      for (int t = 0; t < 3; ++t) {
        uint32_t a[4];
        const int arow = (lane % 8) + ((lane / 8) % 2) * 8;
        const int acol = c * kProC + kk * 16 + (lane / 16) * 8;
        ldmatrix_x4(a, hat_s + (uint32_t)(((t * kProR + arow) * hstride + acol) * 2));
        mma_bf16(wacc[t][0], a, b[0], b[1]);
        mma_bf16(wacc[t][1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int j = j0 + lane / 4 + half * 8;
      if (j < Jpad) {
        float v0 = wacc[0][nt][half * 2] + (wacc[1][nt][half * 2] + wacc[2][nt][half * 2]);
        float v1 = wacc[0][nt][half * 2 + 1] + (wacc[1][nt][half * 2 + 1] + wacc[2][nt][half * 2 + 1]);
        if (j >= J) v0 = v1 = 0.f;
        const bf16 h0 = __float2bfloat16_rn(v0), h1 = __float2bfloat16_rn(v1);
        const bf16 l0 = __float2bfloat16_rn(v0 - __bfloat162float(h0)), l1 = __float2bfloat16_rn(v1 - __bfloat162float(h1));
        const int64_t o = ((int64_t)bh * Jpad + j) * kHeadDim + warp * 16 + nt * 8 + 2 * (lane % 4);
        __nv_bfloat162 hv, lv;
        hv.x = h0; hv.y = h1; lv.x = l0; lv.y = l1;
        *reinterpret_cast<__nv_bfloat162*>(w_hi + o) = hv;
        *reinterpret_cast<__nv_bfloat162*>(w_lo + o) = lv;
      }
    }
}

// ---------------------------------------------------------------------------------------
// Stable counting sort of labels (three kernels).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) label_hist_kernel(const int32_t* __restrict__ labels,
                                                         int32_t* __restrict__ chunk_hist, int N, int K, int nchunks) {
  __shared__ int hist[SVOO_MAX_CLUSTERS];
  pdl_trigger();
  const int bh = blockIdx.y, chunk = blockIdx.x;
  for (int k = threadIdx.x; k < K; k += 256) hist[k] = 0;
  __syncthreads();
  pdl_wait();
  const int base = chunk * kSortChunk;
  for (int i = threadIdx.x; i < kSortChunk; i += 256) {
    const int n = base + i;
    if (n < N) {
      const int l = labels[(int64_t)bh * N + n];
      if (l >= 0 && l < K) atomicAdd(&hist[l], 1);
    }
  }
  __syncthreads();
  int32_t* out = chunk_hist + ((int64_t)bh * nchunks + chunk) * K;
  for (int k = threadIdx.x; k < K; k += 256) out[k] = hist[k];
}

// One CTA per head: per-cluster exclusive prefix over chunks (in place), totals, offsets.
__global__ void __launch_bounds__(1024) label_scan_kernel(int32_t* __restrict__ chunk_hist, int32_t* __restrict__ offsets,
                                                          int32_t* __restrict__ sizes, int K, int nchunks) {
  __shared__ int warp_tot[32];
  pdl_trigger();
  pdl_wait();
  const int bh = blockIdx.x, k = threadIdx.x, lane = k % 32, warp = k / 32;
  int total = 0;
  if (k < K) {
    int32_t* col = chunk_hist + (int64_t)bh * nchunks * K + k;
    for (int c0 = 0; c0 < nchunks; c0 += 8) {          // 8 independent loads in flight, then the stores
      int v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = (c0 + u < nchunks) ? col[(int64_t)(c0 + u) * K] : 0;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (c0 + u < nchunks) col[(int64_t)(c0 + u) * K] = total;
        total += v[u];
      }
    }
    if (sizes) sizes[(int64_t)bh * K + k] = total;
  }
  int incl = total;
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, incl, s);
    if (lane >= s) incl += o;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int v = warp_tot[lane];
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, v, s);
      if (lane >= s) v += o;
    }
    warp_tot[lane] = v;
  }
  __syncthreads();
  const int excl = incl - total + (warp ? warp_tot[warp - 1] : 0);
  if (k < K) offsets[(int64_t)bh * (K + 1) + k] = excl;
  if (k == K - 1) offsets[(int64_t)bh * (K + 1) + K] = excl + total;
}

__global__ void __launch_bounds__(256) label_scatter_kernel(const int32_t* __restrict__ labels,
                                                            const int32_t* __restrict__ chunk_base,
                                                            const int32_t* __restrict__ offsets,
                                                            int32_t* __restrict__ sorted_idx, int N, int K, int nchunks) {
  extern __shared__ int wh[];          // [8][K] per-warp histogram, then per-warp running position
  pdl_trigger();
  const int bh = blockIdx.y, chunk = blockIdx.x;
  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  for (int i = tid; i < 8 * K; i += 256) wh[i] = 0;
  __syncthreads();
  pdl_wait();
  const int wbase = chunk * kSortChunk + warp * (kSortChunk / 8);
  const int32_t* lb = labels + (int64_t)bh * N;
  int mine[8];
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    const int n = wbase + s * 32 + lane;
    int l = (n < N) ? lb[n] : -1;
    if (l >= K) l = -1;
    mine[s] = l;
    if (l >= 0) atomicAdd(&wh[warp * K + l], 1);
  }
  __syncthreads();
  const int32_t* cb = chunk_base + ((int64_t)bh * nchunks + chunk) * K;
  const int32_t* ob = offsets + (int64_t)bh * (K + 1);
  for (int k = tid; k < K; k += 256) {
    int run = ob[k] + cb[k];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int t = wh[w * K + k];
      wh[w * K + k] = run;
      run += t;
    }
  }
  __syncthreads();
  int32_t* out = sorted_idx + (int64_t)bh * N;
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    const int l = mine[s];
    const unsigned key = (l >= 0) ? (unsigned)l : (unsigned)(SVOO_MAX_CLUSTERS + lane);
    const unsigned grp = __match_any_sync(0xffffffffu, key);
    const int rank = __popc(grp & ((1u << lane) - 1u));
    int base = 0;
    if (l >= 0) base = wh[warp * K + l];
    __syncwarp();
    if (l >= 0 && rank == 0) wh[warp * K + l] = base + __popc(grp);
    __syncwarp();
    if (l >= 0) {
      const int pos = base + rank;
      if (pos < N) out[pos] = wbase + s * 32 + lane;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Centroid update: fixed-order fp32 sums over the sorted order, then mean / keep-old.
// ---------------------------------------------------------------------------------------
constexpr int kSlabMin = 256;

// Rows [s0, s1) of slab z when a cluster is cut into `nslabs` pieces of at least kSlabMin rows.
__device__ __forceinline__ void slab_range(int begin, int end, int z, int nslabs, int& s0, int& s1) {
  const int size = end - begin;
  int per = (size + nslabs - 1) / nslabs;
  per = per < kSlabMin ? kSlabMin : per;
  s0 = begin + z * per;
  s1 = s0 + per < end ? s0 + per : end;
}

__global__ void __launch_bounds__(256) centroid_partial_kernel(const bf16* __restrict__ x,
                                                               const int32_t* __restrict__ sorted_idx,
                                                               const int32_t* __restrict__ offsets,
                                                               float* __restrict__ partial, int N, int K, int nslabs) {
  __shared__ float red[16][kHeadDim + 4];
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x, z = blockIdx.y, bh = blockIdx.z;
  const int begin = offsets[(int64_t)bh * (K + 1) + c], end = offsets[(int64_t)bh * (K + 1) + c + 1];
  int s0, s1;
  slab_range(begin, end, z, nslabs, s0, s1);
  if (s0 >= s1) return;
  const int grp = threadIdx.x / 16, lane = threadIdx.x % 16;
  const int32_t* idx = sorted_idx + (int64_t)bh * N;
  const bf16* xb = x + (int64_t)bh * N * kHeadDim;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  // a thread adds rows s0 + grp + 16 k, k = 0, 1, 2, ... in that order; eight gathers are in flight
  for (int s = s0 + grp; s < s1; s += 128) {
    int row[8];
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int ss = s + u * 16;
      row[u] = ss < s1 ? idx[ss] : -1;
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (row[u] >= 0) {
        v[u] = __ldg(reinterpret_cast<const uint4*>(xb + (int64_t)row[u] * kHeadDim) + lane);
      } else {
        v[u] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] += __low2float(h[i]);
        acc[2 * i + 1] += __high2float(h[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[grp][lane * 8 + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < kHeadDim) {
    float s = 0.f;
#pragma unroll
    for (int g = 0; g < 16; ++g) s += red[g][threadIdx.x];
    partial[(((int64_t)bh * K + c) * kCentroidSlabs + z) * kHeadDim + threadIdx.x] = s;
  }
}

// Four clusters per CTA (one per group of 128 threads): a CTA per cluster would be 20,000 CTAs of
// a few hundred bytes of work each at 40 heads x 500 clusters.
constexpr int kFinalizePerCta = 4;
__global__ void __launch_bounds__(128 * kFinalizePerCta) centroid_finalize_kernel(
    const float* __restrict__ partial, const int32_t* __restrict__ offsets, const bf16* __restrict__ old_c,
    bf16* __restrict__ new_c, int32_t* __restrict__ sizes, int K, int nslabs) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * kFinalizePerCta + threadIdx.x / 128, bh = blockIdx.y, d = threadIdx.x % 128;
  if (c >= K) return;
  const int begin = offsets[(int64_t)bh * (K + 1) + c], end = offsets[(int64_t)bh * (K + 1) + c + 1];
  const int cnt = end - begin;
  const int64_t o = ((int64_t)bh * K + c) * kHeadDim + d;
  float s = 0.f;
  for (int z = 0; z < nslabs; ++z) {
    int s0, s1;
    slab_range(begin, end, z, nslabs, s0, s1);
    if (s0 < s1) s += partial[(((int64_t)bh * K + c) * kCentroidSlabs + z) * kHeadDim + d];
  }
  const bf16 keep = old_c[o];
  new_c[o] = cnt > 0 ? __float2bfloat16_rn(s / (float)cnt) : keep;
  if (d == 0 && sizes) sizes[(int64_t)bh * K + c] = cnt;
}

// sizes [BH,K] -> offsets [BH,K+1]; thread k owns entries 2k and 2k + 1 (K <= 2048)
__global__ void __launch_bounds__(1024) offsets_from_sizes_kernel(const int32_t* __restrict__ sizes,
                                                                  int32_t* __restrict__ offsets, int K) {
  __shared__ int warp_tot[32];
  const int bh = blockIdx.x, k = threadIdx.x, lane = k % 32, warp = k / 32;
  const int v0 = 2 * k < K ? sizes[(int64_t)bh * K + 2 * k] : 0;
  const int v1 = 2 * k + 1 < K ? sizes[(int64_t)bh * K + 2 * k + 1] : 0;
  const int v = v0 + v1;
  int incl = v;
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
  const int excl = incl - v + (warp ? warp_tot[warp - 1] : 0);
  int32_t* out = offsets + (int64_t)bh * (K + 1);
  if (2 * k < K) out[2 * k] = excl;
  if (2 * k + 1 < K) out[2 * k + 1] = excl + v0;
  if (2 * k == K - 1) out[K] = excl + v0;
  if (2 * k + 1 == K - 1) out[K] = excl + v;
}

// ---------------------------------------------------------------------------------------
// Host launchers (called from api.cu)
// ---------------------------------------------------------------------------------------
cudaError_t launch_gather_rows(const void* x, const int32_t* idx, void* out, int64_t BH, int64_t N, int64_t K,
                               cudaStream_t st) {
  dim3 grid((unsigned)ceil_div64(K, 16), (unsigned)BH);
  count_launches(1);
  return launch_pdl(gather_rows_kernel, grid, dim3(256), 0, st, (const bf16*)x, idx, (bf16*)out, (int)N, (int)K);
}

cudaError_t launch_prologue(const void* own, const void* form, void* w_hi, void* w_lo, int64_t BH, int64_t J,
                            int64_t K, cudaStream_t st) {
  const int Jpad = pad_clusters(J);
  const size_t smem = pro_smem_bytes((int)K);
  cudaError_t e = cudaFuncSetAttribute(profile_prologue_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)(Jpad / kProR), (unsigned)BH);
  count_launches(1);
  return launch_pdl(profile_prologue_kernel, grid, dim3(256), smem, st, (const bf16*)own, (const bf16*)form, (bf16*)w_hi,
                    (bf16*)w_lo, (int)J, (int)K, Jpad);
}

// hist_done: chunk_hist already holds the per-chunk label histograms (written by the assignment's
// reduction), so the first pass is skipped.
cudaError_t launch_sort_labels(const int32_t* labels, int64_t BH, int64_t N, int64_t K, int32_t* sorted_idx,
                               int32_t* offsets, int32_t* sizes, int32_t* chunk_hist, cudaStream_t st, bool hist_done) {
  const int nchunks = sort_chunks(N);
  // label_scatter_kernel uses 8 * K * 4 <= 32 KB of dynamic shared memory: inside the default limit
  dim3 grid((unsigned)nchunks, (unsigned)BH);
  cudaError_t e = cudaSuccess;
  if (!hist_done) e = launch_pdl(label_hist_kernel, grid, dim3(256), 0, st, labels, chunk_hist, (int)N, (int)K, nchunks);
  if (e != cudaSuccess) return e;
  e = launch_pdl(label_scan_kernel, dim3((unsigned)BH), dim3(1024), 0, st, chunk_hist, offsets, sizes, (int)K, nchunks);
  if (e != cudaSuccess) return e;
  count_launches(hist_done ? 2 : 3);
  return launch_pdl(label_scatter_kernel, grid, dim3(256), (size_t)(8 * K * 4), st, labels, (const int32_t*)chunk_hist,
                    (const int32_t*)offsets, sorted_idx, (int)N, (int)K, nchunks);
}

cudaError_t launch_centroid_update(const void* x, const int32_t* sorted_idx, const int32_t* offsets,
                                   const void* old_c, void* new_c, int32_t* sizes, float* partial, int64_t BH,
                                   int64_t N, int64_t K, cudaStream_t st) {
  // slabs per cluster: enough for clusters of four times the mean size to keep the 256-row minimum,
  // at most kCentroidSlabs; larger clusters just get longer slabs (most launched CTAs of a finer
  // split would find their slab empty)
  int nslabs = (int)ceil_div64(4 * ceil_div64(N, K), kSlabMin);
  nslabs = nslabs < 1 ? 1 : (nslabs > kCentroidSlabs ? kCentroidSlabs : nslabs);
  dim3 grid((unsigned)K, (unsigned)nslabs, (unsigned)BH);
  cudaError_t e = launch_pdl(centroid_partial_kernel, grid, dim3(256), 0, st, (const bf16*)x, sorted_idx, offsets, partial,
                             (int)N, (int)K, nslabs);
  if (e != cudaSuccess) return e;
  dim3 grid2((unsigned)ceil_div64(K, kFinalizePerCta), (unsigned)BH);
  count_launches(2);
  return launch_pdl(centroid_finalize_kernel, grid2, dim3(128 * kFinalizePerCta), 0, st, (const float*)partial, offsets, (const bf16*)old_c,
                    (bf16*)new_c, sizes, (int)K, nslabs);
}

cudaError_t launch_offsets_from_sizes(const int32_t* sizes, int32_t* offsets, int64_t BH, int64_t K, cudaStream_t st) {
  offsets_from_sizes_kernel<<<(unsigned)BH, 1024, 0, st>>>(sizes, offsets, (int)K);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo

// ---------------------------------------------------------------------------------------
// svoo_b200_sort_labels_static: the label sort for callers that cannot hand over a workspace.
//
// Some hosts of this library are not allowed to allocate device memory at the point where
// they call it: a serving process whose HBM is carved up once at start-up, a plug-in that
// only ever receives raw pointers from its host framework and has no allocator of its own,
// or a latency-critical loop that must not risk the implicit device synchronisation of an
// allocation.  For them the per-chunk histogram scratch of the sort lives in the array
// below instead of a caller-provided workspace.  The price is a fixed 4 MiB of device
// memory on every GPU that loads the library, held until the process exits, and a size
// limit: BH * ceil(N / 2048) * K must not exceed kStaticSortInts.
//
// `g_static_sort_scratch` names the array for device code.  In host code the same name is
// only a stand-in symbol, not a device address, so the launcher asks the runtime for the
// real address once per device (cudaGetSymbolAddress, with that device current) and
// passes that pointer to the kernels.
// ---------------------------------------------------------------------------------------
namespace svoo {
constexpr int64_t kStaticSortInts = 1 << 20;                       // 4 MiB of int32
constexpr int kMaxDevices = 64;
static __device__ __align__(256) int32_t g_static_sort_scratch[kStaticSortInts];
}  // namespace svoo

extern "C" int svoo_b200_sort_labels_static(const int32_t* labels, int64_t BH, int64_t N, int64_t K,
                                            int32_t* sorted_idx, int32_t* offsets, void* stream) {
  using namespace svoo;
  if (!labels || !sorted_idx || !offsets) return SVOO_ERR_NULL;
  if (BH < 1 || BH > 65535 || N < 1 || N > (1 << 24) || K < 1 || BH * N > (int64_t)INT32_MAX) return SVOO_ERR_SHAPE;
  if (K > SVOO_MAX_CLUSTERS) return SVOO_ERR_CLUSTERS;
  if (BH * (int64_t)sort_chunks(N) * K > kStaticSortInts) return SVOO_ERR_STATIC_SCRATCH;
  // Address of the array on the current device, looked up on the first call made with that
  // device current.  Two host threads racing here would store the same value.
  static int32_t* scratch_of_device[kMaxDevices] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return SVOO_ERR_SHAPE;
  int32_t* scratch = scratch_of_device[dev];
  if (!scratch) {
    e = cudaGetSymbolAddress((void**)&scratch, g_static_sort_scratch);
    if (e != cudaSuccess) return (int)e;
    scratch_of_device[dev] = scratch;
  }
  // Nothing in the array has to start at zero: label_hist_kernel writes every
  // [head, chunk, cluster] entry that the scan and scatter kernels read afterwards.
  e = launch_sort_labels(labels, BH, N, K, sorted_idx, offsets, nullptr, scratch, (cudaStream_t)stream, false);
  return e == cudaSuccess ? SVOO_OK : (int)e;
}
