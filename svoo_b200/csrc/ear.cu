// Error-aware routing ("EAR") on top of the co-clustered layout: value centroids and per-token
// value statistics, the estimated error of replacing a key cluster by its centroid for every
// (query cluster, key cluster) pair, the budgeted block selection, and the key-row runs of the
// attention kernel with the head's centroid rows appended as virtual keys.
//
// Reference: svoo/models/wan/attention.py:594-610 (value centroids), svoo/co_clustering.py:1314-1395
// (value statistics), :1398-1565 (block error estimate), :1691-1798 (selection), :1800-1921
// (centroid compensation, here folded into the attention kernel as extra keys).
#include <math.h>

#include "map_common.cuh"

namespace svoo {

// ---------------------------------------------------------------------------------------------
// Value centroids and statistics.  One CTA per (key cluster, head): the cluster's rows of the
// cluster-ordered V are contiguous.  Pass 1: fp32 column sums -> mean -> bf16 centroid and the sum
// of its squares.  Pass 2 (rows now in L1/L2): per row |v|^2 and v.vc.  As in the reference's
// kernel on bf16 tensors, every product is rounded to bf16 before the fp32 sum.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) ear_value_stats_kernel(const bf16* __restrict__ v_perm,
                                                              const int32_t* __restrict__ k_off, bf16* __restrict__ vc,
                                                              float* __restrict__ vnorm, float* __restrict__ cvd,
                                                              float* __restrict__ vcsq, int N, int KC) {
  __shared__ float red[8][kHeadDim];
  __shared__ float vc_s[kHeadDim];
  __shared__ float sq_s[4];
  const int j = blockIdx.x, bh = blockIdx.y, tid = threadIdx.x, sub = tid % 16, rg = tid / 16;
  const int begin = k_off[(int64_t)bh * (KC + 1) + j], n = k_off[(int64_t)bh * (KC + 1) + j + 1] - begin;
  const bf16* rows = v_perm + ((int64_t)bh * N + begin) * kHeadDim;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int r = rg; r < n; r += 8) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(rows + (int64_t)r * kHeadDim) + sub);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc[2 * e] += __low2float(h[e]);
      acc[2 * e + 1] += __high2float(h[e]);
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) red[rg][sub * 8 + e] = acc[e];
  __syncthreads();
  {
    float s = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) s += red[g][tid];
    const bf16 c = __float2bfloat16_rn(s / (float)max(n, 1));
    vc[((int64_t)bh * KC + j) * kHeadDim + tid] = c;
    const float cf = __bfloat162float(c);
    vc_s[tid] = cf;
    float sq = bf16_round(cf * cf);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if (tid % 32 == 0) sq_s[tid / 32] = sq;
  }
  __syncthreads();
  if (tid == 0) vcsq[(int64_t)bh * KC + j] = (sq_s[0] + sq_s[1]) + (sq_s[2] + sq_s[3]);
  float c8[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) c8[e] = vc_s[sub * 8 + e];
  for (int r0 = 0; r0 < n; r0 += 8) {                 // whole half-warps stay together for the shuffles
    const int r = r0 + rg;
    float vn = 0.f, cv = 0.f;
    if (r < n) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(rows + (int64_t)r * kHeadDim) + sub);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a = __low2float(h[e]), b = __high2float(h[e]);
        vn += bf16_round(a * a) + bf16_round(b * b);
        cv += bf16_round(c8[2 * e] * a) + bf16_round(c8[2 * e + 1] * b);
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) {
      vn += __shfl_xor_sync(0xffffffffu, vn, o);
      cv += __shfl_xor_sync(0xffffffffu, cv, o);
    }
    if (sub == 0 && r < n) {
      vnorm[(int64_t)bh * N + begin + r] = vn;
      cvd[(int64_t)bh * N + begin + r] = cv;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Centroid logits c_ij = bf16(bf16(qc_i . kc_j) * D^-0.5), the dot accumulated d ascending in fp32
// with separate multiply and add: the value torch's bf16 einsum followed by `* scale` gives, in an
// order the CPU side mirrors.  One CTA = 8 query clusters of one head.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ear_centroid_logits_kernel(const bf16* __restrict__ qc, const bf16* __restrict__ kc,
                                                                  float* __restrict__ c_logits, int QC, int KC,
                                                                  float scale) {
  __shared__ float q_s[8][kHeadDim];
  const int i0 = blockIdx.x * 8, bh = blockIdx.y, tid = threadIdx.x;
  for (int t = tid; t < 8 * kHeadDim; t += 256) {
    const int r = t / kHeadDim, d = t % kHeadDim;
    q_s[r][d] = i0 + r < QC ? __bfloat162float(qc[((int64_t)bh * QC + i0 + r) * kHeadDim + d]) : 0.f;
  }
  __syncthreads();
  for (int j = tid; j < KC; j += 256) {
    const uint4* row = reinterpret_cast<const uint4*>(kc + ((int64_t)bh * KC + j) * kHeadDim);
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) acc[r] = 0.f;
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
      for (int r = 0; r < 8; ++r) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[r] = __fadd_rn(acc[r], __fmul_rn(q_s[r][c * 8 + e], kv[e]));
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (i0 + r < QC) c_logits[((int64_t)bh * QC + i0 + r) * KC + j] = bf16_round(__fmul_rn(bf16_round(acc[r]), scale));
  }
}

// ---------------------------------------------------------------------------------------------
// Block error estimate.  For query centroid i and key cluster j
//     err_ij = sum_{t in K_j} | e^{a_it} v_t - e^{c_ij} vc_j |^2,   a_it = qc_i . k_t D^-0.5
// expanded into sum e^{2a}|v|^2 - 2 e^c sum e^a (v.vc) + e^{2c} |vc|^2 |K_j| and evaluated relative to
// a running maximum as the reference does; score = log(max(err, eps)) - gamma log(max(|Q_i||K_j|, eps)).
// One CTA = 128 query centroids (16 per warp, their A fragments stay in registers) x four key
// clusters; the clusters' key rows go through a three-deep cp.async ring 64 at a time (the next two
// chunks, of this cluster or the following ones, are in flight while this one is used) and the logits come from
// mma.sync m16n8k16 (bf16 in, fp32 out).
// ---------------------------------------------------------------------------------------------
constexpr int kEarQ = 128, kEarTok = 64, kEarStride = kHeadDim + 8, kEarClustersPerCta = 4, kEarThreads = 256;
constexpr int kEarStages = 3;
constexpr int kEarSmemBytes = (kEarQ + kEarStages * kEarTok) * kEarStride * 2 + 2 * kEarStages * kEarTok * 4;

__global__ void __launch_bounds__(kEarThreads) ear_scores_kernel(const bf16* __restrict__ qc, const bf16* __restrict__ k_perm,
                                                                 const int32_t* __restrict__ k_off,
                                                                 const int32_t* __restrict__ q_off,
                                                                 const float* __restrict__ c_logits,
                                                                 const float* __restrict__ vnorm, const float* __restrict__ cvd,
                                                                 const float* __restrict__ vcsq, float* __restrict__ scores,
                                                                 int N, int QC, int KC, float scale, float gamma, float eps) {
  extern __shared__ __align__(16) unsigned char ear_sc_sm[];
  bf16* q_s = reinterpret_cast<bf16*>(ear_sc_sm);                          // [128][136]
  bf16* k_s = q_s + kEarQ * kEarStride;                                    // [3][64][136]: a three-deep ring
  float* vn_s = reinterpret_cast<float*>(k_s + kEarStages * kEarTok * kEarStride);   // [3][64]
  float* cv_s = vn_s + kEarStages * kEarTok;                               // [3][64]
  const int bh = blockIdx.z, qt = blockIdx.y, tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int g = lane / 4, tq = lane % 4;
  for (int t = tid; t < kEarQ * 16; t += kEarThreads) {
    const int r = t / 16, c = t % 16, qi = qt * kEarQ + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (qi < QC) v = __ldg(reinterpret_cast<const uint4*>(qc + ((int64_t)bh * QC + qi) * kHeadDim) + c);
    *reinterpret_cast<uint4*>(&q_s[r * kEarStride + c * 8]) = v;
  }
  __syncthreads();
  uint32_t a[8][4];
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const bf16* base = &q_s[(warp * 16 + g) * kEarStride + kk * 16 + 2 * tq];
    a[kk][0] = *reinterpret_cast<const uint32_t*>(base);
    a[kk][1] = *reinterpret_cast<const uint32_t*>(base + 8 * kEarStride);
    a[kk][2] = *reinterpret_cast<const uint32_t*>(base + 8);
    a[kk][3] = *reinterpret_cast<const uint32_t*>(base + 8 * kEarStride + 8);
  }
  const int qi0 = qt * kEarQ + warp * 16 + g, qi1 = qi0 + 8;
  const int32_t* off = k_off + (int64_t)bh * (KC + 1);
  const int32_t* qo = q_off + (int64_t)bh * (QC + 1);
  const float qsz0 = qi0 < QC ? (float)(qo[qi0 + 1] - qo[qi0]) : 0.f;
  const float qsz1 = qi1 < QC ? (float)(qo[qi1 + 1] - qo[qi1]) : 0.f;
  const int j_begin = blockIdx.x * kEarClustersPerCta, j_end = min(j_begin + kEarClustersPerCta, KC);

  // chunk (cluster jc, first token tc) -> buffer b: 64 key rows and their value statistics by cp.async
  // (zero-filled past the cluster's end)
  auto load_chunk = [&](int jc, int tc, int b) {
    const int begin = off[jc], n = off[jc + 1] - begin;
    const uint32_t dst = smem_u32(k_s + b * kEarTok * kEarStride);
    for (int t = tid; t < kEarTok * 16; t += kEarThreads) {
      const int r = t / 16, c = t % 16;
      const bool ok = tc + r < n;
      cp_async16(dst + (r * kEarStride + c * 8) * 2, k_perm + ((int64_t)bh * N + begin + (ok ? tc + r : 0)) * kHeadDim + c * 8, ok);
    }
    if (tid < 2 * kEarTok) {
      const int r = tid % kEarTok;
      const bool ok = tc + r < n;
      const float* src = (tid < kEarTok ? vnorm : cvd) + (int64_t)bh * N + begin + (ok ? tc + r : 0);
      const uint32_t d4 = smem_u32((tid < kEarTok ? vn_s : cv_s) + b * kEarTok + r);
      const int sz = ok ? 4 : 0;
      asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d4), "l"(src), "r"(sz));
    }
    cp_async_commit();
  };
  // the chunk after (jc, tc): the next one of the same cluster, else the first of the next non-empty one
  auto next_chunk = [&](int& jc, int& tc) {
    tc += kEarTok;
    while (jc < j_end && tc >= off[jc + 1] - off[jc]) {
      ++jc;
      tc = 0;
    }
  };
  // (pj, pt): the next chunk to load; chunks are consumed in the same order, two loads ahead
  int pj = j_begin, pt = -kEarTok;
  next_chunk(pj, pt);
  int issued = 0, consumed = 0;
  for (int k = 0; k < kEarStages - 1 && pj < j_end; ++k) {
    load_chunk(pj, pt, issued % kEarStages);
    ++issued;
    next_chunk(pj, pt);
  }
  // the running maximum and every exponent are kept in base 2 (ex2.approx; the estimate feeds a ranking
  // and tolerates its 2 ulp): a' = a log2(e), c' = c log2(e)
  const float kLog2e = 1.4426950408889634f;
  const float scale2 = scale * kLog2e;
  const bool warp_has_rows = qt * kEarQ + warp * 16 < QC;
  for (int j = j_begin; j < j_end; ++j) {
    const int n = off[j + 1] - off[j];
    const float c0 = qi0 < QC ? c_logits[((int64_t)bh * QC + qi0) * KC + j] * kLog2e : 0.f;
    const float c1 = qi1 < QC ? c_logits[((int64_t)bh * QC + qi1) * KC + j] * kLog2e : 0.f;
    float run0 = c0, run1 = c1, sq0 = 0.f, sq1 = 0.f, cr0 = 0.f, cr1 = 0.f;
    for (int t0 = 0; t0 < n; t0 += kEarTok) {
      // wait for this chunk; the barrier also says that everyone is done with the chunk before it, whose
      // buffer the next load reuses
      if (issued - consumed >= 2) cp_async_wait<1>(); else cp_async_wait<0>();
      __syncthreads();
      if (pj < j_end) {
        load_chunk(pj, pt, issued % kEarStages);
        ++issued;
        next_chunk(pj, pt);
      }
      const int buf = consumed % kEarStages;
      ++consumed;
      if (warp_has_rows) {
        const bf16* kb = k_s + buf * kEarTok * kEarStride;
        const float* vn = vn_s + buf * kEarTok;
        const float* cv = cv_s + buf * kEarTok;
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const bf16* base = &kb[(nt * 8 + g) * kEarStride + kk * 16 + 2 * tq];
            mma_bf16(s[nt], a[kk], *reinterpret_cast<const uint32_t*>(base), *reinterpret_cast<const uint32_t*>(base + 8));
          }
        }
        float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const bool ok = t0 + nt * 8 + 2 * tq + e < n;
            s[nt][e] = ok ? s[nt][e] * scale2 : -INFINITY;
            s[nt][2 + e] = ok ? s[nt][2 + e] * scale2 : -INFINITY;
            m0 = fmaxf(m0, s[nt][e]);
            m1 = fmaxf(m1, s[nt][2 + e]);
          }
        }
        m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1));
        m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
        m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1));
        m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
        const float new0 = fmaxf(run0, m0), new1 = fmaxf(run1, m1);
        const float r0 = exp2f(run0 - new0), r1 = exp2f(run1 - new1);
        sq0 *= r0 * r0;
        cr0 *= r0;
        sq1 *= r1 * r1;
        cr1 *= r1;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = nt * 8 + 2 * tq + e;
            float p0, p1;                                  // ex2(-inf) = 0 for the padding
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(s[nt][e] - new0));
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(s[nt][2 + e] - new1));
            sq0 += p0 * p0 * vn[c];
            cr0 += p0 * cv[c];
            sq1 += p1 * p1 * vn[c];
            cr1 += p1 * cv[c];
          }
        }
        run0 = new0;
        run1 = new1;
      }
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      sq0 += __shfl_xor_sync(0xffffffffu, sq0, o);
      cr0 += __shfl_xor_sync(0xffffffffu, cr0, o);
      sq1 += __shfl_xor_sync(0xffffffffu, sq1, o);
      cr1 += __shfl_xor_sync(0xffffffffu, cr1, o);
    }
    if (tq == 0) {
      // err = (sq - 2 cp cr + cp^2 |vc|^2 n) 2^(2 run): its logarithm is taken piecewise so that a large
      // running maximum cannot overflow the product (the reference multiplies and clamps; the two agree
      // wherever that product is finite)
      const float vs = vcsq[(int64_t)bh * KC + j], nf = (float)n;
      const float kLn2 = 0.6931471805599453f;
      if (qi0 < QC) {
        const float cp = exp2f(c0 - run0);
        const float err = sq0 - 2.0f * cp * cr0 + cp * cp * vs * nf;
        const float le = err > 0.f ? logf(err) + 2.0f * run0 * kLn2 : -INFINITY;
        scores[((int64_t)bh * QC + qi0) * KC + j] = fmaxf(le, logf(eps)) - gamma * logf(fmaxf(qsz0 * nf, eps));
      }
      if (qi1 < QC) {
        const float cp = exp2f(c1 - run1);
        const float err = sq1 - 2.0f * cp * cr1 + cp * cp * vs * nf;
        const float le = err > 0.f ? logf(err) + 2.0f * run1 * kLn2 : -INFINITY;
        scores[((int64_t)bh * QC + qi1) * KC + j] = fmaxf(le, logf(eps)) - gamma * logf(fmaxf(qsz1 * nf, eps));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Budgeted selection (identify_dynamic_map_estimated after the scores).  Arithmetic fixed as on the
// CPU side so that the map is reproducible bit for bit from (c_logits, scores, sizes):
//   log size = bf16(log_fixed(bf16(bf16(size) + 1e-8)));  budget logit = bf16(c_ij + log size_j)
//   prob     = bf16(exp_fixed(x - max) / sum_j)            (sum j ascending, fp32)
//   order    = descending prob, ties by lower index; prefix = running fp32 sum, each rounded to bf16;
//              keep[0], keep[r] = prefix[r-1] <= bf16(top_p), keep[r < budget_preserve]
//   budget   = running fp32 sum of |Q_i||K_j| over the kept positions, in sorted order
//   guaranteed = first `preserve` positions; cost = their areas summed j ascending
//   candidates = score (guaranteed: -1e10) descending, ties by lower index; kept while
//              (running sum - own area) < max(budget - cost, 0)
// One warp per (head, query cluster), eight per CTA.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float log_f32_fixed(float x) {
  // ln(x), x > 0 normal, from fp32 add/mul/div only; mirrored operation by operation on the CPU side
  const int bits = __float_as_int(x);
  int e = ((bits >> 23) & 0xFF) - 127;
  float m = __int_as_float((bits & 0x007FFFFF) | 0x3F800000);
  if (m > 1.41421354f) {
    m = __fmul_rn(m, 0.5f);
    e += 1;
  }
  const float f = __fsub_rn(m, 1.0f);
  const float s = __fdiv_rn(f, __fadd_rn(f, 2.0f));
  const float z = __fmul_rn(s, s);
  float p = (float)(1.0 / 11);
  p = __fadd_rn(__fmul_rn(p, z), (float)(1.0 / 9));
  p = __fadd_rn(__fmul_rn(p, z), (float)(1.0 / 7));
  p = __fadd_rn(__fmul_rn(p, z), (float)(1.0 / 5));
  p = __fadd_rn(__fmul_rn(p, z), (float)(1.0 / 3));
  p = __fadd_rn(__fmul_rn(p, z), 1.0f);
  const float lm = __fmul_rn(__fadd_rn(s, s), p);
  const float ef = (float)e;
  const float lo = __fadd_rn(__fmul_rn(ef, (float)1.428606765330187e-06), lm);
  return __fadd_rn(__fmul_rn(ef, 0.693145751953125f), lo);
}

struct EarLimits {
  int32_t preserve[SVOO_MAX_HEADS];
  int32_t budget_preserve[SVOO_MAX_HEADS];
};

template <int M>
__device__ __forceinline__ void ear_sort_probs(const float* vw, uint32_t* kw, float tot, int KC, int KCpad, int lane) {
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

template <int M>
__device__ __forceinline__ void ear_sort_scores(const float* sc, const uint8_t* guaranteed, uint32_t* order, int KC,
                                                int KCpad, int lane) {
  unsigned long long v[M];
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const int j = lane + 32 * m;
    unsigned long long kk = 0;
    if (j < KC) {
      const float x = guaranteed[j] ? -1e10f : sc[j];
      uint32_t u = __float_as_uint(x);
      u ^= (u >> 31) ? 0xFFFFFFFFu : 0x80000000u;             // order-preserving map of fp32 to unsigned
      kk = ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFu - j) | 0x10000ull;   // above the zero padding
    }
    v[m] = kk;
  }
  warp_sort_desc<M, unsigned long long>(v, lane);
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const int t = lane + 32 * m;
    if (t < KCpad) order[t] = (v[m] & 0x10000ull) ? (uint32_t)(0xFFFFu - (v[m] & 0xFFFFull)) : 0xFFFFFFFFu;
  }
}

__global__ void __launch_bounds__(256) ear_select_kernel(const float* __restrict__ c_logits, const float* __restrict__ scores,
                                                         const int32_t* __restrict__ q_off, const int32_t* __restrict__ k_off,
                                                         uint8_t* __restrict__ map, int QC, int KC, int KCpad, float top_p,
                                                         const __grid_constant__ EarLimits lim) {
  extern __shared__ __align__(16) unsigned char ear_sm[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, bh = blockIdx.y, i = blockIdx.x * 8 + warp;
  if (i >= QC) return;
  float* vw = reinterpret_cast<float*>(ear_sm) + warp * KCpad;                            // [8][KCpad]
  uint32_t* kw = reinterpret_cast<uint32_t*>(ear_sm) + 8 * KCpad + warp * KCpad;          // [8][KCpad]
  float* area = reinterpret_cast<float*>(ear_sm) + 16 * KCpad + warp * KCpad;             // [8][KCpad]
  uint8_t* gflag = ear_sm + 24 * KCpad * 4 + warp * KCpad;                                // [8][KCpad]
  const int32_t* ko = k_off + (int64_t)bh * (KC + 1);
  const long long qsz = q_off[(int64_t)bh * (QC + 1) + i + 1] - q_off[(int64_t)bh * (QC + 1) + i];
  const float* cl = c_logits + ((int64_t)bh * QC + i) * KC;
  const float* sc = scores + ((int64_t)bh * QC + i) * KC;
  float mx = -INFINITY;
  for (int j = lane; j < KC; j += 32) {
    const int ks = ko[j + 1] - ko[j];
    const float ls = bf16_round(log_f32_fixed(bf16_round(__fadd_rn(bf16_round((float)ks), 1e-8f))));
    const float x = bf16_round(__fadd_rn(cl[j], ls));
    vw[j] = x;
    area[j] = __ll2float_rn(qsz * (long long)ks);
    gflag[j] = 0;
    mx = fmaxf(mx, x);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  for (int j = lane; j < KC; j += 32) vw[j] = exp_f32_fixed(__fsub_rn(vw[j], mx));
  __syncwarp();
  float tot = 0.f;
  if (lane == 0)
    for (int j = 0; j < KC; ++j) tot = __fadd_rn(tot, vw[j]);
  tot = __shfl_sync(0xffffffffu, tot, 0);
  switch (KCpad <= 32 ? 1 : KCpad / 32) {
    case 1: ear_sort_probs<1>(vw, kw, tot, KC, KCpad, lane); break;
    case 2: ear_sort_probs<2>(vw, kw, tot, KC, KCpad, lane); break;
    case 4: ear_sort_probs<4>(vw, kw, tot, KC, KCpad, lane); break;
    case 8: ear_sort_probs<8>(vw, kw, tot, KC, KCpad, lane); break;
    case 16: ear_sort_probs<16>(vw, kw, tot, KC, KCpad, lane); break;
    default: ear_sort_probs<32>(vw, kw, tot, KC, KCpad, lane); break;
  }
  __syncwarp();
  const int preserve = lim.preserve[bh], bpres = lim.budget_preserve[bh];
  // The sequential passes below run on lane 0 in the fixed order the CPU side uses; everything that is
  // a gather or a scatter is done by the whole warp before or after them, so that a pass reads its
  // operands in order from shared memory and carries only its fp32 sums.
  for (int r = lane; r < KC; r += 32) {              // areas in budget order (vw is free: the probabilities live in kw)
    const int j = 0xFFFF - (int)(kw[r] & 0xFFFFu);
    vw[r] = area[j];
    if (r < preserve) gflag[j] = 1;
  }
  __syncwarp();
  float remaining = 0.f;
  if (lane == 0) {
    const float p_b = bf16_round(top_p);
    float run = 0.f, budget = 0.f;
    bool keep = true;                                   // position 0 is always kept
    for (int r = 0; r < KC; ++r) {
      if (keep || r < bpres) budget = __fadd_rn(budget, vw[r]);
      run = __fadd_rn(run, __uint_as_float(kw[r] & 0xFFFF0000u));
      keep = bf16_round(run) <= p_b;                    // decides position r + 1
    }
    float cost = 0.f;
    for (int j = 0; j < KC; ++j)
      if (gflag[j]) cost = __fadd_rn(cost, area[j]);
    remaining = fmaxf(__fsub_rn(budget, cost), 0.f);
  }
  __syncwarp();
  switch (KCpad <= 32 ? 1 : KCpad / 32) {
    case 1: ear_sort_scores<1>(sc, gflag, kw, KC, KCpad, lane); break;
    case 2: ear_sort_scores<2>(sc, gflag, kw, KC, KCpad, lane); break;
    case 4: ear_sort_scores<4>(sc, gflag, kw, KC, KCpad, lane); break;
    case 8: ear_sort_scores<8>(sc, gflag, kw, KC, KCpad, lane); break;
    case 16: ear_sort_scores<16>(sc, gflag, kw, KC, KCpad, lane); break;
    default: ear_sort_scores<32>(sc, gflag, kw, KC, KCpad, lane); break;
  }
  __syncwarp();
  for (int r = lane; r < KC; r += 32) vw[r] = area[kw[r]];      // areas in candidate order
  __syncwarp();
  if (lane == 0) {                                    // position r is kept while (running sum - own area) < remaining
    float run = 0.f;
    for (int r = 0; r < KC; ++r) {
      const float aj = vw[r];
      run = __fadd_rn(run, aj);
      if (__fsub_rn(run, aj) < remaining) kw[r] |= 0x80000000u;
    }
  }
  __syncwarp();
  for (int r = lane; r < KC; r += 32)
    if (kw[r] & 0x80000000u) gflag[kw[r] & 0xFFFFu] |= 2;     // distinct clusters: no two lanes write one byte
  __syncwarp();
  uint8_t* out = map + ((int64_t)bh * QC + i) * KC;
  for (int j = lane; j < KC; j += 32) out[j] = gflag[j] ? 1 : 0;
}

// ---------------------------------------------------------------------------------------------
// Key-row runs of the attention kernel in EAR mode.  The K/V tensors the kernel reads are the
// cluster-ordered rows of all heads followed by the centroid rows of all heads ([BH*S + BH*KC, 128]);
// a query cluster's key list is the token runs of its selected clusters, then ONE run: the KC
// centroid rows of its head (whole 128-row TMA boxes; the kernel masks the centroids of the selected
// clusters, see the bias table there).  One warp per (head, query cluster); entries as in
// build_runs_kernel, rows relative to the head's first token row.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) ear_build_runs_kernel(const uint8_t* __restrict__ map, const int32_t* __restrict__ k_off,
                                                             int2* __restrict__ runs, int32_t* __restrict__ nruns, int QC,
                                                             int KC, int max_runs, int rows_total, int BH, int S) {
  const int row = blockIdx.x * 8 + threadIdx.x / 32;
  if (row >= rows_total) return;
  const int lane = threadIdx.x % 32;
  const int bh = row / QC;
  const uint8_t* m = map + (int64_t)row * KC;
  const int32_t* off = k_off + (int64_t)bh * (KC + 1);
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
  const int n = n_start < max_runs - 2 ? n_start : max_runs - 2;
  __syncwarp();
  if (lane == 0) {
    int vbeg = 0;
    for (int r = 0; r < n; ++r) {
      const int2 se = out[r];
      out[r] = make_int2(se.x, vbeg);
      vbeg += se.y - se.x;
    }
    out[n] = make_int2((BH - bh) * S + bh * KC, vbeg);          // the head's centroid rows
    out[n + 1] = make_int2(0, vbeg + KC);
    nruns[row] = n + 1;
  }
}

// ---------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------
cudaError_t launch_ear_value_stats(const void* v_perm, const int32_t* k_off, void* vc, float* vnorm, float* cvd, float* vcsq,
                                   int64_t BH, int64_t N, int64_t KC, cudaStream_t st) {
  ear_value_stats_kernel<<<dim3((unsigned)KC, (unsigned)BH), 128, 0, st>>>((const bf16*)v_perm, k_off, (bf16*)vc, vnorm, cvd,
                                                                          vcsq, (int)N, (int)KC);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t launch_ear_scores(const void* qc, const void* kc, const void* k_perm, const int32_t* q_off, const int32_t* k_off,
                              const float* vnorm, const float* cvd, const float* vcsq, float* c_logits, float* scores,
                              int64_t BH, int64_t N, int64_t QC, int64_t KC, float gamma, cudaStream_t st) {
  const float scale = (float)(1.0 / sqrt((double)kHeadDim));
  ear_centroid_logits_kernel<<<dim3((unsigned)ceil_div64(QC, 8), (unsigned)BH), 256, 0, st>>>(
      (const bf16*)qc, (const bf16*)kc, c_logits, (int)QC, (int)KC, scale);
  dim3 grid((unsigned)ceil_div64(KC, kEarClustersPerCta), (unsigned)ceil_div64(QC, kEarQ), (unsigned)BH);
  cudaError_t e = cudaFuncSetAttribute(ear_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kEarSmemBytes);
  if (e != cudaSuccess) return e;
  ear_scores_kernel<<<grid, kEarThreads, kEarSmemBytes, st>>>((const bf16*)qc, (const bf16*)k_perm, k_off, q_off, c_logits, vnorm, cvd, vcsq, scores,
                                          (int)N, (int)QC, (int)KC, scale, gamma, 1e-8f);
  count_launches(2);
  return cudaGetLastError();
}

cudaError_t launch_ear_select(const float* c_logits, const float* scores, const int32_t* q_off, const int32_t* k_off,
                              uint8_t* map, int64_t BH, int64_t QC, int64_t KC, float top_p, const int32_t* preserve_host,
                              const int32_t* budget_preserve_host, cudaStream_t st) {
  EarLimits lim;
  for (int h = 0; h < SVOO_MAX_HEADS; ++h) {
    lim.preserve[h] = h < BH ? preserve_host[h] : 0;
    lim.budget_preserve[h] = h < BH ? budget_preserve_host[h] : 0;
  }
  int KCpad = 32;
  while (KCpad < KC) KCpad <<= 1;
  const size_t smem = (size_t)8 * KCpad * (3 * 4 + 1);                    // at most 104 KB (1024 clusters)
  cudaError_t e = cudaFuncSetAttribute(ear_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
  if (e != cudaSuccess) return e;
  ear_select_kernel<<<dim3((unsigned)ceil_div64(QC, 8), (unsigned)BH), 256, smem, st>>>(c_logits, scores, q_off, k_off, map,
                                                                                         (int)QC, (int)KC, KCpad, top_p, lim);
  count_launches(1);
  return cudaGetLastError();
}

cudaError_t launch_ear_build_runs(const uint8_t* map, const int32_t* k_off, int2* runs, int32_t* nruns, int64_t BH,
                                  int64_t S, int64_t QC, int64_t KC, int max_runs, cudaStream_t st) {
  const int rows = (int)(BH * QC);
  ear_build_runs_kernel<<<(rows + 7) / 8, 256, 0, st>>>(map, k_off, runs, nruns, (int)QC, (int)KC, max_runs, rows, (int)BH,
                                                        (int)S);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo
