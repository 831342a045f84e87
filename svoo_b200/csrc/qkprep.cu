// Producer of the path's inputs: RMS norm over the whole projection row, rotary embedding and the
// [S, H*128] -> [H, S, 128] head transpose in ONE pass over the projection output.
//
// Reference (three to four passes): triton_rmsnorm_forward, svoo/kernels/triton/rmsnorm.py:9-46
// (y = bf16(x * rstd * w), rstd = 1 / sqrt(mean(x^2) + eps), fp32 arithmetic), the interleaved-pair
// rotation of svoo/models/wan/attention.py:179-190 (out[2i] = x[2i] cos[2i] - x[2i+1] sin[2i+1],
// out[2i+1] = x[2i] sin[2i+1] + x[2i+1] cos[2i], fp32 arithmetic on the bf16-rounded normed values,
// rounded to bf16) and transpose(1, 2).contiguous() of svoo/models/wan/attention.py:127-131.
// The roundings are kept where the reference has them, so results differ from it only through the
// order of the sum of squares (at most one bf16 ulp on isolated elements).
//
// One CTA per token: 256 threads hold the row in registers (8 bf16 per 128-bit chunk, up to 8
// chunks per thread, H*128 <= 16384), reduce the sum of squares in a fixed order, and store every
// head's 128 values as one 256-byte segment -- into this GPU's [H, S, 128] array or, for a
// sequence-parallel caller, straight into the arrays of the ranks that own the heads (the same
// destination rule as push_heads), which folds the re-shard's send pass into the producer.
// HBM-bound: 2 * H*128*2 bytes per token.
#include "common.cuh"

namespace svoo {

constexpr int kPrepThreads = 256;
constexpr int kPrepMinBlocks = 4;

struct PrepDest {
  uint4* dst[16];       // [0] only when world == 0 (local [H, S, 128]); else every rank's [H/world, N, 128]
  int16_t owner[128];
  int16_t slot[128];
  int world;            // 0: local
  int rank;
  int64_t n_loc;        // tokens of this rank (== S); N = n_loc * world
};

// One CTA per token, for rows too wide for the warp kernel below (H > 48).  CPT = chunks per
// thread (ceil(H * 16 / 256)).  For CPT <= 4 the norm weights of the thread's chunks are fetched
// together with the row, before the reduction, so the CTA pays one memory latency instead of two.
template <int CPT>
__global__ void __launch_bounds__(kPrepThreads, kPrepMinBlocks) qk_prep_kernel(const uint4* __restrict__ x, const float* __restrict__ weight,
                                                               float eps, const float* __restrict__ cosv,
                                                               const float* __restrict__ sinv, int64_t S, int H,
                                                               const __grid_constant__ PrepDest dest) {
  constexpr bool kPrefetch = CPT <= 4;
  __shared__ float warp_sum[kPrepThreads / 32];
  __shared__ float rstd_s;
  const int64_t s = blockIdx.x;
  const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32;
  const int nchunks = H * 16;                                       // 16 chunks of 8 values per head
  const uint4* row = x + s * nchunks;
  uint4 v[CPT];
  float4 wv[kPrefetch ? CPT : 1][2];
  // every chunk of a thread starts at the same head-dim offset ((tid + 256 u) & 15 == tid & 15), so
  // the thread's rotary coefficients are fetched once
  float ce[4] = {1.f, 1.f, 1.f, 1.f}, so[4] = {0.f, 0.f, 0.f, 0.f};
  if (cosv) {
    const float* cb = cosv + s * kHeadDim + (tid & 15) * 8;
    const float* sb = sinv + s * kHeadDim + (tid & 15) * 8;
    const float4 c0 = __ldg(reinterpret_cast<const float4*>(cb)), c1 = __ldg(reinterpret_cast<const float4*>(cb + 4));
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(sb)), s1 = __ldg(reinterpret_cast<const float4*>(sb + 4));
    ce[0] = c0.x; ce[1] = c0.z; ce[2] = c1.x; ce[3] = c1.z;                        // cos[..., 0::2]
    so[0] = s0.y; so[1] = s0.w; so[2] = s1.y; so[3] = s1.w;                        // sin[..., 1::2]
  }
#pragma unroll
  for (int u = 0; u < CPT; ++u) {
    const int c = tid + u * kPrepThreads;
    if (c < nchunks) {
      v[u] = __ldcs(row + c);
      if (kPrefetch) {
        if (weight) {
          wv[u][0] = __ldg(reinterpret_cast<const float4*>(weight + c * 8));
          wv[u][1] = __ldg(reinterpret_cast<const float4*>(weight + c * 8 + 4));
        }
      }
    }
  }
  float ss = 0.f;
  if (weight) {
#pragma unroll
    for (int u = 0; u < CPT; ++u) {
      const int c = tid + u * kPrepThreads;
      if (c < nchunks) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = __low2float(h[i]), b = __high2float(h[i]);
          ss = fmaf(a, a, ss);
          ss = fmaf(b, b, ss);
        }
      }
    }
  }
  float rstd = 1.f;
  if (weight) {                                                      // fixed-order block reduction
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) warp_sum[warp] = ss;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < kPrepThreads / 32; ++w) t += warp_sum[w];
      rstd_s = 1.0f / sqrtf(t / (float)(H * kHeadDim) + eps);
    }
    __syncthreads();
    rstd = rstd_s;
  }
#pragma unroll
  for (int u = 0; u < CPT; ++u) {
    const int c = tid + u * kPrepThreads;
    if (c >= nchunks) continue;
    const int h = c >> 4;
    const __nv_bfloat162* hin = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
    float y[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      y[2 * i] = __low2float(hin[i]);
      y[2 * i + 1] = __high2float(hin[i]);
    }
    if (weight) {
      const float4 w0 = kPrefetch ? wv[kPrefetch ? u : 0][0] : __ldg(reinterpret_cast<const float4*>(weight + c * 8));
      const float4 w1 = kPrefetch ? wv[kPrefetch ? u : 0][1] : __ldg(reinterpret_cast<const float4*>(weight + c * 8 + 4));
      const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = bf16_round(y[i] * rstd * wf[i]);          // the norm's output is bf16
    }
    if (cosv) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = y[2 * i], b = y[2 * i + 1];
        // two rounded products, then the sum: the reference evaluates x1 * cos - x2 * sin with
        // separate multiply and subtract kernels, not a fused multiply-add
        y[2 * i] = __fsub_rn(__fmul_rn(a, ce[i]), __fmul_rn(b, so[i]));
        y[2 * i + 1] = __fadd_rn(__fmul_rn(a, so[i]), __fmul_rn(b, ce[i]));
      }
    }
    uint4 o;
    o.x = pack_bf16x2(y[0], y[1]);
    o.y = pack_bf16x2(y[2], y[3]);
    o.z = pack_bf16x2(y[4], y[5]);
    o.w = pack_bf16x2(y[6], y[7]);
    uint4* d;
    if (dest.world == 0) {
      d = dest.dst[0] + ((int64_t)h * S + s) * 16;
    } else {
      const int64_t N = dest.n_loc * dest.world;
      d = dest.dst[dest.owner[h]] + ((int64_t)dest.slot[h] * N + (int64_t)dest.rank * dest.n_loc + s) * 16;
    }
    d[c & 15] = o;
  }
}

// One WARP per token (rows of at most 24 * 32 chunks, i.e. H <= 48): the row lives in the
// registers of 32 lanes (CPL chunks each), the sum of squares is a shuffle reduction, and nothing
// waits on a block barrier, so many more bytes are in flight per SM than with one CTA per token.
constexpr int kPrepWarpMinBlocks = 3;
template <int CPL>
__global__ void __launch_bounds__(128, kPrepWarpMinBlocks) qk_prep_warp_kernel(const uint4* __restrict__ x, const float* __restrict__ weight,
                                                           float eps, const float* __restrict__ cosv,
                                                           const float* __restrict__ sinv, int64_t S, int H,
                                                           const __grid_constant__ PrepDest dest) {
  const int lane = threadIdx.x % 32;
  const int64_t s = (int64_t)blockIdx.x * 4 + threadIdx.x / 32;
  if (s >= S) return;
  const int nchunks = H * 16;
  const uint4* row = x + s * nchunks;
  uint4 v[CPL];
#pragma unroll
  for (int u = 0; u < CPL; ++u) {
    const int c = lane + u * 32;
    if (c < nchunks) v[u] = __ldcs(row + c);
  }
  float rstd = 1.f;
  if (weight) {
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < CPL; ++u) {
      const int c = lane + u * 32;
      if (c < nchunks) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = __low2float(h[i]), b = __high2float(h[i]);
          ss = fmaf(a, a, ss);
          ss = fmaf(b, b, ss);
        }
      }
    }
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    rstd = 1.0f / sqrtf(ss / (float)(H * kHeadDim) + eps);
  }
  const int64_t N = dest.n_loc * (dest.world > 0 ? dest.world : 1);
  // every chunk of a lane starts at the same head-dim offset ((lane + 32 u) & 15 == lane & 15), so
  // the lane's rotary coefficients are fetched once per token
  const int d0 = (lane & 15) * 8;
  float ce[4] = {1.f, 1.f, 1.f, 1.f}, so[4] = {0.f, 0.f, 0.f, 0.f};
  if (cosv) {
    const float* cb = cosv + s * kHeadDim + d0;
    const float* sb = sinv + s * kHeadDim + d0;
    const float4 c0 = __ldg(reinterpret_cast<const float4*>(cb)), c1 = __ldg(reinterpret_cast<const float4*>(cb + 4));
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(sb)), s1 = __ldg(reinterpret_cast<const float4*>(sb + 4));
    ce[0] = c0.x; ce[1] = c0.z; ce[2] = c1.x; ce[3] = c1.z;                        // cos[..., 0::2]
    so[0] = s0.y; so[1] = s0.w; so[2] = s1.y; so[3] = s1.w;                        // sin[..., 1::2]
  }
#pragma unroll
  for (int u = 0; u < CPL; ++u) {
    const int c = lane + u * 32;
    if (c >= nchunks) continue;
    const int h = c >> 4;
    const __nv_bfloat162* hin = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
    float y[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      y[2 * i] = __low2float(hin[i]);
      y[2 * i + 1] = __high2float(hin[i]);
    }
    if (weight) {
      const float4 w0 = __ldg(reinterpret_cast<const float4*>(weight + c * 8));
      const float4 w1 = __ldg(reinterpret_cast<const float4*>(weight + c * 8 + 4));
      const float wf[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) y[i] = bf16_round(y[i] * rstd * wf[i]);
    }
    if (cosv) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = y[2 * i], b = y[2 * i + 1];
        y[2 * i] = __fsub_rn(__fmul_rn(a, ce[i]), __fmul_rn(b, so[i]));          // separate products and sum, as above
        y[2 * i + 1] = __fadd_rn(__fmul_rn(a, so[i]), __fmul_rn(b, ce[i]));
      }
    }
    uint4 o;
    o.x = pack_bf16x2(y[0], y[1]);
    o.y = pack_bf16x2(y[2], y[3]);
    o.z = pack_bf16x2(y[4], y[5]);
    o.w = pack_bf16x2(y[6], y[7]);
    uint4* d;
    if (dest.world == 0)
      d = dest.dst[0] + ((int64_t)h * S + s) * 16;
    else
      d = dest.dst[dest.owner[h]] + ((int64_t)dest.slot[h] * N + (int64_t)dest.rank * dest.n_loc + s) * 16;
    d[c & 15] = o;
  }
}

template <int CPL>
static void launch_prep_warp(const uint4* xp, const float* weight, float eps, const float* cosv, const float* sinv, int64_t S,
                             int H, const PrepDest& dest, cudaStream_t st) {
  qk_prep_warp_kernel<CPL><<<(unsigned)ceil_div64(S, 4), 128, 0, st>>>(xp, weight, eps, cosv, sinv, S, H, dest);
}

cudaError_t launch_qk_prep(const void* x, const float* weight, float eps, const float* cosv, const float* sinv, int64_t S,
                           int H, void* out_local, void* const* peer_dst, const int32_t* owner, const int32_t* slot,
                           int world, int rank, cudaStream_t st) {
  PrepDest dest{};
  if (peer_dst) {
    for (int p = 0; p < world; ++p) dest.dst[p] = (uint4*)peer_dst[p];
    for (int h = 0; h < H; ++h) {
      dest.owner[h] = (int16_t)owner[h];
      dest.slot[h] = (int16_t)slot[h];
    }
    dest.world = world;
    dest.rank = rank;
    dest.n_loc = S;
  } else {
    dest.dst[0] = (uint4*)out_local;
    dest.world = 0;
  }
  const uint4* xp = (const uint4*)x;
  const int cpl = ceil_div(H * 16, 32);                 // chunks per lane of the warp-per-token kernel
  if (cpl <= 4) launch_prep_warp<4>(xp, weight, eps, cosv, sinv, S, H, dest, st);
  else if (cpl <= 8) launch_prep_warp<8>(xp, weight, eps, cosv, sinv, S, H, dest, st);
  else if (cpl <= 12) launch_prep_warp<12>(xp, weight, eps, cosv, sinv, S, H, dest, st);
  else if (cpl <= 16) launch_prep_warp<16>(xp, weight, eps, cosv, sinv, S, H, dest, st);
  else if (cpl <= 20) launch_prep_warp<20>(xp, weight, eps, cosv, sinv, S, H, dest, st);
  else if (cpl <= 24) launch_prep_warp<24>(xp, weight, eps, cosv, sinv, S, H, dest, st);
  else {                                                // wide rows: one CTA per token
    const int cpt = ceil_div(H * 16, kPrepThreads);
    if (cpt <= 4) qk_prep_kernel<4><<<(unsigned)S, kPrepThreads, 0, st>>>(xp, weight, eps, cosv, sinv, S, H, dest);
    else qk_prep_kernel<8><<<(unsigned)S, kPrepThreads, 0, st>>>(xp, weight, eps, cosv, sinv, S, H, dest);
  }
  count_launches(1);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Per-head variant (HunyuanVideo): RMS norm over the 128 values of every (token, head), rotary
// embedding of the first `rope_rows` tokens only (the text tokens at the end of the sequence are not
// rotated) and the head transpose, in one pass.  Arithmetic of the reference's own CUDA kernels:
//   y = bf16((x * rsqrtf(sum(x^2) / 128 + eps)) * w)     rmsnorm_narrow_n_subwarp_reduction,
//                                                         svoo/kernels/include/norm/narrow_rms_norm.cuh:22-74
//   out[i] = bf16(y[i] cos[i] + (i even ? -y[i+1] : y[i-1]) sin[i])
//                                                         vec_apply_llama_rope_cos_sin_interleave,
//                                                         svoo/kernels/include/rope/rope_enc.cuh:17-36, called for
//                                                         the rows before the text by rope_enc_txtlast.cuh:34-78
// One half-warp per (token, head): 16 lanes x 8 values, the sum of squares per lane in element order,
// then a butterfly over the 16 lanes, as there.  The rows of head h go to out[h][out_row0 + s] of an
// [H, out_rows, 128] array, so a caller can place video and text tokens of separate projections in one
// sequence.  HBM-bound: 2 * 256 bytes per (token, head).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) qk_prep_heads_kernel(const uint4* __restrict__ x, const float* __restrict__ weight,
                                                            float eps, const float* __restrict__ cosv,
                                                            const float* __restrict__ sinv, int64_t S, int H,
                                                            int64_t rope_rows, uint4* __restrict__ out, int64_t out_rows,
                                                            int64_t out_row0) {
  const int64_t item = (int64_t)blockIdx.x * 16 + threadIdx.x / 16;
  const int sub = threadIdx.x % 16;
  const bool live = item < S * H;
  const int64_t s = live ? item / H : 0;
  const int h = live ? (int)(item % H) : 0;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (live) v = __ldg(x + item * 16 + sub);
  const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v);
  float y[8];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    y[2 * e] = __low2float(hv[e]);
    y[2 * e + 1] = __high2float(hv[e]);
  }
  if (weight) {
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) sum = fmaf(y[e], y[e], sum);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float rstd = rsqrtf(sum / (float)kHeadDim + eps);
    const float4 w0 = __ldg(reinterpret_cast<const float4*>(weight + sub * 8));
    const float4 w1 = __ldg(reinterpret_cast<const float4*>(weight + sub * 8 + 4));
    const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = bf16_round(__fmul_rn(__fmul_rn(y[e], rstd), w[e]));
  }
  if (cosv && live && s < rope_rows) {
    const float* cb = cosv + s * kHeadDim + sub * 8;
    const float* sb = sinv + s * kHeadDim + sub * 8;
    const float4 c0 = __ldg(reinterpret_cast<const float4*>(cb)), c1 = __ldg(reinterpret_cast<const float4*>(cb + 4));
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(sb)), s1 = __ldg(reinterpret_cast<const float4*>(sb + 4));
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      o[e] = fmaf(-y[e + 1], sn[e], __fmul_rn(y[e], c[e]));
      o[e + 1] = fmaf(y[e], sn[e + 1], __fmul_rn(y[e + 1], c[e + 1]));
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = o[e];
  }
  if (live) {
    uint4 r;
    __nv_bfloat162* hr = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int e = 0; e < 4; ++e) hr[e] = __floats2bfloat162_rn(y[2 * e], y[2 * e + 1]);
    out[((int64_t)h * out_rows + out_row0 + s) * 16 + sub] = r;
  }
}

cudaError_t launch_qk_prep_heads(const void* x, const float* weight, float eps, const float* cosv, const float* sinv, int64_t S,
                                 int H, int64_t rope_rows, void* out, int64_t out_rows, int64_t out_row0, cudaStream_t st) {
  qk_prep_heads_kernel<<<(unsigned)ceil_div64(S * H, 16), 256, 0, st>>>((const uint4*)x, weight, eps, cosv, sinv, S, H, rope_rows,
                                                                      (uint4*)out, out_rows, out_row0);
  count_launches(1);
  return cudaGetLastError();
}

}  // namespace svoo
