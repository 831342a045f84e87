// Shared device helpers for the svoo_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/svoo_b200.h"

namespace svoo {

constexpr int kHeadDim = 128;            // bf16 row = 256 bytes = 16 chunks of 16 bytes
constexpr int kRowBytes = kHeadDim * 2;

typedef __nv_bfloat16 bf16;

__host__ __device__ inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t align_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

// ---------------------------------------------------------------------------------------
// Workspace layout shared by the host entry points.  All offsets are multiples of 256 B.
// ---------------------------------------------------------------------------------------
constexpr int kSortChunk = 2048;         // tokens per CTA in the counting sort
constexpr int kCentroidSlabs = 8;        // partial sums per cluster in the centroid update
constexpr int kAttnBM = 128;             // query rows per attention tile

struct Workspace {
  int64_t chunk_hist;    // int32 [BH, nchunks, Kmax]   per-chunk label histograms / bases
  int64_t partial;       // float [BH, Kmax, slabs, 128] centroid partial sums
  int64_t w_hi;          // bf16  [BH, Jpad, 128]
  int64_t w_lo;          // bf16  [BH, Jpad, 128]
  int64_t assign_partial;  // int2 [Jpad/128, BH, N]: best (score bits, j) per column group
  int64_t status;        // int32 [4]: word 0 != 0 after a kernel gave up on a bounded wait
  int64_t runs;          // int2  [BH, QC, max_runs]: (first_row, virtual_begin) + sentinel (0, total)
  int64_t nruns;         // int32 [BH, QC]
  int64_t qtiles;        // int4  [BH, max_qtiles]
  int64_t nqtiles;       // int32 [BH]
  int64_t total;
};

__host__ inline int sort_chunks(int64_t N) { return (int)ceil_div64(N, kSortChunk); }
__host__ inline int pad_clusters(int64_t K) { return (int)align_up(K, 256); }   // W rows, whole 256-row blocks
__host__ inline int max_runs(int64_t KC) { return (int)(KC / 2 + 2); }   // + one sentinel entry
__host__ inline int max_qtiles(int64_t N, int64_t QC) { return (int)(ceil_div64(N, kAttnBM) + QC); }

__host__ inline Workspace workspace_layout(int64_t BH, int64_t N, int64_t QC, int64_t KC) {
  Workspace w;
  const int64_t Kmax = QC > KC ? QC : KC;
  int64_t o = 0;
  auto take = [&](int64_t bytes) { int64_t at = o; o += align_up(bytes, 256); return at; };
  w.chunk_hist = take(BH * sort_chunks(N) * Kmax * 4);
  w.partial = take(BH * Kmax * kCentroidSlabs * kHeadDim * 4);
  w.w_hi = take(BH * (int64_t)pad_clusters(Kmax) * kRowBytes);
  w.w_lo = take(BH * (int64_t)pad_clusters(Kmax) * kRowBytes);
  w.assign_partial = take((int64_t)(pad_clusters(Kmax) / 128) * BH * N * 8);   // two column groups per 256 rows
  w.status = take(16);
  // sized symmetrically in (QC, KC) so that one workspace serves either side
  w.runs = take(BH * (QC * KC / 2 + 2 * (QC + KC)) * 8);
  w.nruns = take(BH * Kmax * 4);
  w.qtiles = take(BH * (int64_t)max_qtiles(N, Kmax) * 16);
  w.nqtiles = take(BH * 4);
  w.total = o;
  return w;
}

// Process-wide count of kernel launches (read through svoo_b200_launch_count()).
int64_t& launch_counter();
inline void count_launches(int n) { __atomic_fetch_add(&launch_counter(), (int64_t)n, __ATOMIC_RELAXED); }

// ---------------------------------------------------------------------------------------
// Programmatic dependent launch.  The clustering is a chain of short kernels (ten phases of
// seven launches); launched this way, a kernel's CTAs are scheduled and run their set-up while
// the previous kernel drains, and block in pdl_wait() until that kernel has completed and its
// writes are visible.  Every kernel launched with launch_pdl() calls pdl_wait() before its first
// access to memory that an earlier kernel of the stream wrote, and pdl_trigger() at its start
// (the next kernel's CTAs may then be scheduled as soon as every CTA of this one has started).
// Outside such a launch both are no-ops.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---------------------------------------------------------------------------------------
// Small device utilities
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async16(uint32_t smem, const void* gmem, bool valid) {
  int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16) * B(16x8,bf16)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` in a [rows][128] bf16 tile whose
// chunks are XOR-swizzled by the row so that ldmatrix reads are bank-conflict free.
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return (uint32_t)(row * kRowBytes + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace svoo
