// extern "C" entry points of libsvoo_b200.so: argument checks, workspace carving and the
// launch sequences.  No entry point allocates or synchronises.
#include "common.cuh"

namespace svoo {
cudaError_t launch_gather_rows(const void*, const int32_t*, void*, int64_t, int64_t, int64_t, cudaStream_t);
cudaError_t launch_prologue(const void*, const void*, void*, void*, int64_t, int64_t, int64_t, cudaStream_t);
cudaError_t launch_assign_tc(const void*, const void*, const void*, int32_t*, int2*, int32_t*, int64_t, int64_t, int64_t,
                             int32_t*, cudaStream_t);
cudaError_t launch_sort_labels(const int32_t*, int64_t, int64_t, int64_t, int32_t*, int32_t*, int32_t*, int32_t*,
                               cudaStream_t, bool);
cudaError_t launch_centroid_update(const void*, const int32_t*, const int32_t*, const void*, void*, int32_t*, float*,
                                   int64_t, int64_t, int64_t, cudaStream_t);
cudaError_t launch_offsets_from_sizes(const int32_t*, int32_t*, int64_t, int64_t, cudaStream_t);
cudaError_t launch_permute(const void*, const int32_t*, void*, int64_t, int64_t, int64_t, int64_t, bool, cudaStream_t);
cudaError_t launch_block_map(const void*, const void*, const int32_t*, uint8_t*, int64_t, int64_t, int64_t, float,
                             const int32_t*, const int32_t*, cudaStream_t);
cudaError_t launch_build_runs(const uint8_t*, const int32_t*, int2*, int32_t*, int64_t, int64_t, int64_t, cudaStream_t);
cudaError_t launch_build_qtiles(const int32_t*, int4*, int32_t*, int64_t, int64_t, int64_t, int, cudaStream_t);
cudaError_t launch_sparse_attn_tc(const void*, const void*, const void*, void*, const int32_t*, const int4*,
                                  const int32_t*, const int2*, const int32_t*, int32_t*, int64_t, int64_t, int64_t,
                                  int64_t, float, void* const*, const int32_t*, int, int64_t, int, float*, cudaStream_t,
                                  const uint8_t* ear_map = nullptr, const int32_t* ear_k_offsets = nullptr,
                                  int ear_max_runs = 0);
cudaError_t launch_ear_value_stats(const void*, const int32_t*, void*, float*, float*, float*, int64_t, int64_t, int64_t,
                                   cudaStream_t);
cudaError_t launch_ear_scores(const void*, const void*, const void*, const int32_t*, const int32_t*, const float*,
                              const float*, const float*, float*, float*, int64_t, int64_t, int64_t, int64_t, float,
                              cudaStream_t);
cudaError_t launch_ear_select(const float*, const float*, const int32_t*, const int32_t*, uint8_t*, int64_t, int64_t, int64_t,
                              float, const int32_t*, const int32_t*, cudaStream_t);
cudaError_t launch_ear_build_runs(const uint8_t*, const int32_t*, int2*, int32_t*, int64_t, int64_t, int64_t, int64_t, int,
                                  cudaStream_t);
cudaError_t launch_euclid_assign_tc(const void*, const void*, float*, int32_t*, int2*, int32_t*, int64_t, int64_t, int64_t,
                                    int32_t*, cudaStream_t);
cudaError_t launch_append_text_blocks(const uint8_t*, const int32_t*, const int32_t*, const int32_t*, const int32_t*,
                                      uint8_t*, int32_t*, int32_t*, int32_t*, int32_t*, int64_t, int64_t, int64_t, int64_t,
                                      int64_t, int64_t, cudaStream_t);
cudaError_t launch_sparse_attn_mma(const void*, const void*, const void*, void*, const int32_t*, const int4*,
                                   const int32_t*, const int2*, const int32_t*, int64_t, int64_t, int64_t, int64_t,
                                   float, cudaStream_t);
cudaError_t launch_push_heads(const void*, void* const*, const int32_t*, const int32_t*, int, int, int64_t, int,
                              cudaStream_t);
cudaError_t launch_push_seq(const void*, void* const*, const int32_t*, int, int64_t, int, int, cudaStream_t);
cudaError_t launch_peer_barrier(void* const*, int, int, int, uint32_t, int32_t*, cudaStream_t);
cudaError_t launch_qk_prep(const void*, const float*, float, const float*, const float*, int64_t, int, void*, void* const*,
                           const int32_t*, const int32_t*, int, int, cudaStream_t);
cudaError_t launch_qk_prep_heads(const void*, const float*, float, const float*, const float*, int64_t, int, int64_t, void*,
                                 int64_t, int64_t, cudaStream_t);
}  // namespace svoo

namespace svoo {
int64_t& launch_counter() {
  static int64_t n = 0;
  return n;
}
}  // namespace svoo

using namespace svoo;

namespace {
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_tokens(int64_t BH, int64_t N, int64_t D) {
  if (D != kHeadDim) return SVOO_ERR_HEAD_DIM;
  if (BH < 1 || BH > 65535 || N < 1 || N > (1 << 24)) return SVOO_ERR_SHAPE;
  if (BH * N > (int64_t)INT32_MAX) return SVOO_ERR_SHAPE;         // the kernels index token rows with 32-bit ints
  return SVOO_OK;
}
int check_clusters(int64_t K) {
  if (K < 1) return SVOO_ERR_SHAPE;
  if (K > SVOO_MAX_CLUSTERS) return SVOO_ERR_CLUSTERS;
  return SVOO_OK;
}
// attention side: the clusters plus the two text blocks of a joint-attention layer
int check_attn_clusters(int64_t K) {
  if (K < 1) return SVOO_ERR_SHAPE;
  if (K > SVOO_MAX_ATTN_CLUSTERS) return SVOO_ERR_CLUSTERS;
  return SVOO_OK;
}
#define SVOO_TRY(expr) do { int _rc = (expr); if (_rc != SVOO_OK) return _rc; } while (0)
#define SVOO_CUDA(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) return (int)_e; } while (0)

template <typename T>
inline T* ws_at(void* ws, int64_t off) { return reinterpret_cast<T*>(static_cast<char*>(ws) + off); }
}  // namespace

extern "C" {

int svoo_b200_version(void) { return SVOO_B200_VERSION; }

int64_t svoo_b200_launch_count(void) { return __atomic_load_n(&launch_counter(), __ATOMIC_RELAXED); }

const char* svoo_b200_error_string(int code) {
  switch (code) {
    case SVOO_OK: return "ok";
    case SVOO_ERR_NULL: return "a required pointer is null";
    case SVOO_ERR_SHAPE: return "a size is out of the supported range";
    case SVOO_ERR_HEAD_DIM: return "head dimension must be 128";
    case SVOO_ERR_WORKSPACE: return "workspace too small";
    case SVOO_ERR_ALIGN: return "tensor pointer is not 16-byte aligned";
    case SVOO_ERR_CLUSTERS: return "cluster count above 1024 (1026 blocks for the attention)";
    case SVOO_ERR_STATIC_SCRATCH: return "problem too large for the built-in scratch array (BH*ceil(N/2048)*K > 1048576)";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown svoo_b200 error";
  }
}

int svoo_b200_workspace_bytes(int64_t BH, int64_t N, int64_t QC, int64_t KC, int64_t* bytes_out) {
  if (!bytes_out) return SVOO_ERR_NULL;
  SVOO_TRY(check_tokens(BH, N, kHeadDim));
  SVOO_TRY(check_attn_clusters(QC));
  SVOO_TRY(check_attn_clusters(KC));
  *bytes_out = workspace_layout(BH, N, QC, KC).total;
  return SVOO_OK;
}

int svoo_b200_cocluster_assign(const void* x, const void* form_centroids, const void* own_centroids, int64_t BH,
                               int64_t N, int64_t D, int64_t K, int64_t J, int32_t* labels, void* workspace,
                               int64_t workspace_bytes, void* stream) {
  if (!x || !form_centroids || !own_centroids || !labels || !workspace) return SVOO_ERR_NULL;
  SVOO_TRY(check_tokens(BH, N, D));
  SVOO_TRY(check_clusters(K));
  SVOO_TRY(check_clusters(J));
  if (!aligned16(x) || !aligned16(form_centroids) || !aligned16(own_centroids) || !aligned16(workspace))
    return SVOO_ERR_ALIGN;
  const Workspace w = workspace_layout(BH, N, K, J);
  if (workspace_bytes < w.total) return SVOO_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  SVOO_CUDA(launch_prologue(own_centroids, form_centroids, ws_at<void>(workspace, w.w_hi),
                            ws_at<void>(workspace, w.w_lo), BH, J, K, st));
  SVOO_CUDA(cudaMemsetAsync(ws_at<int32_t>(workspace, w.status) + 1, 0, 4, st));
  SVOO_CUDA(launch_assign_tc(x, ws_at<void>(workspace, w.w_hi), ws_at<void>(workspace, w.w_lo), labels,
                             ws_at<int2>(workspace, w.assign_partial), ws_at<int32_t>(workspace, w.status) + 1, BH, N, J, nullptr,
                             st));
  return SVOO_OK;
}

int svoo_b200_euclid_assign(const void* x, const void* centroids, int64_t BH, int64_t N, int64_t D, int64_t K,
                            int32_t* labels, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!x || !centroids || !labels || !workspace) return SVOO_ERR_NULL;
  SVOO_TRY(check_tokens(BH, N, D));
  SVOO_TRY(check_clusters(K));
  if (!aligned16(x) || !aligned16(centroids) || !aligned16(workspace)) return SVOO_ERR_ALIGN;
  const Workspace w = workspace_layout(BH, N, K, K);
  if (workspace_bytes < w.total) return SVOO_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  int32_t* status = ws_at<int32_t>(workspace, w.status) + 1;
  SVOO_CUDA(cudaMemsetAsync(status, 0, 4, st));
  SVOO_CUDA(launch_euclid_assign_tc(x, centroids, ws_at<float>(workspace, w.w_hi), labels,
                                    ws_at<int2>(workspace, w.assign_partial), status, BH, N, K, nullptr, st));
  return SVOO_OK;
}

int svoo_b200_sort_labels(const int32_t* labels, int64_t BH, int64_t N, int64_t K, int32_t* sorted_idx,
                          int32_t* offsets, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!labels || !sorted_idx || !offsets || !workspace) return SVOO_ERR_NULL;
  SVOO_TRY(check_tokens(BH, N, kHeadDim));
  SVOO_TRY(check_clusters(K));
  const Workspace w = workspace_layout(BH, N, K, K);
  if (workspace_bytes < w.total) return SVOO_ERR_WORKSPACE;
  SVOO_CUDA(launch_sort_labels(labels, BH, N, K, sorted_idx, offsets, nullptr, ws_at<int32_t>(workspace, w.chunk_hist),
                               (cudaStream_t)stream, false));
  return SVOO_OK;
}

int svoo_b200_centroid_update(const void* x, const int32_t* sorted_idx, const int32_t* offsets,
                              const void* old_centroids, int64_t BH, int64_t N, int64_t D, int64_t K,
                              void* new_centroids, int32_t* sizes, void* workspace, int64_t workspace_bytes,
                              void* stream) {
  if (!x || !sorted_idx || !offsets || !old_centroids || !new_centroids || !workspace) return SVOO_ERR_NULL;
  SVOO_TRY(check_tokens(BH, N, D));
  SVOO_TRY(check_clusters(K));
  if (!aligned16(x)) return SVOO_ERR_ALIGN;
  const Workspace w = workspace_layout(BH, N, K, K);
  if (workspace_bytes < w.total) return SVOO_ERR_WORKSPACE;
  SVOO_CUDA(launch_centroid_update(x, sorted_idx, offsets, old_centroids, new_centroids, sizes,
                                   ws_at<float>(workspace, w.partial), BH, N, K, (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_cocluster(const void* q, const void* k, const int32_t* q_init_idx, const int32_t* k_init_idx, int64_t BH,
                        int64_t N, int64_t D, int64_t QC, int64_t KC, int32_t iters, int32_t* qlabels,
                        int32_t* klabels, void* qcentroids, void* kcentroids, int32_t* qsizes, int32_t* ksizes,
                        int32_t* q_sorted_idx, int32_t* q_offsets, int32_t* k_sorted_idx, int32_t* k_offsets,
                        void* workspace, int64_t workspace_bytes, void* stream) {
  if (!q || !k || !qlabels || !klabels || !qcentroids || !kcentroids || !qsizes || !ksizes || !q_sorted_idx ||
      !q_offsets || !k_sorted_idx || !k_offsets || !workspace)
    return SVOO_ERR_NULL;
  if ((q_init_idx == nullptr) != (k_init_idx == nullptr)) return SVOO_ERR_NULL;   // both (fresh start) or neither (warm start)
  SVOO_TRY(check_tokens(BH, N, D));
  SVOO_TRY(check_clusters(QC));
  SVOO_TRY(check_clusters(KC));
  if (iters < 1 || iters > 1000) return SVOO_ERR_SHAPE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(qcentroids) || !aligned16(kcentroids) || !aligned16(workspace))
    return SVOO_ERR_ALIGN;
  const Workspace w = workspace_layout(BH, N, QC, KC);
  if (workspace_bytes < w.total) return SVOO_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  void* w_hi = ws_at<void>(workspace, w.w_hi);
  void* w_lo = ws_at<void>(workspace, w.w_lo);
  int32_t* hist = ws_at<int32_t>(workspace, w.chunk_hist);
  float* partial = ws_at<float>(workspace, w.partial);
  int2* apart = ws_at<int2>(workspace, w.assign_partial);
  int32_t* status = ws_at<int32_t>(workspace, w.status) + 1;       // word 1: assignment kernel

  SVOO_CUDA(cudaMemsetAsync(status, 0, 4, st));
  if (q_init_idx) {
    SVOO_CUDA(launch_gather_rows(q, q_init_idx, qcentroids, BH, N, QC, st));
    SVOO_CUDA(launch_gather_rows(k, k_init_idx, kcentroids, BH, N, KC, st));
  }
  for (int it = 0; it < iters; ++it) {
    // keys: profile over the query centroids
    SVOO_CUDA(launch_prologue(kcentroids, qcentroids, w_hi, w_lo, BH, KC, QC, st));
    SVOO_CUDA(launch_assign_tc(k, w_hi, w_lo, klabels, apart, status, BH, N, KC, hist, st));
    SVOO_CUDA(launch_sort_labels(klabels, BH, N, KC, k_sorted_idx, k_offsets, nullptr, hist, st, true));
    SVOO_CUDA(launch_centroid_update(k, k_sorted_idx, k_offsets, kcentroids, kcentroids, ksizes, partial, BH, N, KC, st));
    // queries: profile over the just-updated key centroids
    SVOO_CUDA(launch_prologue(qcentroids, kcentroids, w_hi, w_lo, BH, QC, KC, st));
    SVOO_CUDA(launch_assign_tc(q, w_hi, w_lo, qlabels, apart, status, BH, N, QC, hist, st));
    SVOO_CUDA(launch_sort_labels(qlabels, BH, N, QC, q_sorted_idx, q_offsets, nullptr, hist, st, true));
    SVOO_CUDA(launch_centroid_update(q, q_sorted_idx, q_offsets, qcentroids, qcentroids, qsizes, partial, BH, N, QC, st));
  }
  return SVOO_OK;
}

int svoo_b200_permute(const void* x, const int32_t* sorted_idx, int64_t BH, int64_t N, int64_t D,
                      int64_t x_head_rows, int64_t y_head_rows, void* y, void* stream) {
  if (!x || !sorted_idx || !y) return SVOO_ERR_NULL;
  SVOO_TRY(check_tokens(BH, N, D));
  if (x_head_rows < N || y_head_rows < N) return SVOO_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(y)) return SVOO_ERR_ALIGN;
  SVOO_CUDA(launch_permute(x, sorted_idx, y, BH, N, x_head_rows, y_head_rows, false, (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_inverse_permute(const void* x, const int32_t* sorted_idx, int64_t BH, int64_t N, int64_t D,
                              int64_t x_head_rows, int64_t y_head_rows, void* y, void* stream) {
  if (!x || !sorted_idx || !y) return SVOO_ERR_NULL;
  SVOO_TRY(check_tokens(BH, N, D));
  if (x_head_rows < N || y_head_rows < N) return SVOO_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(y)) return SVOO_ERR_ALIGN;
  SVOO_CUDA(launch_permute(x, sorted_idx, y, BH, N, x_head_rows, y_head_rows, true, (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_block_map(const void* qcentroids, const void* kcentroids, const int32_t* ksizes, int64_t BH, int64_t QC,
                        int64_t KC, int64_t D, float top_p, const int32_t* preserve_host, const int32_t* cap_host,
                        uint8_t* map_out, void* stream) {
  if (!qcentroids || !kcentroids || !ksizes || !preserve_host || !cap_host || !map_out) return SVOO_ERR_NULL;
  if (D != kHeadDim) return SVOO_ERR_HEAD_DIM;
  if (BH < 1 || BH > SVOO_MAX_HEADS) return SVOO_ERR_SHAPE;
  SVOO_TRY(check_clusters(QC));
  SVOO_TRY(check_clusters(KC));
  if (!aligned16(qcentroids) || !aligned16(kcentroids)) return SVOO_ERR_ALIGN;
  SVOO_CUDA(launch_block_map(qcentroids, kcentroids, ksizes, map_out, BH, QC, KC, top_p, preserve_host, cap_host,
                             (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_offsets_from_sizes(const int32_t* sizes, int64_t BH, int64_t K, int32_t* offsets, void* stream) {
  if (!sizes || !offsets) return SVOO_ERR_NULL;
  if (BH < 1 || BH > 65535) return SVOO_ERR_SHAPE;
  SVOO_TRY(check_attn_clusters(K));
  SVOO_CUDA(launch_offsets_from_sizes(sizes, offsets, BH, K, (cudaStream_t)stream));
  return SVOO_OK;
}

namespace {
int check_exchange(void* const* peer_dst, int32_t world, int64_t n_loc, int64_t H, int64_t D) {
  if (!peer_dst) return SVOO_ERR_NULL;
  if (D != kHeadDim) return SVOO_ERR_HEAD_DIM;
  if (world < 1 || world > 16 || H < world || H > 128 || n_loc < 1 || n_loc * world > (int64_t)1 << 30)
    return SVOO_ERR_SHAPE;
  for (int p = 0; p < world; ++p) {
    if (!peer_dst[p]) return SVOO_ERR_NULL;
    if (!aligned16(peer_dst[p])) return SVOO_ERR_ALIGN;
  }
  return SVOO_OK;
}
}  // namespace

static int sparse_attn_impl(bool tensor_core, const void* q, const void* k, const void* v, const uint8_t* map,
                            const int32_t* q_offsets, const int32_t* k_offsets, int64_t BH, int64_t S, int64_t D,
                            int64_t QC, int64_t KC, float sm_scale, void* out, const int32_t* out_row_idx,
                            void* workspace, int64_t workspace_bytes, void* stream, void* const* peer_dst = nullptr,
                            const int32_t* my_heads = nullptr, int world = 0, int64_t n_loc = 0, int H = 0,
                            float* lse = nullptr) {
  if (!q || !k || !v || !map || !q_offsets || !k_offsets || (!out && !peer_dst) || !workspace) return SVOO_ERR_NULL;
  SVOO_TRY(check_tokens(BH, S, D));
  SVOO_TRY(check_attn_clusters(QC));
  SVOO_TRY(check_attn_clusters(KC));
  if (lse && !tensor_core) return SVOO_ERR_SHAPE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(workspace))
    return SVOO_ERR_ALIGN;
  if (!tensor_core && peer_dst) return SVOO_ERR_SHAPE;
  const Workspace w = workspace_layout(BH, S, QC, KC);
  if (workspace_bytes < w.total) return SVOO_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  int2* runs = ws_at<int2>(workspace, w.runs);
  int32_t* nruns = ws_at<int32_t>(workspace, w.nruns);
  int4* qtiles = ws_at<int4>(workspace, w.qtiles);
  int32_t* nqtiles = ws_at<int32_t>(workspace, w.nqtiles);
  int32_t* status = ws_at<int32_t>(workspace, w.status);
  SVOO_CUDA(launch_build_runs(map, k_offsets, runs, nruns, BH, QC, KC, st));
  SVOO_CUDA(launch_build_qtiles(q_offsets, qtiles, nqtiles, BH, S, QC, tensor_core ? 256 : 128, st));
  if (tensor_core) {
    SVOO_CUDA(cudaMemsetAsync(status, 0, 4, st));                     // word 0: attention kernel
    SVOO_CUDA(launch_sparse_attn_tc(q, k, v, out, out_row_idx, qtiles, nqtiles, runs, nruns, status, BH, S, QC, KC,
                                    sm_scale, peer_dst, my_heads, world, n_loc, H, lse, st));
  } else {
    SVOO_CUDA(launch_sparse_attn_mma(q, k, v, out, out_row_idx, qtiles, nqtiles, runs, nruns, BH, S, QC, KC, sm_scale,
                                     st));
  }
  return SVOO_OK;
}

int svoo_b200_sparse_attn(const void* q, const void* k, const void* v, const uint8_t* map, const int32_t* q_offsets,
                          const int32_t* k_offsets, int64_t BH, int64_t S, int64_t D, int64_t QC, int64_t KC,
                          float sm_scale, void* out, const int32_t* out_row_idx, float* lse, void* workspace,
                          int64_t workspace_bytes, void* stream) {
  return sparse_attn_impl(true, q, k, v, map, q_offsets, k_offsets, BH, S, D, QC, KC, sm_scale, out, out_row_idx,
                          workspace, workspace_bytes, stream, nullptr, nullptr, 0, 0, 0, lse);
}

int svoo_b200_sparse_attn_push(const void* q, const void* k, const void* v, const uint8_t* map,
                               const int32_t* q_offsets, const int32_t* k_offsets, int64_t BH, int64_t S, int64_t D,
                               int64_t QC, int64_t KC, float sm_scale, void* const* peer_dst, const int32_t* my_heads,
                               int32_t world, int64_t n_loc, int64_t H, const int32_t* out_row_idx, void* workspace,
                               int64_t workspace_bytes, void* stream) {
  if (!my_heads) return SVOO_ERR_NULL;
  SVOO_TRY(check_exchange(peer_dst, world, n_loc, H, D));
  if (BH < 1 || BH > ceil_div64(H, world) || S != n_loc * world) return SVOO_ERR_SHAPE;
  bool seen[128] = {};
  for (int64_t i = 0; i < BH; ++i) {
    if (my_heads[i] < 0 || my_heads[i] >= H || seen[my_heads[i]]) return SVOO_ERR_SHAPE;
    seen[my_heads[i]] = true;
  }
  return sparse_attn_impl(true, q, k, v, map, q_offsets, k_offsets, BH, S, D, QC, KC, sm_scale, nullptr, out_row_idx,
                          workspace, workspace_bytes, stream, peer_dst, my_heads, world, n_loc, (int)H);
}

int svoo_b200_sparse_attn_simt(const void* q, const void* k, const void* v, const uint8_t* map,
                               const int32_t* q_offsets, const int32_t* k_offsets, int64_t BH, int64_t S, int64_t D,
                               int64_t QC, int64_t KC, float sm_scale, void* out, const int32_t* out_row_idx,
                               void* workspace, int64_t workspace_bytes, void* stream) {
  return sparse_attn_impl(false, q, k, v, map, q_offsets, k_offsets, BH, S, D, QC, KC, sm_scale, out, out_row_idx,
                          workspace, workspace_bytes, stream);
}

// ---------------------------------------------------------------------------------------
// Error-aware routing (EAR)
// ---------------------------------------------------------------------------------------
namespace {
struct EarWorkspace {
  int64_t vnorm, cvd, vcsq, runs, nruns, qtiles, nqtiles, status, total;
};
inline int ear_max_runs(int64_t KC) { return (int)(KC / 2 + 4); }   // token runs + the centroid run + sentinel
inline EarWorkspace ear_layout(int64_t BH, int64_t N, int64_t QC, int64_t KC) {
  EarWorkspace w;
  int64_t o = 0;
  auto take = [&](int64_t bytes) { int64_t at = o; o += align_up(bytes, 256); return at; };
  w.vnorm = take(BH * N * 4);
  w.cvd = take(BH * N * 4);
  w.vcsq = take(BH * KC * 4);
  w.runs = take(BH * QC * (int64_t)ear_max_runs(KC) * 8);
  w.nruns = take(BH * QC * 4);
  w.qtiles = take(BH * (int64_t)max_qtiles(N, QC) * 16);
  w.nqtiles = take(BH * 4);
  w.status = take(16);
  w.total = o;
  return w;
}
int check_ear(int64_t BH, int64_t N, int64_t D, int64_t QC, int64_t KC) {
  SVOO_TRY(check_tokens(BH, N, D));
  if (QC < 1 || KC < 1 || QC > SVOO_MAX_CLUSTERS || KC > SVOO_MAX_CLUSTERS) return SVOO_ERR_CLUSTERS;
  return SVOO_OK;
}
}  // namespace

int svoo_b200_ear_workspace_bytes(int64_t BH, int64_t N, int64_t QC, int64_t KC, int64_t* bytes_out,
                                  int64_t* status_offset_out) {
  if (!bytes_out) return SVOO_ERR_NULL;
  SVOO_TRY(check_ear(BH, N, kHeadDim, QC, KC));
  const EarWorkspace w = ear_layout(BH, N, QC, KC);
  *bytes_out = w.total;
  if (status_offset_out) *status_offset_out = w.status;
  return SVOO_OK;
}

int svoo_b200_ear_value_centroids(const void* v_perm, const int32_t* k_offsets, int64_t BH, int64_t N, int64_t D,
                                  int64_t QC, int64_t KC, void* vcentroids_out, void* ear_workspace,
                                  int64_t ear_workspace_bytes, void* stream) {
  if (!v_perm || !k_offsets || !vcentroids_out || !ear_workspace) return SVOO_ERR_NULL;
  SVOO_TRY(check_ear(BH, N, D, QC, KC));
  if (!aligned16(v_perm) || !aligned16(vcentroids_out) || !aligned16(ear_workspace)) return SVOO_ERR_ALIGN;
  const EarWorkspace w = ear_layout(BH, N, QC, KC);
  if (ear_workspace_bytes < w.total) return SVOO_ERR_WORKSPACE;
  SVOO_CUDA(launch_ear_value_stats(v_perm, k_offsets, vcentroids_out, ws_at<float>(ear_workspace, w.vnorm),
                                   ws_at<float>(ear_workspace, w.cvd), ws_at<float>(ear_workspace, w.vcsq), BH, N, KC,
                                   (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_ear_block_scores(const void* qcentroids, const void* kcentroids, const void* k_perm, const int32_t* q_offsets,
                               const int32_t* k_offsets, int64_t BH, int64_t N, int64_t D, int64_t QC, int64_t KC,
                               float gamma, float* c_logits_out, float* scores_out, void* ear_workspace,
                               int64_t ear_workspace_bytes, void* stream) {
  if (!qcentroids || !kcentroids || !k_perm || !q_offsets || !k_offsets || !c_logits_out || !scores_out || !ear_workspace)
    return SVOO_ERR_NULL;
  SVOO_TRY(check_ear(BH, N, D, QC, KC));
  if (!aligned16(qcentroids) || !aligned16(kcentroids) || !aligned16(k_perm) || !aligned16(ear_workspace)) return SVOO_ERR_ALIGN;
  const EarWorkspace w = ear_layout(BH, N, QC, KC);
  if (ear_workspace_bytes < w.total) return SVOO_ERR_WORKSPACE;
  SVOO_CUDA(launch_ear_scores(qcentroids, kcentroids, k_perm, q_offsets, k_offsets, ws_at<float>(ear_workspace, w.vnorm),
                              ws_at<float>(ear_workspace, w.cvd), ws_at<float>(ear_workspace, w.vcsq), c_logits_out, scores_out,
                              BH, N, QC, KC, gamma, (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_ear_select_blocks(const float* c_logits, const float* scores, const int32_t* q_offsets, const int32_t* k_offsets,
                                int64_t BH, int64_t QC, int64_t KC, float top_p, const int32_t* preserve_host,
                                const int32_t* budget_preserve_host, uint8_t* map_out, void* stream) {
  if (!c_logits || !scores || !q_offsets || !k_offsets || !preserve_host || !budget_preserve_host || !map_out)
    return SVOO_ERR_NULL;
  if (BH < 1 || BH > SVOO_MAX_HEADS) return SVOO_ERR_SHAPE;
  if (QC < 1 || KC < 1 || QC > SVOO_MAX_CLUSTERS || KC > SVOO_MAX_CLUSTERS) return SVOO_ERR_CLUSTERS;
  for (int64_t h = 0; h < BH; ++h)
    if (preserve_host[h] < 0 || budget_preserve_host[h] < 0) return SVOO_ERR_SHAPE;
  SVOO_CUDA(launch_ear_select(c_logits, scores, q_offsets, k_offsets, map_out, BH, QC, KC, top_p, preserve_host,
                              budget_preserve_host, (cudaStream_t)stream));
  return SVOO_OK;
}

static int sparse_attn_ear_impl(const void* q, const void* k_ext, const void* v_ext, const uint8_t* map,
                                const int32_t* q_offsets, const int32_t* k_offsets, int64_t BH, int64_t S, int64_t D,
                                int64_t QC, int64_t KC, float sm_scale, void* out, const int32_t* out_row_idx, float* lse,
                                void* ear_workspace, int64_t ear_workspace_bytes, void* stream, void* const* peer_dst,
                                const int32_t* my_heads, int world, int64_t n_loc, int H) {
  if (!q || !k_ext || !v_ext || !map || !q_offsets || !k_offsets || (!out && !peer_dst) || !ear_workspace) return SVOO_ERR_NULL;
  SVOO_TRY(check_ear(BH, S, D, QC, KC));
  if ((BH * S + BH * KC) > 2147483647LL) return SVOO_ERR_SHAPE;
  if (!aligned16(q) || !aligned16(k_ext) || !aligned16(v_ext) || !aligned16(out) || !aligned16(ear_workspace))
    return SVOO_ERR_ALIGN;
  const EarWorkspace w = ear_layout(BH, S, QC, KC);
  if (ear_workspace_bytes < w.total) return SVOO_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  int2* runs = ws_at<int2>(ear_workspace, w.runs);
  int32_t* nruns = ws_at<int32_t>(ear_workspace, w.nruns);
  int4* qtiles = ws_at<int4>(ear_workspace, w.qtiles);
  int32_t* nqtiles = ws_at<int32_t>(ear_workspace, w.nqtiles);
  int32_t* status = ws_at<int32_t>(ear_workspace, w.status);
  SVOO_CUDA(launch_ear_build_runs(map, k_offsets, runs, nruns, BH, S, QC, KC, ear_max_runs(KC), st));
  SVOO_CUDA(launch_build_qtiles(q_offsets, qtiles, nqtiles, BH, S, QC, 256, st));
  SVOO_CUDA(cudaMemsetAsync(status, 0, 4, st));
  SVOO_CUDA(launch_sparse_attn_tc(q, k_ext, v_ext, out, out_row_idx, qtiles, nqtiles, runs, nruns, status, BH, S, QC, KC,
                                  sm_scale, peer_dst, my_heads, world, n_loc, H, lse, st, map, k_offsets, ear_max_runs(KC)));
  return SVOO_OK;
}

int svoo_b200_sparse_attn_ear(const void* q, const void* k_ext, const void* v_ext, const uint8_t* map,
                              const int32_t* q_offsets, const int32_t* k_offsets, int64_t BH, int64_t S, int64_t D,
                              int64_t QC, int64_t KC, float sm_scale, void* out, const int32_t* out_row_idx, float* lse,
                              void* ear_workspace, int64_t ear_workspace_bytes, void* stream) {
  return sparse_attn_ear_impl(q, k_ext, v_ext, map, q_offsets, k_offsets, BH, S, D, QC, KC, sm_scale, out, out_row_idx, lse,
                              ear_workspace, ear_workspace_bytes, stream, nullptr, nullptr, 0, 0, 0);
}

int svoo_b200_sparse_attn_ear_push(const void* q, const void* k_ext, const void* v_ext, const uint8_t* map,
                                   const int32_t* q_offsets, const int32_t* k_offsets, int64_t BH, int64_t S, int64_t D,
                                   int64_t QC, int64_t KC, float sm_scale, void* const* peer_dst, const int32_t* my_heads,
                                   int32_t world, int64_t n_loc, int64_t H, const int32_t* out_row_idx, void* ear_workspace,
                                   int64_t ear_workspace_bytes, void* stream) {
  if (!my_heads) return SVOO_ERR_NULL;
  SVOO_TRY(check_exchange(peer_dst, world, n_loc, H, D));
  if (BH < 1 || BH > ceil_div64(H, world) || S != n_loc * world) return SVOO_ERR_SHAPE;
  bool seen[128] = {};
  for (int64_t i = 0; i < BH; ++i) {
    if (my_heads[i] < 0 || my_heads[i] >= H || seen[my_heads[i]]) return SVOO_ERR_SHAPE;
    seen[my_heads[i]] = true;
  }
  return sparse_attn_ear_impl(q, k_ext, v_ext, map, q_offsets, k_offsets, BH, S, D, QC, KC, sm_scale, nullptr, out_row_idx,
                              nullptr, ear_workspace, ear_workspace_bytes, stream, peer_dst, my_heads, world, n_loc, (int)H);
}

int svoo_b200_status_offset(int64_t BH, int64_t N, int64_t QC, int64_t KC, int64_t* offset_out) {
  if (!offset_out) return SVOO_ERR_NULL;
  SVOO_TRY(check_tokens(BH, N, kHeadDim));
  SVOO_TRY(check_attn_clusters(QC));
  SVOO_TRY(check_attn_clusters(KC));
  *offset_out = workspace_layout(BH, N, QC, KC).status;
  return SVOO_OK;
}

int svoo_b200_push_heads(const void* x, void* const* peer_dst, const int32_t* owner, const int32_t* slot,
                         int32_t world, int32_t rank, int64_t n_loc, int64_t H, int64_t D, void* stream) {
  if (!x || !owner || !slot) return SVOO_ERR_NULL;
  SVOO_TRY(check_exchange(peer_dst, world, n_loc, H, D));
  if (rank < 0 || rank >= world) return SVOO_ERR_SHAPE;
  if (!aligned16(x)) return SVOO_ERR_ALIGN;
  const int64_t hr = ceil_div64(H, world);
  bool seen[16 * 128] = {};
  for (int64_t h = 0; h < H; ++h) {
    if (owner[h] < 0 || owner[h] >= world || slot[h] < 0 || slot[h] >= hr) return SVOO_ERR_SHAPE;
    bool& s = seen[owner[h] * 128 + slot[h]];
    if (s) return SVOO_ERR_SHAPE;
    s = true;
  }
  SVOO_CUDA(launch_push_heads(x, peer_dst, owner, slot, world, rank, n_loc, (int)H, (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_push_seq(const void* y, void* const* peer_dst, const int32_t* my_heads, int64_t heads_local, int32_t world,
                       int64_t n_loc, int64_t H, int64_t D, void* stream) {
  if (!y || !my_heads) return SVOO_ERR_NULL;
  SVOO_TRY(check_exchange(peer_dst, world, n_loc, H, D));
  if (!aligned16(y)) return SVOO_ERR_ALIGN;
  const int64_t hr = heads_local;
  if (hr < 1 || hr > ceil_div64(H, world)) return SVOO_ERR_SHAPE;
  bool seen[128] = {};
  for (int64_t i = 0; i < hr; ++i) {
    if (my_heads[i] < 0 || my_heads[i] >= H || seen[my_heads[i]]) return SVOO_ERR_SHAPE;
    seen[my_heads[i]] = true;
  }
  SVOO_CUDA(launch_push_seq(y, peer_dst, my_heads, world, n_loc, (int)H, (int)hr, (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_peer_barrier(void* const* peer_flags, int32_t world, int32_t rank, int32_t channel, uint32_t epoch,
                           int32_t* status, void* stream) {
  if (!peer_flags || !status) return SVOO_ERR_NULL;
  if (world < 1 || world > 16 || rank < 0 || rank >= world || channel < 0 || channel >= SVOO_BARRIER_CHANNELS)
    return SVOO_ERR_SHAPE;
  for (int p = 0; p < world; ++p)
    if (!peer_flags[p]) return SVOO_ERR_NULL;
  SVOO_CUDA(launch_peer_barrier(peer_flags, world, rank, channel * 16, epoch, status, (cudaStream_t)stream));
  return SVOO_OK;
}

namespace {
int check_prep(const void* x, const float* weight, const float* cosv, const float* sinv, int64_t S, int64_t H, int64_t D) {
  if (!x) return SVOO_ERR_NULL;
  if ((cosv == nullptr) != (sinv == nullptr)) return SVOO_ERR_NULL;
  if (D != kHeadDim) return SVOO_ERR_HEAD_DIM;
  if (S < 1 || S > ((int64_t)1 << 30) || H < 1 || H > 128) return SVOO_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(cosv) || !aligned16(sinv)) return SVOO_ERR_ALIGN;
  return SVOO_OK;
}
}  // namespace

int svoo_b200_qk_prep(const void* x, const float* weight, float eps, const float* cosv, const float* sinv, int64_t S,
                      int64_t H, int64_t D, void* out, void* stream) {
  SVOO_TRY(check_prep(x, weight, cosv, sinv, S, H, D));
  if (!out) return SVOO_ERR_NULL;
  if (!aligned16(out)) return SVOO_ERR_ALIGN;
  SVOO_CUDA(launch_qk_prep(x, weight, eps, cosv, sinv, S, (int)H, out, nullptr, nullptr, nullptr, 0, 0,
                           (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_qk_prep_heads(const void* x, const float* weight, float eps, const float* cosv, const float* sinv, int64_t S,
                            int64_t H, int64_t D, int64_t rope_rows, void* out, int64_t out_rows, int64_t out_row0,
                            void* stream) {
  SVOO_TRY(check_prep(x, weight, cosv, sinv, S, H, D));
  if (!out) return SVOO_ERR_NULL;
  if (!aligned16(out)) return SVOO_ERR_ALIGN;
  if (rope_rows < 0 || rope_rows > S || out_row0 < 0 || out_rows < out_row0 + S) return SVOO_ERR_SHAPE;
  if (H * out_rows > 2147483647LL) return SVOO_ERR_SHAPE;
  SVOO_CUDA(launch_qk_prep_heads(x, weight, eps, cosv, sinv, S, (int)H, rope_rows, out, out_rows, out_row0,
                                 (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_qk_prep_push(const void* x, const float* weight, float eps, const float* cosv, const float* sinv,
                           void* const* peer_dst, const int32_t* owner, const int32_t* slot, int32_t world, int32_t rank,
                           int64_t n_loc, int64_t H, int64_t D, void* stream) {
  SVOO_TRY(check_prep(x, weight, cosv, sinv, n_loc, H, D));
  if (!owner || !slot) return SVOO_ERR_NULL;
  SVOO_TRY(check_exchange(peer_dst, world, n_loc, H, D));
  if (rank < 0 || rank >= world) return SVOO_ERR_SHAPE;
  const int64_t hr = ceil_div64(H, world);
  bool seen[16 * 128] = {};
  for (int64_t h = 0; h < H; ++h) {
    if (owner[h] < 0 || owner[h] >= world || slot[h] < 0 || slot[h] >= hr) return SVOO_ERR_SHAPE;
    bool& sref = seen[owner[h] * 128 + slot[h]];
    if (sref) return SVOO_ERR_SHAPE;
    sref = true;
  }
  SVOO_CUDA(launch_qk_prep(x, weight, eps, cosv, sinv, n_loc, (int)H, nullptr, peer_dst, owner, slot, world, rank,
                           (cudaStream_t)stream));
  return SVOO_OK;
}

int svoo_b200_append_text_blocks(const uint8_t* map, const int32_t* q_offsets, const int32_t* k_offsets,
                                 const int32_t* q_sorted_idx, const int32_t* k_sorted_idx, int64_t BH, int64_t N, int64_t QC,
                                 int64_t KC, int64_t text, int64_t prompt, uint8_t* map_out, int32_t* q_offsets_out,
                                 int32_t* k_offsets_out, int32_t* q_idx_out, int32_t* k_idx_out, void* stream) {
  if (!map || !q_offsets || !k_offsets || !q_sorted_idx || !k_sorted_idx || !map_out || !q_offsets_out || !k_offsets_out ||
      !q_idx_out || !k_idx_out)
    return SVOO_ERR_NULL;
  if (text < 1 || prompt < 0 || prompt > text) return SVOO_ERR_SHAPE;
  SVOO_TRY(check_tokens(BH, N + text, kHeadDim));
  SVOO_TRY(check_clusters(QC));
  SVOO_TRY(check_clusters(KC));
  SVOO_CUDA(launch_append_text_blocks(map, q_offsets, k_offsets, q_sorted_idx, k_sorted_idx, map_out, q_offsets_out,
                                      k_offsets_out, q_idx_out, k_idx_out, BH, N, QC, KC, text, prompt, (cudaStream_t)stream));
  return SVOO_OK;
}

// --------------------------------------------------------------------------------------------
// The whole layer behind one call: every intermediate lives in a caller-provided scratch block.
// --------------------------------------------------------------------------------------------
namespace {
struct LayerScratch {
  int64_t qp, kp, vp, qlabels, klabels, qsorted, ksorted, qoff, koff, qcent, kcent, qsizes, ksizes, map;
  int64_t map_full, qoff_full, koff_full, qidx_full, kidx_full, total;
};
LayerScratch layer_scratch_layout(int64_t BH, int64_t S, int64_t QC, int64_t KC, int64_t text) {
  LayerScratch l{};
  const int64_t N = S - text;
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    const int64_t at = off;
    off += align_up(bytes, 256);
    return at;
  };
  l.qp = take(BH * S * kRowBytes);
  l.kp = take(BH * S * kRowBytes);
  l.vp = take(BH * S * kRowBytes);
  l.qlabels = take(BH * N * 4);
  l.klabels = take(BH * N * 4);
  l.qsorted = take(BH * N * 4);
  l.ksorted = take(BH * N * 4);
  l.qoff = take(BH * (QC + 1) * 4);
  l.koff = take(BH * (KC + 1) * 4);
  l.qcent = take(BH * QC * kRowBytes);
  l.kcent = take(BH * KC * kRowBytes);
  l.qsizes = take(BH * QC * 4);
  l.ksizes = take(BH * KC * 4);
  l.map = take(BH * QC * KC);
  if (text > 0) {
    l.map_full = take(BH * (QC + 2) * (KC + 2));
    l.qoff_full = take(BH * (QC + 3) * 4);
    l.koff_full = take(BH * (KC + 3) * 4);
    l.qidx_full = take(BH * S * 4);
    l.kidx_full = take(BH * S * 4);
  }
  l.total = off;
  return l;
}
int check_layer_shape(int64_t BH, int64_t S, int64_t QC, int64_t KC, int64_t text, int64_t prompt) {
  SVOO_TRY(check_tokens(BH, S, kHeadDim));
  SVOO_TRY(check_clusters(QC));
  SVOO_TRY(check_clusters(KC));
  if (text < 0 || text >= S || prompt < 0 || prompt > text) return SVOO_ERR_SHAPE;
  return SVOO_OK;
}
}  // namespace

int svoo_b200_layer_scratch_bytes(int64_t BH, int64_t S, int64_t QC, int64_t KC, int64_t text, int64_t* bytes_out) {
  if (!bytes_out) return SVOO_ERR_NULL;
  SVOO_TRY(check_layer_shape(BH, S, QC, KC, text, 0));
  *bytes_out = layer_scratch_layout(BH, S, QC, KC, text).total;
  return SVOO_OK;
}

int svoo_b200_layer(const void* q, const void* k, const void* v, const int32_t* q_init_idx, const int32_t* k_init_idx,
                    int64_t BH, int64_t S, int64_t D, int64_t QC, int64_t KC, int32_t iters, float top_p,
                    const int32_t* preserve_host, const int32_t* cap_host, float sm_scale, int64_t text, int64_t prompt,
                    void* out, void* scratch, int64_t scratch_bytes, void* workspace, int64_t workspace_bytes,
                    void* stream) {
  if (!scratch || !q || !k || !v || !out) return SVOO_ERR_NULL;
  if (D != kHeadDim) return SVOO_ERR_HEAD_DIM;
  SVOO_TRY(check_layer_shape(BH, S, QC, KC, text, prompt));
  if (BH > SVOO_MAX_HEADS) return SVOO_ERR_SHAPE;
  if (!aligned16(scratch) || !aligned16(q) || !aligned16(k)) return SVOO_ERR_ALIGN;
  const LayerScratch l = layer_scratch_layout(BH, S, QC, KC, text);
  if (scratch_bytes < l.total) return SVOO_ERR_WORKSPACE;
  if (text > 0 && workspace_bytes < workspace_layout(BH, S, QC + 2, KC + 2).total) return SVOO_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t N = S - text;
  auto at = [&](int64_t off) { return static_cast<void*>(static_cast<char*>(scratch) + off); };
  int32_t* qsorted = static_cast<int32_t*>(at(l.qsorted));
  int32_t* ksorted = static_cast<int32_t*>(at(l.ksorted));
  int32_t* qoff = static_cast<int32_t*>(at(l.qoff));
  int32_t* koff = static_cast<int32_t*>(at(l.koff));
  const void* qv = q;
  const void* kv = k;
  if (text > 0) {
    // the clustering reads dense [BH, N, 128] video rows: stage them where the permuted Q and K
    // will be written once the clustering is done
    SVOO_CUDA(cudaMemcpy2DAsync(at(l.qp), (size_t)N * kRowBytes, q, (size_t)S * kRowBytes, (size_t)N * kRowBytes, (size_t)BH,
                                cudaMemcpyDeviceToDevice, st));
    SVOO_CUDA(cudaMemcpy2DAsync(at(l.kp), (size_t)N * kRowBytes, k, (size_t)S * kRowBytes, (size_t)N * kRowBytes, (size_t)BH,
                                cudaMemcpyDeviceToDevice, st));
    qv = at(l.qp);
    kv = at(l.kp);
  }
  SVOO_TRY(svoo_b200_cocluster(qv, kv, q_init_idx, k_init_idx, BH, N, D, QC, KC, iters, static_cast<int32_t*>(at(l.qlabels)),
                               static_cast<int32_t*>(at(l.klabels)), at(l.qcent), at(l.kcent),
                               static_cast<int32_t*>(at(l.qsizes)), static_cast<int32_t*>(at(l.ksizes)), qsorted, qoff,
                               ksorted, koff, workspace, workspace_bytes, stream));
  uint8_t* map = static_cast<uint8_t*>(at(l.map));
  if (top_p >= 1.0f) {
    SVOO_CUDA(cudaMemsetAsync(map, 1, (size_t)(BH * QC * KC), st));
  } else {
    SVOO_TRY(svoo_b200_block_map(at(l.qcent), at(l.kcent), static_cast<int32_t*>(at(l.ksizes)), BH, QC, KC, D, top_p,
                                 preserve_host, cap_host, map, stream));
  }
  const int32_t* qidx = qsorted;
  const int32_t* kidx = ksorted;
  int64_t QCa = QC, KCa = KC;
  if (text > 0) {
    SVOO_TRY(svoo_b200_append_text_blocks(map, qoff, koff, qsorted, ksorted, BH, N, QC, KC, text, prompt,
                                          static_cast<uint8_t*>(at(l.map_full)), static_cast<int32_t*>(at(l.qoff_full)),
                                          static_cast<int32_t*>(at(l.koff_full)), static_cast<int32_t*>(at(l.qidx_full)),
                                          static_cast<int32_t*>(at(l.kidx_full)), stream));
    map = static_cast<uint8_t*>(at(l.map_full));
    qoff = static_cast<int32_t*>(at(l.qoff_full));
    koff = static_cast<int32_t*>(at(l.koff_full));
    qidx = static_cast<int32_t*>(at(l.qidx_full));
    kidx = static_cast<int32_t*>(at(l.kidx_full));
    QCa = QC + 2;
    KCa = KC + 2;
  }
  SVOO_TRY(svoo_b200_permute(q, qidx, BH, S, D, S, S, at(l.qp), stream));
  SVOO_TRY(svoo_b200_permute(k, kidx, BH, S, D, S, S, at(l.kp), stream));
  SVOO_TRY(svoo_b200_permute(v, kidx, BH, S, D, S, S, at(l.vp), stream));
  return svoo_b200_sparse_attn(at(l.qp), at(l.kp), at(l.vp), map, qoff, koff, BH, S, D, QCa, KCa, sm_scale, out, qidx,
                               nullptr, workspace, workspace_bytes, stream);
}

}  // extern "C"
