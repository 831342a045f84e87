/*
 * svoo_b200 -- C ABI of the B200 (sm_100a) implementation of SVOO's online
 * sparse-attention path: QK co-clustering, cluster-order permute / inverse
 * permute, cluster-block map, block-sparse attention.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its name ends in `_host`.
 *   - Token tensors are bf16, row-major [BH, N, 128] (BH = batch*heads flattened,
 *     head dim D must be 128).  Labels, indices, sizes, offsets are int32.
 *     bf16 is the only element type: there is no dtype argument, and a caller that
 *     holds fp16 or fp32 activations casts them before the call (the Python front end
 *     does that and casts results back).  BH * N must be below 2^31.
 *   - The library allocates nothing: outputs and the workspace are caller-owned.
 *     `stream` is a cudaStream_t passed as void*; all work is enqueued on it and
 *     no entry point synchronises with the host.
 *   - Return value: 0 on success; < 0 an SVOO_ERR_* argument error detected on the
 *     host before anything is launched; > 0 a cudaError_t from a launch.
 *
 * Each entry point names the reference interface it replaces (paths inside the
 * SVOO project).
 */
#ifndef SVOO_B200_H
#define SVOO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SVOO_B200_VERSION 104

enum {
  SVOO_OK = 0,
  SVOO_ERR_NULL = -1,        /* a required pointer is null                       */
  SVOO_ERR_SHAPE = -2,       /* a size is out of the supported range             */
  SVOO_ERR_HEAD_DIM = -3,    /* D != 128                                         */
  SVOO_ERR_WORKSPACE = -4,   /* workspace too small (see *_workspace_bytes)      */
  SVOO_ERR_ALIGN = -5,       /* a tensor pointer is not 16-byte aligned          */
  SVOO_ERR_CLUSTERS = -6,    /* cluster count above SVOO_MAX_CLUSTERS            */
  SVOO_ERR_STATIC_SCRATCH = -7 /* problem too large for the built-in scratch array */
};

#define SVOO_MAX_CLUSTERS 1024   /* per side; the reference ships QC=256, KC=1024 */
/* Blocks per side that the attention-side entry points accept (svoo_b200_sparse_attn*,
 * svoo_b200_offsets_from_sizes, svoo_b200_workspace_bytes): the clusters plus the two text
 * blocks of a joint-attention layer. */
#define SVOO_MAX_ATTN_CLUSTERS (SVOO_MAX_CLUSTERS + 2)
#define SVOO_MAX_HEADS 256       /* BH limit of svoo_b200_block_map              */
#define SVOO_BARRIER_CHANNELS 4  /* independent flag sets of svoo_b200_peer_barrier */

int svoo_b200_version(void);
const char* svoo_b200_error_string(int code);

/* Number of kernels this library has launched in the calling process so far
 * (instrumentation for benchmarks; no counterpart in the reference). */
int64_t svoo_b200_launch_count(void);

/* Bytes of scratch that svoo_b200_cocluster / svoo_b200_sort_labels /
 * svoo_b200_sparse_attn need for these sizes (one value covers all three). */
int svoo_b200_workspace_bytes(int64_t BH, int64_t N, int64_t QC, int64_t KC, int64_t* bytes_out);

/* Replaces co_cluster_tokens (svoo/co_clustering.py:2402-2451) together with the
 * kernels it drives (profile norm :2088-2144, fused assign :2148-2255, centroid
 * update :181-303, l2norm svoo/kernels/triton/l2norm.py:9-80).  The random initial
 * centroid token indices, which the reference draws inside the call, are inputs.
 * Also returns the stable cluster-order permutation of each side (sorted_idx,
 * offsets[BH,K+1]), which the reference recomputes with torch.argsort in
 * svoo/kernels/triton/permute.py:90.  Centroids are bf16 [BH,K,128].
 * Warm start (no counterpart in the reference, which re-draws the centroids at every call,
 * svoo/models/wan/attention.py:641-647): with q_init_idx == NULL and k_init_idx == NULL the
 * iterations start from the values already in qcentroids / kcentroids, for example the
 * centroids of the previous denoising step. */
int svoo_b200_cocluster(const void* q, const void* k,
                        const int32_t* q_init_idx, const int32_t* k_init_idx,
                        int64_t BH, int64_t N, int64_t D, int64_t QC, int64_t KC, int32_t iters,
                        int32_t* qlabels, int32_t* klabels,
                        void* qcentroids, void* kcentroids,
                        int32_t* qsizes, int32_t* ksizes,
                        int32_t* q_sorted_idx, int32_t* q_offsets,
                        int32_t* k_sorted_idx, int32_t* k_offsets,
                        void* workspace, int64_t workspace_bytes, void* stream);

/* One assignment step of the co-clustering: labels[n] = argmax_j <profile(x_n), P_j>
 * for tokens x against the profile-forming centroids `form` [BH,K,128] and the
 * centroids being assigned `own` [BH,J,128] (svoo/co_clustering.py:2427-2433). */
int svoo_b200_cocluster_assign(const void* x, const void* form_centroids, const void* own_centroids,
                               int64_t BH, int64_t N, int64_t D, int64_t K, int64_t J,
                               int32_t* labels, void* workspace, int64_t workspace_bytes, void* stream);

/* Nearest centroid in Euclidean distance: labels[bh,n] = first argmin_j |x_n - c_j|^2 with the
 * centroid norms taken as in the reference's kernel for bf16 inputs (every c_d^2 rounded to bf16,
 * summed in fp32).  Replaces _euclid_assign_kernel / euclid_assign_triton
 * (svoo/co_clustering.py:335-483), the assignment step of batch_kmeans_Euclid (:502-541); the
 * reference's clamp of negative distances to zero is not applied (it only matters when a token
 * is within rounding error of two distinct centroids).  centroids: bf16 [BH,K,128]. */
int svoo_b200_euclid_assign(const void* x, const void* centroids, int64_t BH, int64_t N, int64_t D, int64_t K,
                            int32_t* labels, void* workspace, int64_t workspace_bytes, void* stream);

/* Stable counting sort of labels in [0,K): sorted_idx[BH,N] and offsets[BH,K+1]
 * (replaces torch.argsort in svoo/kernels/triton/permute.py:90 and torch.sort in
 * svoo/co_clustering.py:274). */
int svoo_b200_sort_labels(const int32_t* labels, int64_t BH, int64_t N, int64_t K,
                          int32_t* sorted_idx, int32_t* offsets,
                          void* workspace, int64_t workspace_bytes, void* stream);

/* svoo_b200_sort_labels without a workspace argument, for callers that are not able to
 * allocate device memory when they call the library (a process whose GPU memory is
 * partitioned once at start-up, a plug-in that only gets raw pointers from its host, a
 * loop that must not hit the synchronisation an allocation implies).  This entry point has
 * no counterpart in the reference.  Same inputs, outputs and results as
 * svoo_b200_sort_labels; its scratch is a 4 MiB array built into the library image, which
 * every GPU that loads the library keeps resident until the process exits.
 *   - Limit: BH * ceil(N / 2048) * K <= 1,048,576, otherwise SVOO_ERR_STATIC_SCRATCH is
 *     returned and nothing is launched (40 heads x 75,600 tokens x 500 clusters fits).
 *   - It calls no allocating routine.  The first call made with a given device current
 *     looks up the array's device address; make that first call outside any stream capture.
 *   - All calls on one GPU share the one array.  It holds whatever the previous call left
 *     (the kernels overwrite every entry they later read, so no clearing is needed), and
 *     two calls that run concurrently on the same GPU -- different streams, or different
 *     host threads -- would overwrite each other's histograms: order them.
 *   - The looked-up address is kept for the life of the process.  cudaDeviceReset() destroys the
 *     context it belongs to, so a process that resets a device must not call this entry point
 *     on that device afterwards. */
int svoo_b200_sort_labels_static(const int32_t* labels, int64_t BH, int64_t N, int64_t K,
                                 int32_t* sorted_idx, int32_t* offsets, void* stream);

/* Mean of the tokens of each cluster (fp32 sums in a fixed order, bf16 result),
 * empty clusters keep `old_centroids` (svoo/co_clustering.py:253-303).  In place
 * update is allowed (new_centroids == old_centroids). */
int svoo_b200_centroid_update(const void* x, const int32_t* sorted_idx, const int32_t* offsets,
                              const void* old_centroids, int64_t BH, int64_t N, int64_t D, int64_t K,
                              void* new_centroids, int32_t* sizes,
                              void* workspace, int64_t workspace_bytes, void* stream);

/* y[bh,s,:] = x[bh,idx[bh,s],:] for s < N  (svoo/kernels/triton/permute.py:10-35,68-102).
 * x_head_rows / y_head_rows are the rows between consecutive heads in x and y (>= N;
 * N for dense [BH,N,128] tensors), so a [BH,N] block of a longer sequence can be
 * permuted in place of the copy in svoo/models/hunyuan10/attention.py:995-997. */
int svoo_b200_permute(const void* x, const int32_t* sorted_idx, int64_t BH, int64_t N, int64_t D,
                      int64_t x_head_rows, int64_t y_head_rows, void* y, void* stream);

/* y[bh,idx[bh,s],:] = x[bh,s,:]  (svoo/kernels/triton/permute.py:39-65,105-130). */
int svoo_b200_inverse_permute(const void* x, const int32_t* sorted_idx, int64_t BH, int64_t N, int64_t D,
                              int64_t x_head_rows, int64_t y_head_rows, void* y, void* stream);

/* Cluster-block map (identify_dynamic_map, svoo/co_clustering.py:556-633, with
 * weighted_softmax :544-553) for bf16 centroids.  preserve_host[h] / cap_host[h]
 * are the per-head floor and cap in numbers of key clusters (cap = KC: no cap);
 * both are HOST arrays of length BH.  map_out is uint8 [BH,QC,KC], 1 = keep. */
int svoo_b200_block_map(const void* qcentroids, const void* kcentroids, const int32_t* ksizes,
                        int64_t BH, int64_t QC, int64_t KC, int64_t D, float top_p,
                        const int32_t* preserve_host, const int32_t* cap_host,
                        uint8_t* map_out, void* stream);

/* Block-sparse attention over cluster-ordered q,k,v [BH,S,128]
 * (dynamic_block_sparse_fwd_flashinfer, svoo/co_clustering.py:1231-1311, whose
 * semantics are those of _dynamic_block_sparse_fwd_kernel :949-1108): query
 * cluster i of head bh attends the key clusters j with map[bh,i,j] != 0; rows
 * without a selected key give 0.  q_offsets [BH,QC+1], k_offsets [BH,KC+1] are
 * the cluster row offsets.  If out_row_idx is not null the result row s is
 * written to row out_row_idx[bh,s] (the inverse permutation fused into the
 * store); otherwise to row s.  QC, KC <= SVOO_MAX_ATTN_CLUSTERS.
 * lse (may be NULL): fp32 [BH,S]; entry [bh,r], r the row the output row is written to, receives
 * log2(sum_j exp(s_j * sm_scale)) over the selected keys -- the base-2 log-sum-exp that FlashInfer
 * returns with return_lse=True and that the reference's error-aware merge consumes
 * (svoo/co_clustering.py:1866-1868, 1998); -inf for a row without keys. */
int svoo_b200_sparse_attn(const void* q, const void* k, const void* v, const uint8_t* map,
                          const int32_t* q_offsets, const int32_t* k_offsets,
                          int64_t BH, int64_t S, int64_t D, int64_t QC, int64_t KC, float sm_scale,
                          void* out, const int32_t* out_row_idx, float* lse,
                          void* workspace, int64_t workspace_bytes, void* stream);

/* Same contract as svoo_b200_sparse_attn, computed by the warp-level-MMA (mma.sync)
 * kernel instead of the tcgen05 one.  Kept as an independent on-device cross-check of
 * the tensor-core kernel at sizes the CPU oracle cannot reach; not used by the layer. */
int svoo_b200_sparse_attn_simt(const void* q, const void* k, const void* v, const uint8_t* map,
                               const int32_t* q_offsets, const int32_t* k_offsets,
                               int64_t BH, int64_t S, int64_t D, int64_t QC, int64_t KC, float sm_scale,
                               void* out, const int32_t* out_row_idx,
                               void* workspace, int64_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * Error-aware routing ("EAR"): the reference's alternative block selection and forward of the
 * Wan processor (svoo/models/wan/attention.py:1047-1076, 1184-1196).  All tensors bf16 and in
 * cluster order; QC, KC <= SVOO_MAX_CLUSTERS.  The four calls share one scratch buffer of
 * svoo_b200_ear_workspace_bytes() bytes, which carries the value statistics from the first call to
 * the second (same stream).
 * ------------------------------------------------------------------------------------------ */

/* Scratch size of the EAR calls; *status_offset_out (optional) = byte offset of the int32 status
 * word that svoo_b200_sparse_attn_ear clears and its kernel sets when a bounded wait expires. */
int svoo_b200_ear_workspace_bytes(int64_t BH, int64_t N, int64_t QC, int64_t KC, int64_t* bytes_out,
                                  int64_t* status_offset_out);

/* Replaces _compute_value_centroids (svoo/models/wan/attention.py:594-610) and
 * _precompute_v_stats_kernel (svoo/co_clustering.py:1314-1395).  v_perm [BH,N,128] in key-cluster
 * order, k_offsets [BH,KC+1].  vcentroids_out [BH,KC,128]: mean value row of every key cluster
 * (fp32 sums, rounded once; zero for an empty cluster).  The per-token |v|^2 and v.vc and the
 * per-cluster |vc|^2 stay in the scratch buffer. */
int svoo_b200_ear_value_centroids(const void* v_perm, const int32_t* k_offsets, int64_t BH, int64_t N, int64_t D,
                                  int64_t QC, int64_t KC, void* vcentroids_out, void* ear_workspace,
                                  int64_t ear_workspace_bytes, void* stream);

/* Replaces the centroid-logit einsum of identify_dynamic_map_estimated (svoo/co_clustering.py:1724)
 * and error_estimation_triton / _error_estimation_kernel (:1398-1689).  After
 * svoo_b200_ear_value_centroids on the same scratch buffer.  c_logits_out, scores_out: fp32
 * [BH,QC,KC]; c_logits = bf16(bf16(qc.kc) D^-0.5); scores = log(max(err,1e-8)) - gamma
 * log(max(|Q_i||K_j|,1e-8)) with err the squared error of replacing the cluster's keys by its
 * centroid. */
int svoo_b200_ear_block_scores(const void* qcentroids, const void* kcentroids, const void* k_perm,
                               const int32_t* q_offsets, const int32_t* k_offsets, int64_t BH, int64_t N, int64_t D,
                               int64_t QC, int64_t KC, float gamma, float* c_logits_out, float* scores_out,
                               void* ear_workspace, int64_t ear_workspace_bytes, void* stream);

/* Replaces the selection of identify_dynamic_map_estimated (svoo/co_clustering.py:1738-1798):
 * budget from the size-weighted centroid softmax and top_p, `preserve_host[h]` guaranteed clusters
 * (max(1, int(ratio*KC)) there, 0 for ratio <= 0), `budget_preserve_host[h]` = max(1, int(ratio*KC*2)),
 * then the highest-score candidates that fit the remaining budget.  Host arrays of BH ints.
 * map_out uint8 [BH,QC,KC].  Bit-reproducible from its inputs (fixed-order fp32 arithmetic, ties by
 * lower cluster index; the reference's torch.sort is unstable). */
int svoo_b200_ear_select_blocks(const float* c_logits, const float* scores, const int32_t* q_offsets,
                                const int32_t* k_offsets, int64_t BH, int64_t QC, int64_t KC, float top_p,
                                const int32_t* preserve_host, const int32_t* budget_preserve_host, uint8_t* map_out,
                                void* stream);

/* Replaces dynamic_block_sparse_prune_fwd_flashinfer + _fused_qc_kernel_opt
 * (svoo/co_clustering.py:1800-2050) in one pass: a query of cluster i attends the key tokens of the
 * clusters map[i] selects and, for every other cluster j, one virtual key (key centroid j, value
 * centroid j, logit bias log(|K_j| + 1e-6)); the softmax runs over the union, which is what the
 * reference's merge of FlashInfer's (output, log-sum-exp) with the centroid part computes.  (The
 * kernel reads all KC centroid rows of the head and masks those of the selected clusters.)
 * k_ext, v_ext: [BH*S + BH*KC, 128] -- the cluster-ordered rows of all heads, then the centroid rows
 * of all heads.  out, out_row_idx, lse as in svoo_b200_sparse_attn. */
int svoo_b200_sparse_attn_ear(const void* q, const void* k_ext, const void* v_ext, const uint8_t* map,
                              const int32_t* q_offsets, const int32_t* k_offsets, int64_t BH, int64_t S, int64_t D,
                              int64_t QC, int64_t KC, float sm_scale, void* out, const int32_t* out_row_idx, float* lse,
                              void* ear_workspace, int64_t ear_workspace_bytes, void* stream);

/* The same with the output rows stored straight into the ranks' sequence shards, as
 * svoo_b200_sparse_attn_push does for the plain kernel (peer_dst, my_heads, world, n_loc, H as there).
 * No counterpart in the reference (its EAR mode runs on one GPU). */
int svoo_b200_sparse_attn_ear_push(const void* q, const void* k_ext, const void* v_ext, const uint8_t* map,
                                   const int32_t* q_offsets, const int32_t* k_offsets, int64_t BH, int64_t S, int64_t D,
                                   int64_t QC, int64_t KC, float sm_scale, void* const* peer_dst, const int32_t* my_heads,
                                   int32_t world, int64_t n_loc, int64_t H, const int32_t* out_row_idx, void* ear_workspace,
                                   int64_t ear_workspace_bytes, void* stream);

/* Byte offset, inside a workspace of these sizes, of a 4-word int32 status block that
 * the tensor-core kernels report into.  Word 0 is cleared by svoo_b200_sparse_attn and
 * becomes non-zero if a CTA of the attention kernel gave up on one of its bounded barrier
 * waits (its output rows are then not written); word 1 is the same for the assignment
 * kernel of svoo_b200_cocluster / svoo_b200_cocluster_assign.  No counterpart in the
 * reference. */
int svoo_b200_status_offset(int64_t BH, int64_t N, int64_t QC, int64_t KC, int64_t* offset_out);

/* Exclusive prefix of cluster sizes [BH,K] -> offsets [BH,K+1]
 * (the torch.cumsum of svoo/co_clustering.py:1147-1148). */
int svoo_b200_offsets_from_sizes(const int32_t* sizes, int64_t BH, int64_t K, int32_t* offsets, void* stream);

/* Text tokens of a joint-attention layer as two extra blocks (dynamic_map_post_processing,
 * svoo/models/hunyuan10/attention.py:999-1019): `text` rows follow the N clustered video rows of
 * every head; the first `prompt` of them form the "prompt" block, the rest the "unused prompt"
 * block.  map [BH,QC,KC] -> map_out [BH,QC+2,KC+2] (prompt queries attend all video and prompt
 * keys, all queries except the unused prompt attend the prompt keys, the unused prompt attends
 * itself); offsets [BH,K+1] -> [BH,K+3]; sorted_idx [BH,N] -> [BH,N+text], identity on the text
 * rows.  0 <= prompt <= text. */
int svoo_b200_append_text_blocks(const uint8_t* map, const int32_t* q_offsets, const int32_t* k_offsets,
                                 const int32_t* q_sorted_idx, const int32_t* k_sorted_idx, int64_t BH, int64_t N,
                                 int64_t QC, int64_t KC, int64_t text, int64_t prompt, uint8_t* map_out,
                                 int32_t* q_offsets_out, int32_t* k_offsets_out, int32_t* q_idx_out, int32_t* k_idx_out,
                                 void* stream);

/* Multi-GPU re-sharding by stores into peer memory.  The reference runs on one GPU (its
 * processors, svoo/models/wan/attention.py:153-260, receive all heads of the whole sequence);
 * these entry points have no counterpart there.  They move [*,128] bf16 rows between the "sequence
 * shard" layout of a sequence-parallel caller ([n_loc, H, 128] per rank, N = world *
 * n_loc tokens) and the "head shard" layout the path computes in ([H / world, N, 128]
 * per rank), over NVLink, with no wait on another GPU inside the kernels.
 *
 * peer_dst: HOST array of `world` device pointers, entry p = rank p's destination
 * array, mapped into this process (CUDA IPC / symmetric memory).  The caller orders the
 * launches against the other ranks: a stream-ordered collective after the call before a
 * destination is read, and before a destination is overwritten again.
 *   - world in [1,16], H in [world,128], n_loc >= 1.  A rank owns at most hr = ceil(H / world)
 *     heads (12 heads on 8 ranks: four ranks own two, four own one); every receive array has
 *     room for hr heads.
 *
 * svoo_b200_push_heads: x = this rank's [n_loc, H, 128]; row (r, h) is stored into rank
 *   owner[h] at [slot[h], rank * n_loc + r, :] of its [hr, N, 128] array.
 *   owner/slot: HOST int32 [H]; every (owner, slot) pair must be distinct, slot < hr.
 * svoo_b200_push_seq: y = this rank's [heads_local, N, 128]; row (i, n) is stored into rank
 *   n / n_loc at [n % n_loc, my_heads[i], :] of its [n_loc, H, 128] array.
 *   my_heads: HOST int32 [heads_local], distinct, in [0, H); 1 <= heads_local <= hr. */
/* svoo_b200_sparse_attn with the head -> sequence re-shard fused into its store: output row
 * n of local head i (after out_row_idx, if given) is written by the attention kernel straight
 * into rank n / n_loc at [n % n_loc, my_heads[i], :] of that rank's [n_loc, H, 128] array
 * (peer_dst as for svoo_b200_push_seq).  BH is this rank's head count (1 <= BH <= ceil(H / world))
 * and S must equal world * n_loc.  The caller fences as after svoo_b200_push_seq.  No counterpart in the
 * reference. */
int svoo_b200_sparse_attn_push(const void* q, const void* k, const void* v, const uint8_t* map,
                               const int32_t* q_offsets, const int32_t* k_offsets, int64_t BH, int64_t S, int64_t D,
                               int64_t QC, int64_t KC, float sm_scale, void* const* peer_dst, const int32_t* my_heads,
                               int32_t world, int64_t n_loc, int64_t H, const int32_t* out_row_idx, void* workspace,
                               int64_t workspace_bytes, void* stream);
int svoo_b200_push_heads(const void* x, void* const* peer_dst, const int32_t* owner, const int32_t* slot,
                         int32_t world, int32_t rank, int64_t n_loc, int64_t H, int64_t D, void* stream);
int svoo_b200_push_seq(const void* y, void* const* peer_dst, const int32_t* my_heads, int64_t heads_local, int32_t world,
                       int64_t n_loc, int64_t H, int64_t D, void* stream);

/* The whole layer in one call, for hosts that bind only one entry point: co-clustering
 * (svoo_b200_cocluster), cluster-block map (svoo_b200_block_map; top_p >= 1 gives the all-ones
 * map, svoo/co_clustering.py:575-576), cluster-order gathers of Q, K, V and the block-sparse
 * attention with the inverse permutation fused into its store -- the sparse branch of
 * attention_core_logic, svoo/models/wan/attention.py:1110-1216, and, with text > 0, of the joint
 * attention of svoo/models/hunyuan10/attention.py:1031-1110 (the last `text` rows of every head
 * are text tokens: never clustered, appended as the two blocks of svoo_b200_append_text_blocks).
 * q, k, v, out: [BH, S, D] bf16 in the original token order, S = video tokens + text; init
 * indices (into the video tokens) and the per-head preserve / cap arrays as in the calls it
 * wraps.  Every intermediate lives in `scratch` (svoo_b200_layer_scratch_bytes) and stays valid
 * after the call: permuted Q/K/V [BH,S,D], labels, permutations, offsets, centroids, sizes, map,
 * then (text > 0 only) the padded map, offsets and row indices, each 256-byte aligned.  The
 * workspace must cover svoo_b200_workspace_bytes(BH, S, QC + 2, KC + 2) when text > 0. */
int svoo_b200_layer_scratch_bytes(int64_t BH, int64_t S, int64_t QC, int64_t KC, int64_t text, int64_t* bytes_out);
int svoo_b200_layer(const void* q, const void* k, const void* v, const int32_t* q_init_idx, const int32_t* k_init_idx,
                    int64_t BH, int64_t S, int64_t D, int64_t QC, int64_t KC, int32_t iters, float top_p,
                    const int32_t* preserve_host, const int32_t* cap_host, float sm_scale, int64_t text, int64_t prompt,
                    void* out, void* scratch, int64_t scratch_bytes, void* workspace, int64_t workspace_bytes,
                    void* stream);

/* The producer of the path's Q and K (and V), one pass over the projection output:
 *   y = bf16(x * rstd * weight), rstd = 1 / sqrt(mean_row(x^2) + eps)      if weight != NULL
 *       (triton_rmsnorm_forward, svoo/kernels/triton/rmsnorm.py:9-46, called from
 *        get_qk_norm, svoo/models/wan/attention.py:112-125; the norm runs over all H*D columns)
 *   out[2i]   = y[2i] cos[2i] - y[2i+1] sin[2i+1]                          if cos != NULL
 *   out[2i+1] = y[2i] sin[2i+1] + y[2i+1] cos[2i]       (apply_rotary_emb, attention.py:179-190)
 *   result stored as [H, S, D]                 (transpose(1, 2).contiguous(), attention.py:127-131)
 * x: [S, H*D] bf16; weight: [H*D] fp32; cos, sin: [S, D] fp32 (the full-width tables the
 * caller's rotary module produces; even entries of cos and odd entries of sin are used).
 * With weight == NULL and cos == NULL it is the plain head transpose (V).  H <= 128. */
int svoo_b200_qk_prep(const void* x, const float* weight, float eps, const float* cos, const float* sin, int64_t S,
                      int64_t H, int64_t D, void* out, void* stream);
/* The per-head producer of HunyuanVideo's blocks, one pass: RMS norm over the D values of every
 * (token, head) with weight [D] (fp32), y = bf16((x * rsqrt(mean(x^2) + eps)) * w)
 * (rmsnorm_narrow_n_subwarp_reduction, svoo/kernels/include/norm/narrow_rms_norm.cuh:22-74, called from
 * apply_qk_norm, svoo/models/hunyuan10/attention.py:262-270); interleaved-pair rotation of the first
 * `rope_rows` tokens, out[i] = bf16(y[i] cos[i] + (i even ? -y[i+1] : y[i-1]) sin[i]) with cos, sin
 * [rope_rows, D] fp32 (ApplyQKRotaryCosSinTXTLASTCacheInPlace, svoo/kernels/include/rope/rope_enc_txtlast.cuh:34-110:
 * the text tokens at the end of the sequence are not rotated); head transpose
 * (get_transpose_qkv, hunyuan10/attention.py:471-476).  x: [S, H*D] bf16; row s of head h is stored at
 * out[h][out_row0 + s] of an [H, out_rows, D] array, so the video and the text tokens of a
 * double-stream block (separate projections) can be placed in one sequence.  weight == NULL / cos ==
 * NULL skip that part. */
int svoo_b200_qk_prep_heads(const void* x, const float* weight, float eps, const float* cos, const float* sin, int64_t S,
                            int64_t H, int64_t D, int64_t rope_rows, void* out, int64_t out_rows, int64_t out_row0,
                            void* stream);
/* The same for a sequence-parallel caller: x is this rank's [n_loc, H*D] rows (cos, sin
 * [n_loc, D]) and every head's row is stored straight into the rank that owns the head, at
 * [slot[h], rank * n_loc + r, :] of its [ceil(H/world), N, D] array -- svoo_b200_push_heads fused
 * into the producer (peer_dst, owner, slot as there).  No counterpart in the reference. */
int svoo_b200_qk_prep_push(const void* x, const float* weight, float eps, const float* cos, const float* sin,
                           void* const* peer_dst, const int32_t* owner, const int32_t* slot, int32_t world, int32_t rank,
                           int64_t n_loc, int64_t H, int64_t D, void* stream);

/* Barrier over the ranks of one node, as a kernel on `stream`: publishes this rank's earlier
 * peer stores on that stream and waits (at most ~2 s) for the same call of every other rank.
 * peer_flags: HOST array of `world` device pointers, entry p = rank p's flag array of
 * SVOO_BARRIER_CHANNELS * 16 uint32 words (zeroed before the first call, mapped into every
 * process).  `epoch` must grow by one per call and be the same on all ranks for the same
 * call; calls that may overlap in time (different streams) use different channels.  *status
 * (device int32) is set to 1 if a rank did not arrive in time.  Every rank runs its call on
 * its own GPU.  No counterpart in the reference (one GPU). */
int svoo_b200_peer_barrier(void* const* peer_flags, int32_t world, int32_t rank, int32_t channel, uint32_t epoch,
                           int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SVOO_B200_H */
