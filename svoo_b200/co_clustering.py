"""The reference's operator interface for the sparse-attention path, on the B200 kernels.

Same names, argument meaning and error behaviour as svoo/co_clustering.py of the
reference: co_cluster_tokens (:2402), identify_dynamic_map (:556),
dynamic_block_sparse_fwd_flashinfer (:1231) / dynamic_block_sparse_fwd_triton (:1111).
Inputs other than bf16 are computed in bf16 and returned in the input dtype.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple, Union

import torch

from . import ops

Ratio = Union[float, int, Sequence[float], torch.Tensor, None]


def _as_bf16(x: torch.Tensor) -> torch.Tensor:
    return x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)


def draw_init_indices(BH: int, N: int, num_q: int, num_k: int, device, generator=None):
    """Initial centroid token indices in the reference's draw order: q first, then k
    (svoo/co_clustering.py:2417-2421)."""
    q_idx = torch.randint(0, N, (BH, num_q), device=device, generator=generator)
    k_idx = torch.randint(0, N, (BH, num_k), device=device, generator=generator)
    return q_idx, k_idx


def co_cluster(q_flat: torch.Tensor, k_flat: torch.Tensor, num_q_centroids: int, num_k_centroids: int,
               max_iters: int = 10, *, init_indices=None, generator=None, init_centroids=None) -> ops.Clustering:
    """co_cluster_tokens returning the full device-side result (labels, centroids, sizes and
    the stable cluster-order permutations), everything int32 / bf16.  `init_centroids` =
    (q centroids, k centroids) starts from those instead of drawing tokens (warm start; the
    reference always draws, svoo/models/wan/attention.py:641-647)."""
    assert q_flat.is_cuda and k_flat.is_cuda, "tensors must be on CUDA"
    BH, N, D = q_flat.shape
    if init_centroids is not None:
        qc0, kc0 = init_centroids
        return ops.cocluster(_as_bf16(q_flat).contiguous(), _as_bf16(k_flat).contiguous(), None, None, max_iters,
                             init_centroids=(_as_bf16(qc0).contiguous(), _as_bf16(kc0).contiguous()))
    if init_indices is None:
        init_indices = draw_init_indices(BH, N, num_q_centroids, num_k_centroids, q_flat.device, generator)
    q_idx, k_idx = init_indices
    assert q_idx.shape == (BH, num_q_centroids) and k_idx.shape == (BH, num_k_centroids)
    return ops.cocluster(_as_bf16(q_flat).contiguous(), _as_bf16(k_flat).contiguous(),
                         q_idx.to(q_flat.device), k_idx.to(q_flat.device), max_iters)


def co_cluster_tokens(q_flat, k_flat, num_q_centroids, num_k_centroids, max_iters=10, *, init_indices=None,
                      generator=None):
    """Drop-in for the reference's co_cluster_tokens: returns
    (qlabels int64, qcentroids, q_cluster_sizes int32, klabels int64, kcentroids, k_cluster_sizes int32)."""
    c = co_cluster(q_flat, k_flat, num_q_centroids, num_k_centroids, max_iters, init_indices=init_indices,
                   generator=generator)
    dt = q_flat.dtype
    return (c.qlabels.long(), c.qcentroids.to(dt), c.qsizes, c.klabels.long(), c.kcentroids.to(dt), c.ksizes)


def euclid_assign_triton(x: torch.Tensor, centroids: torch.Tensor, x_sq: Optional[torch.Tensor] = None,
                         out: Optional[torch.Tensor] = None, **_tile_sizes) -> torch.Tensor:
    """Nearest-centroid labels [B, N] int64 (svoo/co_clustering.py:420-483).  `x_sq` (the token
    norms) does not change the argmin and is ignored; tile-size keywords are accepted and unused."""
    assert x.is_cuda and centroids.is_cuda, "All tensors must be on CUDA"
    assert centroids.dtype == x.dtype, "centroids dtype mismatch"
    B, N, D = x.shape
    assert centroids.shape == (B, centroids.shape[1], D), "centroids shape mismatch"
    lab = ops.euclid_assign(_as_bf16(x).contiguous(), _as_bf16(centroids).contiguous()).long()
    if out is not None:
        out.copy_(lab)
        return out
    return lab


def batch_kmeans_Euclid(x, n_clusters, max_iters=100, tol=1e-4, init_centroids=None, verbose=False, *,
                        init_indices=None, generator=None):
    """Batched Euclidean k-means with the reference's loop (svoo/co_clustering.py:502-541):
    assign, centroid update, stop when the largest centroid shift is below `tol` (one host read
    per iteration, as there).  Returns (cluster_ids int64 [B,N], centroids [B,K,D],
    cluster_sizes int32 [B,K], iterations run).  As in the reference the returned centroids
    are the ones the last assignment used when the loop stops on `tol`, else the updated ones."""
    assert x.is_cuda, "tensors must be on CUDA"
    B, N, D = x.shape
    xb = _as_bf16(x).contiguous()
    if init_centroids is None:
        if init_indices is None:
            init_indices = torch.randint(0, N, (B, n_clusters), device=x.device, generator=generator)
        centroids = torch.gather(xb, 1, init_indices.to(x.device)[..., None].expand(-1, -1, D))
    else:
        centroids = _as_bf16(init_centroids)
    centroids = centroids.reshape(B, n_clusters, D).contiguous()
    cluster_ids = cluster_sizes = None
    it = -1
    for it in range(max_iters):
        labels = ops.euclid_assign(xb, centroids)
        idx, off = ops.sort_labels(labels, n_clusters)
        new, cluster_sizes = ops.centroid_update(xb, idx, off, centroids)
        cluster_ids = labels
        shift = (new.float() - centroids.float()).norm(dim=-1).max()
        if verbose:
            print(f"Iter {it}, center shift: {shift.item():.6f}")
        if shift < tol:
            break
        centroids = new
    return cluster_ids.long(), centroids.to(x.dtype), cluster_sizes, it + 1


def _ratio_values(r: Ratio, H: int):
    if r is None:
        return None, "none"
    if isinstance(r, (list, tuple)) or (hasattr(r, "__len__") and len(r) == H):
        # like the reference: through a float32 tensor, then python floats
        return [float(v) for v in torch.as_tensor(r, dtype=torch.float32).tolist()], "list"
    if isinstance(r, (int, float)):
        return float(r), "scalar"
    return None, "none"


def keep_limits(kc_num: int, H: int, min_kc_ratio: Ratio, max_kc_ratio: Ratio):
    """Per-head (floor, cap) in numbers of key clusters, with the reference's int() truncation
    and list/scalar dispatch (svoo/co_clustering.py:589-627).  cap == kc_num means no cap."""
    mn, mn_kind = _ratio_values(min_kc_ratio, H)
    mx, mx_kind = _ratio_values(max_kc_ratio, H)
    preserve = [0] * H
    if mn_kind == "list":
        preserve = [int(v * kc_num) if v > 0 else 0 for v in mn]
    elif mn_kind == "scalar" and mn > 0:
        preserve = [int(mn * kc_num)] * H
    cap = [kc_num] * H
    if mx_kind == "list":
        for h in range(H):
            if mx[h] > 0:
                c = max(1, int(mx[h] * kc_num))
                if mn_kind == "list":
                    c = max(c, int(mn[h] * kc_num))
                cap[h] = c
    elif mx_kind == "scalar" and mx > 0:
        c0 = max(1, int(mx * kc_num))
        for h in range(H):
            c = c0
            if mn_kind == "list":
                if mn[h] > 0:
                    c = max(c, int(mn[h] * kc_num))
                c = max(1, c)
            elif mn_kind == "scalar" and mn > 0:
                c = max(c, int(mn * kc_num))
            cap[h] = c
    return [min(p, kc_num) for p in preserve], [min(c, kc_num) for c in cap]


def identify_dynamic_map(query_centroids, key_centroids, q_cluster_sizes, k_cluster_sizes, p, min_kc_ratio=0,
                         max_kc_ratio=0):
    """Bool map [B, H, QC, KC] of the key clusters each query cluster keeps
    (svoo/co_clustering.py:556-633).  No host synchronisation."""
    B, H, qc_num, D = query_centroids.shape
    kc_num = key_centroids.shape[2]
    if p >= 1.0:
        return torch.ones(B, H, qc_num, kc_num, dtype=torch.bool, device=query_centroids.device)
    preserve, cap = keep_limits(kc_num, H, min_kc_ratio, max_kc_ratio)
    m = ops.block_map(_as_bf16(query_centroids).reshape(B * H, qc_num, D).contiguous(),
                      _as_bf16(key_centroids).reshape(B * H, kc_num, D).contiguous(),
                      k_cluster_sizes.reshape(B * H, kc_num), float(p), preserve * B, cap * B)
    return m.view(B, H, qc_num, kc_num).view(torch.bool)


def dynamic_block_sparse_fwd(q, k, v, block_mask_map, block_row_sz, block_col_sz, sm_scale=None,
                             out_row_idx=None):
    """Block-sparse attention over cluster-ordered q,k,v [B,H,S,D]; returns [B,H,S,D]."""
    B, H, S, D = q.shape
    qc_num = block_row_sz.shape[-1]
    kc_num = block_col_sz.shape[-1]
    assert block_mask_map.shape == (B, H, qc_num, kc_num)
    assert q.is_cuda and k.is_cuda and v.is_cuda, "Inputs must be CUDA tensors"
    assert q.dtype == k.dtype == v.dtype, "Input dtypes must match"
    dev = q.device
    q_off = ops.offsets_from_sizes(block_row_sz.reshape(B * H, qc_num).to(dev))
    k_off = ops.offsets_from_sizes(block_col_sz.reshape(B * H, kc_num).to(dev))
    m = block_mask_map.to(dev).reshape(B * H, qc_num, kc_num).contiguous()
    m = m.view(torch.uint8) if m.dtype == torch.bool else m.to(torch.uint8)
    o = ops.sparse_attn(_as_bf16(q).reshape(B * H, S, D).contiguous(), _as_bf16(k).reshape(B * H, S, D).contiguous(),
                        _as_bf16(v).reshape(B * H, S, D).contiguous(), m, q_off, k_off, sm_scale,
                        None if out_row_idx is None else out_row_idx.reshape(B * H, S).contiguous())
    return o.view(B, H, S, D).to(q.dtype)


def dynamic_block_sparse_fwd_flashinfer(q, k, v, block_mask_map, block_row_sz, block_col_sz, is_cpu: bool = True):
    """Name and signature of the reference's default backend (svoo/co_clustering.py:1231-1239).
    `is_cpu` only says where the map and sizes live; they are moved to the device either way."""
    return dynamic_block_sparse_fwd(q, k, v, block_mask_map, block_row_sz, block_col_sz)


def dynamic_block_sparse_fwd_triton(q, k, v, dynamic_map, qc_size, kc_size):
    """Name and signature of the reference's alternative backend (svoo/co_clustering.py:1111)."""
    return dynamic_block_sparse_fwd(q, k, v, dynamic_map, qc_size, kc_size)


# ----------------------------------------------------------------------------------------------
# Error-aware routing (EAR): names and signatures of svoo/co_clustering.py:1570-2050
# ----------------------------------------------------------------------------------------------
def ear_limits(kc_num: int, H: int, min_kc_ratio: Ratio):
    """Per-head (guaranteed, budget-preserved) numbers of key clusters of identify_dynamic_map_estimated:
    max(1, int(r * KC)) and max(1, int(r * KC * 2)) for a positive ratio r, else 0, with the reference's
    list / one-element / scalar dispatch (svoo/co_clustering.py:1748-1774)."""
    vals = [0.0] * H
    if isinstance(min_kc_ratio, torch.Tensor):
        if min_kc_ratio.numel() == H:
            vals = [float(v) for v in min_kc_ratio.to(dtype=torch.float32).flatten().tolist()]
        elif min_kc_ratio.numel() == 1:
            vals = [float(min_kc_ratio.item())] * H
    elif isinstance(min_kc_ratio, (list, tuple)):
        if len(min_kc_ratio) == H:
            vals = [float(v) for v in torch.tensor(min_kc_ratio, dtype=torch.float32).tolist()]
        elif len(min_kc_ratio) == 1:
            vals = [float(min_kc_ratio[0])] * H
    elif isinstance(min_kc_ratio, (int, float)):
        vals = [float(min_kc_ratio)] * H
    preserve = [min(kc_num, max(1, int(r * kc_num))) if r > 0 else 0 for r in vals]
    budget = [min(kc_num, max(1, int(r * kc_num * 2))) if r > 0 else 0 for r in vals]
    return preserve, budget


def _offsets(sizes: torch.Tensor, device) -> torch.Tensor:
    B, H, K = sizes.shape
    return ops.offsets_from_sizes(sizes.reshape(B * H, K).to(device))


def compute_value_centroids(v_perm: torch.Tensor, k_cluster_sizes: torch.Tensor) -> torch.Tensor:
    """Mean value row of every key cluster from the cluster-ordered values [B,H,S,D]: what the Wan
    processor's _compute_value_centroids (svoo/models/wan/attention.py:594-610) yields from the
    unpermuted values and the labels.  Returns bf16 [B,H,KC,D]."""
    B, H, S, D = v_perm.shape
    KC = k_cluster_sizes.shape[-1]
    vc = ops.ear_value_centroids(_as_bf16(v_perm).reshape(B * H, S, D).contiguous(), _offsets(k_cluster_sizes, v_perm.device), 1)
    return vc.view(B, H, KC, D)


def _ear_scores(query_centroids, key_centroids, permuted_K, permuted_V, qc_sz, kc_sz, gamma):
    B, H, qc_num, D = query_centroids.shape
    kc_num = key_centroids.shape[2]
    S = permuted_K.shape[2]
    dev = permuted_K.device
    q_off, k_off = _offsets(qc_sz, dev), _offsets(kc_sz, dev)
    ops.ear_value_centroids(_as_bf16(permuted_V).reshape(B * H, S, D).contiguous(), k_off, qc_num)
    clog, sc = ops.ear_block_scores(_as_bf16(query_centroids).reshape(B * H, qc_num, D),
                                    _as_bf16(key_centroids).reshape(B * H, kc_num, D),
                                    _as_bf16(permuted_K).reshape(B * H, S, D).contiguous(), q_off, k_off, gamma)
    return clog, sc, q_off, k_off


def error_estimation_triton(query_centroids, key_centroids, value_centroids, permuted_K, permuted_V, qc_sz, kc_sz,
                            c_logits=None, gamma: float = 1.0, eps: float = 1e-8, BLOCK_SIZE_Q: int = 64,
                            BLOCK_SIZE_K: int = 32):
    """Log-efficiency score of every (query cluster, key cluster) pair, fp32 [B,H,QC,KC]
    (svoo/co_clustering.py:1570-1689).  The value centroids and the centroid logits are recomputed by the
    kernels (as the key-cluster means of permuted_V and bf16(bf16(qc.kc) D^-0.5)); `value_centroids`,
    `c_logits`, `eps` (1e-8) and the block sizes are accepted for signature compatibility."""
    B, H, qc_num, _ = query_centroids.shape
    _, sc, _, _ = _ear_scores(query_centroids, key_centroids, permuted_K, permuted_V, qc_sz, kc_sz, gamma)
    return sc.view(B, H, qc_num, -1)


def identify_dynamic_map_estimated(q_perm, k_perm, v_perm, qc_sz, kc_sz, qcentroids, kcentroids, vcentroids, top_p=0.9,
                                   gamma=1.0, min_kc_ratio=0.0):
    """Bool map [B,H,QC,KC] under the error-aware budget (svoo/co_clustering.py:1691-1798): per-block
    error estimate, budget from the size-weighted centroid softmax and top_p, guaranteed minimum
    coverage, then the highest-score blocks that fit.  No host synchronisation."""
    B, H, qc_num, D = qcentroids.shape
    kc_num = kcentroids.shape[2]
    clog, sc, q_off, k_off = _ear_scores(qcentroids, kcentroids, k_perm, v_perm, qc_sz, kc_sz, gamma)
    preserve, budget = ear_limits(kc_num, H, min_kc_ratio)
    m = ops.ear_select_blocks(clog, sc, q_off, k_off, float(top_p), preserve * B, budget * B)
    return m.view(B, H, qc_num, kc_num).view(torch.bool)


def dynamic_block_sparse_prune_fwd_flashinfer(q, k, v, k_centroids, v_centroids, block_mask_map, block_row_sz, block_col_sz,
                                              is_cpu: bool = True, out_row_idx=None):
    """EAR forward over cluster-ordered q,k,v [B,H,S,D] (svoo/co_clustering.py:1924-2050): selected blocks
    at token granularity, every other key cluster through its centroids.  One kernel pass; this wrapper
    concatenates the token and centroid rows into the layout the kernel reads (the layer path writes
    them there directly)."""
    B, H, S, D = q.shape
    qc_num, kc_num = block_row_sz.shape[-1], block_col_sz.shape[-1]
    assert block_mask_map.shape == (B, H, qc_num, kc_num)
    assert k_centroids.shape == (B, H, kc_num, D) and v_centroids.shape == (B, H, kc_num, D)
    dev = q.device
    q_off, k_off = _offsets(block_row_sz, dev), _offsets(block_col_sz, dev)
    m = block_mask_map.to(dev).reshape(B * H, qc_num, kc_num).contiguous()
    m = m.view(torch.uint8) if m.dtype == torch.bool else m.to(torch.uint8)
    k_ext = torch.cat([_as_bf16(k).reshape(-1, D), _as_bf16(k_centroids).reshape(-1, D)])
    v_ext = torch.cat([_as_bf16(v).reshape(-1, D), _as_bf16(v_centroids).reshape(-1, D)])
    o = ops.sparse_attn_ear(_as_bf16(q).reshape(B * H, S, D).contiguous(), k_ext, v_ext, m, q_off, k_off,
                            out_row_idx=None if out_row_idx is None else out_row_idx.reshape(B * H, S).contiguous())
    return o.view(B, H, S, D).to(q.dtype)

