"""CPU oracle for SVOO's online sparse-attention path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain torch-CPU / numpy arithmetic, the algorithm of the
reference's hot path so the CUDA kernels can be checked against it.  Nothing in
the product package imports it; only the test-suite, the smoke check and the
benchmark's CPU-baseline leg do.

Parity status: PINNED.  Every function below is checked (tests/test_oracle_golden.py)
against outputs of the reference's own functions, executed unmodified on CPU
(Triton kernels under the Triton interpreter) by tests/golden/make_golden.py and
committed as fixtures under tests/golden/.  One exception, parity unpinned: qk_prep_heads
restates two CUDA kernels of the reference, which cannot be executed without a GPU.

Reference locations restated here (paths inside the reference project):
  * co_cluster_tokens                 svoo/co_clustering.py:2402-2451
  * profile row norm                  svoo/co_clustering.py:2088-2144
  * fused profile-space assign        svoo/co_clustering.py:2148-2255
  * centroid update                   svoo/co_clustering.py:181-303
  * row l2norm                        svoo/kernels/triton/l2norm.py:9-80
  * permute / inverse permute         svoo/kernels/triton/permute.py:10-130
  * weighted_softmax / dynamic map    svoo/co_clustering.py:544-633
  * block-sparse attention semantics  svoo/co_clustering.py:949-1108
  * Hunyuan text-block post-process   svoo/models/hunyuan10/attention.py:977-1021
  * producer of Q, K, V (RMS norm, rotary embedding, head transpose)
                                      svoo/kernels/triton/rmsnorm.py:9-46,
                                      svoo/models/wan/attention.py:112-131,177-195
  * HunyuanVideo's producer (per-head RMS norm, text-last rotary embedding; restated from CUDA
    source, not pinned)               svoo/kernels/include/norm/narrow_rms_norm.cuh:22-74,
                                      svoo/kernels/include/rope/rope_enc.cuh:17-36
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple, Union

import numpy as np
import torch

Ratio = Union[float, int, Sequence[float], torch.Tensor, None]


# --------------------------------------------------------------------------------------
# Producer of the path's inputs
# --------------------------------------------------------------------------------------
def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, truncate: bool = False) -> torch.Tensor:
    """y = (x * rstd * w) in fp32, rounded to x's dtype; rstd = 1 / sqrt(mean(x^2) + eps) over the
    last dimension (svoo/kernels/triton/rmsnorm.py:32-42).  `truncate`: drop the low 16 bits
    instead of rounding to nearest even -- what the Triton *interpreter* does for an in-kernel
    fp32 -> bf16 cast (on a GPU the cast rounds to nearest even); only used to compare with
    fixtures that were produced under the interpreter."""
    xf = x.float()
    var = (xf * xf).sum(-1, keepdim=True) / x.shape[-1]
    rstd = 1.0 / torch.sqrt(var + eps)
    y = xf * rstd * weight.float()
    if truncate and x.dtype == torch.bfloat16:
        return (y.view(torch.int32) & -65536).view(torch.float32).to(x.dtype)
    return y.to(x.dtype)


def rotary_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B,S,H,D]; cos, sin broadcastable [.,S,1,D]: pairs (2i, 2i+1) rotated with cos[2i], sin[2i+1]
    (svoo/models/wan/attention.py:179-190); fp32 arithmetic, result in x's dtype."""
    x1, x2 = x.unflatten(-1, (-1, 2)).unbind(-1)
    c, s_ = cos[..., 0::2], sin[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = x1 * c - x2 * s_
    out[..., 1::2] = x1 * s_ + x2 * c
    return out


def qk_prep(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
            sin: Optional[torch.Tensor], heads: int, truncate_norm: bool = False) -> torch.Tensor:
    """x [B,S,H*D] -> [B,H,S,D]: norm over all H*D columns, rotary embedding, head transpose
    (svoo/models/wan/attention.py:112-131,173-195)."""
    y = x if weight is None else rmsnorm_rows(x, weight, eps, truncate_norm)
    y = y.unflatten(2, (heads, -1))
    if cos is not None:
        y = rotary_interleaved(y, cos, sin)
    return y.transpose(1, 2).contiguous()


# --------------------------------------------------------------------------------------
# co-clustering
# --------------------------------------------------------------------------------------

def qk_prep_heads(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
                  sin: Optional[torch.Tensor], rope_rows: int, heads: int) -> torch.Tensor:
    """HunyuanVideo's producer, [S, H*128] -> [H, S, 128], as the reference's own CUDA kernels compute it
    (restated from their source; they cannot run without a GPU, so this function is not pinned by a
    fixture): y = dtype((x * rsqrt(sum(x^2)/128 + eps)) * w) per (token, head)
    (svoo/kernels/include/norm/narrow_rms_norm.cuh:22-74); for the first `rope_rows` tokens
    out[i] = dtype(y[i] cos[i] + (i even ? -y[i+1] : y[i-1]) sin[i]) (svoo/kernels/include/rope/rope_enc.cuh:17-36,
    rope_enc_txtlast.cuh:34-78); head transpose.  fp32 arithmetic."""
    S = x.shape[0]
    y = x.view(S, heads, 128).float()
    if weight is not None:
        rstd = torch.rsqrt((y * y).sum(-1, keepdim=True) / 128.0 + eps)
        y = ((y * rstd) * weight.float()).to(x.dtype).float()
    if cos is not None and rope_rows > 0:
        c, sn = cos.float()[:rope_rows, None], sin.float()[:rope_rows, None]
        v = y[:rope_rows]
        rot = torch.stack([-v[..., 1::2], v[..., 0::2]], -1).flatten(-2)
        y = torch.cat([(v * c + rot * sn).to(x.dtype).float(), y[rope_rows:]], 0)
    return y.to(x.dtype).transpose(0, 1).contiguous()


def l2norm_rows(x: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    """x / sqrt(sum(x^2) + eps) along the last dim, fp32 out (l2norm.py:36-41)."""
    x = x.float()
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def profile_norm(x: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """norm[b,n] = sqrt(sum_k (x[b,n]·c[b,k])^2 + 1e-8) (co_clustering.py:2123-2142)."""
    dot = torch.matmul(x.float(), c.float().transpose(-1, -2))
    return torch.sqrt((dot * dot).sum(-1) + 1e-8)


def round_tf32(t: torch.Tensor) -> torch.Tensor:
    """fp32 -> TF32 (10 mantissa bits, round to nearest, ties away from zero) -> fp32: what a
    tensor-core dot with allow_tf32=True does to its fp32 operands on a GPU."""
    bits = t.float().contiguous().view(torch.int32)
    return ((bits + 0x1000) & -0x2000).view(torch.float32)


def cocluster_assign(x, c, pc, norms, tf32: bool = False) -> torch.Tensor:
    """label = first argmin_j 2 - 2*<(x·c^T)/norm, pc_j> (co_clustering.py:2203-2252).

    x [B,N,D], c [B,K,D], pc [B,J,K] fp32, norms [B,N] -> int64 [B,N].
    tf32=True rounds the operands of the second product to TF32, as the reference's kernel does on a
    GPU (tl.dot(..., allow_tf32=True), :2242; the first product's operands are bf16 values, which
    TF32 holds exactly).  The fixtures were made by the Triton interpreter, which multiplies in
    fp32, so the default is the fp32 evaluation.
    """
    prof = torch.matmul(x.float(), c.float().transpose(-1, -2)) / norms[..., None]
    pcf = pc.float()
    if tf32:
        prof, pcf = round_tf32(prof), round_tf32(pcf)
    dist = 2.0 - 2.0 * torch.matmul(prof, pcf.transpose(-1, -2))
    # torch.argmin returns the first minimal index on CPU, which is the rule the
    # reference's running (strict <) update across J tiles produces.
    return torch.argmin(dist, dim=-1)


def centroid_update(x, labels, old_centroids) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-cluster mean in fp32, empty clusters keep the old centroid, cast to x dtype;
    int32 counts (co_clustering.py:253-303)."""
    B, N, D = x.shape
    K = old_centroids.shape[1]
    sums = torch.zeros(B, K, D, dtype=torch.float64)
    for b in range(B):
        sums[b].index_add_(0, labels[b], x[b].double())
    counts = torch.zeros(B, K, dtype=torch.int64)
    counts.scatter_add_(1, labels, torch.ones_like(labels))
    means = (sums / counts.clamp(min=1).double()[..., None]).float()
    means = torch.where((counts == 0)[..., None], old_centroids.float(), means)
    return means.to(x.dtype), counts.to(torch.int32)


def co_cluster_tokens(q, k, q_init_idx, k_init_idx, max_iters: int, tf32: bool = False):
    """Restates co_cluster_tokens (co_clustering.py:2402-2451) with the random
    initial token indices passed in (the reference draws q indices, then k
    indices, with torch.randint).  Returns the reference's tuple order:
    (qlabels, qcentroids, qsizes, klabels, kcentroids, ksizes).  tf32: see cocluster_assign."""
    B, N, D = q.shape
    qc = torch.gather(q, 1, q_init_idx[..., None].expand(-1, -1, D))
    kc = torch.gather(k, 1, k_init_idx[..., None].expand(-1, -1, D))
    ql = kl = qs = ks = None
    for _ in range(max_iters):
        pk = l2norm_rows(torch.matmul(kc, qc.transpose(-1, -2)))
        kl = cocluster_assign(k, qc, pk, profile_norm(k, qc), tf32)
        kc, ks = centroid_update(k, kl, kc)
        pq = l2norm_rows(torch.matmul(qc, kc.transpose(-1, -2)))
        ql = cocluster_assign(q, kc, pq, profile_norm(q, kc), tf32)
        qc, qs = centroid_update(q, ql, qc)
    return ql, qc, qs, kl, kc, ks


def cocluster_assign_one_gemm(x, c, own) -> torch.Tensor:
    """The same assignment in a different fp32 evaluation order: label = first argmax_j x . W_j with
    W = l2norm(own . c^T) . c (the token's norm does not depend on j and the double sum is linear
    in x).  Not a restatement of reference code: a second, equally valid fp32 implementation, kept
    to measure how far two correct implementations drift apart over k-means iterations."""
    pc = l2norm_rows(torch.matmul(own, c.transpose(-1, -2)))
    w = torch.matmul(pc, c.float())
    return torch.argmax(torch.matmul(x.float(), w.transpose(-1, -2)), dim=-1)


def co_cluster_tokens_one_gemm(q, k, q_init_idx, k_init_idx, max_iters: int):
    """co_cluster_tokens with cocluster_assign_one_gemm as the assignment step."""
    B, N, D = q.shape
    qc = torch.gather(q, 1, q_init_idx[..., None].expand(-1, -1, D))
    kc = torch.gather(k, 1, k_init_idx[..., None].expand(-1, -1, D))
    ql = kl = qs = ks = None
    for _ in range(max_iters):
        kl = cocluster_assign_one_gemm(k, qc, kc)
        kc, ks = centroid_update(k, kl, kc)
        ql = cocluster_assign_one_gemm(q, kc, qc)
        qc, qs = centroid_update(q, ql, qc)
    return ql, qc, qs, kl, kc, ks


def clustering_objective(x, form, own, labels) -> float:
    """Mean cosine between a token's profile over `form` and the profile of its own centroid: the
    quantity the assignment maximises, a measure of a clustering that does not depend on which of
    two near-tied centroids a token went to."""
    pc = l2norm_rows(torch.matmul(own, form.transpose(-1, -2)))                  # [B,J,K]
    prof = torch.matmul(x.float(), form.float().transpose(-1, -2))
    prof = prof / profile_norm(x, form)[..., None]
    mine = torch.gather(pc, 1, labels[..., None].expand(-1, -1, pc.shape[-1]))
    return float((prof * mine).sum(-1).mean())


# --------------------------------------------------------------------------------------
# permutation
# --------------------------------------------------------------------------------------

def sort_labels(labels: torch.Tensor, num_clusters: int):
    """Stable ascending sort of labels per head: (sorted_idx int32 [B,N],
    offsets int32 [B,K+1]).  The reference calls torch.argsort (permute.py:90),
    whose order inside one cluster is unspecified; the stable order is the
    convention adopted here (same cluster membership, same cluster offsets)."""
    idx = torch.argsort(labels, dim=-1, stable=True).to(torch.int32)
    B = labels.shape[0]
    counts = torch.zeros(B, num_clusters, dtype=torch.int64)
    counts.scatter_add_(1, labels.long(), torch.ones_like(labels, dtype=torch.int64))
    offsets = torch.zeros(B, num_clusters + 1, dtype=torch.int32)
    offsets[:, 1:] = torch.cumsum(counts, -1).to(torch.int32)
    return idx, offsets


def permute(x: torch.Tensor, sorted_idx: torch.Tensor) -> torch.Tensor:
    """Y[b,s,:] = X[b,idx[b,s],:] (permute.py:10-35).  x [B,N,D]."""
    return torch.gather(x, 1, sorted_idx.long()[..., None].expand(-1, -1, x.shape[-1]))


def inverse_permute(y: torch.Tensor, sorted_idx: torch.Tensor) -> torch.Tensor:
    """X[b,idx[b,s],:] = Y[b,s,:] (permute.py:39-65)."""
    out = torch.empty_like(y)
    out.scatter_(1, sorted_idx.long()[..., None].expand(-1, -1, y.shape[-1]), y)
    return out


# --------------------------------------------------------------------------------------
# cluster-block map
# --------------------------------------------------------------------------------------

_LOG2E = np.float32(1.4426950408889634)
_LN2_HI = np.float32(0.693145751953125)          # 0x3f317200
_LN2_LO = np.float32(1.428606765330187e-06)      # ln2 - LN2_HI
_EXP_POLY = [np.float32(v) for v in (1.0 / 720, 1.0 / 120, 1.0 / 24, 1.0 / 6, 0.5, 1.0, 1.0)]


def exp_f32(x: np.ndarray) -> np.ndarray:
    """exp(x) for x <= 0 from IEEE fp32 add/mul only (no fma), so that the CUDA
    kernel, which runs the same sequence with __fmul_rn/__fadd_rn, gets the same bits."""
    x = x.astype(np.float32)
    n = np.rint(x * _LOG2E).astype(np.float32)
    r = (x - n * _LN2_HI).astype(np.float32)
    r = (r - n * _LN2_LO).astype(np.float32)
    p = np.full_like(r, _EXP_POLY[0])
    for c in _EXP_POLY[1:]:
        p = (p * r).astype(np.float32)
        p = (p + c).astype(np.float32)
    n_i = np.maximum(n, np.float32(-126.0)).astype(np.int32)
    out = np.ldexp(p, n_i).astype(np.float32)
    return np.where(x < np.float32(-87.0), np.float32(0.0), out)


def _round_to_bf16(a: np.ndarray) -> np.ndarray:
    """fp32 -> nearest-even bf16 -> fp32."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).bfloat16().float().numpy()


def _ratio_list(r: Ratio, H: int):
    """Mirror of the reference's scalar / per-head-list dispatch (co_clustering.py:589-627)."""
    if r is None:
        return None, "none"
    if isinstance(r, (list, tuple)) or (hasattr(r, "__len__") and len(r) == H):
        # the reference goes through a float32 tensor and .item()
        vals = torch.as_tensor(r, dtype=torch.float32).tolist()
        return [float(v) for v in vals], "list"
    if isinstance(r, (int, float)):
        return float(r), "scalar"
    return None, "none"


def keep_counts(kc_num: int, H: int, min_kc_ratio: Ratio, max_kc_ratio: Ratio):
    """Per-head (preserve_length, cap) of identify_dynamic_map; cap = kc_num means
    no cap (co_clustering.py:589-627)."""
    mn, mn_kind = _ratio_list(min_kc_ratio, H)
    mx, mx_kind = _ratio_list(max_kc_ratio, H)
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
                # the reference only enters this branch when min is a tensor; a python
                # list has been converted to a tensor by the floor step before
                if mn[h] > 0:
                    c = max(c, int(mn[h] * kc_num))
                c = max(1, c)
            elif mn_kind == "scalar" and mn > 0:
                c = max(c, int(mn * kc_num))
            cap[h] = c
    return preserve, cap


def identify_dynamic_map(qc, kc, q_sizes, k_sizes, p: float, min_kc_ratio: Ratio = 0,
                         max_kc_ratio: Ratio = 0, return_order: bool = False, return_probs: bool = False):
    """Restates identify_dynamic_map (co_clustering.py:556-633).

    qc [B,H,QC,D], kc [B,H,KC,D] (fp32 or bf16), sizes int [B,H,*].  Returns bool
    [B,H,QC,KC].  Arithmetic is fixed so that it can be reproduced bit for bit:
      score  = dot(q_i, k_j) accumulated d = 0..D-1 in fp32 (products of bf16 values
               are exact in fp32), rounded to the centroid dtype, divided by
               fp32(sqrt(D)), rounded to the centroid dtype again;
      prob   = size_j * exp(score - max) / max(sum, 1e-12), the sum taken j = 0..KC-1
               in fp32, rounded to the centroid dtype;
      order  = descending prob, ties by lower cluster index;
      cumsum = running fp32 sum of the sorted probs, each prefix rounded to the
               centroid dtype, compared with p rounded to the centroid dtype.
    """
    B, H, QC, D = qc.shape
    KC = kc.shape[2]
    if p >= 1.0:
        m = torch.ones(B, H, QC, KC, dtype=torch.bool)
        return (m, None) if (return_order or return_probs) else m
    lowp = qc.dtype == torch.bfloat16
    rnd = _round_to_bf16 if lowp else (lambda a: a.astype(np.float32))
    q = qc.float().numpy()
    k = kc.float().numpy()
    acc = np.zeros((B, H, QC, KC), dtype=np.float32)
    for d in range(D):
        prod = (q[..., :, None, d] * k[..., None, :, d]).astype(np.float32)
        acc = (acc + prod).astype(np.float32)
    s = rnd(acc)
    s = rnd((s / np.float32(D ** 0.5)).astype(np.float32))
    w = k_sizes.float().numpy()[..., None, :]
    mx = s.max(-1, keepdims=True)
    e = exp_f32((s - mx).astype(np.float32))
    we = (w * e).astype(np.float32)
    tot = np.zeros(we.shape[:-1], dtype=np.float32)
    for j in range(KC):
        tot = (tot + we[..., j]).astype(np.float32)
    tot = np.maximum(tot, np.float32(1e-12))
    prob = rnd((we / tot[..., None]).astype(np.float32))
    # descending, stable on ties
    order = np.argsort(-prob.astype(np.float64), axis=-1, kind="stable")
    sp = np.take_along_axis(prob, order, -1)
    run = np.zeros(sp.shape[:-1], dtype=np.float32)
    cum = np.empty_like(sp)
    for j in range(KC):
        run = (run + sp[..., j]).astype(np.float32)
        cum[..., j] = run
    cum = rnd(cum)
    p_cmp = rnd(np.array([p], dtype=np.float32))[0] if lowp else np.float32(p)
    remove = cum > p_cmp
    remove[..., 1:] = remove[..., :-1].copy()
    remove[..., 0] = False
    preserve, cap = keep_counts(KC, H, min_kc_ratio, max_kc_ratio)
    for h in range(H):
        if preserve[h] > 0:
            remove[:, h, :, :preserve[h]] = False
        if cap[h] < KC:
            remove[:, h, :, cap[h]:] = True
    keep_sorted = ~remove
    out = np.zeros((B, H, QC, KC), dtype=bool)
    np.put_along_axis(out, order, keep_sorted, -1)
    m = torch.from_numpy(out)
    if return_probs:
        return m, torch.from_numpy(prob)
    return (m, torch.from_numpy(order)) if return_order else m


def hunyuan_text_blocks(dyn_map, q_sizes, k_sizes, q_sorted_idx, video_length, context_length,
                        prompt_length):
    """Append the prompt / unused-prompt blocks (hunyuan10/attention.py:999-1019).
    dyn_map [B,H,QC,KC] bool; sizes [B,H,*]; q_sorted_idx [H,video_length]."""
    import torch.nn.functional as F
    unprompt = context_length - prompt_length
    m = F.pad(dyn_map, (0, 2, 0, 2), value=False)
    m[:, :, -2, :-1] = True
    m[:, :, :-1, -2] = True
    m[:, :, -1, -1] = True
    qs = F.pad(q_sizes, (0, 2), value=0)
    qs[:, :, -2] = prompt_length
    qs[:, :, -1] = unprompt
    ks = F.pad(k_sizes, (0, 2), value=0)
    ks[:, :, -2] = prompt_length
    ks[:, :, -1] = unprompt
    idx = F.pad(q_sorted_idx, (0, context_length), value=0)
    idx[:, video_length:] = torch.arange(video_length, video_length + context_length)
    return m, qs, ks, idx


# --------------------------------------------------------------------------------------
# block-sparse attention
# --------------------------------------------------------------------------------------

def block_sparse_attention(q, k, v, dyn_map, q_sizes, k_sizes, sm_scale: Optional[float] = None):
    """softmax(Q K_sel^T * scale) V_sel per query cluster over the key clusters its
    map row selects; rows with no selected key token give 0
    (co_clustering.py:1040-1108).  q,k,v [B,H,S,D] already in cluster order;
    fp32 math; output in q's dtype."""
    B, H, S, D = q.shape
    scale = D ** -0.5 if sm_scale is None else sm_scale
    out = torch.zeros(B, H, S, D, dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            qo = np.concatenate([[0], np.cumsum(q_sizes[b, h].numpy())])
            ko = np.concatenate([[0], np.cumsum(k_sizes[b, h].numpy())])
            kf = k[b, h].float()
            vf = v[b, h].float()
            for i in range(len(qo) - 1):
                if qo[i + 1] == qo[i]:
                    continue
                sel = [torch.arange(ko[j], ko[j + 1]) for j in np.nonzero(dyn_map[b, h, i].numpy())[0]
                       if ko[j + 1] > ko[j]]
                if not sel:
                    continue
                sel = torch.cat(sel)
                qi = q[b, h, qo[i]:qo[i + 1]].float()
                sc = (qi @ kf[sel].T) * scale
                out[b, h, qo[i]:qo[i + 1]] = torch.softmax(sc, -1) @ vf[sel]
    return out.to(q.dtype)


def realised_density(dyn_map, q_sizes, k_sizes) -> torch.Tensor:
    """rho_h = sum_ij map[h,i,j] |Q_i| |K_j| / N^2 per head -> [B,H] float64."""
    qs = q_sizes.double()
    ks = k_sizes.double()
    n = qs.sum(-1)
    return torch.einsum("bhi,bhij,bhj->bh", qs, dyn_map.double(), ks) / (n * n)


def attention_given_clustering(q, k, v, clustering, top_p, min_kc_ratio=0, max_kc_ratio=0, context_length=0,
                                prompt_length=0):
    """Everything after the clustering for [1,H,S,D] inputs whose last `context_length` rows are
    text tokens: stable permute of the video rows, map (+ the two text blocks), masked attention,
    inverse permute.  `clustering` = (qlabels, qcentroids, qsizes, klabels, kcentroids, ksizes) of the
    video rows -- fresh, or cached from an earlier denoising step as the reference's processors reuse
    it (wan/attention.py:682-715; hunyuan10/attention.py:977-1110).  Returns (out [1,H,S,D], aux)."""
    ql, qc, qs, kl, kc, ks = clustering
    B, H, S, D = q.shape
    assert B == 1
    n = S - context_length
    num_q, num_k = qc.shape[1], kc.shape[1]
    q_idx, q_off = sort_labels(ql, num_q)
    k_idx, k_off = sort_labels(kl, num_k)
    qp, kp, vp = permute(q[0, :, :n], q_idx), permute(k[0, :, :n], k_idx), permute(v[0, :, :n], k_idx)
    m = identify_dynamic_map(qc[None], kc[None], qs[None], ks[None], top_p, min_kc_ratio, max_kc_ratio)
    m_video = m
    qs_b, ks_b, idx_full = qs[None], ks[None], q_idx
    if context_length:
        qp, kp, vp = (torch.cat([a, b[0, :, n:]], 1) for a, b in ((qp, q), (kp, k), (vp, v)))
        m, qs_b, ks_b, idx_full = hunyuan_text_blocks(m, qs[None], ks[None], q_idx, n, context_length, prompt_length)
    op = block_sparse_attention(qp[None], kp[None], vp[None], m, qs_b, ks_b)
    out = inverse_permute(op[0], idx_full)[None]
    return out, dict(qlabels=ql, klabels=kl, qcentroids=qc, kcentroids=kc, qsizes=qs, ksizes=ks, q_idx=q_idx,
                     k_idx=k_idx, q_off=q_off, k_off=k_off, map=m, map_video=m_video, out_permuted=op)


def sparse_attention_layer(q, k, v, q_init_idx, k_init_idx, num_q, num_k, iters, top_p,
                           min_kc_ratio=0, max_kc_ratio=0, context_length=0, prompt_length=0):
    """The whole path for [1,H,S,D] inputs: co-clustering (of the video rows) -> stable permute ->
    map -> masked attention -> inverse permute (wan/attention.py:958-1088,1159-1216).
    Returns (out [1,H,S,D], dict of intermediates)."""
    B, H, S, D = q.shape
    assert B == 1
    n = S - context_length
    clustering = co_cluster_tokens(q[0, :, :n].contiguous(), k[0, :, :n].contiguous(), q_init_idx, k_init_idx, iters)
    return attention_given_clustering(q, k, v, clustering, top_p, min_kc_ratio, max_kc_ratio, context_length,
                                      prompt_length)


# --------------------------------------------------------------------------------------
# Euclidean k-means (the reference's non-co-clustering mode)
# --------------------------------------------------------------------------------------
def euclid_assign(x, centroids):
    """first argmin_j max(|x|^2 + |c_j|^2 - 2 x.c_j, 0) (co_clustering.py:335-416).  For bf16 inputs the
    squares are rounded to bf16 before they are summed, as `c_tile * c_tile` and `x ** 2` are there;
    the token norm is rounded to bf16 once more (torch.sum of a bf16 tensor, :516)."""
    lowp = x.dtype == torch.bfloat16
    sq = (lambda t: (t * t).float()) if lowp else (lambda t: t.float() * t.float())
    x_sq = sq(x).sum(-1)
    if lowp:
        x_sq = x_sq.bfloat16().float()
    c_sq = sq(centroids).sum(-1)
    cross = torch.matmul(x.float(), centroids.float().transpose(-1, -2))
    dist = (x_sq[..., None] + c_sq[..., None, :] - 2.0 * cross).clamp_min(0.0)
    return torch.argmin(dist, dim=-1)


def batch_kmeans_euclid(x, init_centroids, max_iters, tol=1e-4):
    """batch_kmeans_Euclid from given initial centroids (co_clustering.py:502-541): returns
    (labels, centroids, sizes, iterations); on a `tol` stop the centroids of the last assignment."""
    centroids = init_centroids
    labels = sizes = None
    it = -1
    for it in range(max_iters):
        labels = euclid_assign(x, centroids)
        new, sizes = centroid_update(x, labels, centroids)
        shift = (new.float() - centroids.float()).norm(dim=-1).max()
        if shift < tol:
            break
        centroids = new
    return labels, centroids, sizes, it + 1
