"""CPU oracle for the error-aware routing ("EAR") variant of the sparse-attention path.
TEST INFRASTRUCTURE ONLY: nothing in the product package imports it.

Parity status: PINNED by tests/test_oracle_golden.py against outputs of the reference's own
functions (tests/golden/ear_*.npz, made by tests/golden/make_golden.py: Triton kernels under the
interpreter, the torch part as written).

Reference locations restated here (paths inside the reference project):
  * value centroids                  svoo/models/wan/attention.py:594-610
  * value statistics per key token   svoo/co_clustering.py:1314-1395
  * block error estimate             svoo/co_clustering.py:1398-1565 (wrapper :1570-1689)
  * budgeted block selection         svoo/co_clustering.py:1691-1798
  * centroid compensation            svoo/co_clustering.py:1800-1921 (wrapper :1924-2050)
"""
from __future__ import annotations

import math

import numpy as np
import torch

from . import svoo_oracle as O

_LN2_HI = np.float32(0.693145751953125)
_LN2_LO = np.float32(1.428606765330187e-06)
_SQRT2 = np.float32(1.41421354)
_LOG_POLY = [np.float32(v) for v in (1.0 / 11, 1.0 / 9, 1.0 / 7, 1.0 / 5, 1.0 / 3, 1.0)]
EPS = 1e-8


def log_f32(x: np.ndarray) -> np.ndarray:
    """ln(x) for normal x > 0 from IEEE fp32 add/mul/div only (no fma), so that the CUDA kernel,
    which runs the same sequence with __fadd_rn/__fmul_rn/__fdiv_rn, gets the same bits:
    x = m 2^e with m in (sqrt(1/2), sqrt(2)], s = (m-1)/(m+1), ln m = 2 s (1 + z/3 + ... + z^5/11)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.int32)
    e = ((bits >> 23) & 0xFF) - 127
    m = ((bits & 0x007FFFFF) | 0x3F800000).view(np.float32)
    big = m > _SQRT2
    m = np.where(big, (m * np.float32(0.5)).astype(np.float32), m)
    e = (e + big).astype(np.float32)
    f = (m - np.float32(1.0)).astype(np.float32)
    s = (f / (f + np.float32(2.0)).astype(np.float32)).astype(np.float32)
    z = (s * s).astype(np.float32)
    p = np.full_like(z, _LOG_POLY[0])
    for c in _LOG_POLY[1:]:
        p = (p * z).astype(np.float32)
        p = (p + c).astype(np.float32)
    lm = ((s + s).astype(np.float32) * p).astype(np.float32)
    lo = ((e * _LN2_LO).astype(np.float32) + lm).astype(np.float32)
    return ((e * _LN2_HI).astype(np.float32) + lo).astype(np.float32)


def value_centroids(v: torch.Tensor, labels: torch.Tensor, sizes: torch.Tensor, num_clusters: int) -> torch.Tensor:
    """Mean of the value rows of every key cluster, zero for an empty one (wan/attention.py:594-610).
    v [H,N,D], labels [H,N], sizes [H,KC] -> [H,KC,D] in v's dtype.  The reference accumulates with
    scatter_add_ in the tokens' dtype (for bf16 its result depends on the order of the atomics); here the
    sums are fp32 and rounded once."""
    H, N, D = v.shape
    acc = torch.zeros(H, num_clusters, D, dtype=torch.float32)
    acc.scatter_add_(1, labels.long()[..., None].expand(-1, -1, D), v.float())
    return (acc / sizes.clamp_min(1).float()[..., None]).to(v.dtype)


def value_stats(v_perm: torch.Tensor, vc: torch.Tensor, k_off: torch.Tensor):
    """Per key token (cluster order) |v|^2 and v.vc of its cluster, per cluster |vc|^2
    (co_clustering.py:1314-1395).  For bf16 inputs every product is rounded to bf16 before the fp32
    sum, as `value_block * value_block` is there.  Returns fp32 ([H,N], [H,N], [H,KC])."""
    H, N, D = v_perm.shape
    KC = vc.shape[1]
    lowp = v_perm.dtype == torch.bfloat16
    prod = (lambda a, b: (a * b).float()) if lowp else (lambda a, b: a.float() * b.float())
    vn = prod(v_perm, v_perm).sum(-1)
    vc_sq = prod(vc, vc).sum(-1)
    cvd = torch.zeros(H, N, dtype=torch.float32)
    for h in range(H):
        off = k_off[h].tolist()
        for j in range(KC):
            if off[j + 1] > off[j]:
                cvd[h, off[j]:off[j + 1]] = prod(vc[h, j][None, :], v_perm[h, off[j]:off[j + 1]]).sum(-1)
    return vn, cvd, vc_sq


def centroid_logits(qc: torch.Tensor, kc: torch.Tensor) -> np.ndarray:
    """einsum(qc, kc) * D^-0.5 as torch evaluates it in the centroids' dtype (co_clustering.py:1724):
    the dot accumulated d = 0..D-1 in fp32, rounded to the dtype, times fp32(D^-0.5), rounded again."""
    H, QC, D = qc.shape
    lowp = qc.dtype == torch.bfloat16
    rnd = O._round_to_bf16 if lowp else (lambda a: a.astype(np.float32))
    q = qc.float().numpy()
    k = kc.float().numpy()
    acc = np.zeros((H, QC, kc.shape[1]), dtype=np.float32)
    for d in range(D):
        acc = (acc + (q[:, :, None, d] * k[:, None, :, d]).astype(np.float32)).astype(np.float32)
    return rnd((rnd(acc) * np.float32(D ** -0.5)).astype(np.float32))


def error_scores(qc, k_perm, k_off, q_sizes, k_sizes, c_logits, vn, cvd, vc_sq, gamma: float, eps: float = EPS):
    """log-efficiency of every (query cluster i, key cluster j) pair (co_clustering.py:1398-1565):
        err_ij  = sum_{t in K_j} | e^{a_it} v_t - e^{c_ij} vc_j |^2,  a_it = qc_i.k_t D^-0.5,
                  evaluated as there: everything relative to M = max(c_ij, max_t a_it), then * e^{2M};
        score   = log(max(err, eps)) - gamma log(max(|Q_i| |K_j|, eps)).
    fp32 throughout; returns [H,QC,KC] float32 (torch)."""
    H, QC, D = qc.shape
    KC = k_sizes.shape[1]
    scale = D ** -0.5
    out = torch.empty(H, QC, KC, dtype=torch.float32)
    clog = torch.as_tensor(c_logits, dtype=torch.float32)
    for h in range(H):
        attn = (qc[h].float() @ k_perm[h].float().T) * scale           # [QC, N]
        off = k_off[h].tolist()
        qs = q_sizes[h].float()
        for j in range(KC):
            a = attn[:, off[j]:off[j + 1]]
            c = clog[h, :, j]
            M = torch.maximum(c, a.max(-1).values) if a.shape[1] else c
            p = torch.exp(a - M[:, None])
            sq = (p * p * vn[h, off[j]:off[j + 1]][None, :]).sum(-1)
            cr = (p * cvd[h, off[j]:off[j + 1]][None, :]).sum(-1)
            cp = torch.exp(c - M)
            n_j = float(k_sizes[h, j])
            err = sq - 2.0 * cp * cr + cp * cp * vc_sq[h, j] * n_j
            err = (err * torch.exp(2.0 * M)).clamp_min(eps)
            area = (qs * n_j).clamp_min(eps)
            out[h, :, j] = torch.log(err) - gamma * torch.log(area)
    return out


def ratio_lengths(KC: int, H: int, min_kc_ratio):
    """(preserve_len, budget_preserve_len) per head, 0 where the ratio is not positive
    (co_clustering.py:1748-1774)."""
    if isinstance(min_kc_ratio, torch.Tensor) and min_kc_ratio.numel() == 1 and H != 1:
        mn, kind = float(min_kc_ratio.item()), "scalar"
    elif isinstance(min_kc_ratio, (list, tuple)) and len(min_kc_ratio) == 1 and H != 1:
        mn, kind = float(min_kc_ratio[0]), "scalar"
    elif isinstance(min_kc_ratio, torch.Tensor):
        mn, kind = O._ratio_list(min_kc_ratio.flatten(), H) if min_kc_ratio.numel() == H else (None, "none")
    else:
        mn, kind = O._ratio_list(min_kc_ratio, H)
    if kind == "scalar":
        mn = [mn] * H
    elif kind != "list":
        mn = [0.0] * H
    pres = [max(1, int(r * KC)) if r > 0 else 0 for r in mn]
    bud = [max(1, int(r * KC * 2)) if r > 0 else 0 for r in mn]
    return pres, bud


def select_blocks(c_logits: np.ndarray, scores, q_sizes, k_sizes, top_p: float, min_kc_ratio, lowp: bool,
                  return_aux: bool = False):
    """The torch part of identify_dynamic_map_estimated (co_clustering.py:1738-1798) with its arithmetic
    fixed so that it can be reproduced bit for bit:
      log size   = log_f32(rnd(rnd(size) + 1e-8)) rounded (rnd = round to the centroids' dtype);
      budget     = softmax_j(rnd(c_ij + log size_j)): exp_f32(x - max) / sum (j ascending, fp32), rounded;
      order      = descending probability, ties by lower cluster index; prefix sums as running fp32
                   sums, each rounded, compared with rnd(top_p); keep[0] always, keep[r] = cum[r-1] <= p;
                   the first budget_preserve_len positions kept;
      budget_i   = sum of |Q_i||K_j| (as fp32) over the kept positions in sorted order, running fp32 sum;
      guaranteed = the first preserve_len positions; their cost summed j ascending;
      remaining  = max(budget - guaranteed cost, 0);
      candidates = score (guaranteed ones -1e10) descending, ties by lower index; running fp32 sum of
                   their areas; kept while (cum - area) < remaining.
    c_logits, scores [H,QC,KC]; returns bool [H,QC,KC]."""
    H, QC, KC = c_logits.shape
    rnd = O._round_to_bf16 if lowp else (lambda a: np.asarray(a, dtype=np.float32))
    ks = k_sizes.numpy().astype(np.float32)
    logsz = rnd(log_f32(rnd((rnd(ks) + np.float32(EPS)).astype(np.float32))))
    bl = rnd((np.asarray(c_logits, dtype=np.float32) + logsz[:, None, :]).astype(np.float32))
    mx = bl.max(-1, keepdims=True)
    e = O.exp_f32((bl - mx).astype(np.float32))
    tot = np.zeros(e.shape[:-1], dtype=np.float32)
    for j in range(KC):
        tot = (tot + e[..., j]).astype(np.float32)
    prob = rnd((e / tot[..., None]).astype(np.float32))
    order = np.argsort(-prob.astype(np.float64), axis=-1, kind="stable")
    sp = np.take_along_axis(prob, order, -1)
    run = np.zeros(sp.shape[:-1], dtype=np.float32)
    cum = np.empty_like(sp)
    for j in range(KC):
        run = (run + sp[..., j]).astype(np.float32)
        cum[..., j] = run
    cum = rnd(cum)
    p_cmp = rnd(np.array([top_p], dtype=np.float32))[0] if lowp else np.float32(top_p)
    keep = np.ones((H, QC, KC), dtype=bool)
    keep[..., 1:] = cum[..., :-1] <= p_cmp
    pres, bud = ratio_lengths(KC, H, min_kc_ratio)
    guaranteed_sorted = np.zeros((H, QC, KC), dtype=bool)
    for h in range(H):
        if pres[h] > 0:
            keep[h, :, :bud[h]] = True
            guaranteed_sorted[h, :, :pres[h]] = True
    guaranteed = np.zeros((H, QC, KC), dtype=bool)
    np.put_along_axis(guaranteed, order, guaranteed_sorted, -1)
    area = (q_sizes.numpy().astype(np.int64)[:, :, None] * k_sizes.numpy().astype(np.int64)[:, None, :]).astype(np.float32)
    sa = np.take_along_axis(area, order, -1)
    budget = np.zeros((H, QC), dtype=np.float32)
    for r in range(KC):
        budget = np.where(keep[..., r], (budget + sa[..., r]).astype(np.float32), budget)
    gcost = np.zeros((H, QC), dtype=np.float32)
    for j in range(KC):
        gcost = np.where(guaranteed[..., j], (gcost + area[..., j]).astype(np.float32), gcost)
    remaining = np.maximum((budget - gcost).astype(np.float32), np.float32(0.0))
    sc = np.where(guaranteed, np.float32(-1e10), np.asarray(scores, dtype=np.float32))
    order2 = np.argsort(-sc.astype(np.float64), axis=-1, kind="stable")
    ca = np.take_along_axis(area, order2, -1)
    run = np.zeros((H, QC), dtype=np.float32)
    dyn_sorted = np.zeros((H, QC, KC), dtype=bool)
    for r in range(KC):
        run = (run + ca[..., r]).astype(np.float32)
        dyn_sorted[..., r] = (run - ca[..., r]).astype(np.float32) < remaining
    dyn = np.zeros((H, QC, KC), dtype=bool)
    np.put_along_axis(dyn, order2, dyn_sorted, -1)
    out = torch.from_numpy(guaranteed | dyn)
    if return_aux:
        return out, dict(prob=prob, order=order, guaranteed=guaranteed, remaining=remaining, budget=budget,
                         scores_masked=sc, area=area, budget_kept=keep, preserve=pres)
    return out


def identify_dynamic_map_estimated(k_perm, v_perm, q_sizes, k_sizes, qc, kc, vc, top_p: float = 0.9, gamma: float = 1.0,
                                   min_kc_ratio=0.0, scores=None, return_aux: bool = False):
    """identify_dynamic_map_estimated (co_clustering.py:1691-1798) for one batch entry: k_perm, v_perm
    [H,N,D] in cluster order, sizes [H,*], centroids [H,*,D].  `scores`: use these block scores
    instead of estimating them (to test the selection alone)."""
    H = qc.shape[0]
    k_off = torch.zeros(H, k_sizes.shape[1] + 1, dtype=torch.int64)
    k_off[:, 1:] = torch.cumsum(k_sizes.long(), -1)
    clog = centroid_logits(qc, kc)
    if scores is None:
        vn, cvd, vc_sq = value_stats(v_perm, vc, k_off)
        scores = error_scores(qc, k_perm, k_off, q_sizes, k_sizes, clog, vn, cvd, vc_sq, gamma)
    res = select_blocks(clog, scores, q_sizes, k_sizes, top_p, min_kc_ratio, qc.dtype == torch.bfloat16, return_aux)
    if return_aux:
        res[1]["scores"] = scores
        res[1]["c_logits"] = clog
    return res


def token_attention_with_lse(q_perm, k_perm, v_perm, dyn_map, q_sizes, k_sizes):
    """The token part alone: softmax attention over the selected key tokens, with its log-sum-exp in
    base 2 as FlashInfer returns it (co_clustering.py:1866-1868; -inf and a zero row without keys).
    fp32; returns (o [H,S,D] fp32, lse2 [H,S] fp32)."""
    H, S, D = q_perm.shape
    scale = D ** -0.5
    o = torch.zeros(H, S, D, dtype=torch.float32)
    lse2 = torch.full((H, S), -float("inf"), dtype=torch.float32)
    for h in range(H):
        qo = np.concatenate([[0], np.cumsum(q_sizes[h].numpy())])
        ko = np.concatenate([[0], np.cumsum(k_sizes[h].numpy())])
        for i in range(len(qo) - 1):
            sel = [torch.arange(ko[j], ko[j + 1]) for j in np.nonzero(dyn_map[h, i].numpy())[0] if ko[j + 1] > ko[j]]
            if qo[i + 1] == qo[i] or not sel:
                continue
            sel = torch.cat(sel)
            sc = (q_perm[h, qo[i]:qo[i + 1]].float() @ k_perm[h].float()[sel].T) * scale
            o[h, qo[i]:qo[i + 1]] = torch.softmax(sc, -1) @ v_perm[h].float()[sel]
            lse2[h, qo[i]:qo[i + 1]] = torch.logsumexp(sc, -1) / math.log(2.0)
    return o, lse2


def compensated_attention(q_perm, k_perm, v_perm, kc, vc, dyn_map, q_sizes, k_sizes):
    """EAR forward (co_clustering.py:1800-2050) for one batch entry, everything [H,...] in cluster order:
    a query of cluster i attends the key tokens of the clusters its map row selects and, for every
    other cluster j, one virtual key kc_j with value vc_j and logit bias ln(|K_j| + 1e-6).
    The reference evaluates the two parts separately (token part by FlashInfer, rounded to the
    tensors' dtype, then an online-softmax merge over the centroids); the result is the softmax over
    the union.  fp32 math; returns (out [H,S,D] in q's dtype, lse [H,S] natural log, fp32)."""
    H, S, D = q_perm.shape
    KC = kc.shape[1]
    scale = D ** -0.5
    out = torch.zeros(H, S, D, dtype=torch.float32)
    lse = torch.full((H, S), -float("inf"), dtype=torch.float32)
    for h in range(H):
        qo = np.concatenate([[0], np.cumsum(q_sizes[h].numpy())])
        ko = np.concatenate([[0], np.cumsum(k_sizes[h].numpy())])
        kf, vf = k_perm[h].float(), v_perm[h].float()
        bias = torch.log(k_sizes[h].float() + 1e-6)
        for i in range(len(qo) - 1):
            if qo[i + 1] == qo[i]:
                continue
            row = dyn_map[h, i].numpy().astype(bool)
            sel = [torch.arange(ko[j], ko[j + 1]) for j in np.nonzero(row)[0] if ko[j + 1] > ko[j]]
            qi = q_perm[h, qo[i]:qo[i + 1]].float()
            parts_s, parts_v = [], []
            if sel:
                sel = torch.cat(sel)
                parts_s.append((qi @ kf[sel].T) * scale)
                parts_v.append(vf[sel])
            rest = torch.from_numpy(np.nonzero(~row)[0])
            if len(rest):
                parts_s.append((qi @ kc[h, rest].float().T) * scale + bias[rest][None, :])
                parts_v.append(vc[h, rest].float())
            if not parts_s:
                continue
            sc = torch.cat(parts_s, 1)
            out[h, qo[i]:qo[i + 1]] = torch.softmax(sc, -1) @ torch.cat(parts_v, 0)
            lse[h, qo[i]:qo[i + 1]] = torch.logsumexp(sc, -1)
    return out.to(q_perm.dtype), lse
