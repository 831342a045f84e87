"""Torch-tensor front end of the C ABI: one function per entry point.

Tensors are CUDA, contiguous; token tensors are bf16 [BH, N, 128].  Work is enqueued
on torch's current stream; nothing here synchronises with the host.
"""
from __future__ import annotations

import ctypes
import dataclasses
from typing import Dict, Optional, Sequence, Tuple

import torch

from ._lib import LIB, check

HEAD_DIM = 128
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("svoo_b200 ops need CUDA tensors; there is no CPU path")
        if not t.is_contiguous():
            raise ValueError("svoo_b200 ops need contiguous tensors")


def _tokens(x: torch.Tensor) -> Tuple[int, int, int]:
    if x.dim() != 3 or x.dtype != torch.bfloat16:
        raise ValueError(f"expected bf16 [BH, N, {HEAD_DIM}] tokens, got {x.dtype} {tuple(x.shape)}")
    return x.shape


def workspace_bytes(BH: int, N: int, QC: int, KC: int) -> int:
    out = ctypes.c_int64(0)
    check(LIB.svoo_b200_workspace_bytes(BH, N, QC, KC, ctypes.byref(out)), "workspace_bytes")
    return out.value


def workspace(device: torch.device, BH: int, N: int, QC: int, KC: int) -> torch.Tensor:
    """A cached uint8 scratch tensor of at least the needed size, one per device and stream."""
    need = workspace_bytes(BH, N, QC, KC)
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


@dataclasses.dataclass
class Clustering:
    """Everything one co-clustering call produces (all on device)."""
    qlabels: torch.Tensor      # int32 [BH, N]
    klabels: torch.Tensor
    qcentroids: torch.Tensor   # bf16 [BH, QC, 128]
    kcentroids: torch.Tensor
    qsizes: torch.Tensor       # int32 [BH, QC]
    ksizes: torch.Tensor
    q_sorted_idx: torch.Tensor  # int32 [BH, N] stable cluster-order permutation
    k_sorted_idx: torch.Tensor
    q_offsets: torch.Tensor     # int32 [BH, QC+1]
    k_offsets: torch.Tensor


def cocluster(q: torch.Tensor, k: torch.Tensor, q_init_idx: Optional[torch.Tensor],
              k_init_idx: Optional[torch.Tensor], iters: int,
              init_centroids: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> Clustering:
    """Co-clustering from initial centroid token indices, or (warm start) from `init_centroids` =
    (q centroids [BH,QC,128], k centroids [BH,KC,128]), which are not modified."""
    _need_cuda(q, k)
    BH, N, D = _tokens(q)
    if k.shape != q.shape or k.dtype != q.dtype:
        raise ValueError("q and k must have the same shape and dtype")
    dev = q.device
    i32 = dict(dtype=torch.int32, device=dev)
    if init_centroids is not None:
        qc0, kc0 = init_centroids
        _need_cuda(qc0, kc0)
        QC, KC = qc0.shape[1], kc0.shape[1]
        if qc0.shape != (BH, QC, D) or kc0.shape != (BH, KC, D) or qc0.dtype != q.dtype or kc0.dtype != q.dtype:
            raise ValueError("initial centroids must be bf16 [BH, QC, 128] and [BH, KC, 128]")
        qcent, kcent = qc0.clone(), kc0.clone()
        qi_ptr = ki_ptr = 0
    else:
        if q_init_idx is None or k_init_idx is None:
            raise ValueError("cocluster needs both initial index tensors, or init_centroids")
        _need_cuda(q_init_idx, k_init_idx)
        QC, KC = q_init_idx.shape[-1], k_init_idx.shape[-1]
        qi = q_init_idx.to(torch.int32).contiguous()
        ki = k_init_idx.to(torch.int32).contiguous()
        qi_ptr, ki_ptr = qi.data_ptr(), ki.data_ptr()
        qcent = torch.empty(BH, QC, D, dtype=q.dtype, device=dev)
        kcent = torch.empty(BH, KC, D, dtype=q.dtype, device=dev)
    c = Clustering(
        torch.empty(BH, N, **i32), torch.empty(BH, N, **i32), qcent, kcent,
        torch.empty(BH, QC, **i32), torch.empty(BH, KC, **i32),
        torch.empty(BH, N, **i32), torch.empty(BH, N, **i32),
        torch.empty(BH, QC + 1, **i32), torch.empty(BH, KC + 1, **i32))
    ws = workspace(dev, BH, N, QC, KC)
    check(LIB.svoo_b200_cocluster(
        q.data_ptr(), k.data_ptr(), qi_ptr, ki_ptr, BH, N, D, QC, KC, int(iters),
        c.qlabels.data_ptr(), c.klabels.data_ptr(), c.qcentroids.data_ptr(), c.kcentroids.data_ptr(),
        c.qsizes.data_ptr(), c.ksizes.data_ptr(), c.q_sorted_idx.data_ptr(), c.q_offsets.data_ptr(),
        c.k_sorted_idx.data_ptr(), c.k_offsets.data_ptr(), ws.data_ptr(), ws.numel(), _stream()), "cocluster")
    return c


def cocluster_assign(x: torch.Tensor, form_centroids: torch.Tensor, own_centroids: torch.Tensor) -> torch.Tensor:
    """int32 labels [BH, N] of tokens x among own_centroids, profiles formed over form_centroids."""
    _need_cuda(x, form_centroids, own_centroids)
    BH, N, D = _tokens(x)
    K, J = form_centroids.shape[1], own_centroids.shape[1]
    labels = torch.empty(BH, N, dtype=torch.int32, device=x.device)
    ws = workspace(x.device, BH, N, K, J)
    check(LIB.svoo_b200_cocluster_assign(x.data_ptr(), form_centroids.data_ptr(), own_centroids.data_ptr(), BH, N, D,
                                         K, J, labels.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
          "cocluster_assign")
    return labels


def euclid_assign(x: torch.Tensor, centroids: torch.Tensor) -> torch.Tensor:
    """int32 labels [BH, N]: the nearest centroid of every token in Euclidean distance."""
    _need_cuda(x, centroids)
    BH, N, D = _tokens(x)
    K = centroids.shape[1]
    if centroids.shape != (BH, K, D) or centroids.dtype != x.dtype:
        raise ValueError("centroids must be bf16 [BH, K, 128]")
    labels = torch.empty(BH, N, dtype=torch.int32, device=x.device)
    ws = workspace(x.device, BH, N, K, K)
    check(LIB.svoo_b200_euclid_assign(x.data_ptr(), centroids.data_ptr(), BH, N, D, K, labels.data_ptr(), ws.data_ptr(),
                                      ws.numel(), _stream()), "euclid_assign")
    return labels


def append_text_blocks(block_map_u8: torch.Tensor, q_offsets: torch.Tensor, k_offsets: torch.Tensor,
                       q_sorted_idx: torch.Tensor, k_sorted_idx: torch.Tensor, text: int, prompt: int):
    """Map, offsets and row indices of a joint-attention layer whose `text` text rows follow the
    clustered video rows: (map [BH,QC+2,KC+2], q_off [BH,QC+3], k_off [BH,KC+3], q_idx, k_idx [BH,N+text])."""
    _need_cuda(block_map_u8, q_offsets, k_offsets, q_sorted_idx, k_sorted_idx)
    BH, QC, KC = block_map_u8.shape
    N = q_sorted_idx.shape[1]
    dev = block_map_u8.device
    i32 = dict(dtype=torch.int32, device=dev)
    m = torch.empty(BH, QC + 2, KC + 2, dtype=torch.uint8, device=dev)
    qo, ko = torch.empty(BH, QC + 3, **i32), torch.empty(BH, KC + 3, **i32)
    qi, ki = torch.empty(BH, N + text, **i32), torch.empty(BH, N + text, **i32)
    src = block_map_u8.view(torch.uint8) if block_map_u8.dtype == torch.bool else block_map_u8
    check(LIB.svoo_b200_append_text_blocks(src.data_ptr(), q_offsets.data_ptr(), k_offsets.data_ptr(),
                                           q_sorted_idx.data_ptr(), k_sorted_idx.data_ptr(), BH, N, QC, KC, int(text),
                                           int(prompt), m.data_ptr(), qo.data_ptr(), ko.data_ptr(), qi.data_ptr(),
                                           ki.data_ptr(), _stream()), "append_text_blocks")
    return m, qo, ko, qi, ki


def sort_labels(labels: torch.Tensor, num_clusters: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Stable cluster-order permutation: (sorted_idx int32 [BH,N], offsets int32 [BH,K+1]).
    Labels must lie in [0, num_clusters)."""
    _need_cuda(labels)
    lab = labels.to(torch.int32).contiguous()
    BH, N = lab.shape
    idx = torch.empty_like(lab)
    off = torch.empty(BH, num_clusters + 1, dtype=torch.int32, device=lab.device)
    ws = workspace(lab.device, BH, N, num_clusters, num_clusters)
    check(LIB.svoo_b200_sort_labels(lab.data_ptr(), BH, N, num_clusters, idx.data_ptr(), off.data_ptr(),
                                    ws.data_ptr(), ws.numel(), _stream()), "sort_labels")
    return idx, off


def centroid_update(x: torch.Tensor, sorted_idx: torch.Tensor, offsets: torch.Tensor,
                    old_centroids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    _need_cuda(x, sorted_idx, offsets, old_centroids)
    BH, N, D = _tokens(x)
    K = old_centroids.shape[1]
    new = torch.empty_like(old_centroids)
    sizes = torch.empty(BH, K, dtype=torch.int32, device=x.device)
    ws = workspace(x.device, BH, N, K, K)
    check(LIB.svoo_b200_centroid_update(x.data_ptr(), sorted_idx.data_ptr(), offsets.data_ptr(),
                                        old_centroids.data_ptr(), BH, N, D, K, new.data_ptr(), sizes.data_ptr(),
                                        ws.data_ptr(), ws.numel(), _stream()), "centroid_update")
    return new, sizes


def _head_rows(t: torch.Tensor, n: int) -> int:
    """Rows between consecutive heads of a [BH, >=n, 128] tensor whose rows are dense."""
    if t.dim() != 3 or t.shape[-1] != HEAD_DIM or t.stride(-1) != 1 or t.stride(1) != HEAD_DIM or t.shape[1] < n:
        raise ValueError("expected [BH, rows, 128] with dense rows")
    if t.shape[0] > 1 and t.stride(0) % HEAD_DIM:
        raise ValueError("head stride must be a whole number of rows")
    return t.stride(0) // HEAD_DIM if t.shape[0] > 1 else max(t.shape[1], n)


def permute(x: torch.Tensor, sorted_idx: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[bh, s] = x[bh, idx[bh, s]] for s < N = idx.shape[1]; x and out may be [BH, N, 128]
    views (leading rows) of longer per-head sequences."""
    N = sorted_idx.shape[1]
    BH = sorted_idx.shape[0]
    if not (x.is_cuda and sorted_idx.is_cuda and sorted_idx.is_contiguous() and x.dtype == torch.bfloat16):
        raise ValueError("permute needs CUDA bf16 tokens and a contiguous int32 index")
    y = torch.empty(BH, N, HEAD_DIM, dtype=x.dtype, device=x.device) if out is None else out
    check(LIB.svoo_b200_permute(x.data_ptr(), sorted_idx.data_ptr(), BH, N, HEAD_DIM, _head_rows(x, N),
                                _head_rows(y, N), y.data_ptr(), _stream()), "permute")
    return y


def inverse_permute(x: torch.Tensor, sorted_idx: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[bh, idx[bh, s]] = x[bh, s] for s < N = idx.shape[1]."""
    N = sorted_idx.shape[1]
    BH = sorted_idx.shape[0]
    if not (x.is_cuda and sorted_idx.is_cuda and sorted_idx.is_contiguous() and x.dtype == torch.bfloat16):
        raise ValueError("inverse_permute needs CUDA bf16 tokens and a contiguous int32 index")
    y = torch.empty(BH, N, HEAD_DIM, dtype=x.dtype, device=x.device) if out is None else out
    check(LIB.svoo_b200_inverse_permute(x.data_ptr(), sorted_idx.data_ptr(), BH, N, HEAD_DIM, _head_rows(x, N),
                                        _head_rows(y, N), y.data_ptr(), _stream()), "inverse_permute")
    return y


def block_map(qcentroids: torch.Tensor, kcentroids: torch.Tensor, ksizes: torch.Tensor, top_p: float,
              preserve: Sequence[int], cap: Sequence[int]) -> torch.Tensor:
    """uint8 [BH, QC, KC]; preserve / cap are per-head python ints (numbers of key clusters)."""
    _need_cuda(qcentroids, kcentroids, ksizes)
    BH, QC, D = qcentroids.shape
    KC = kcentroids.shape[1]
    if qcentroids.dtype != torch.bfloat16 or kcentroids.dtype != torch.bfloat16:
        raise ValueError("block_map needs bf16 centroids")
    if len(preserve) != BH or len(cap) != BH:
        raise ValueError("preserve and cap need one entry per head")
    out = torch.empty(BH, QC, KC, dtype=torch.uint8, device=qcentroids.device)
    arr = ctypes.c_int32 * BH
    ks = ksizes.to(torch.int32).contiguous()
    check(LIB.svoo_b200_block_map(qcentroids.data_ptr(), kcentroids.data_ptr(), ks.data_ptr(), BH, QC, KC, D,
                                  float(top_p), arr(*[int(v) for v in preserve]), arr(*[int(v) for v in cap]),
                                  out.data_ptr(), _stream()), "block_map")
    return out


def offsets_from_sizes(sizes: torch.Tensor) -> torch.Tensor:
    _need_cuda(sizes)
    s = sizes.to(torch.int32).contiguous()
    BH, K = s.shape
    off = torch.empty(BH, K + 1, dtype=torch.int32, device=s.device)
    check(LIB.svoo_b200_offsets_from_sizes(s.data_ptr(), BH, K, off.data_ptr(), _stream()), "offsets_from_sizes")
    return off


def sparse_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, block_map_u8: torch.Tensor,
                q_offsets: torch.Tensor, k_offsets: torch.Tensor, sm_scale: Optional[float] = None,
                out_row_idx: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                kernel: str = "tcgen05", peer_out=None, return_lse: bool = False):
    """Block-sparse attention over cluster-ordered q,k,v [BH,S,128].  With out_row_idx the
    result rows are scattered to their original positions (fused inverse permutation).
    kernel="simt" selects the mma.sync cross-check kernel.  peer_out = (peer pointer array,
    head id array, world, n_loc, H): the rows are stored into the ranks' sequence shards
    instead of a local tensor (svoo_b200_sparse_attn_push) and nothing is returned.
    return_lse: also return fp32 [BH, S], log2 of every row's softmax denominator (-inf for a row
    without keys), indexed like the output rows."""
    _need_cuda(q, k, v, block_map_u8, q_offsets, k_offsets)
    BH, S, D = _tokens(q)
    QC, KC = q_offsets.shape[1] - 1, k_offsets.shape[1] - 1
    if tuple(block_map_u8.shape) != (BH, QC, KC) or block_map_u8.dtype not in (torch.uint8, torch.bool):
        raise ValueError("block map must be uint8/bool [BH, QC, KC]")
    if kernel not in ("tcgen05", "simt"):
        raise ValueError("kernel must be 'tcgen05' or 'simt'")
    ws = workspace(q.device, BH, S, QC, KC)
    scale = D ** -0.5 if sm_scale is None else float(sm_scale)
    ridx = 0 if out_row_idx is None else out_row_idx.data_ptr()
    if peer_out is not None:
        if kernel != "tcgen05":
            raise ValueError("peer stores need the tcgen05 kernel")
        ptrs, heads, world, n_loc, H = peer_out
        rc = LIB.svoo_b200_sparse_attn_push(q.data_ptr(), k.data_ptr(), v.data_ptr(), block_map_u8.data_ptr(),
                                            q_offsets.data_ptr(), k_offsets.data_ptr(), BH, S, D, QC, KC, scale, ptrs,
                                            heads, world, n_loc, H, ridx, ws.data_ptr(), ws.numel(), _stream())
        check(rc, "sparse_attn_push")
        return None
    y = torch.empty_like(q) if out is None else out
    head = (q.data_ptr(), k.data_ptr(), v.data_ptr(), block_map_u8.data_ptr(), q_offsets.data_ptr(),
            k_offsets.data_ptr(), BH, S, D, QC, KC, scale, y.data_ptr())
    if kernel == "tcgen05":
        lse = torch.empty(BH, S, dtype=torch.float32, device=q.device) if return_lse else None
        rc = LIB.svoo_b200_sparse_attn(*head, ridx, 0 if lse is None else lse.data_ptr(), ws.data_ptr(), ws.numel(),
                                       _stream())
        check(rc, "sparse_attn")
        return (y, lse) if return_lse else y
    if return_lse:
        raise ValueError("the log-sum-exp output needs the tcgen05 kernel")
    check(LIB.svoo_b200_sparse_attn_simt(*head, ridx, ws.data_ptr(), ws.numel(), _stream()), "sparse_attn")
    return y


def attention_status(device: torch.device, BH: int, S: int, QC: int, KC: int) -> int:
    """Status word of the last svoo_b200_sparse_attn call that used this device's cached
    workspace with these sizes (synchronises).  0 = every CTA completed; non-zero = a CTA gave
    up on a bounded barrier wait and left its rows unwritten."""
    off = ctypes.c_int64(0)
    check(LIB.svoo_b200_status_offset(BH, S, QC, KC, ctypes.byref(off)), "status_offset")
    ws = workspace(device, BH, S, QC, KC)
    return int(ws[off.value:off.value + 4].view(torch.int32).item())


def cluster_status(device: torch.device, BH: int, N: int, QC: int, KC: int) -> int:
    """Same as attention_status for the assignment kernel of the last cocluster /
    cocluster_assign call (status word 1)."""
    off = ctypes.c_int64(0)
    check(LIB.svoo_b200_status_offset(BH, N, QC, KC, ctypes.byref(off)), "status_offset")
    ws = workspace(device, BH, N, QC, KC)
    return int(ws[off.value + 4:off.value + 8].view(torch.int32).item())


def qk_prep(x: torch.Tensor, heads: int, weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
            cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The producer of the path's inputs in one pass: x [S, H*128] bf16 (a projection output) ->
    [H, S, 128] with the RMS norm over all H*128 columns (weight [H*128], any float dtype),
    the interleaved-pair rotary embedding (cos, sin [S, 128], the full-width tables; even cos and
    odd sin entries are used) and the head transpose.  weight / cos None skip that part (V)."""
    _need_cuda(x)
    if x.dim() != 2 or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.shape[1] != heads * 128:
        raise ValueError("x must be contiguous bf16 [S, H*128]")
    S = x.shape[0]
    w = None if weight is None else weight.detach().to(device=x.device, dtype=torch.float32).contiguous()
    if w is not None and w.numel() != heads * 128:
        raise ValueError("weight must have H*128 entries")
    c = s_ = None
    if cos is not None:
        c = cos.to(device=x.device, dtype=torch.float32).reshape(S, 128).contiguous()
        s_ = sin.to(device=x.device, dtype=torch.float32).reshape(S, 128).contiguous()
    out = torch.empty(heads, S, 128, dtype=torch.bfloat16, device=x.device)
    check(LIB.svoo_b200_qk_prep(x.data_ptr(), 0 if w is None else w.data_ptr(), float(eps), 0 if c is None else c.data_ptr(),
                                0 if s_ is None else s_.data_ptr(), S, heads, 128, out.data_ptr(), _stream()), "qk_prep")
    return out


def qk_prep_heads(x: torch.Tensor, heads: int, weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                  cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None, rope_rows: Optional[int] = None,
                  out: Optional[torch.Tensor] = None, out_row0: int = 0) -> torch.Tensor:
    """HunyuanVideo's producer in one pass: x [S, H*128] bf16 -> rows [out_row0, out_row0 + S) of
    out [H, rows, 128] with the RMS norm over the 128 values of every (token, head) (weight [128]),
    the interleaved-pair rotary embedding of the first `rope_rows` tokens (cos, sin [>= rope_rows, 128]) and
    the head transpose.  weight / cos None skip that part."""
    _need_cuda(x)
    if x.dim() != 2 or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.shape[1] != heads * 128:
        raise ValueError("x must be contiguous bf16 [S, H*128]")
    S = x.shape[0]
    w = None if weight is None else weight.detach().to(device=x.device, dtype=torch.float32).contiguous()
    if w is not None and w.numel() != 128:
        raise ValueError("weight must have 128 entries")
    rr = 0
    c = s_ = None
    if cos is not None:
        rr = S if rope_rows is None else int(rope_rows)
        c = cos.to(device=x.device, dtype=torch.float32).reshape(-1, 128).contiguous()
        s_ = sin.to(device=x.device, dtype=torch.float32).reshape(-1, 128).contiguous()
        if c.shape[0] < rr or s_.shape[0] < rr:
            raise ValueError("cos / sin need at least rope_rows rows")
    if out is None:
        out = torch.empty(heads, out_row0 + S, 128, dtype=torch.bfloat16, device=x.device)
    if out.dim() != 3 or out.shape[0] != heads or out.shape[2] != 128 or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be contiguous bf16 [H, rows, 128]")
    check(LIB.svoo_b200_qk_prep_heads(x.data_ptr(), 0 if w is None else w.data_ptr(), float(eps),
                                      0 if c is None else c.data_ptr(), 0 if s_ is None else s_.data_ptr(), S, heads, 128, rr,
                                      out.data_ptr(), out.shape[1], int(out_row0), _stream()), "qk_prep_heads")
    return out


def layer(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_init_idx: torch.Tensor, k_init_idx: torch.Tensor,
          iters: int, top_p: float, preserve: Sequence[int], cap: Sequence[int],
          sm_scale: Optional[float] = None, text: int = 0, prompt: int = 0) -> torch.Tensor:
    """The whole layer through the single C entry point svoo_b200_layer: q, k, v [BH, S, 128] bf16
    in token order -> out [BH, S, 128]; the last `text` rows of every head are text tokens, of
    which the first `prompt` are the prompt.  Intermediates live in a scratch block that is
    released with the returned tensor's call frame; use the separate ops when they are needed."""
    _need_cuda(q, k, v, q_init_idx, k_init_idx)
    BH, S, D = _tokens(q)
    QC, KC = q_init_idx.shape[-1], k_init_idx.shape[-1]
    if len(preserve) != BH or len(cap) != BH:
        raise ValueError("preserve and cap need one entry per head")
    nbytes = ctypes.c_int64(0)
    check(LIB.svoo_b200_layer_scratch_bytes(BH, S, QC, KC, int(text), ctypes.byref(nbytes)), "layer_scratch_bytes")
    scratch = torch.empty(nbytes.value, dtype=torch.uint8, device=q.device)
    ws = workspace(q.device, BH, S, QC + 2, KC + 2) if text else workspace(q.device, BH, S, QC, KC)
    out = torch.empty_like(q)
    arr = ctypes.c_int32 * BH
    qi, ki = q_init_idx.to(torch.int32).contiguous(), k_init_idx.to(torch.int32).contiguous()
    check(LIB.svoo_b200_layer(q.data_ptr(), k.data_ptr(), v.data_ptr(), qi.data_ptr(), ki.data_ptr(), BH, S, D, QC, KC,
                              int(iters), float(top_p), arr(*[int(x) for x in preserve]), arr(*[int(x) for x in cap]),
                              D ** -0.5 if sm_scale is None else float(sm_scale), int(text), int(prompt), out.data_ptr(),
                              scratch.data_ptr(), scratch.numel(), ws.data_ptr(), ws.numel(), _stream()), "layer")
    return out


# ----------------------------------------------------------------------------------------------
# Error-aware routing (EAR)
# ----------------------------------------------------------------------------------------------
_ear_workspaces = {}


def ear_workspace(device: torch.device, BH: int, N: int, QC: int, KC: int) -> torch.Tensor:
    """Cached scratch of the EAR calls (one per device and stream); it carries the value statistics
    from ear_value_centroids to ear_block_scores."""
    need, _ = _ear_sizes(BH, N, QC, KC)
    key = (device.index if device.index is not None else torch.cuda.current_device(), _stream())
    ws = _ear_workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        _ear_workspaces[key] = ws
    return ws


def _ear_sizes(BH, N, QC, KC):
    need, status = ctypes.c_int64(0), ctypes.c_int64(0)
    check(LIB.svoo_b200_ear_workspace_bytes(BH, N, QC, KC, ctypes.byref(need), ctypes.byref(status)), "ear_workspace_bytes")
    return need.value, status.value


def ear_value_centroids(v_perm: torch.Tensor, k_offsets: torch.Tensor, QC: int, out: Optional[torch.Tensor] = None):
    """Mean value row of every key cluster, bf16 [BH, KC, 128] (written into `out` when given, e.g. the
    centroid rows of an extended V tensor); the per-token statistics the block scores need stay in
    the EAR scratch of this device and stream."""
    _need_cuda(v_perm, k_offsets)
    BH, N, D = _tokens(v_perm)
    KC = k_offsets.shape[1] - 1
    vc = torch.empty(BH, KC, HEAD_DIM, dtype=torch.bfloat16, device=v_perm.device) if out is None else out
    ws = ear_workspace(v_perm.device, BH, N, QC, KC)
    check(LIB.svoo_b200_ear_value_centroids(v_perm.data_ptr(), k_offsets.data_ptr(), BH, N, D, QC, KC, vc.data_ptr(),
                                            ws.data_ptr(), ws.numel(), _stream()), "ear_value_centroids")
    return vc


def ear_block_scores(qcentroids: torch.Tensor, kcentroids: torch.Tensor, k_perm: torch.Tensor, q_offsets: torch.Tensor,
                     k_offsets: torch.Tensor, gamma: float):
    """(centroid logits, log-efficiency scores), fp32 [BH, QC, KC]; after ear_value_centroids on this
    device and stream."""
    _need_cuda(qcentroids, kcentroids, k_perm, q_offsets, k_offsets)
    BH, N, D = _tokens(k_perm)
    QC, KC = q_offsets.shape[1] - 1, k_offsets.shape[1] - 1
    if qcentroids.dtype != torch.bfloat16 or kcentroids.dtype != torch.bfloat16:
        raise ValueError("ear_block_scores needs bf16 centroids")
    clog = torch.empty(BH, QC, KC, dtype=torch.float32, device=k_perm.device)
    scores = torch.empty_like(clog)
    ws = ear_workspace(k_perm.device, BH, N, QC, KC)
    check(LIB.svoo_b200_ear_block_scores(qcentroids.contiguous().data_ptr(), kcentroids.contiguous().data_ptr(),
                                         k_perm.data_ptr(), q_offsets.data_ptr(), k_offsets.data_ptr(), BH, N, D, QC, KC,
                                         float(gamma), clog.data_ptr(), scores.data_ptr(), ws.data_ptr(), ws.numel(),
                                         _stream()), "ear_block_scores")
    return clog, scores


def ear_select_blocks(c_logits: torch.Tensor, scores: torch.Tensor, q_offsets: torch.Tensor, k_offsets: torch.Tensor,
                      top_p: float, preserve: Sequence[int], budget_preserve: Sequence[int]) -> torch.Tensor:
    """uint8 [BH, QC, KC]; preserve / budget_preserve are per-head python ints (numbers of key clusters)."""
    _need_cuda(c_logits, scores, q_offsets, k_offsets)
    BH, QC, KC = c_logits.shape
    if len(preserve) != BH or len(budget_preserve) != BH:
        raise ValueError("preserve and budget_preserve need one entry per head")
    if c_logits.dtype != torch.float32 or scores.dtype != torch.float32 or tuple(scores.shape) != (BH, QC, KC):
        raise ValueError("c_logits and scores must be fp32 [BH, QC, KC]")
    out = torch.empty(BH, QC, KC, dtype=torch.uint8, device=c_logits.device)
    arr = ctypes.c_int32 * BH
    check(LIB.svoo_b200_ear_select_blocks(c_logits.contiguous().data_ptr(), scores.contiguous().data_ptr(),
                                          q_offsets.data_ptr(), k_offsets.data_ptr(), BH, QC, KC, float(top_p),
                                          arr(*[int(v) for v in preserve]), arr(*[int(v) for v in budget_preserve]),
                                          out.data_ptr(), _stream()), "ear_select_blocks")
    return out


def sparse_attn_ear(q: torch.Tensor, k_ext: torch.Tensor, v_ext: torch.Tensor, block_map_u8: torch.Tensor,
                    q_offsets: torch.Tensor, k_offsets: torch.Tensor, sm_scale: Optional[float] = None,
                    out_row_idx: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                    return_lse: bool = False, peer_out=None):
    """EAR forward: q [BH,S,128] in cluster order; k_ext, v_ext [BH*S + BH*KC, 128] = the cluster-ordered
    rows of all heads followed by the key / value centroid rows of all heads.  Output, out_row_idx, the
    log2-sum-exp and peer_out as in sparse_attn."""
    _need_cuda(q, k_ext, v_ext, block_map_u8, q_offsets, k_offsets)
    BH, S, D = _tokens(q)
    QC, KC = q_offsets.shape[1] - 1, k_offsets.shape[1] - 1
    if tuple(block_map_u8.shape) != (BH, QC, KC) or block_map_u8.dtype not in (torch.uint8, torch.bool):
        raise ValueError("block map must be uint8/bool [BH, QC, KC]")
    for t in (k_ext, v_ext):
        if tuple(t.shape) != (BH * S + BH * KC, HEAD_DIM) or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError("k_ext and v_ext must be contiguous bf16 [BH*S + BH*KC, 128]")
    ws = ear_workspace(q.device, BH, S, QC, KC)
    if peer_out is not None:
        ptrs, heads, world, n_loc, H = peer_out
        check(LIB.svoo_b200_sparse_attn_ear_push(q.data_ptr(), k_ext.data_ptr(), v_ext.data_ptr(), block_map_u8.data_ptr(),
                                                 q_offsets.data_ptr(), k_offsets.data_ptr(), BH, S, D, QC, KC,
                                                 D ** -0.5 if sm_scale is None else float(sm_scale), ptrs, heads, world, n_loc,
                                                 H, 0 if out_row_idx is None else out_row_idx.data_ptr(), ws.data_ptr(),
                                                 ws.numel(), _stream()), "sparse_attn_ear_push")
        return None
    y = torch.empty_like(q) if out is None else out
    lse = torch.empty(BH, S, dtype=torch.float32, device=q.device) if return_lse else None
    check(LIB.svoo_b200_sparse_attn_ear(q.data_ptr(), k_ext.data_ptr(), v_ext.data_ptr(), block_map_u8.data_ptr(),
                                        q_offsets.data_ptr(), k_offsets.data_ptr(), BH, S, D, QC, KC,
                                        D ** -0.5 if sm_scale is None else float(sm_scale), y.data_ptr(),
                                        0 if out_row_idx is None else out_row_idx.data_ptr(),
                                        0 if lse is None else lse.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
          "sparse_attn_ear")
    return (y, lse) if return_lse else y


def ear_attention_status(device: torch.device, BH: int, S: int, QC: int, KC: int) -> int:
    """Status word of the last sparse_attn_ear on this device and stream (0 = no bounded wait expired)."""
    _, off = _ear_sizes(BH, S, QC, KC)
    ws = ear_workspace(device, BH, S, QC, KC)
    return int(ws[off:off + 4].view(torch.int32).item())
