"""The whole sparse-attention layer as one stream-ordered sequence of kernels:
co-clustering -> cluster-order permute -> cluster-block map -> block-sparse attention with
the inverse permutation fused into its store.

Replaces semantic_aware_permutation + the sparse branch of attention_core_logic
(svoo/models/wan/attention.py:958-1088,1159-1216) and, with text tokens, the
Hunyuan variant (svoo/models/hunyuan10/attention.py:977-1110).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from . import co_clustering as cc
from . import ops


class StageTimer:
    """CUDA-event marks on the launching stream, one per stage boundary of a layer call.
    After a synchronize, `stage_ms()` gives the device time between consecutive marks."""

    def __init__(self):
        self.marks = []

    def mark(self, name: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream())
        self.marks.append((name, ev))

    def stage_ms(self):
        out = {}
        for (_, a), (name, b) in zip(self.marks[:-1], self.marks[1:]):
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out


@dataclasses.dataclass
class LayerState:
    """What a layer call leaves behind; `clustering` can be fed back in to reuse it."""
    clustering: ops.Clustering
    block_map: torch.Tensor          # uint8 [H, QC(+2), KC(+2)]
    q_offsets: torch.Tensor
    k_offsets: torch.Tensor


def sparse_attention_layer(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, *, num_q_centroids: int,
                           num_k_centroids: int, kmeans_iters: int, top_p: float, min_kc_ratio=0, max_kc_ratio=0,
                           init_indices=None, clustering: Optional[ops.Clustering] = None,
                           context_length: int = 0, prompt_length: Optional[int] = None,
                           return_state: bool = False, timer: Optional[StageTimer] = None,
                           value_ready: Optional[torch.cuda.Event] = None, peer_out=None,
                           ear_gamma: Optional[float] = None):
    """query/key/value: [1, H, S, 128] bf16 CUDA, S = video tokens + context_length text
    tokens (text last, never clustered).  Returns [1, H, S, 128] in the original token order.
    `value_ready`: an event the launching stream waits for before it first reads `value`
    (the clustering only reads query and key, so V may still be arriving while it runs).
    `peer_out` (see ops.sparse_attn): the output rows are stored into the ranks' sequence
    shards by the attention kernel itself and the returned tensor is None."""
    cfg, H, S, D = query.shape
    assert cfg == 1, "Batch size must be 1 for kmeans block sparse attention"
    assert query.is_cuda and query.dtype == torch.bfloat16, "bf16 CUDA tensors expected"
    n_video = S - context_length
    q, k, v = query[0], key[0], value[0]
    mark = timer.mark if timer is not None else (lambda name: None)
    mark("start")
    c = clustering
    if c is None:
        if context_length:
            qv, kv = q[:, :n_video].contiguous(), k[:, :n_video].contiguous()
        else:
            qv, kv = q.contiguous(), k.contiguous()
        c = cc.co_cluster(qv, kv, num_q_centroids, num_k_centroids, kmeans_iters, init_indices=init_indices)
        del qv, kv
    mark("cocluster")
    if ear_gamma is not None:
        return _ear_layer(q, k, v, c, top_p, min_kc_ratio, float(ear_gamma), context_length, peer_out, value_ready, mark,
                          return_state)
    preserve, cap = cc.keep_limits(num_k_centroids, H, min_kc_ratio, max_kc_ratio)
    if top_p >= 1.0:
        m = torch.ones(H, num_q_centroids, num_k_centroids, dtype=torch.uint8, device=q.device)
    else:
        m = ops.block_map(c.qcentroids, c.kcentroids, c.ksizes, top_p, preserve, cap)
    mark("block_map")

    if context_length == 0:
        m_full, q_off, k_off = m, c.q_offsets, c.k_offsets
        q_idx, k_idx = c.q_sorted_idx, c.k_sorted_idx
    else:
        # text tokens stay where they are, as two extra blocks (prompt, unused prompt)
        prompt = context_length if prompt_length is None else prompt_length
        m_full, q_off, k_off, q_idx, k_idx = ops.append_text_blocks(m, c.q_offsets, c.k_offsets, c.q_sorted_idx,
                                                                    c.k_sorted_idx, context_length, prompt)
    m = m_full
    if value_ready is not None:
        torch.cuda.current_stream(q.device).wait_event(value_ready)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    qp, kp, vp = ops.permute(q, q_idx), ops.permute(k, k_idx), ops.permute(v, k_idx)
    mark("permute")
    out = ops.sparse_attn(qp, kp, vp, m.contiguous(), q_off, k_off, D ** -0.5, out_row_idx=q_idx, peer_out=peer_out)
    mark("attention")
    if out is not None:
        out = out.unsqueeze(0)
    if return_state:
        return out, LayerState(c, m, q_off, k_off)
    return out


def _ear_layer(q, k, v, c, top_p, min_kc_ratio, gamma, context_length, peer_out, value_ready, mark, return_state):
    """The error-aware routing variant after the clustering (svoo/models/wan/attention.py:1037-1076,
    1184-1196): permute, value centroids, block scores, budgeted selection, attention with one virtual
    key per pruned cluster.  K and V are permuted straight into the [H*S + H*KC, 128] tensors the
    kernel reads (token rows of all heads, then centroid rows of all heads)."""
    if context_length:
        raise ValueError("the EAR variant covers video-only self attention, as in the reference")
    H, S, D = q.shape
    QC, KC = c.qcentroids.shape[1], c.kcentroids.shape[1]
    if value_ready is not None:
        torch.cuda.current_stream(q.device).wait_event(value_ready)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    k_ext = torch.empty(H * S + H * KC, D, dtype=q.dtype, device=q.device)
    v_ext = torch.empty_like(k_ext)
    kp, vp = k_ext[:H * S].view(H, S, D), v_ext[:H * S].view(H, S, D)
    qp = ops.permute(q, c.q_sorted_idx)
    ops.permute(k, c.k_sorted_idx, out=kp)
    ops.permute(v, c.k_sorted_idx, out=vp)
    k_ext[H * S:].view(H, KC, D).copy_(c.kcentroids)
    mark("permute")
    ops.ear_value_centroids(vp, c.k_offsets, QC, out=v_ext[H * S:].view(H, KC, D))
    clog, scores = ops.ear_block_scores(c.qcentroids, c.kcentroids, kp, c.q_offsets, c.k_offsets, gamma)
    preserve, budget = cc.ear_limits(KC, H, min_kc_ratio)
    m = ops.ear_select_blocks(clog, scores, c.q_offsets, c.k_offsets, top_p, preserve, budget)
    mark("block_map")
    out = ops.sparse_attn_ear(qp, k_ext, v_ext, m, c.q_offsets, c.k_offsets, D ** -0.5, out_row_idx=c.q_sorted_idx,
                              peer_out=peer_out)
    mark("attention")
    if out is not None:
        out = out.unsqueeze(0)
    if return_state:
        return out, LayerState(c, m, c.q_offsets, c.k_offsets)
    return out


class HostLayerPipeline:
    """The layer for callers whose Q, K, V live in (pinned) host memory: heads are processed in
    groups, and the host-to-device copy of group g+1 and the device-to-host copy of group g-1
    run on their own streams while group g computes (heads are independent, so nothing else
    changes).  Buffers are allocated once and reused by every call; the buffer hand-over events
    persist across calls, so the copies of a call also overlap the tail of the previous one.
    A call returns when its work is enqueued: `wait()` (or a device synchronize) before `out_host`
    is read or the input tensors are overwritten."""

    def __init__(self, device: torch.device, heads: int, tokens: int, heads_per_group: int = 5):
        self.device = device
        self.group = max(1, min(heads_per_group, heads))
        self.copy_in = torch.cuda.Stream(device)
        self.copy_out = torch.cuda.Stream(device)
        shape = (1, self.group, tokens, 128)
        self.bufs = [[torch.empty(shape, dtype=torch.bfloat16, device=device) for _ in range(3)] for _ in range(2)]
        self.outs = [torch.empty(shape, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.in_free = [None, None]         # event: compute finished reading input buffer set b
        self.out_free = [None, None]        # event: device-to-host copy of output buffer b finished
        self.n_groups = 0                   # groups processed so far (buffer parity runs on across calls)

    def wait(self) -> None:
        """Blocks the host until every copy and kernel of the calls so far has finished."""
        self.copy_out.synchronize()
        torch.cuda.current_stream(self.device).synchronize()

    def __call__(self, q_host, k_host, v_host, out_host, *, min_kc_ratio, max_kc_ratio, init_indices, **layer_kw):
        """q/k/v_host, out_host: [1, H, S, 128] bf16 pinned host tensors; per-head ratio lists and
        init index tensors [H, *] cover all heads."""
        H = q_host.shape[1]
        compute = torch.cuda.current_stream(self.device)
        groups = [(h0, min(h0 + self.group, H)) for h0 in range(0, H, self.group)]
        qi, ki = init_indices
        for h0, h1 in groups:
            b, n = self.n_groups % 2, h1 - h0
            self.n_groups += 1
            with torch.cuda.stream(self.copy_in):
                if self.in_free[b] is not None:
                    self.copy_in.wait_event(self.in_free[b])
                for dst, src in zip(self.bufs[b], (q_host, k_host, v_host)):
                    dst[:, :n].copy_(src[:, h0:h1], non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(self.copy_in)
            compute.wait_event(loaded)
            if self.out_free[b] is not None:
                compute.wait_event(self.out_free[b])
            qd, kd, vd = (t[:, :n] for t in self.bufs[b])
            out = sparse_attention_layer(qd, kd, vd, min_kc_ratio=list(min_kc_ratio[h0:h1]),
                                         max_kc_ratio=list(max_kc_ratio[h0:h1]),
                                         init_indices=(qi[h0:h1], ki[h0:h1]), **layer_kw)
            self.outs[b][:, :n].copy_(out)
            done = torch.cuda.Event()
            done.record(compute)
            self.in_free[b] = done
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(done)
                out_host[:, h0:h1].copy_(self.outs[b][:, :n], non_blocking=True)
                stored = torch.cuda.Event()
                stored.record(self.copy_out)
            self.out_free[b] = stored
        return out_host
