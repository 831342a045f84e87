"""Head-sharded execution of the sparse-attention layer over torch.distributed.

The reference runs on one GPU.  Every stage of the path is independent per head, so
with P ranks each rank computes H/P heads; when the activations arrive sharded by
sequence (Ulysses layout), one all-to-all turns [N/P, H, D] per rank into [H/P, N, D]
and a second one brings the result back.  There is no other exchange: no collective
touches labels, centroids or the map.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def head_partition(num_heads: int, world: int, weights: Optional[Sequence[float]] = None) -> List[List[int]]:
    """Heads of each rank.  Equal counts per rank (the all-to-all below needs that when H
    divides by P; otherwise the first H % P ranks take one more).  With `weights` (for
    example the per-head density budget) heads are dealt greedily, heaviest first, to the
    rank with the least total weight that still has room, which evens out the attention work."""
    base, extra = divmod(num_heads, world)
    room = [base + (1 if r < extra else 0) for r in range(world)]
    parts: List[List[int]] = [[] for _ in range(world)]
    if weights is None:
        h = 0
        for r in range(world):
            parts[r] = list(range(h, h + room[r]))
            h += room[r]
        return parts
    load = [0.0] * world
    for h in sorted(range(num_heads), key=lambda i: (-float(weights[i]), i)):
        r = min((r for r in range(world) if len(parts[r]) < room[r]), key=lambda r: (load[r], r))
        parts[r].append(h)
        load[r] += float(weights[h])
    return [sorted(p) for p in parts]


_order_cache = {}


def _order(parts: List[List[int]], device) -> torch.Tensor:
    """Head index vector [hr * P]: entry i * P + p is the i-th head of rank p (cached per device)."""
    key = (tuple(tuple(p) for p in parts), str(device))
    t = _order_cache.get(key)
    if t is None:
        hr = len(parts[0])
        t = torch.tensor([parts[p][i] for i in range(hr) for p in range(len(parts))], dtype=torch.long, device=device)
        _order_cache[key] = t
    return t


def seq_to_head_shard(x: torch.Tensor, parts: List[List[int]], group=None) -> torch.Tensor:
    """x: this rank's sequence shard [N/P, H, D] -> this rank's heads over the whole
    sequence [H_r, N, D].  Needs the same number of heads on every rank.

    One pass packs the shard as [hr, P, N/P, D] (block (i, p) = the i-th head of rank p); then
    one all-to-all per local head index i exchanges its [P, N/P, D] blocks, which land as that
    head's [N, D] rows directly -- no copy after the exchange."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n_loc, H, D = x.shape
    hr = len(parts[rank])
    assert all(len(p) == hr for p in parts), "equal head counts per rank are required"
    send = x.transpose(0, 1)[_order(parts, x.device)]                    # [hr * P, N/P, D], the one copy
    out = torch.empty(hr, world * n_loc, D, dtype=x.dtype, device=x.device)
    for i in range(hr):
        dist.all_to_all_single(out[i], send[i * world:(i + 1) * world].view(world * n_loc, D), group=group)
    return out


def head_to_seq_shard(y: torch.Tensor, parts: List[List[int]], group=None) -> torch.Tensor:
    """Inverse of seq_to_head_shard: [H_r, N, D] -> [N/P, H, D].  The head rows are sent as
    they lie; one pass unpacks the received [hr, P, N/P, D] blocks."""
    world = dist.get_world_size(group)
    hr, N, D = y.shape
    n_loc = N // world
    recv = torch.empty(hr * world, n_loc, D, dtype=y.dtype, device=y.device)
    for i in range(hr):
        dist.all_to_all_single(recv[i * world:(i + 1) * world].view(N, D), y[i], group=group)
    out = torch.empty(n_loc, world * hr, D, dtype=y.dtype, device=y.device)
    out[:, _order(parts, y.device)] = recv.transpose(0, 1)
    return out


def sparse_attention_layer_sharded(q_seq, k_seq, v_seq, parts, *, densities, init_indices, group=None, **layer_kw):
    """Ulysses-style layer: q/k/v_seq are this rank's [N/P, H, 128] shards; returns the
    [N/P, H, 128] shard of the output.  `densities` and `init_indices` are for all H heads;
    each rank takes the entries of its own heads."""
    from .layer import sparse_attention_layer
    rank = dist.get_rank(group)
    mine = parts[rank]
    q = seq_to_head_shard(q_seq, parts, group)
    k = seq_to_head_shard(k_seq, parts, group)
    v = seq_to_head_shard(v_seq, parts, group)
    qi, ki = init_indices
    d = [densities[h] for h in mine]
    out = sparse_attention_layer(q[None], k[None], v[None], min_kc_ratio=d, max_kc_ratio=d,
                                 init_indices=(qi[mine], ki[mine]), **layer_kw)
    return head_to_seq_shard(out[0], parts, group)
