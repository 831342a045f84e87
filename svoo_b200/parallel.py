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
    # refinement: swap one head of the heaviest rank with one of another rank while that lowers
    # the larger of the two loads (counts stay equal); deterministic, a few dozen swaps at most
    for _ in range(16 * num_heads):
        hi = max(range(world), key=lambda r: (load[r], -r))
        best = None
        for r in range(world):
            if r == hi:
                continue
            for a in parts[hi]:
                for b in parts[r]:
                    delta = float(weights[a]) - float(weights[b])
                    if delta <= 0:
                        continue
                    new_max = max(load[hi] - delta, load[r] + delta)
                    if new_max < load[hi] - 1e-12 and (best is None or new_max < best[0]):
                        best = (new_max, r, a, b)
        if best is None:
            break
        _, r, a, b = best
        parts[hi].remove(a); parts[r].remove(b)
        parts[hi].append(b); parts[r].append(a)
        delta = float(weights[a]) - float(weights[b])
        load[hi] -= delta
        load[r] += delta
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


def exchange_tables(parts: List[List[int]]) -> Tuple[List[int], List[int]]:
    """owner[h] = rank that computes head h, slot[h] = index of h among that rank's heads."""
    H = sum(len(p) for p in parts)
    owner, slot = [0] * H, [0] * H
    for r, heads in enumerate(parts):
        for i, h in enumerate(heads):
            owner[h], slot[h] = r, i
    return owner, slot


class PeerExchange:
    """The two re-shardings of the layer as stores into the peers' memory (one kernel launch
    per tensor, no library all-to-all).  The receive arrays live in symmetric memory that
    every rank of the group maps; a flag barrier kernel on the launching stream
    (svoo_b200_peer_barrier; `fence="nccl"` selects a one-element all-reduce instead) is the
    ordering point between "my stores are issued" and "my array is complete".

    Per layer call: push q, k -> fence -> clustering ... attention -> push out -> fence; V is
    pushed (and fenced) on a side stream while the clustering runs and joined through
    `value_ready` before its first use.  A rank passes a fence only after every peer has
    finished the previous call, so the receive arrays are reused without further ordering."""

    def __init__(self, parts: List[List[int]], n_tokens: int, device, group=None, head_dim: int = 128,
                 fence: str = "flags"):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.parts = parts
        self.H = sum(len(p) for p in parts)
        self.hr = len(parts[self.rank])                      # heads of this rank
        self.hr_max = -(-self.H // self.world)               # room in every receive array
        if n_tokens % self.world:
            raise ValueError("tokens must split evenly over the ranks")
        if min(len(p) for p in parts) < 1 or max(len(p) for p in parts) > self.hr_max:
            raise ValueError("every rank needs between 1 and ceil(H / world) heads")
        self.N, self.n_loc, self.D = n_tokens, n_tokens // self.world, head_dim
        self.heads_in = symm_mem.empty((3, self.hr_max, self.N, head_dim), dtype=torch.bfloat16, device=device)
        self.seq_out = symm_mem.empty((self.n_loc, self.H, head_dim), dtype=torch.bfloat16, device=device)
        h_in = symm_mem.rendezvous(self.heads_in, self.group)
        h_out = symm_mem.rendezvous(self.seq_out, self.group)
        per = self.hr_max * self.N * head_dim * 2
        self._in_ptrs = [(ctypes.c_void_p * self.world)(*[int(p) + t * per for p in h_in.buffer_ptrs]) for t in range(3)]
        self._out_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in h_out.buffer_ptrs])
        owner, slot = exchange_tables(parts)
        self._owner = (ctypes.c_int32 * self.H)(*owner)
        self._slot = (ctypes.c_int32 * self.H)(*slot)
        self._mine = (ctypes.c_int32 * self.hr)(*parts[self.rank])
        self._flag = torch.zeros(2, dtype=torch.int32, device=device)
        if fence not in ("flags", "nccl"):
            raise ValueError("fence must be 'flags' or 'nccl'")
        self._fence_kind = fence
        self._flags = symm_mem.empty((64,), dtype=torch.int32, device=device)     # 4 channels x 16 ranks
        self._flags.zero_()
        h_flags = symm_mem.rendezvous(self._flags, self.group)
        self._flag_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in h_flags.buffer_ptrs])
        self._epoch = [0, 0, 0, 0]
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)                       # every rank's flags are zero before the first epoch
        self._handles = (h_in, h_out, h_flags)
        self._side = torch.cuda.Stream(device)
        self.value_ready: Optional[torch.cuda.Event] = None

    def fence(self, which: int = 0):
        """Orders this rank's earlier peer stores on the current stream before every rank's later
        kernels.  Channel `which` must be used from one stream at a time."""
        if self._fence_kind == "nccl":
            dist.all_reduce(self._flag[which:which + 1], group=self.group)
            return
        from . import _lib
        self._epoch[which] += 1
        stream = torch.cuda.current_stream(self._status.device).cuda_stream
        _lib.check(_lib.LIB.svoo_b200_peer_barrier(self._flag_ptrs, self.world, self.rank, which, self._epoch[which],
                                                   self._status.data_ptr(), stream), "peer_barrier")

    def status(self) -> int:
        """Non-zero if a flag barrier gave up waiting for a rank (synchronises)."""
        return int(self._status.item())

    def _push_heads(self, t: int, x: torch.Tensor, stream: int):
        from . import _lib
        if tuple(x.shape) != (self.n_loc, self.H, self.D) or x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError("sequence shards must be contiguous bf16 [N/P, H, 128]")
        _lib.check(_lib.LIB.svoo_b200_push_heads(x.data_ptr(), self._in_ptrs[t], self._owner, self._slot, self.world,
                                                 self.rank, self.n_loc, self.H, self.D, stream), "push_heads")

    def to_heads(self, q_seq, k_seq, v_seq, overlap_value: bool = True, v_host: Optional[torch.Tensor] = None):
        """[N/P, H, 128] shards of q, k, v -> views [H_r, N, 128] of the receive arrays.  With
        `overlap_value` the V array is complete only after `self.value_ready`.  `v_host`: a pinned
        host copy of the V shard that the side stream first copies into `v_seq` (so that this
        transfer, too, runs behind the clustering)."""
        main = torch.cuda.current_stream(q_seq.device)
        self._push_heads(0, q_seq, main.cuda_stream)
        self._push_heads(1, k_seq, main.cuda_stream)
        if not overlap_value:
            self._push_heads(2, v_seq, main.cuda_stream)
            self.value_ready = None
            self.fence()
        else:
            here = torch.cuda.Event()
            here.record(main)
            self.fence()
            self._side.wait_event(here)
            with torch.cuda.stream(self._side):
                if v_host is not None:
                    v_seq.copy_(v_host, non_blocking=True)
                self._push_heads(2, v_seq, self._side.cuda_stream)
                self.fence(1)
                self.value_ready = torch.cuda.Event()
                self.value_ready.record(self._side)
        return self.heads_in[0, :self.hr], self.heads_in[1, :self.hr], self.heads_in[2, :self.hr]

    def producer_to_heads(self, xq, xk, xv, norm_q, norm_k, cos, sin):
        """to_heads fused with the producer: xq, xk, xv are this rank's [N/P, H*128] projection
        outputs; the RMS norm (norm_q / norm_k = (weight, eps)), the rotary embedding (cos, sin
        [N/P, 128] fp32, this rank's rows) and the head transpose run in the kernel that stores the
        rows into the owning ranks (svoo_b200_qk_prep_push).  Returns the [H_r, N, 128] views;
        V is complete after `self.value_ready`."""
        from . import _lib
        main = torch.cuda.current_stream(xq.device)
        cos = cos.to(torch.float32).reshape(self.n_loc, self.D).contiguous()
        sin = sin.to(torch.float32).reshape(self.n_loc, self.D).contiguous()

        def push(t, x, norm, rope, stream):
            if tuple(x.shape) != (self.n_loc, self.H * self.D) or x.dtype != torch.bfloat16 or not x.is_contiguous():
                raise ValueError("projection outputs must be contiguous bf16 [N/P, H*128]")
            w = None if norm is None else norm[0].detach().to(device=x.device, dtype=torch.float32).contiguous()
            rc = _lib.LIB.svoo_b200_qk_prep_push(x.data_ptr(), 0 if w is None else w.data_ptr(),
                                                 0.0 if norm is None else float(norm[1]),
                                                 cos.data_ptr() if rope else 0, sin.data_ptr() if rope else 0,
                                                 self._in_ptrs[t], self._owner, self._slot, self.world, self.rank,
                                                 self.n_loc, self.H, self.D, stream)
            _lib.check(rc, "qk_prep_push")
            return w                                                  # keep the fp32 weight alive until the launch is queued

        keep = [push(0, xq, norm_q, True, main.cuda_stream), push(1, xk, norm_k, True, main.cuda_stream)]
        here = torch.cuda.Event()
        here.record(main)
        self.fence()
        self._side.wait_event(here)
        with torch.cuda.stream(self._side):
            push(2, xv, None, False, self._side.cuda_stream)
            self.fence(1)
            self.value_ready = torch.cuda.Event()
            self.value_ready.record(self._side)
        del keep
        return self.heads_in[0, :self.hr], self.heads_in[1, :self.hr], self.heads_in[2, :self.hr]

    @property
    def peer_out(self):
        """Argument for sparse_attention_layer(peer_out=...): the attention kernel then stores its
        rows into the ranks' sequence shards itself; call `seq_result()` afterwards."""
        return (self._out_ptrs, self._mine, self.world, self.n_loc, self.H)

    def seq_result(self):
        """After a layer call with `peer_out`: fence, then this rank's [N/P, H, 128] shard."""
        self.fence()
        return self.seq_out

    def to_seq(self, y):
        """This rank's [H_r, N, 128] result -> the [N/P, H, 128] shard (a view of the receive array)."""
        from . import _lib
        if tuple(y.shape) != (self.hr, self.N, self.D) or y.dtype != torch.bfloat16 or not y.is_contiguous():
            raise ValueError("head-sharded result must be contiguous bf16 [H_r, N, 128]")
        stream = torch.cuda.current_stream(y.device).cuda_stream
        _lib.check(_lib.LIB.svoo_b200_push_seq(y.data_ptr(), self._out_ptrs, self._mine, self.hr, self.world, self.n_loc,
                                               self.H, self.D, stream), "push_seq")
        self.fence()
        return self.seq_out


def sparse_attention_layer_sharded(q_seq, k_seq, v_seq, parts, *, densities, init_indices, group=None, exchange=None,
                                   fused_store: bool = True, **layer_kw):
    """Ulysses-style layer: q/k/v_seq are this rank's [N/P, H, 128] shards; returns the
    [N/P, H, 128] shard of the output.  `densities` and `init_indices` are for all H heads;
    each rank takes the entries of its own heads.  With `exchange` (a PeerExchange) the two
    re-shardings are peer stores (the second one issued by the attention kernel itself when
    `fused_store`); without it they are torch.distributed all-to-alls."""
    from .layer import sparse_attention_layer
    rank = dist.get_rank(group)
    mine = parts[rank]
    if exchange is not None:
        q, k, v = exchange.to_heads(q_seq, k_seq, v_seq)
    else:
        q = seq_to_head_shard(q_seq, parts, group)
        k = seq_to_head_shard(k_seq, parts, group)
        v = seq_to_head_shard(v_seq, parts, group)
    qi, ki = init_indices
    d = [densities[h] for h in mine]
    out = sparse_attention_layer(q[None], k[None], v[None], min_kc_ratio=d, max_kc_ratio=d,
                                 init_indices=(qi[mine], ki[mine]),
                                 value_ready=exchange.value_ready if exchange is not None else None,
                                 peer_out=exchange.peer_out if (exchange is not None and fused_store) else None,
                                 **layer_kw)
    if exchange is not None:
        return exchange.seq_result() if fused_store else exchange.to_seq(out[0])
    return head_to_seq_shard(out[0], parts, group)


class HostShardPipeline:
    """The sharded layer for a sequence-parallel caller whose activations live in (pinned) host
    memory: this rank's [N/P, H, 128] shards of q, k, v come from the host and the [N/P, H, 128]
    result shard goes back.  Device buffers are double: the host-to-device copies of call i+1 and
    the device-to-host copy of call i-1 run on their own streams while call i computes.  A call
    returns when its work is enqueued: `wait()` before `out_host` is read or the inputs are
    overwritten."""

    def __init__(self, exchange: PeerExchange, device):
        self.x = exchange
        self.device = device
        shape = (exchange.n_loc, exchange.H, exchange.D)
        self.bufs = [[torch.empty(shape, dtype=torch.bfloat16, device=device) for _ in range(3)] for _ in range(2)]
        self.outs = [torch.empty(shape, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.copy_in = torch.cuda.Stream(device)
        self.copy_out = torch.cuda.Stream(device)
        self.in_free = [None, None]
        self.out_free = [None, None]
        self.calls = 0

    def wait(self) -> None:
        self.copy_out.synchronize()
        torch.cuda.current_stream(self.device).synchronize()

    def __call__(self, q_host, k_host, v_host, out_host, parts, *, densities, init_indices, **layer_kw):
        from .layer import sparse_attention_layer
        x = self.x
        b = self.calls % 2
        self.calls += 1
        compute = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.copy_in):
            if self.in_free[b] is not None:
                self.copy_in.wait_event(self.in_free[b])
            for dst, src in zip(self.bufs[b], (q_host, k_host, v_host)):
                dst.copy_(src, non_blocking=True)
            loaded = torch.cuda.Event()
            loaded.record(self.copy_in)
        compute.wait_event(loaded)
        if self.out_free[b] is not None:
            compute.wait_event(self.out_free[b])
        q, k, v = x.to_heads(*self.bufs[b])
        mine = parts[x.rank]
        qi, ki = init_indices
        d = [densities[h] for h in mine]
        sparse_attention_layer(q[None], k[None], v[None], min_kc_ratio=d, max_kc_ratio=d, init_indices=(qi[mine], ki[mine]),
                               value_ready=x.value_ready, peer_out=x.peer_out, **layer_kw)
        self.outs[b].copy_(x.seq_result())
        done = torch.cuda.Event()
        done.record(compute)
        self.in_free[b] = done
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(done)
            out_host.copy_(self.outs[b], non_blocking=True)
            stored = torch.cuda.Event()
            stored.record(self.copy_out)
        self.out_free[b] = stored
        return out_host
