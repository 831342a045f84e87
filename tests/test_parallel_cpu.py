"""Head sharding and the Ulysses all-to-all layouts, world_size 2 and 4 over gloo on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from svoo_b200 import parallel


def test_head_partition():
    assert parallel.head_partition(40, 8) == [list(range(i * 5, i * 5 + 5)) for i in range(8)]
    parts = parallel.head_partition(12, 8)
    assert [len(p) for p in parts] == [2, 2, 2, 2, 1, 1, 1, 1]
    assert sorted(h for p in parts for h in p) == list(range(12))
    w = [0.25, 0.05, 0.24, 0.06, 0.2, 0.1, 0.15, 0.15]
    parts = parallel.head_partition(8, 4, w)
    assert sorted(h for p in parts for h in p) == list(range(8)) and all(len(p) == 2 for p in parts)
    loads = [sum(w[h] for h in p) for p in parts]
    assert max(loads) - min(loads) < 0.011                    # contiguous split would give 0.30 vs 0.30 vs ... worse
    contiguous = [sum(w[2 * r:2 * r + 2]) for r in range(4)]
    assert max(loads) <= max(contiguous)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, H, N, weights):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        D = 8
        g = torch.Generator().manual_seed(0)
        full = torch.randn(N, H, D, generator=g)              # the same on every rank
        n_loc = N // world
        mine = full[rank * n_loc:(rank + 1) * n_loc].contiguous()
        parts = parallel.head_partition(H, world, weights)
        heads = parallel.seq_to_head_shard(mine, parts)
        expect = full[:, parts[rank], :].permute(1, 0, 2)
        assert torch.equal(heads, expect), "sequence -> head shard layout"
        back = parallel.head_to_seq_shard(heads * 2.0, parts)
        assert torch.equal(back, mine * 2.0), "head -> sequence shard layout"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,H,weights", [(2, 4, None), (2, 6, [0.3, 0.1, 0.2, 0.05, 0.25, 0.1]), (4, 8, None)])
def test_ulysses_layout_round_trip(world, H, weights):
    mp.spawn(_worker, args=(world, _free_port(), H, 24, weights), nprocs=world, join=True)


def test_exchange_tables_reproduce_the_all_to_all_layout():
    """The owner/slot tables the peer-store kernels index with, replayed in numpy with the
    kernels' row arithmetic, give the head-shard layout and its inverse."""
    import numpy as np
    from svoo_b200.parallel import exchange_tables, head_partition
    world, H, n_loc, D = 4, 8, 5, 3
    N = world * n_loc
    parts = head_partition(H, world, [0.3, 0.1, 0.2, 0.25, 0.05, 0.15, 0.22, 0.12])
    owner, slot = exchange_tables(parts)
    hr = H // world
    assert sorted(zip(owner, slot)) == [(r, i) for r in range(world) for i in range(hr)]
    rng = np.random.default_rng(0)
    full = rng.standard_normal((H, N, D)).astype(np.float32)
    recv = [np.zeros((hr, N, D), np.float32) for _ in range(world)]
    for rank in range(world):                                   # push_heads of every rank
        x = full[:, rank * n_loc:(rank + 1) * n_loc].transpose(1, 0, 2).reshape(n_loc * H, D)
        for t in range(n_loc * H):
            r, h = divmod(t, H)
            recv[owner[h]].reshape(hr * N, D)[slot[h] * N + rank * n_loc + r] = x[t]
    for rank in range(world):
        assert np.array_equal(recv[rank], full[parts[rank]])
    seq = [np.zeros((n_loc * H, D), np.float32) for _ in range(world)]
    for rank in range(world):                                   # push_seq of every rank
        y = recv[rank].reshape(hr * N, D)
        for t in range(hr * N):
            i, n = divmod(t, N)
            p = n // n_loc
            seq[p][(n - p * n_loc) * H + parts[rank][i]] = y[t]
    for rank in range(world):
        want = full[:, rank * n_loc:(rank + 1) * n_loc].transpose(1, 0, 2).reshape(n_loc * H, D)
        assert np.array_equal(seq[rank], want)


def test_head_partition_properties():
    """Every head exactly once, equal counts when H divides by P, deterministic, and the heaviest
    rank never heavier than with contiguous blocks of heads."""
    import random
    from svoo_b200.parallel import head_partition
    rnd = random.Random(3)
    for H, P in ((40, 8), (40, 4), (24, 8), (12, 4), (7, 3), (5, 5)):
        w = [rnd.uniform(0.05, 0.3) for _ in range(H)]
        parts = head_partition(H, P, w)
        assert parts == head_partition(H, P, w)
        assert sorted(h for p in parts for h in p) == list(range(H))
        sizes = sorted(len(p) for p in parts)
        assert sizes[-1] - sizes[0] <= 1
        load = max(sum(w[h] for h in p) for p in parts)
        plain = head_partition(H, P)
        assert load <= max(sum(w[h] for h in p) for p in plain) + 1e-12
    # the bench configuration: 40 heads with the seeded density budget over 8 ranks
    from svoo_b200 import synth
    d = synth.head_densities(synth.CONFIGS["cfg2"])
    loads = [sum(d[h] for h in p) for p in head_partition(40, 8, d)]
    assert max(loads) / (sum(loads) / 8) < 1.01


def test_exchange_tables_uneven_split():
    """12 heads on 8 ranks (the Wan-1.3B head count on a full node): four ranks own two heads, four
    own one; every receive array has ceil(12 / 8) = 2 head slots, and the kernels' row arithmetic
    (replayed in numpy) still puts every row where the head-shard layout wants it, both ways."""
    import numpy as np
    from svoo_b200.parallel import exchange_tables, head_partition
    world, H, n_loc, D = 8, 12, 3, 2
    N = world * n_loc
    rng = np.random.default_rng(1)
    parts = head_partition(H, world, list(rng.uniform(0.05, 0.3, H)))
    assert sorted(len(p) for p in parts) == [1, 1, 1, 1, 2, 2, 2, 2]
    owner, slot = exchange_tables(parts)
    hr = -(-H // world)
    assert len(set(zip(owner, slot))) == H and max(slot) < hr
    full = rng.standard_normal((H, N, D)).astype(np.float32)
    recv = [np.full((hr, N, D), np.nan, np.float32) for _ in range(world)]
    for rank in range(world):
        x = full[:, rank * n_loc:(rank + 1) * n_loc].transpose(1, 0, 2).reshape(n_loc * H, D)
        for t in range(n_loc * H):
            r, h = divmod(t, H)
            recv[owner[h]].reshape(hr * N, D)[slot[h] * N + rank * n_loc + r] = x[t]
    seq = [np.full((n_loc * H, D), np.nan, np.float32) for _ in range(world)]
    for rank in range(world):
        mine = parts[rank]
        assert np.array_equal(recv[rank][:len(mine)], full[mine])
        y = recv[rank][:len(mine)].reshape(len(mine) * N, D)
        for t in range(len(mine) * N):
            i, n = divmod(t, N)
            p = n // n_loc
            seq[p][(n - p * n_loc) * H + mine[i]] = y[t]
    for rank in range(world):
        want = full[:, rank * n_loc:(rank + 1) * n_loc].transpose(1, 0, 2).reshape(n_loc * H, D)
        assert np.array_equal(seq[rank], want)
