"""Two-GPU checks of the head-sharded layer: the peer-store re-shard against the
torch.distributed all-to-all, and the sharded layer against the one-GPU layer.
Runs as child processes (one per GPU); skipped with fewer than two GPUs."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["SVOO_ROOT"])
from svoo_b200 import layer, parallel, synth
import dataclasses
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local); dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
cfg = dataclasses.replace(synth.CONFIGS["cfg1"], heads=4)
H, N = cfg.heads, cfg.n_tokens
assert N % world == 0
dens = synth.head_densities(cfg)
parts = parallel.head_partition(H, world, dens)
q, k, v = (t.to(dev) for t in synth.make_qkv(cfg))                      # all heads, on every rank
n_loc = N // world
shard = lambda t: t[0, :, rank * n_loc:(rank + 1) * n_loc].transpose(0, 1).contiguous()   # [n_loc, H, D]
qs, ks, vs = shard(q), shard(k), shard(v)
x = parallel.PeerExchange(parts, N, dev)
for rep in range(2):                                                    # twice: the receive arrays are reused
    got = x.to_heads(qs, ks, vs, overlap_value=bool(rep))
    if x.value_ready is not None:
        torch.cuda.current_stream().wait_event(x.value_ready)
    want = [parallel.seq_to_head_shard(t, parts) for t in (qs, ks, vs)]
    for g, w, full in zip(got, want, (q, k, v)):
        assert torch.equal(g, w), "push_heads differs from the all-to-all"
        assert torch.equal(g, full[0, parts[rank]]), "push_heads differs from the unsharded heads"
    y = got[0].clone()
    back = x.to_seq(y)
    assert torch.equal(back, parallel.head_to_seq_shard(y, parts)), "push_seq differs from the all-to-all"
    assert torch.equal(back, qs), "round trip"
qi, ki = synth.init_indices(cfg)
kw = dict(num_q_centroids=cfg.num_q, num_k_centroids=cfg.num_k, kmeans_iters=cfg.iters, top_p=cfg.top_p)
outs = [parallel.sparse_attention_layer_sharded(qs, ks, vs, parts, densities=dens, init_indices=(qi.to(dev), ki.to(dev)),
                                                exchange=x, fused_store=f, **kw).clone() for f in (False, True)]
assert torch.equal(outs[0], outs[1]), "fused peer store differs from push_seq"
out = outs[1]
ref = layer.sparse_attention_layer(q, k, v, min_kc_ratio=dens, max_kc_ratio=dens, init_indices=(qi.to(dev), ki.to(dev)), **kw)
assert torch.equal(out, shard(ref)), "sharded layer differs from the one-GPU layer"
assert x.status() == 0, "a flag barrier timed out"
y = parallel.PeerExchange(parts, N, dev, fence="nccl")
out2 = parallel.sparse_attention_layer_sharded(qs, ks, vs, parts, densities=dens, init_indices=(qi.to(dev), ki.to(dev)),
                                               exchange=y, **kw)
assert torch.equal(out2, out), "NCCL-fenced run differs from the flag-fenced run"
# producer fused with the re-shard: projections of this rank's tokens -> heads on their owners
g = torch.Generator("cpu").manual_seed(5)
xq, xk, xv = ((torch.randn(N, H * 128, generator=g) * 1.3).bfloat16() for _ in range(3))
wq, wk = ((1.0 + 0.2 * torch.randn(H * 128, generator=g)).bfloat16() for _ in range(2))
ang = torch.rand(N, 64, generator=g) * 6.2831853
cos, sin = torch.cos(ang).repeat_interleave(2, -1), torch.sin(ang).repeat_interleave(2, -1)
lo, hi = rank * n_loc, (rank + 1) * n_loc
from svoo_b200 import ops
full = [ops.qk_prep(xq.to(dev), H, wq.to(dev), 1e-6, cos.to(dev), sin.to(dev)),
        ops.qk_prep(xk.to(dev), H, wk.to(dev), 1e-6, cos.to(dev), sin.to(dev)), ops.qk_prep(xv.to(dev), H)]
got = x.producer_to_heads(xq[lo:hi].contiguous().to(dev), xk[lo:hi].contiguous().to(dev), xv[lo:hi].contiguous().to(dev),
                          (wq, 1e-6), (wk, 1e-6), cos[lo:hi].to(dev), sin[lo:hi].to(dev))
torch.cuda.current_stream().wait_event(x.value_ready)
for gt, fl in zip(got, full):
    assert torch.equal(gt, fl[parts[rank]]), "fused producer + re-shard differs from the one-GPU producer"
assert x.status() == 0
torch.cuda.synchronize(); dist.barrier(); dist.destroy_process_group()
print("OK", rank)
'''


@pytest.mark.gpu
def test_peer_exchange_and_sharded_layer_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, SVOO_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("OK") == 2


CHILD_MORE = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["SVOO_ROOT"])
from svoo_b200 import layer, parallel, processor, synth, wan_dit
import dataclasses
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local); dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)

def sharded_equals_single(cfg, parts, **extra):
    H, N = cfg.heads, cfg.n_tokens
    n_loc = N // world
    dens = synth.head_densities(cfg)
    q, k, v = (t.to(dev) for t in synth.make_qkv(cfg))
    shard = lambda t: t[0, :, rank * n_loc:(rank + 1) * n_loc].transpose(0, 1).contiguous()
    qi, ki = (t.to(dev) for t in synth.init_indices(cfg))
    kw = dict(num_q_centroids=cfg.num_q, num_k_centroids=cfg.num_k, kmeans_iters=2, top_p=cfg.top_p, **extra)
    x = parallel.PeerExchange(parts, N, dev)
    out = parallel.sparse_attention_layer_sharded(shard(q), shard(k), shard(v), parts, densities=dens, init_indices=(qi, ki),
                                                  exchange=x, **kw)
    ref = layer.sparse_attention_layer(q, k, v, min_kc_ratio=dens, max_kc_ratio=dens, init_indices=(qi, ki), **kw)
    assert torch.equal(out, shard(ref)) and x.status() == 0

# 1. uneven head split: 3 heads on 2 ranks (the 12-heads-on-8-GPUs case in small)
cfg = dataclasses.replace(synth.CONFIGS["cfg1"], heads=3, grid=(7, 30, 52))
parts = parallel.head_partition(3, world, synth.head_densities(cfg))
assert sorted(len(p) for p in parts) == [1, 2]
sharded_equals_single(cfg, parts)
# 2. text tokens after the video tokens (joint attention): the sequence, text included, is split evenly
cfg = dataclasses.replace(synth.CONFIGS["cfg1"], heads=2, grid=(7, 30, 52), text_tokens=256, cfg_id=97)
sharded_equals_single(cfg, parallel.head_partition(2, world), context_length=256, prompt_length=200)
# 2b. the error-aware routing variant through the peer-store re-shard (3 heads, uneven)
cfg = dataclasses.replace(synth.CONFIGS["cfg1"], heads=3, grid=(7, 30, 52), top_p=0.3)
sharded_equals_single(cfg, parallel.head_partition(3, world, synth.head_densities(cfg)), ear_gamma=1.0)

# 3. sequence-parallel DiT step against the one-GPU model (same weights, same initial indices)
dcfg = wan_dit.WanDiTConfig(num_layers=2, dim=512, heads=4, ffn_dim=1024, text_dim=64, text_len=16, latent=(4, 32, 40))
S = dcfg.tokens
kw = dict(num_q_centroids=12, num_k_centroids=40, top_p_kmeans=0.9, min_kc_ratio=0.2, kmeans_iter_init=2, kmeans_iter_step=1)
g = torch.Generator("cpu").manual_seed(0)
lat = torch.randn(1, 16, *dcfg.latent, generator=g).bfloat16().to(dev)
text = torch.randn(1, 16, 64, generator=g).bfloat16().to(dev)
idx = [(torch.randint(0, S, (4, 12), generator=g), torch.randint(0, S, (4, 40), generator=g)) for _ in range(2)]
def build(cls, shard):
    m = wan_dit.WanDiT(dcfg).init_weights(1).to(device=dev, dtype=torch.bfloat16).eval()
    procs = wan_dit.install_processors(m, cls, dcfg.grid, **kw)
    m.seq_shard = shard
    return m, procs
single, p1 = build(type("P1", (processor.WanAttn_SAPAttn_Processor,), {}), None)
sp_cls = type("P2", (wan_dit.SequenceParallelWanProcessor,), {})
parts = parallel.head_partition(4, world)
sp_cls.exchange = parallel.PeerExchange(parts, S, dev)
sp, p2 = build(sp_cls, (rank, world))
for l in range(2):
    qi, ki = idx[l]
    p1[l].draw_init_indices = lambda BH, n, d, qi=qi, ki=ki: (qi.to(d), ki.to(d))
    mine = parts[rank]
    p2[l].draw_init_indices = lambda BH, n, d, qi=qi, ki=ki, mine=mine: (qi[mine].to(d), ki[mine].to(d))
for step in (1, 2):
    wan_dit.set_attention_step(single, step); wan_dit.set_attention_step(sp, step)
    t = torch.tensor([800.0 - 100 * step], device=dev)
    with torch.no_grad():
        want = single(lat, t, text)
        got = sp(lat, t, text)                                # [1, S/P, C*patch]
    T, Hh, W = dcfg.grid
    rows = want.reshape(1, 16, T, 1, Hh, 2, W, 2).permute(0, 2, 4, 6, 3, 5, 7, 1).reshape(1, S, -1)
    n_loc = S // world
    mine_rows = rows[:, rank * n_loc:(rank + 1) * n_loc].float().flatten()
    a = got.float().flatten()
    cos = float(a @ mine_rows / (a.norm() * mine_rows.norm()))
    assert cos >= 0.999, cos
    for l in range(2):
        p2[l].check_status()
        full = p1[l]._cached_clustering_results.qlabels[parts[rank]]
        assert (p2[l]._cached_clustering_results.qlabels == full).float().mean() >= 0.98
assert sp_cls.exchange.status() == 0
torch.cuda.synchronize(); dist.barrier(); dist.destroy_process_group()
print("OK", rank)
'''


@pytest.mark.gpu
def test_uneven_heads_text_tokens_and_sequence_parallel_dit_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "child_more.py"
    script.write_text(CHILD_MORE)
    env = dict(os.environ, SVOO_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29534", str(script)],
                         env=env, capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("OK") == 2
