"""Benchmark of the sparse-attention layer (co-clustering + permute + block map +
block-sparse attention + inverse permute) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config cfg2] [--impl reference]

N = 1: the Wan-14B 720p layer (40 heads x 75,600 tokens, 100/500 clusters, 5 iterations,
per-head density U[0.05, 0.25]) on one GPU.  N > 1 (under torch.distributed.run): the same
layer, heads sharded over the ranks, activations arriving and leaving sharded by sequence
(one peer-store re-shard each way inside the timed region) -- total work is fixed ("strong" scaling).

`value` is effective TFLOP/s: the reference algorithm's flops for this layer
    F = iters*H*[2*N*D*(QC+KC) + 4*N*QC*KC]  +  sum_h 4*N^2*D*rho_h
(rho_h = realised token-pair density of head h) divided by the step time.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch

from svoo_b200 import synth

D = 128
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


# ------------------------------------------------------------------------------------------
# work model
# ------------------------------------------------------------------------------------------
def cluster_flops_reference(cfg, heads):
    n = cfg.n_video
    return cfg.iters * heads * (2.0 * n * D * (cfg.num_q + cfg.num_k) + 4.0 * n * cfg.num_q * cfg.num_k)


def cluster_flops_executed(cfg, heads):
    """Flops the assignment GEMMs of this implementation run: one [N,128]x[128,J] product per
    side and iteration, twice (W is a bf16 hi/lo pair)."""
    n = cfg.n_video
    return cfg.iters * heads * 2.0 * (2.0 * n * D * (cfg.num_q + cfg.num_k))


def attention_flops(rho, n_tokens):
    return float(sum(4.0 * n_tokens * n_tokens * D * r for r in rho))


def realised_density(block_map, q_off, k_off):
    """rho_h = sum_ij map[h,i,j] |Q_i| |K_j| / S^2 for every head (device tensors)."""
    qs = (q_off[:, 1:] - q_off[:, :-1]).double()
    ks = (k_off[:, 1:] - k_off[:, :-1]).double()
    s = qs.sum(-1)
    return (torch.einsum("hi,hij,hj->h", qs, block_map.double(), ks) / (s * s)).tolist()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS if k in p}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi samples (SM clock, throttle reasons) of one GPU while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index),
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=5)

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                mhz.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except ValueError:
                continue
            for name, val in zip(names, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ------------------------------------------------------------------------------------------
# CPU arm (the oracle port of the reference's algorithm, on the host cores)
# ------------------------------------------------------------------------------------------
def centroid_key_flops(block_map, q_off):
    """EAR: 4 * 128 flops per (query row, pruned key cluster) pair -- one virtual key each."""
    qs = (q_off[:, 1:] - q_off[:, :-1]).double()
    pruned = (block_map.shape[-1] - block_map.double().sum(-1))
    return float((qs * pruned).sum()) * 4.0 * 128.0


def cpu_ear_sample(cfg, head: int):
    """One head of the workload through the CPU restatement of the reference's EAR path."""
    from oracle import ear_oracle as E
    from oracle import svoo_oracle as O
    one = dataclasses.replace(cfg, heads=1)
    q, k, v = synth.make_qkv(cfg, heads=[head])
    qi, ki = synth.init_indices(cfg)
    d = synth.head_densities(cfg)[head]
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    ql, qc, qs, kl, kc, ks = O.co_cluster_tokens(q[0], k[0], qi[head:head + 1], ki[head:head + 1], cfg.iters)
    q_idx, q_off = O.sort_labels(ql, cfg.num_q)
    k_idx, k_off = O.sort_labels(kl, cfg.num_k)
    qp, kp, vp = O.permute(q[0], q_idx), O.permute(k[0], k_idx), O.permute(v[0], k_idx)
    vc = E.value_centroids(v[0], kl, ks, cfg.num_k)
    m = E.identify_dynamic_map_estimated(kp, vp, qs, ks, qc, kc, vc, cfg.top_p, 1.0, [d])
    out_p, _ = E.compensated_attention(qp, kp, vp, kc, vc, m, qs, ks)
    O.inverse_permute(out_p, q_idx)
    dt = time.perf_counter() - t0
    rho = O.realised_density(m[None], qs[None], ks[None])[0].tolist()
    return dt, cluster_flops_reference(one, 1) + attention_flops(rho, cfg.n_tokens) + centroid_key_flops(m, q_off)


def cpu_layer_sample(cfg, head: int, pattern: str = "svoo"):
    """One head of the workload through the CPU restatement of the reference path.
    Returns (seconds, reference-algorithm flops of that head)."""
    if pattern == "ear":
        return cpu_ear_sample(cfg, head)
    from oracle import svoo_oracle as O
    one = dataclasses.replace(cfg, heads=1)
    q, k, v = synth.make_qkv(cfg, heads=[head])
    qi, ki = synth.init_indices(cfg)
    d = synth.head_densities(cfg)[head]
    torch.set_num_threads(os.cpu_count() or 1)
    t0 = time.perf_counter()
    out, aux = O.sparse_attention_layer(q, k, v, qi[head:head + 1], ki[head:head + 1], cfg.num_q, cfg.num_k, cfg.iters,
                                        cfg.top_p, [d], [d], cfg.text_tokens, cfg.text_tokens)
    dt = time.perf_counter() - t0
    qs, ks = aux["qsizes"][None], aux["ksizes"][None]
    if cfg.text_tokens:                                      # the two text blocks (prompt = all text tokens)
        tail = torch.tensor([cfg.text_tokens, 0], dtype=qs.dtype).expand(1, 1, 2)
        qs, ks = torch.cat([qs, tail], -1), torch.cat([ks, tail], -1)
    rho = O.realised_density(aux["map"], qs, ks)[0].tolist()
    return dt, cluster_flops_reference(one, 1) + attention_flops(rho, cfg.n_tokens)


def run_reference_arm(args, cfg):
    """--impl reference: the reference algorithm on the host cores (CPU restatement; the
    reference's own kernels are Triton/CUDA-only), one head of the layer per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    for _ in range(args.warmup):
        cpu_layer_sample(cfg, 0, args.pattern)
    tot_t, tot_f = 0.0, 0.0
    for s in range(args.steps):
        dt, fl = cpu_layer_sample(cfg, s % cfg.heads, args.pattern)
        tot_t += dt
        tot_f += fl
    val = tot_f / tot_t / 1e12
    sample = f"1 of {cfg.heads} heads of the {cfg.name} layer per step (full {cfg.n_video} tokens)"
    line = {
        "impl": "reference", "metric": "sparse_attn_layer_effective_tflops", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": tot_t / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg.name + ("-ear" if args.pattern == "ear" else ""), "heads": cfg.heads, "tokens": cfg.n_tokens,
                   "q_clusters": cfg.num_q, "k_clusters": cfg.num_k, "kmeans_iters": cfg.iters, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def run_gpu_arm(args, cfg):
    import torch.distributed as dist
    from svoo_b200 import _lib, layer, parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    H, N = cfg.heads, cfg.n_tokens
    if N % world:
        raise SystemExit(f"{N} tokens do not split evenly over {world} ranks")
    dens = synth.head_densities(cfg)
    parts = parallel.head_partition(H, world, dens if world > 1 else None)
    if world > 1 and len({len(p) for p in parts}) != 1:
        raise SystemExit(f"{H} heads do not split evenly over {world} ranks")
    mine = parts[rank]
    qi_all, ki_all = synth.init_indices(cfg)
    q_h, k_h, v_h = synth.make_qkv(cfg, heads=mine, pin_memory=True)          # [1, H_r, N, 128] pinned host
    qi, ki = qi_all[mine].to(dev), ki_all[mine].to(dev)
    d_mine = [dens[h] for h in mine]
    kw = dict(num_q_centroids=cfg.num_q, num_k_centroids=cfg.num_k, kmeans_iters=cfg.iters, top_p=cfg.top_p,
              context_length=cfg.text_tokens)
    ear = args.pattern == "ear"
    if ear:
        if cfg.text_tokens:
            raise SystemExit("--pattern ear: video-only self attention, as in the reference")
        kw["ear_gamma"] = 1.0

    q_d, k_d, v_d = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    if world > 1:
        # sequence-sharded activations, as a sequence-parallel DiT block holds them
        q_s = parallel.head_to_seq_shard(q_d[0], parts)
        k_s = parallel.head_to_seq_shard(k_d[0], parts)
        v_s = parallel.head_to_seq_shard(v_d[0], parts)
        del q_d, k_d, v_d
        host_in = [t.cpu().pin_memory() for t in (q_s, k_s, v_s)]
        host_out = torch.empty_like(host_in[0]).pin_memory()
    else:
        host_in = [q_h, k_h, v_h]
        host_out = torch.empty_like(q_h).pin_memory()

    state = {}
    xchg = parallel.PeerExchange(parts, N, dev) if world > 1 else None

    def step(timer=None):
        if world > 1:
            if timer is not None:
                timer.mark("begin")
            q, k, v = (t[None] for t in xchg.to_heads(q_s, k_s, v_s))
        else:
            q, k, v = q_d, k_d, v_d
        out, st = layer.sparse_attention_layer(q, k, v, min_kc_ratio=d_mine, max_kc_ratio=d_mine,
                                               init_indices=(qi, ki), return_state=True, timer=timer,
                                               value_ready=xchg.value_ready if xchg else None,
                                               peer_out=xchg.peer_out if xchg else None, **kw)
        state["st"] = st
        if world > 1:
            res = xchg.seq_result()
            if timer is not None:
                timer.mark("reshard_out")
            return res
        return out

    if world > 1:
        # host shards in, host shard out: the copies of one call overlap the compute of its neighbours
        pipe = parallel.HostShardPipeline(xchg, dev)
        qi_dev, ki_dev = qi_all.to(dev), ki_all.to(dev)

        def step_e2e():
            pipe(*host_in, host_out, parts, densities=dens, init_indices=(qi_dev, ki_dev), **kw)
    else:
        # host buffers in, host buffer out: copies of one head group overlap the compute of another
        pipe = layer.HostLayerPipeline(dev, H, N, heads_per_group=args.e2e_group)

        def step_e2e():
            pipe(q_h, k_h, v_h, host_out, min_kc_ratio=d_mine, max_kc_ratio=d_mine, init_indices=(qi, ki), **kw)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, with_timers=False, finish=None):
        """`finish` runs after the last step and before the closing event: it makes the timing
        stream wait for work that the steps left on other streams (the last device-to-host copy)."""
        timers = []
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            t = layer.StageTimer() if with_timers else None
            fn(t) if with_timers else fn()
            if t is not None:
                timers.append(t)
        if finish is not None:
            finish()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), timers

    with ClockSampler(local) as clocks:            # samples cover the warm-up and the timed steps (same load)
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        launches0 = _lib.LIB.svoo_b200_launch_count()
        total_ms, timers = timed(step, args.steps, with_timers=True)
    launches = _lib.LIB.svoo_b200_launch_count() - launches0
    for _ in range(min(args.warmup, 2)):
        step_e2e()
    e2e_ms, _ = timed(step_e2e, args.steps, finish=lambda: torch.cuda.current_stream().wait_stream(pipe.copy_out))

    producer = measure_producer(cfg, dev, peaks_hbm=measured_peaks()[0]["hbm_gbs"]) if world == 1 else None

    parity = None
    if world > 1:
        # one untimed step through the library all-to-all path (torch.distributed all_to_all_single both ways,
        # unfused store): the peer-store path must give the same bits
        got = step().clone()
        want = parallel.sparse_attention_layer_sharded(q_s, k_s, v_s, parts, densities=dens,
                                                       init_indices=(qi_all.to(dev), ki_all.to(dev)), exchange=None, **kw)
        same = torch.tensor([1 if torch.equal(got, want) else 0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        parity = {"vs": "nccl all_to_all path", "equal": bool(same.item())}
        del got, want

    st = state["st"]
    rho = realised_density(st.block_map, st.q_offsets, st.k_offsets)
    extra = centroid_key_flops(st.block_map, st.q_offsets) if ear else 0.0
    flops = torch.tensor([cluster_flops_reference(cfg, len(mine)) + attention_flops(rho, N) + extra,
                          attention_flops(rho, N) + extra], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(flops)
    flops_total, flops_attn_all = flops.tolist()
    ms_per_step = total_ms / args.steps
    stage = {}
    for t in timers:
        for name, ms in t.stage_ms().items():
            name = "reshard_in" if name == "start" else name
            stage[name] = stage.get(name, 0.0) + ms / len(timers)
    peaks, peak_kind = measured_peaks()
    attn_ms = stage.get("attention", float("nan"))
    attn_flops_rank = attention_flops(rho, N) + extra
    achieved = attn_flops_rank / (attn_ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops_sustained"]

    if rank == 0:
        bytes_in = sum(t.numel() * t.element_size() for t in host_in)
        bytes_out = host_out.numel() * host_out.element_size()
        line = {
            "metric": "sparse_attn_layer_effective_tflops", "value": flops_total / (ms_per_step * 1e-3) / 1e12,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": cfg.name + ("-ear" if ear else ""), "heads": H, "tokens": N, "q_clusters": cfg.num_q,
                       "k_clusters": cfg.num_k, "kmeans_iters": cfg.iters, "top_p": cfg.top_p, "density_budget": list(cfg.density),
                       "realised_density_mean_rank0": sum(rho) / len(rho),
                       "parallelism": f"heads/{world}" + ("+peer-store re-shard" if world > 1 else ""),
                       "l2": f"inputs ({3 * len(mine) * N * D * 2 / 1e9:.2f} GB of Q,K,V on rank 0) are larger than the 126 MB L2; "
                             "no flush between steps"},
            "stage_ms_rank0": {k: round(v, 4) for k, v in stage.items()},
            "roofline": {"kernel": "sparse_attn", "bound": "tensor", "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": achieved / peak, "peak_source": f"{peak_kind} sustained bf16",
                         "traffic": ATTN_DRAM_TRAFFIC_BYTES_PER_HEAD * len(mine) * (N / 75600.0),
                         "traffic_source": "ncu capture at 4 heads x 75,600 tokens, scaled by heads and tokens",
                         "algorithmic_flops_per_launch": attn_flops_rank},
            "roofline_layer": {"time_at_roofline_ms": layer_roofline_ms(cfg, len(mine), rho, N, peaks),
                               "frac": layer_roofline_ms(cfg, len(mine), rho, N, peaks) / ms_per_step},
            "e2e": {"value": flops_total / (e2e_ms / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": bytes_in, "d2h_bytes_per_step": bytes_out},
            "gpu_launches": int(launches),
            "producer": producer,
            "exchange_status": (xchg.status() if xchg else 0),
            "parity_check": parity,
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            dt, fl = cpu_layer_sample(cfg, 0, args.pattern)
            line["cpu_baseline"] = {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count() or 1,
                                    "kind": "port", "seconds": dt,
                                    "sample": f"head 0 of {H} of the {cfg.name} layer, full {cfg.n_video} tokens, once"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["equal"]:
        raise SystemExit("the peer-store path and the all-to-all path disagree")


def measure_producer(cfg, dev, peaks_hbm, reps=5):
    """The step before the layer (RMS norm + rotary embedding + head transpose of the Q, K, V
    projections, one kernel launch per tensor), timed on its own: not part of `value`."""
    from svoo_b200 import ops
    H, S = cfg.heads, cfg.n_tokens
    joint = cfg.text_tokens > 0                              # HunyuanVideo: per-head norm, text rows not rotated
    rows = S - cfg.text_tokens
    g = torch.Generator("cpu").manual_seed(3)
    x = [torch.randn(S, H * D, generator=g, dtype=torch.float32).bfloat16().to(dev) for _ in range(3)]
    w = [(1.0 + 0.1 * torch.randn(D if joint else H * D, generator=g)).to(dev) for _ in range(2)]
    ang = torch.rand(rows, D // 2, generator=g) * 6.2831853
    cos, sin = torch.cos(ang).repeat_interleave(2, -1).to(dev), torch.sin(ang).repeat_interleave(2, -1).to(dev)

    def run():
        if joint:
            ops.qk_prep_heads(x[0], H, w[0], 1e-6, cos, sin, rows)
            ops.qk_prep_heads(x[1], H, w[1], 1e-6, cos, sin, rows)
            ops.qk_prep_heads(x[2], H)
            return
        ops.qk_prep(x[0], H, w[0], 1e-6, cos, sin)
        ops.qk_prep(x[1], H, w[1], 1e-6, cos, sin)
        ops.qk_prep(x[2], H)

    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    nbytes = 3 * 2 * S * H * D * 2 + 2 * 2 * rows * D * 4       # x read + y written per tensor; cos, sin for Q and K
    gbs = nbytes / (ms * 1e-3) / 1e9
    what = ("per-head rmsnorm + text-last rope + head transpose" if joint else "rmsnorm + rope + head transpose")
    return {"what": what + " of the Q, K, V projections (3 launches)", "ms": ms,
            "algorithmic_bytes": nbytes, "achieved": gbs, "peak": peaks_hbm, "unit": "GB/s", "frac": gbs / peaks_hbm,
            "bound": "hbm"}


# dram__bytes_read.sum + dram__bytes_write.sum of one sparse_attn launch per head of 75,600
# tokens, from an ncu capture of a 4-head launch (profiles/sparse_attn_tc_kernel_wan14b_4heads.md).
ATTN_DRAM_TRAFFIC_BYTES_PER_HEAD = 282.5e6 / 4


def layer_roofline_ms(cfg, heads, rho, n_tokens, peaks):
    """Time of the whole layer on `heads` heads at the measured peaks: executed GEMM flops of
    the clustering and the attention flops at the tensor peak, permute / centroid / sort
    bytes at the HBM peak."""
    n = cfg.n_video
    tensor = (cluster_flops_executed(cfg, heads) + attention_flops(rho, n_tokens)) / (peaks["bf16_tflops_sustained"] * 1e12)
    row = n * D * 2
    bytes_cent = cfg.iters * heads * 2 * (2 * row + 3 * 4 * n)       # assign read + centroid gather, labels/idx
    bytes_perm = heads * (3 * 2 * row + 2 * row + 4 * 4 * n)         # Q,K,V gather; attention output scatter
    return (tensor + (bytes_cent + bytes_perm) / (peaks["hbm_gbs"] * 1e9)) * 1e3


# ------------------------------------------------------------------------------------------
# cfg4: one denoising step of a Wan2.1-1.3B-shaped DiT with the sparse processor in every block
# ------------------------------------------------------------------------------------------
DIT_DENSITY = (0.05, 0.30)
# top_p_kmeans = 0 makes the per-head floor the whole selection (the first sorted cluster plus the
# floor, svoo/co_clustering.py:585-596): every query cluster keeps exactly max(1, int(d_h * 500)) key
# clusters, i.e. the table's density is the budget, as in configs 1-3.  (With top-p 0.9 the nearly
# uniform attention of a random-weight model would keep ~90 % of the clusters.)
DIT_CLUSTERS = dict(num_q_centroids=100, num_k_centroids=500, top_p_kmeans=0.0, min_kc_ratio=0.05, kmeans_iter_init=5,
                    kmeans_iter_step=5)


def dit_inputs(cfg, seed=11):
    g = torch.Generator("cpu").manual_seed(seed)
    latents = torch.randn(1, cfg.in_channels, *cfg.latent, generator=g)
    text = torch.randn(1, cfg.text_len, cfg.text_dim, generator=g).bfloat16()
    return latents.bfloat16(), text


def run_dit_arm(args):
    """--config cfg4: K denoising steps (one transformer forward each) of a random-init DiT with
    Wan2.1-1.3B's shape (30 blocks, dim 1536, 12 heads, FFN 8960, cross attention to 512 x 4096 text
    tokens) at 480p / 81 frames (32,760 tokens).  Self-attention of every block runs through
    WanAttn_SAPAttn_Processor: 100 / 500 clusters, 5 iterations, top-p 0.9 with the per-(step,
    layer, head) floor read through SparsityLookup from a seeded U[0.05, 0.30] CSV; the step index
    is set before every step as the pipeline callback does.  N > 1: sequence parallel, the
    self-attention re-shards to heads through peer stores."""
    import tempfile
    import torch.distributed as dist
    from svoo_b200 import _lib, parallel, wan_dit
    from svoo_b200.sparsity import SparsityLookup

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs WORLD_SIZE={args.gpus} (launch with torch.distributed.run)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = wan_dit.WanDiTConfig(num_layers=args.dit_layers)
    S, H = cfg.tokens, cfg.heads
    if S % world:
        raise SystemExit(f"{S} tokens do not split evenly over {world} ranks")
    model = wan_dit.WanDiT(cfg).init_weights(seed=1).to(device=dev, dtype=torch.bfloat16).eval()
    steps_total = args.warmup + args.steps
    csv_path = os.path.join(tempfile.mkdtemp(), "density.csv")
    wan_dit.write_density_table(csv_path, steps_total, cfg.num_layers, H, *DIT_DENSITY, seed=1004)
    lookup = SparsityLookup(csv_path)
    base = wan_dit.SequenceParallelWanProcessor if world > 1 else wan_dit.WanAttn_SAPAttn_Processor
    proc_cls = type("BenchProcessor", (base,), {"_seen_timesteps": set()})
    if world > 1:
        parts = parallel.head_partition(H, world)
        proc_cls.exchange = parallel.PeerExchange(parts, S, dev)
        model.seq_shard = (rank, world)
    procs = wan_dit.install_processors(model, proc_cls, cfg.grid, sparsity_lookup=lookup,
                                       dynamic_min_kc_ratio_min=DIT_DENSITY[0], dynamic_min_kc_ratio_max=DIT_DENSITY[1],
                                       **DIT_CLUSTERS)
    latents_h, text_h = dit_inputs(cfg)
    latents_h, text_h = latents_h.pin_memory(), text_h.pin_memory()
    latents, text = latents_h.to(dev), text_h.to(dev)
    attn_events = []

    def pre(_m, _a, _k):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        attn_events.append([e, None])

    def post(_m, _a, _k, _out):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        attn_events[-1][1] = e

    for blk in model.blocks:
        blk.attn1.register_forward_pre_hook(pre, with_kwargs=True)
        blk.attn1.register_forward_hook(post, with_kwargs=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run_steps(first, count, e2e=False):
        out = None
        for s in range(first, first + count):
            wan_dit.set_attention_step(model, s + 1)
            t = torch.tensor([1000.0 - 20.0 * s], device=dev)
            with torch.no_grad():
                if e2e:
                    lat = latents_h.to(dev, non_blocking=True)
                    out = model(lat, t, text_h.to(dev, non_blocking=True))
                    out_h.copy_(out, non_blocking=True)
                else:
                    out = model(latents, t, text)
        return out

    with torch.no_grad():
        out_h = torch.empty_like(model(latents, torch.tensor([1000.0], device=dev), text), device="cpu").pin_memory()
    for p in procs:                                         # that probe call clustered once: start the schedule afresh
        p.centroids_init, p._cached_clustering_results = False, None
    with ClockSampler(local) as clocks:
        run_steps(0, args.warmup)
        barrier()
        attn_events.clear()
        launches0 = _lib.LIB.svoo_b200_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run_steps(args.warmup, args.steps)
        e1.record()
        barrier()
    launches = _lib.LIB.svoo_b200_launch_count() - launches0
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps, sum(a.elapsed_time(b) for a, b in attn_events) / args.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    step_ms, attn_ms = ms.tolist()
    for p in procs:
        p.check_status()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_steps(args.warmup, args.steps, e2e=True)
    e1.record()
    barrier()
    e2e_ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        line = {
            "metric": "dit_denoising_step_ms", "value": step_ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "wan1.3b-dit-480p", "blocks": cfg.num_layers, "dim": cfg.dim, "heads": H, "tokens": S,
                       "q_clusters": 100, "k_clusters": 500, "kmeans_iters": 5, "density_floor_table": list(DIT_DENSITY),
                       "parallelism": "one GPU" if world == 1 else f"sequence parallel x{world}, heads re-sharded by peer stores",
                       "l2": "activations of one block (100 MB per tensor) and 2.6 GB of weights exceed the L2; no flush"},
            "sparse_attention_ms_per_step": attn_ms, "sparse_attention_share": attn_ms / step_ms,
            "e2e": {"value": float(e2e_ms.item()), "unit": "ms", "ms_per_step": float(e2e_ms.item()),
                    "h2d_bytes_per_step": latents_h.numel() * 2 + text_h.numel() * 2, "d2h_bytes_per_step": out_h.numel() * 2},
            "gpu_launches": int(launches), "clocks": clocks.summary(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_dit_reference_arm(args):
    """--impl reference --config cfg4: one block of the DiT per step on the host cores, its
    self-attention through the CPU restatement of the reference's processor."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle.wan_processor import OracleWanProcessor
    from svoo_b200 import wan_dit
    torch.set_num_threads(os.cpu_count() or 1)
    cfg = wan_dit.WanDiTConfig(num_layers=1)
    model = wan_dit.WanDiT(cfg).init_weights(seed=1).to(dtype=torch.bfloat16).eval()
    cls = type("CpuProcessor", (OracleWanProcessor,), {})
    wan_dit.install_processors(model, cls, cfg.grid, **DIT_CLUSTERS)
    latents, text = dit_inputs(cfg)
    times = []
    for s in range(args.warmup + args.steps):
        wan_dit.set_attention_step(model, s + 1)
        t0 = time.perf_counter()
        with torch.no_grad():
            model(latents, torch.tensor([1000.0 - 20.0 * s]), text)
        times.append(time.perf_counter() - t0)
    ms = sum(times[args.warmup:]) / args.steps * 1e3 * 30
    sample = "1 of 30 blocks per step (time x 30), full 32,760 tokens"
    line = {"impl": "reference", "metric": "dit_denoising_step_ms", "value": ms, "unit": "ms", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "wan1.3b-dit-480p", "sample": sample},
            "cpu_baseline": {"value": ms, "unit": "ms", "cores": os.cpu_count() or 1, "kind": "port", "sample": sample},
            "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="svoo_b200", choices=["svoo_b200", "reference"])
    ap.add_argument("--config", default="cfg2", choices=sorted(synth.CONFIGS) + ["cfg4"])
    ap.add_argument("--dit-layers", type=int, default=30, help="blocks of the cfg4 DiT (debugging)")
    ap.add_argument("--heads", type=int, default=0, help="override the head count (debugging)")
    ap.add_argument("--top-p", type=float, default=None, help="override the config's top-p of the block selection")
    ap.add_argument("--pattern", default="svoo", choices=["svoo", "ear"],
                    help="ear: the error-aware routing variant of the layer (one GPU, video-only configs)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-group", type=int, default=4, help="heads per copy/compute group of the host-buffer path")
    args = ap.parse_args()
    if args.config == "cfg4":
        return run_dit_reference_arm(args) if args.impl == "reference" else run_dit_arm(args)
    cfg = synth.CONFIGS[args.config]
    if args.heads:
        cfg = dataclasses.replace(cfg, heads=args.heads)
    if args.top_p is not None:
        cfg = dataclasses.replace(cfg, top_p=args.top_p)
    if args.impl == "reference":
        run_reference_arm(args, cfg)
    else:
        run_gpu_arm(args, cfg)


if __name__ == "__main__":
    main()
