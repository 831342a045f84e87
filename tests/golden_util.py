"""Helpers shared by the tests that read tests/golden/*.npz."""
import dataclasses
import os

import numpy as np
import torch

from svoo_b200 import synth

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

TINY_FP32 = synth.LayerConfig("tiny-fp32", 90, 2, (4, 16, 16), torch.float32, 8, 16, 3, (0.25, 0.25), 1, False)
TINY_BF16 = dataclasses.replace(TINY_FP32, name="tiny-bf16", cfg_id=91, dtype=torch.bfloat16, rope=True,
                                num_q=12, num_k=40, grid=(3, 16, 20))
LAYER_CASES = {
    "layer_tiny_fp32": TINY_FP32,
    "layer_tiny_bf16": TINY_BF16,
    "layer_cfg0": synth.CONFIGS["cfg0"],
}
EUCLID_CASE = dataclasses.replace(TINY_FP32, name="euclid-fp32", cfg_id=98, num_q=24, grid=(4, 16, 24))
# name -> (config, [(top_p, gamma, min_kc_ratio), ...]); the compensation is recorded for the last setting
EAR_CASES = {
    "ear_fp32": (dataclasses.replace(TINY_FP32, name="ear-fp32", cfg_id=97, num_q=12, num_k=40, grid=(4, 16, 24)),
                 [(0.9, 1.0, 0.0), (0.7, 0.5, 0.1), (0.8, 1.0, [0.05, 0.2]), (0.4, 1.0, 0.05)]),
    "ear_bf16": (dataclasses.replace(TINY_BF16, name="ear-bf16", cfg_id=96, num_q=12, num_k=40, grid=(4, 16, 24)),
                 [(0.9, 1.0, 0.0), (0.8, 1.0, [0.05, 0.2]), (0.4, 1.0, [0.1, 0.05])]),
}
MAP_CASES = ["map_bf16_budget", "map_bf16_topp_floor", "map_bf16_scalar", "map_fp32_topp",
             "map_fp32_cap_scalar", "map_bf16_big", "map_all_ones"]


def load(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def from_bf16_bits(a):
    """int16 bit patterns (as stored by the fixture generator) -> bf16 tensor."""
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


def unpack_map(z, suffix=""):
    if suffix:
        shape = tuple(int(x) for x in z["map_shape" + suffix])
        return np.unpackbits(z["map_bits" + suffix])[: int(np.prod(shape))].reshape(shape).astype(bool)
    return _unpack_map(z)


def _unpack_map(z):
    shape = tuple(int(x) for x in z["map_shape"])
    return np.unpackbits(z["map_bits"])[: int(np.prod(shape))].reshape(shape).astype(bool)


def ratio_arg(arr, is_list):
    if arr[0] < 0:
        return None
    return [float(x) for x in arr] if is_list else float(arr[0])


def layer_ratio(arr, heads):
    """Layer fixtures store a per-head list when its length equals the head count > 1."""
    if arr[0] < 0:
        return None
    return [float(x) for x in arr] if len(arr) > 1 else float(arr[0])


def map_inputs(z):
    """Re-create the centroid inputs of a map fixture from its seed (checked by checksum)."""
    H, QC, KC, seed = int(z["H"][0]), int(z["QC"][0]), int(z["KC"][0]), int(z["seed"][0])
    dtype = torch.bfloat16 if z["is_bf16"][0] else torch.float32
    g = torch.Generator("cpu").manual_seed(seed)
    base = torch.randn(H, 1, 128, generator=g)
    qc = (base + 0.7 * torch.randn(H, QC, 128, generator=g)).to(dtype)[None]
    kc = (base + 0.7 * torch.randn(H, KC, 128, generator=g)).to(dtype)[None]
    ks = torch.randint(0, 400, (1, H, KC), generator=g, dtype=torch.int32)
    ks[0, :, 3] = 0
    qs = torch.randint(1, 900, (1, H, QC), generator=g, dtype=torch.int32)
    assert synth.tensor_checksum(qc, kc, ks, qs)[0] == z["input_checksum"][0], "RNG drift: regenerate fixtures"
    kw = {}
    mn = ratio_arg(z["min_kc_ratio"], bool(z["min_is_list"][0]))
    mx = ratio_arg(z["max_kc_ratio"], bool(z["max_is_list"][0]))
    if mn is not None:
        kw["min_kc_ratio"] = mn
    if mx is not None:
        kw["max_kc_ratio"] = mx
    return qc, kc, qs, ks, float(z["p"][0]), kw


def same_up_to_ties(got, ref, prob):
    """True when two bool maps keep, in every row, clusters of the same probabilities
    (they may differ only in which members of an equal-probability group are kept)."""
    got = np.asarray(got)
    ref = np.asarray(ref)
    if (got.sum(-1) != ref.sum(-1)).any():
        return False
    a = np.sort(np.where(got, prob, -1.0), -1)
    b = np.sort(np.where(ref, prob, -1.0), -1)
    return bool((a == b).all())


def unpack_ear_map(z, n):
    shape = tuple(int(x) for x in z["map_shape"])
    return np.unpackbits(z[f"map_bits_{n}"])[: int(np.prod(shape))].reshape(shape).astype(bool)


def ear_inputs(cfg, z, q, k, v):
    """Tensors of an EAR fixture: the recorded labels / centroids of the reference run, the stable
    permutation of the seeded q, k, v by those labels (the reference's own order inside a cluster may
    differ; nothing that is compared depends on it)."""
    from oracle import svoo_oracle as O
    dt = cfg.dtype
    ql, kl = (torch.from_numpy(z[n].astype(np.int64)) for n in ("qlabels", "klabels"))
    qc, kc, vc = (torch.from_numpy(z[n]).to(dt) for n in ("qcentroids", "kcentroids", "vcentroids"))
    qs, ks = torch.from_numpy(z["qsizes"]), torch.from_numpy(z["ksizes"])
    q_idx, q_off = O.sort_labels(ql, cfg.num_q)
    k_idx, k_off = O.sort_labels(kl, cfg.num_k)
    return dict(ql=ql, kl=kl, qc=qc, kc=kc, vc=vc, qs=qs, ks=ks, q_idx=q_idx, k_idx=k_idx, q_off=q_off, k_off=k_off,
                q=q[0], k=k[0], v=v[0], qp=O.permute(q[0], q_idx), kp=O.permute(k[0], k_idx), vp=O.permute(v[0], k_idx))


def ear_row_has_boundary_tie(prob, preserve, budget_kept, scores, got, ref):
    """Why two selections of one map row may differ although both follow the rule: the reference sorts
    with an unstable sort, so among clusters of equal budget probability it may put a different one
    inside the guaranteed set or inside the budget (which changes the budget by their areas), and among
    candidates of equal score a different one before the cut.  True when the row has such a tie: at the
    guaranteed boundary, at a boundary of the kept budget positions, or between a candidate kept by one
    side only and one kept by the other."""
    sp = np.sort(prob)[::-1]
    if 0 < preserve < len(sp) and sp[preserve - 1] == sp[preserve]:
        return True
    edges = np.nonzero(budget_kept[:-1] != budget_kept[1:])[0]        # sorted positions where keep flips
    if any(sp[e] == sp[e + 1] for e in edges):
        return True
    only_got, only_ref = scores[got & ~ref], scores[ref & ~got]
    return bool(len(only_got) and len(only_ref) and np.isin(only_got, only_ref).any())


# ----------------------------------------------------------------------------------------------
# Processor fixtures: the inputs are rebuilt from seeds by the generator and by the tests alike.
# ----------------------------------------------------------------------------------------------
class RMSNormModule(torch.nn.Module):
    """Weight-only RMS norm over the last dimension (what a DiT block passes as attn.norm_q)."""

    def __init__(self, dim, eps, weight):
        super().__init__()
        self.weight = torch.nn.Parameter(weight)
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + self.eps)
        return (y * self.weight.float()).to(x.dtype)


def smooth_hidden(seed, grid, dim, extra_rows=0, noise=0.35):
    """[1, N(+extra), dim] bf16 activations with low-frequency structure over the latent grid."""
    import math
    T, Hh, W = grid
    g = torch.Generator("cpu").manual_seed(seed)
    t, h, w = torch.meshgrid(torch.arange(T), torch.arange(Hh), torch.arange(W), indexing="ij")
    coords = torch.stack([t.reshape(-1) / T, h.reshape(-1) / Hh, w.reshape(-1) / W], -1).float()
    freqs = torch.randint(0, 3, (12, 3), generator=g).float()
    freqs[freqs.sum(-1) == 0, 0] = 1
    feat = torch.cos(2 * math.pi * coords @ freqs.T + torch.rand(12, generator=g) * 2 * math.pi)
    x = feat @ (torch.randn(12, dim, generator=g) / 3) + noise * torch.randn(coords.shape[0], dim, generator=g)
    if extra_rows:
        x = torch.cat([x, torch.randn(extra_rows, dim, generator=g)], 0)
    return x[None].bfloat16()


def make_attn(seed, heads, joint=False, bias=True):
    """A stand-in for a DiT block's attention module: q/k/v/out projections and QK norms, seeded.
    joint=False: Wan layout (norms over all heads*128 columns); joint=True: HunyuanVideo
    single-stream layout (norms over the 128 columns of a head, no added projections)."""
    dim = heads * 128
    g = torch.Generator("cpu").manual_seed(seed)
    attn = torch.nn.Module()
    for nm in ("to_q", "to_k", "to_v", "to_o"):
        lin = torch.nn.Linear(dim, dim, bias=bias)
        with torch.no_grad():
            lin.weight.copy_(torch.randn(dim, dim, generator=g) / dim ** 0.5)
            if bias:
                lin.bias.copy_(torch.randn(dim, generator=g) * 0.05)
        setattr(attn, nm, lin.bfloat16())
    ndim = 128 if joint else dim
    attn.norm_q = RMSNormModule(ndim, 1e-6, (1.0 + 0.2 * torch.randn(ndim, generator=g)).bfloat16())
    attn.norm_k = RMSNormModule(ndim, 1e-6, (1.0 + 0.2 * torch.randn(ndim, generator=g)).bfloat16())
    attn.heads = heads
    attn.add_k_proj = None
    attn.add_q_proj = None
    attn.to_out = torch.nn.ModuleList([attn.to_o, torch.nn.Identity()])
    del attn.to_o
    return attn


def rotary_tables(seed, S):
    """(cos, sin) [1, S, 1, 128] fp32 in the layout a Wan rotary module hands to the processor."""
    g = torch.Generator("cpu").manual_seed(seed)
    ang = torch.rand(S, 64, generator=g) * 6.2831853
    cos = torch.cos(ang).repeat_interleave(2, dim=-1)[None, :, None, :].contiguous()
    sin = torch.sin(ang).repeat_interleave(2, dim=-1)[None, :, None, :].contiguous()
    return cos, sin


WAN_PROC = dict(heads=4, grid=(3, 16, 20), num_q=12, num_k=40, iter_init=2, iter_step=1, top_p=0.9, min_kc_ratio=0.15,
                first_times_fp=900.0, start_reuse_step=2, reuse_interval=5, dyn_min=0.05, dyn_max=0.4,
                # (1-based step from the pipeline callback, scheduler timestep): dense, cluster, reuse, re-cluster
                steps=[(1, 950.0), (2, 800.0), (3, 700.0), (7, 300.0)])
PROC_ROWS_KEPT = 8          # the processor fixtures keep every 8th output row
HUN_PROC = dict(heads=3, grid=(2, 16, 20), num_q=10, num_k=32, iter_init=2, top_p=0.9, min_kc_ratio=0.2,
                context_length=64, prompt_length=40, first_times_fp=900.0, steps=[(1, 500.0)])


def write_density_csv(path, heads, steps, layer=0, seed=5, hole=None):
    """A Step,Layer,Head,Sparsity table; `hole` = (step, head) that is left out."""
    import csv
    g = torch.Generator("cpu").manual_seed(seed)
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["Step", "Layer", "Head", "Sparsity"])
        for s in steps:
            for h in range(heads):
                v = float(torch.rand(1, generator=g)) * 0.5
                if hole is not None and (s, h) == hole:
                    continue
                w.writerow([s, layer, h, f"{v:.6f}"])


def configure_wan_processor(cls, lookup):
    """Class attributes exactly as the reference's installer assigns them
    (svoo/models/wan/inference.py:267-328) for the WAN_PROC case."""
    P = WAN_PROC
    T, Hh, W = P["grid"]
    cls.first_layers_fp = 0
    cls.first_times_fp = P["first_times_fp"]
    cls.context_length = 0
    cls.num_frame = T
    cls.frame_size = Hh * W
    cls.num_q_centroids = P["num_q"]
    cls.num_k_centroids = P["num_k"]
    cls.top_p_kmeans = P["top_p"]
    cls.min_kc_ratio = P["min_kc_ratio"]
    cls.num_layers = 1
    cls.kmeans_iter_init = P["iter_init"]
    cls.kmeans_iter_step = P["iter_step"]
    cls.zero_step_kmeans_init = False
    cls.use_svoo = True
    cls.start_reuse_step = P["start_reuse_step"]
    cls.reuse_interval = P["reuse_interval"]
    cls.sparsity_lookup = lookup
    cls.use_dynamic_min_kc_ratio = True
    cls.dynamic_min_kc_ratio_min = P["dyn_min"]
    cls.dynamic_min_kc_ratio_max = P["dyn_max"]


def configure_hunyuan_processor(cls):
    """Class attributes as svoo/models/hunyuan10/inference.py assigns them, for the HUN_PROC case."""
    P = HUN_PROC
    T, Hh, W = P["grid"]
    cls.first_layers_fp = 0
    cls.first_times_fp = P["first_times_fp"]
    cls.context_length = P["context_length"]
    cls.prompt_length = P["prompt_length"]
    cls.num_frame = T
    cls.frame_size = Hh * W
    cls.num_q_centroids = P["num_q"]
    cls.num_k_centroids = P["num_k"]
    cls.top_p_kmeans = P["top_p"]
    cls.min_kc_ratio = P["min_kc_ratio"]
    cls.kmeans_iter_init = P["iter_init"]
    cls.kmeans_iter_step = P["iter_init"]
    cls.zero_step_kmeans_init = False
    cls.use_svoo = True
    cls.start_reuse_step = None
    cls.reuse_interval = 1
    cls.use_dynamic_min_kc_ratio = False
    cls.sparsity_lookup = None


def wan_step_hidden(step):
    """Activations of denoising step `step`: one smooth field, a little step-dependent noise."""
    P = WAN_PROC
    base = smooth_hidden(300, P["grid"], P["heads"] * 128).float()
    g = torch.Generator("cpu").manual_seed(300 + step)
    return (base + 0.08 * torch.randn(base.shape, generator=g)).bfloat16()


def hunyuan_inputs():
    """(hidden [1,N,dim], encoder [1,ctx,dim], attention mask [1, N+ctx] bool) of the HUN_PROC case."""
    P = HUN_PROC
    T, Hh, W = P["grid"]
    n = T * Hh * W
    x = smooth_hidden(400, P["grid"], P["heads"] * 128, extra_rows=P["context_length"])
    mask = torch.zeros(1, n + P["context_length"], dtype=torch.bool)
    mask[:, :n + P["prompt_length"]] = True
    return x[:, :n].contiguous(), x[:, n:].contiguous(), mask


def comparable_tokens(qlabels, ref_qlabels, video_map, ref_video_map):
    """bool [N]: tokens that, in every head, carry the reference's query label and whose query
    cluster keeps exactly the reference's key clusters.  The reference's torch.sort is unstable, so
    equal-probability clusters at the cut may be swapped in its map; output rows of the affected
    query clusters are compared nowhere, all other rows everywhere.  qlabels [H,N], maps [H,QC,KC]."""
    ql = torch.as_tensor(np.asarray(qlabels).astype(np.int64))
    rl = torch.as_tensor(np.asarray(ref_qlabels).astype(np.int64))
    same_row = torch.as_tensor((np.asarray(video_map) == np.asarray(ref_video_map)).all(-1))
    return ((ql == rl) & torch.gather(same_row, 1, ql)).all(0)


def processor_map_ties_ok(qc, kc, qs, ks, p, ratio, got_video_map, ref_video_map):
    """The two video maps keep clusters of equal probabilities in every row."""
    from oracle import svoo_oracle as O
    _, prob = O.identify_dynamic_map(qc[None], kc[None], qs[None], ks[None], p, ratio, return_probs=True)
    return same_up_to_ties(np.asarray(got_video_map), np.asarray(ref_video_map), prob.numpy()[0])
