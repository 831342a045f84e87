"""A plain-torch DiT with the Wan2.1 block structure, used to run the sparse-attention
processor in situ: every block's self-attention goes through `WanAttn_SAPAttn_Processor`
(the path this package implements); everything else -- patch embedding, condition embedder,
layer norms, AdaLN modulation, cross attention to the text context, feed-forward, output
projection -- is ordinary torch and outside the path.

The block dataflow follows the reference's patched forward (svoo/models/wan/custom_models.py:
22-108 block, :116-197 model), which threads `timestep` into `attn1` (:63).  Weights are
random: real checkpoints are not available offline, and the layer's cost does not depend on them.

Sequence parallelism (one process per GPU): with `exchange` (a parallel.PeerExchange) every rank
holds a contiguous [S/P] shard of the tokens; token-wise layers run on the shard, the self-attention
re-shards to heads and back through peer stores (`SequenceParallelWanProcessor`), the cross
attention needs no exchange (the text context is replicated).
"""
from __future__ import annotations

import dataclasses
import math
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .layer import sparse_attention_layer
from .processor import WanAttn_SAPAttn_Processor


@dataclasses.dataclass(frozen=True)
class WanDiTConfig:
    """Wan2.1-T2V-1.3B shape by default."""
    num_layers: int = 30
    dim: int = 1536
    heads: int = 12
    ffn_dim: int = 8960
    text_dim: int = 4096
    text_len: int = 512
    freq_dim: int = 256
    in_channels: int = 16
    out_channels: int = 16
    patch: Tuple[int, int, int] = (1, 2, 2)
    eps: float = 1e-6
    latent: Tuple[int, int, int] = (21, 60, 104)          # 81 frames at 480 x 832: 21 x 30 x 52 = 32,760 tokens

    @property
    def grid(self) -> Tuple[int, int, int]:
        return tuple(l // p for l, p in zip(self.latent, self.patch))

    @property
    def tokens(self) -> int:
        t, h, w = self.grid
        return t * h * w


class RMSNormAcrossHeads(nn.Module):
    """Weight-only RMS norm over the whole projection (all heads), fp32 statistics."""

    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        return (y * self.weight.float()).to(x.dtype)


class Attention(nn.Module):
    """The attribute surface a Wan attention processor works on (to_q / to_k / to_v / to_out,
    norm_q / norm_k, heads, add_k_proj) and its dispatch: forward hands everything to `processor`."""

    def __init__(self, dim: int, heads: int, eps: float):
        super().__init__()
        self.heads = heads
        self.to_q = nn.Linear(dim, dim)
        self.to_k = nn.Linear(dim, dim)
        self.to_v = nn.Linear(dim, dim)
        self.to_out = nn.ModuleList([nn.Linear(dim, dim), nn.Dropout(0.0)])
        self.norm_q = RMSNormAcrossHeads(dim, eps)
        self.norm_k = RMSNormAcrossHeads(dim, eps)
        self.add_k_proj = None
        self.processor = None

    def set_processor(self, processor) -> None:
        self.processor = processor

    def forward(self, hidden_states, encoder_hidden_states=None, attention_mask=None, **kwargs):
        return self.processor(self, hidden_states, encoder_hidden_states, attention_mask, **kwargs)


class WanBlock(nn.Module):
    def __init__(self, cfg: WanDiTConfig):
        super().__init__()
        d = cfg.dim
        self.norm1 = nn.LayerNorm(d, cfg.eps, elementwise_affine=False)
        self.attn1 = Attention(d, cfg.heads, cfg.eps)
        self.norm2 = nn.LayerNorm(d, cfg.eps, elementwise_affine=True)
        self.attn2 = Attention(d, cfg.heads, cfg.eps)
        self.norm3 = nn.LayerNorm(d, cfg.eps, elementwise_affine=False)
        self.ffn = nn.Sequential(nn.Linear(d, cfg.ffn_dim), nn.GELU(approximate="tanh"), nn.Linear(cfg.ffn_dim, d))
        self.scale_shift_table = nn.Parameter(torch.zeros(1, 6, d))

    @staticmethod
    def _ln(norm: nn.LayerNorm, x):
        w = None if norm.weight is None else norm.weight.float()
        b = None if norm.bias is None else norm.bias.float()
        return F.layer_norm(x.float(), norm.normalized_shape, w, b, norm.eps)

    def forward(self, hidden_states, encoder_hidden_states, temb, rotary_emb, timestep=0):
        shift, scale, gate, c_shift, c_scale, c_gate = (self.scale_shift_table.float() + temb.float()).chunk(6, dim=1)
        x = (self._ln(self.norm1, hidden_states) * (1 + scale) + shift).type_as(hidden_states)
        attn = self.attn1(hidden_states=x, rotary_emb=rotary_emb, timestep=timestep)
        hidden_states = (hidden_states.float() + attn * gate).type_as(hidden_states)
        x = self._ln(self.norm2, hidden_states).type_as(hidden_states)
        hidden_states = hidden_states + self.attn2(hidden_states=x, encoder_hidden_states=encoder_hidden_states)
        x = (self._ln(self.norm3, hidden_states) * (1 + c_scale) + c_shift).type_as(hidden_states)
        ff = self.ffn(x)
        return (hidden_states.float() + ff.float() * c_gate).type_as(hidden_states)


def rope_tables(grid: Tuple[int, int, int], head_dim: int = 128, theta: float = 10000.0):
    """(cos, sin) [1, S, 1, head_dim] fp32 of the 3-D rotary embedding, frame-major token order; the
    head dimension is split 44 / 42 / 42 over (t, h, w) and every frequency fills an (even, odd) pair."""
    T, Hh, W = grid
    d_h = d_w = 2 * (head_dim // 6)
    d_t = head_dim - d_h - d_w
    t, h, w = torch.meshgrid(torch.arange(T), torch.arange(Hh), torch.arange(W), indexing="ij")
    parts = []
    for pos, d in ((t, d_t), (h, d_h), (w, d_w)):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        parts.append(pos.reshape(-1).double()[:, None] * inv[None, :])
    ang = torch.cat(parts, -1)
    cos = torch.cos(ang).float().repeat_interleave(2, dim=-1)[None, :, None, :].contiguous()
    sin = torch.sin(ang).float().repeat_interleave(2, dim=-1)[None, :, None, :].contiguous()
    return cos, sin


class WanDiT(nn.Module):
    def __init__(self, cfg: WanDiTConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.dim
        self.patch_embedding = nn.Conv3d(cfg.in_channels, d, kernel_size=cfg.patch, stride=cfg.patch)
        self.time_embedder = nn.Sequential(nn.Linear(cfg.freq_dim, d), nn.SiLU(), nn.Linear(d, d))
        self.time_proj = nn.Linear(d, 6 * d)
        self.text_embedder = nn.Sequential(nn.Linear(cfg.text_dim, d), nn.GELU(approximate="tanh"), nn.Linear(d, d))
        self.blocks = nn.ModuleList([WanBlock(cfg) for _ in range(cfg.num_layers)])
        self.norm_out = nn.LayerNorm(d, cfg.eps, elementwise_affine=False)
        self.proj_out = nn.Linear(d, cfg.out_channels * math.prod(cfg.patch))
        self.scale_shift_table = nn.Parameter(torch.zeros(1, 2, d))
        self.seq_shard: Optional[Tuple[int, int]] = None      # (rank, world): this process holds tokens [rank*S/P, (rank+1)*S/P)

    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02) -> "WanDiT":
        g = torch.Generator("cpu").manual_seed(seed)
        for name, p in self.named_parameters():
            if "scale_shift_table" in name:
                p.copy_(torch.randn(p.shape, generator=g) / p.shape[-1] ** 0.5)
            elif p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * std)
            elif name.endswith("bias"):
                p.zero_()
            elif "norm_q" in name or "norm_k" in name:
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g))
        return self

    def _timestep_embedding(self, timestep):
        half = self.cfg.freq_dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=timestep.device) / half)
        args = timestep.float()[:, None] * freqs[None]
        return torch.cat([torch.cos(args), torch.sin(args)], -1)

    def forward(self, latents, timestep, encoder_hidden_states):
        """latents [1, C, T, H, W]; timestep [1]; encoder_hidden_states [1, text_len, text_dim].
        Returns the predicted latents [1, C, T, H, W] (with a sequence shard: this rank's token
        rows of the projected output, [1, S/P, C*patch])."""
        cfg = self.cfg
        dtype = self.proj_out.weight.dtype
        cos, sin = rope_tables(cfg.grid)
        x = self.patch_embedding(latents.to(dtype)).flatten(2).transpose(1, 2).contiguous()
        S = x.shape[1]
        lo, hi = 0, S
        if self.seq_shard is not None:
            rank, world = self.seq_shard
            lo, hi = rank * (S // world), (rank + 1) * (S // world)
            x = x[:, lo:hi].contiguous()
        rotary = (cos[:, lo:hi].to(x.device), sin[:, lo:hi].to(x.device))
        temb = self.time_embedder(self._timestep_embedding(timestep).to(dtype))
        timestep_proj = self.time_proj(F.silu(temb)).unflatten(1, (6, -1))
        text = self.text_embedder(encoder_hidden_states.to(dtype))
        for block in self.blocks:
            x = block(x, text, timestep_proj, rotary, timestep=timestep)
        shift, scale = (self.scale_shift_table.float() + temb.float().unsqueeze(1)).chunk(2, dim=1)
        x = (F.layer_norm(x.float(), (cfg.dim,), None, None, cfg.eps) * (1 + scale) + shift).type_as(x)
        x = self.proj_out(x)
        if self.seq_shard is not None:
            return x
        T, Hh, W = cfg.grid
        pt, ph, pw = cfg.patch
        x = x.reshape(1, T, Hh, W, pt, ph, pw, -1).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return x.flatten(6, 7).flatten(4, 5).flatten(2, 3)


class SequenceParallelWanProcessor(WanAttn_SAPAttn_Processor):
    """WanAttn_SAPAttn_Processor for a sequence-parallel caller: `hidden_states` is this rank's
    [1, S/P, H*128] shard.  Self-attention: the projections run on the shard, the producer (norm +
    rotary + head transpose) stores its rows straight into the ranks that own the heads, every rank
    runs the layer on its heads over the whole sequence, and the attention kernel stores the result
    rows back into the sequence shards.  No counterpart in the reference (one GPU).  Class attribute
    `exchange` holds the parallel.PeerExchange shared by all layers."""
    exchange = None

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, attention_mask=None, rotary_emb=None,
                 timestep=None):
        if timestep is None or self.exchange is None:
            return super().__call__(attn, hidden_states, encoder_hidden_states, attention_mask, rotary_emb, timestep)
        x = self.exchange
        query, key, value = self.get_qkv(attn, hidden_states, None)
        cos, sin = rotary_emb
        q, k, v = x.producer_to_heads(query[0], key[0], value[0], (attn.norm_q.weight, attn.norm_q.eps),
                                      (attn.norm_k.weight, attn.norm_k.eps), cos, sin)
        out = self.attention_core_logic(q[None], k[None], v[None], timestep)
        return self.get_o(attn, query, out)

    def flash_attention(self, query, key, value):
        raise NotImplementedError("the dense warm-up branch is not sharded; run it on one GPU")

    def _sparse(self, query, key, value, prompt_length=None):
        x = self.exchange
        if x is None:
            return super()._sparse(query, key, value, prompt_length)
        cfg, H, S, D = query.shape                             # H = this rank's heads
        c = self.kmeans_clustering(query, key, self.layer_idx)
        self._last_shape = (query.device, cfg * H, S, S, self.num_q_centroids, self.num_k_centroids)
        ratio = self._get_min_kc_ratio_for_heads_from_step(self.current_inference_step, x.H)
        if isinstance(ratio, (list, tuple)):
            ratio = [ratio[h] for h in x.parts[x.rank]]
        sparse_attention_layer(query, key, value, num_q_centroids=self.num_q_centroids, num_k_centroids=self.num_k_centroids,
                               kmeans_iters=0, top_p=self.top_p_kmeans, min_kc_ratio=ratio, clustering=c,
                               value_ready=x.value_ready, peer_out=x.peer_out,
                               ear_gamma=self.ear_gamma if self.use_ear else None)
        return x.seq_result()                                  # [S/P, H_all, 128]

    def attention_core_logic(self, query, key, value, timestep):
        if self.exchange is None:
            return super().attention_core_logic(query, key, value, timestep)
        cfg, H, S, D = query.size()
        cb_step = getattr(self, "_step_from_callback", None)
        self.current_inference_step = cb_step if cb_step is not None else self._get_inference_step(timestep)
        assert S == self.num_frame * self.frame_size, f"Query Shape: {S} is not {self.num_frame} * {self.frame_size}"
        if self._full_attention_flag(timestep):
            self.flash_attention(query, key, value)
        out = self._sparse(query, key, value)                 # [S/P, H_all, 128]
        return out.flatten(1, 2)[None]


def install_processors(model: WanDiT, processor_cls, grid: Tuple[int, int, int], *, num_q_centroids: int,
                       num_k_centroids: int, top_p_kmeans: float, min_kc_ratio: float, kmeans_iter_init: int,
                       kmeans_iter_step: int, sparsity_lookup=None, dynamic_min_kc_ratio_min=None,
                       dynamic_min_kc_ratio_max=None, start_reuse_step=None, reuse_interval: int = 1,
                       first_layers_fp: int = 0, first_times_fp: float = float("inf"), pattern: str = "SVOO",
                       ear_gamma: float = 1.0) -> List:
    """Class attributes and per-block processors, the way the reference's installer sets them
    (svoo/models/wan/inference.py:267-355); `pattern == "EAR"` switches the error-aware routing on
    (`:281-282`).  Cross attention (attn2) gets a processor of the same class: it is called without a
    timestep and takes the dense branch.  Returns the attn1 processors."""
    cls = processor_cls
    cls.use_ear, cls.ear_gamma = pattern == "EAR", ear_gamma
    cls.first_layers_fp, cls.first_times_fp = first_layers_fp, first_times_fp
    cls.context_length, cls.num_frame, cls.frame_size = 0, grid[0], grid[1] * grid[2]
    cls.num_q_centroids, cls.num_k_centroids = num_q_centroids, num_k_centroids
    cls.top_p_kmeans, cls.min_kc_ratio = top_p_kmeans, min_kc_ratio
    cls.num_layers = len(model.blocks)
    cls.kmeans_iter_init, cls.kmeans_iter_step, cls.zero_step_kmeans_init = kmeans_iter_init, kmeans_iter_step, False
    cls.use_svoo = True
    cls.start_reuse_step, cls.reuse_interval = start_reuse_step, reuse_interval
    cls.sparsity_lookup = sparsity_lookup
    cls.use_dynamic_min_kc_ratio = sparsity_lookup is not None
    cls.dynamic_min_kc_ratio_min, cls.dynamic_min_kc_ratio_max = dynamic_min_kc_ratio_min, dynamic_min_kc_ratio_max
    procs = []
    for layer_idx, block in enumerate(model.blocks):
        p = cls(layer_idx)
        p.num_layers = len(model.blocks)
        block.attn1.set_processor(p)
        block.attn2.set_processor(cls(layer_idx))
        procs.append(p)
    return procs


def set_attention_step(model: WanDiT, step_1_based: int) -> None:
    """What the pipeline's step callback does (wan_t2v_inference.py:153-173): tell every processor
    which denoising step comes next."""
    for block in model.blocks:
        for attn in (block.attn1, block.attn2):
            if attn.processor is not None:
                attn.processor._step_from_callback = step_1_based


def write_density_table(path: str, steps: int, layers: int, heads: int, lo: float, hi: float, seed: int) -> None:
    """A seeded U[lo, hi] table in the offline profile's CSV format (Step,Layer,Head,Sparsity; steps are 1-based)."""
    import csv
    g = torch.Generator("cpu").manual_seed(seed)
    vals = lo + (hi - lo) * torch.rand(steps, layers, heads, generator=g, dtype=torch.float64)
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["Step", "Layer", "Head", "Sparsity"])
        for s in range(steps):
            for l in range(layers):
                for h in range(heads):
                    w.writerow([s + 1, l, h, f"{float(vals[s, l, h]):.6f}"])
