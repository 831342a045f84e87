"""Seeded synthetic Q/K/V for the sparse-attention layer benchmarks and tests.

Real Wan / HunyuanVideo activations need model weights; these inputs stand in
for them: a smooth low-frequency field over the (t, h, w) latent grid plus
Gaussian noise, so that token clusters exist, optionally RMS-normalised and
rotated with an interleaved-pair 3-D RoPE like the one the Wan processor applies
(reference: svoo/models/wan/attention.py:179-190).

Everything is generated with CPU generators so that the same seed gives the same
tensors on every machine.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, List, Optional, Tuple

import torch


@dataclasses.dataclass(frozen=True)
class LayerConfig:
    """One sparse-attention layer workload."""
    name: str
    cfg_id: int
    heads: int
    grid: Tuple[int, int, int]          # (t, h, w) latent grid; N = t*h*w video tokens
    dtype: torch.dtype
    num_q: int
    num_k: int
    iters: int
    density: Tuple[float, float]        # per-head budget ~ U[lo, hi] (lo == hi: constant)
    density_seed: int
    rope: bool
    text_tokens: int = 0                # dense text tokens appended after video (Hunyuan)
    top_p: float = 0.9

    @property
    def n_video(self) -> int:
        t, h, w = self.grid
        return t * h * w

    @property
    def n_tokens(self) -> int:
        return self.n_video + self.text_tokens


CONFIGS: Dict[str, LayerConfig] = {
    "cfg0": LayerConfig("cfg0-cpu-4k", 0, 2, (4, 32, 32), torch.float32, 32, 128, 10, (0.20, 0.20), 1000, False),
    "cfg1": LayerConfig("wan1.3b-480p", 1, 12, (21, 30, 52), torch.bfloat16, 100, 500, 5, (0.05, 0.30), 1001, True),
    "cfg2": LayerConfig("wan14b-720p", 2, 40, (21, 45, 80), torch.bfloat16, 100, 500, 5, (0.05, 0.25), 1002, True),
    "cfg3": LayerConfig("hunyuan13b-720p", 3, 24, (33, 45, 80), torch.bfloat16, 128, 640, 5, (0.05, 0.20), 1003, True,
                        text_tokens=256),
}


def head_densities(cfg: LayerConfig) -> List[float]:
    """Per-head density budget d_h, seeded."""
    lo, hi = cfg.density
    if lo == hi:
        return [float(lo)] * cfg.heads
    g = torch.Generator("cpu").manual_seed(cfg.density_seed)
    u = torch.rand(cfg.heads, generator=g, dtype=torch.float64)
    return [float(lo + (hi - lo) * x) for x in u]


def init_indices(cfg: LayerConfig, heads: Optional[int] = None, seed: int = 7):
    """Initial centroid token indices drawn the way the reference draws them
    (svoo/co_clustering.py:2417-2421): q indices first, then k indices."""
    H = cfg.heads if heads is None else heads
    g = torch.Generator("cpu").manual_seed(seed)
    q_idx = torch.randint(0, cfg.n_video, (H, cfg.num_q), generator=g)
    k_idx = torch.randint(0, cfg.n_video, (H, cfg.num_k), generator=g)
    return q_idx, k_idx


def _grid_coords(grid):
    T, Hh, W = grid
    t = torch.arange(T, dtype=torch.float32)
    h = torch.arange(Hh, dtype=torch.float32)
    w = torch.arange(W, dtype=torch.float32)
    tt, hh, ww = torch.meshgrid(t, h, w, indexing="ij")       # frame-major token order
    return tt.reshape(-1), hh.reshape(-1), ww.reshape(-1)


def _rope_tables(grid, dim=128, theta=10000.0):
    """cos/sin [N, dim/2] for a t/h/w split of the head dim of 44/42/42."""
    tt, hh, ww = _grid_coords(grid)
    d_h = d_w = 2 * (dim // 6)
    d_t = dim - d_h - d_w
    parts = []
    for pos, d in ((tt, d_t), (hh, d_h), (ww, d_w)):
        inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        parts.append(pos.double()[:, None] * inv[None, :])
    ang = torch.cat(parts, -1)
    return torch.cos(ang).float(), torch.sin(ang).float()


def _apply_rope(x, cos, sin):
    x1 = x[..., 0::2]
    x2 = x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = x1 * cos - x2 * sin
    out[..., 1::2] = x1 * sin + x2 * cos
    return out


def make_head(cfg: LayerConfig, head: int, dim: int = 128):
    """(q, k, v) of one head, each [n_tokens, dim] in cfg.dtype."""
    T, Hh, W = cfg.grid
    tt, hh, ww = _grid_coords(cfg.grid)
    coords = torch.stack([tt / T, hh / Hh, ww / W], -1)                     # [N,3]
    gf = torch.Generator("cpu").manual_seed(1000 * cfg.cfg_id + 10 * head + 9)
    freqs = torch.randint(0, 4, (16, 3), generator=gf)
    zero = freqs.sum(-1) == 0
    freqs[zero, 0] = 1
    phase_base = coords @ freqs.float().T                                   # [N,16]
    rope = _rope_tables(cfg.grid, dim) if cfg.rope else None
    outs = []
    for which in range(3):
        g = torch.Generator("cpu").manual_seed(1000 * cfg.cfg_id + 10 * head + which)
        phi = torch.rand(16, generator=g) * (2 * math.pi)
        G = torch.randn(16, dim, generator=g) / 4
        x = torch.cos(2 * math.pi * phase_base + phi) @ G
        x = x + 0.5 * torch.randn(cfg.n_video, dim, generator=g)
        if cfg.rope:
            x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6)
            if which < 2:
                x = _apply_rope(x, *rope)
        if cfg.text_tokens:
            txt = torch.randn(cfg.text_tokens, dim, generator=g)
            txt = txt / torch.sqrt((txt * txt).mean(-1, keepdim=True) + 1e-6)
            x = torch.cat([x, txt], 0)
        outs.append(x.to(cfg.dtype))
    return tuple(outs)


def make_qkv(cfg: LayerConfig, heads: Optional[List[int]] = None, pin_memory: bool = False):
    """Q, K, V as [1, H, n_tokens, 128] CPU tensors for the listed heads (default: all)."""
    hs = list(range(cfg.heads)) if heads is None else list(heads)
    shape = (1, len(hs), cfg.n_tokens, 128)
    q = torch.empty(shape, dtype=cfg.dtype, pin_memory=pin_memory)
    k = torch.empty(shape, dtype=cfg.dtype, pin_memory=pin_memory)
    v = torch.empty(shape, dtype=cfg.dtype, pin_memory=pin_memory)
    for i, h in enumerate(hs):
        q[0, i], k[0, i], v[0, i] = make_head(cfg, h)
    return q, k, v


def tensor_checksum(*tensors):
    """Order-dependent 64-bit checksum (numpy uint64 [1]) of the raw bytes of the tensors."""
    import numpy as np
    acc = 1469598103934665603
    for t in tensors:
        b = t.contiguous().view(torch.uint8).reshape(-1).numpy().astype(np.uint64)
        w = (np.arange(b.size, dtype=np.uint64) % np.uint64(65521)) + np.uint64(1)
        acc = (acc * 1099511628211 + int((b * w).sum(dtype=np.uint64))) % (1 << 64)
    return np.array([acc], dtype=np.uint64)
