"""Attention processors with the reference's plug-in interface.

`WanAttn_SAPAttn_Processor` follows svoo/models/wan/attention.py (:61-260 call path,
:546-590 class attributes, :669-715 clustering reuse, :931-956 density lookup,
:1110-1216 attention_core_logic); `Hunyuan_SAPAttn_Processor2_0` follows
svoo/models/hunyuan10/attention.py (:536-575, :977-1110).  Configuration is by the
same class attributes an installer assigns; per-instance state is `layer_idx`,
`_step_from_callback`, `current_inference_step` and the clustering cache.

The sparse branch runs on the svoo_b200 kernels.  The dense branch (first layers /
first timesteps, and cross attention) is plain torch SDPA, as in the reference.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import co_clustering as cc
from . import ops
from .layer import sparse_attention_layer
from .sparsity import min_kc_ratio_for_heads


class _SAPBase:
    # geometry
    context_length = 0
    num_frame = 0
    frame_size = 0
    # dense warm-up
    first_layers_fp = 0
    first_times_fp = 0
    zero_step_kmeans_init = False
    # clustering
    num_layers = 0
    num_q_centroids = 0
    num_k_centroids = 0
    top_p_kmeans = 0
    min_kc_ratio = 0
    kmeans_iter_init = 0
    kmeans_iter_step = 0
    use_svoo = True
    # reuse of a clustering across denoising steps
    start_reuse_step = None
    reuse_interval = 1
    # per-(step, layer, head) density from an offline profile
    use_dynamic_min_kc_ratio = False
    sparsity_lookup = None
    dynamic_min_kc_ratio_min = None
    dynamic_min_kc_ratio_max = None

    def __init__(self, layer_idx):
        self.layer_idx = layer_idx
        self.centroids_init = False
        self.current_inference_step = None
        self._cached_clustering_results = None

    # -- clustering with reuse (wan/attention.py:669-715, 793-819) -------------------------
    def _should_recluster(self) -> bool:
        step = getattr(self, "current_inference_step", None)
        if step is not None and self.start_reuse_step is not None and self.start_reuse_step > 0:
            if step >= self.start_reuse_step:
                return (step - self.start_reuse_step) % self.reuse_interval == 0
        return True

    def kmeans_clustering(self, query, key, layer_idx=None) -> ops.Clustering:
        """query/key [1, H, N, 128] (video tokens only).  Returns the device-side clustering;
        a cached one when the reuse schedule says so."""
        if not self._should_recluster() and self._cached_clustering_results is not None:
            return self._cached_clustering_results
        cfg, H, N, D = query.shape
        iters = self.kmeans_iter_step if self.centroids_init else self.kmeans_iter_init
        c = cc.co_cluster(query.reshape(cfg * H, N, D), key.reshape(cfg * H, N, D), self.num_q_centroids,
                          self.num_k_centroids, iters)
        self.centroids_init = True
        self._cached_clustering_results = c
        return c

    def _get_min_kc_ratio_for_heads_from_step(self, inference_step, num_heads):
        return min_kc_ratio_for_heads(self.sparsity_lookup, self.use_dynamic_min_kc_ratio, inference_step,
                                      self.layer_idx, num_heads, self.min_kc_ratio,
                                      self.dynamic_min_kc_ratio_min, self.dynamic_min_kc_ratio_max)

    def _full_attention_flag(self, timestep) -> bool:
        flag = self.layer_idx < self.first_layers_fp
        if timestep is not None:
            if isinstance(timestep, torch.Tensor):
                value = timestep.flatten()[0].item() if timestep.numel() > 0 else None
            else:
                value = timestep
            if value is not None and value > self.first_times_fp:
                flag = True
        return flag

    def flash_attention(self, query, key, value):
        return F.scaled_dot_product_attention(query, key, value, dropout_p=0.0, is_causal=False)

    def _sparse(self, query, key, value, prompt_length=None):
        cfg, H, S, D = query.shape
        n_video = self.num_frame * self.frame_size
        if self.context_length:
            qv, kv = query[:, :, :n_video].contiguous(), key[:, :, :n_video].contiguous()
        else:
            qv, kv = query, key
        c = self.kmeans_clustering(qv, kv, self.layer_idx)
        ratio = self._get_min_kc_ratio_for_heads_from_step(self.current_inference_step, H)
        return sparse_attention_layer(query, key, value, num_q_centroids=self.num_q_centroids,
                                      num_k_centroids=self.num_k_centroids, kmeans_iters=0,
                                      top_p=self.top_p_kmeans, min_kc_ratio=ratio, clustering=c,
                                      context_length=self.context_length, prompt_length=prompt_length)


class WanAttn_SAPAttn_Processor(_SAPBase):
    """Self-attention processor for Wan DiT blocks; cross attention (timestep is None) is dense."""

    def get_qkv(self, attn, hidden_states, encoder_hidden_states):
        if encoder_hidden_states is None:
            encoder_hidden_states = hidden_states
        if getattr(attn, "fused_projections", False) and getattr(attn, "cross_attention_dim_head", None) is None:
            return attn.to_qkv(hidden_states).chunk(3, dim=-1)
        return attn.to_q(hidden_states), attn.to_k(encoder_hidden_states), attn.to_v(encoder_hidden_states)

    def get_qk_norm(self, attn, query, key):
        if getattr(attn, "norm_q", None) is not None:
            query = attn.norm_q(query)
        if getattr(attn, "norm_k", None) is not None:
            key = attn.norm_k(key)
        return query, key

    @staticmethod
    def apply_rotary_emb(hidden_states, freqs_cos, freqs_sin):
        x1, x2 = hidden_states.unflatten(-1, (-1, 2)).unbind(-1)
        cos = freqs_cos[..., 0::2]
        sin = freqs_sin[..., 1::2]
        out = torch.empty_like(hidden_states)
        out[..., 0::2] = x1 * cos - x2 * sin
        out[..., 1::2] = x1 * sin + x2 * cos
        return out.type_as(hidden_states)

    @staticmethod
    def _fused_producer_applies(attn, query, key, rotary_emb) -> bool:
        """One-pass norm + rotary + head transpose (svoo_b200_qk_prep): self-attention on one bf16
        CUDA sample with 128-wide heads and weight-only RMS norms over the whole projection."""
        if not (query.is_cuda and query.dtype == torch.bfloat16 and query.shape[0] == 1 and query.shape == key.shape):
            return False
        if query.shape[-1] != attn.heads * 128 or attn.heads > 128:
            return False
        for name in ("norm_q", "norm_k"):
            n = getattr(attn, name, None)
            if n is None or getattr(n, "weight", None) is None or getattr(n, "bias", None) is not None:
                return False
            if n.weight.numel() != query.shape[-1]:
                return False
        return True

    @staticmethod
    def fused_producer(attn, query, key, value, rotary_emb):
        """Replaces get_qk_norm + apply_rotary_emb + get_transpose_qkv of the reference
        (svoo/models/wan/attention.py:112-131,177-195) for the case _fused_producer_applies accepts."""
        H = attn.heads
        cos, sin = (None, None) if rotary_emb is None else rotary_emb
        q = ops.qk_prep(query[0].contiguous(), H, attn.norm_q.weight, attn.norm_q.eps, cos, sin)
        k = ops.qk_prep(key[0].contiguous(), H, attn.norm_k.weight, attn.norm_k.eps, cos, sin)
        v = ops.qk_prep(value[0].contiguous(), H)
        return q[None], k[None], v[None]

    def get_o(self, attn, query, hidden_states, hidden_states_img=None):
        if hidden_states.dim() == 4:
            hidden_states = hidden_states.transpose(1, 2).flatten(2, 3)
        hidden_states = hidden_states.type_as(query)
        if hidden_states_img is not None:
            hidden_states = hidden_states + hidden_states_img
        hidden_states = attn.to_out[0](hidden_states)
        return attn.to_out[1](hidden_states)

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, attention_mask=None, rotary_emb=None,
                 timestep=None):
        query, key, value = self.get_qkv(attn, hidden_states, encoder_hidden_states)
        if self._fused_producer_applies(attn, query, key, rotary_emb):
            query, key, value = self.fused_producer(attn, query, key, value, rotary_emb)
        else:
            query, key = self.get_qk_norm(attn, query, key)
            query = query.unflatten(2, (attn.heads, -1))
            key = key.unflatten(2, (attn.heads, -1))
            value = value.unflatten(2, (attn.heads, -1))
            if rotary_emb is not None:
                query = self.apply_rotary_emb(query, *rotary_emb)
                key = self.apply_rotary_emb(key, *rotary_emb)
            query, key, value = (t.transpose(1, 2).contiguous() for t in (query, key, value))
        if timestep is None:
            out = F.scaled_dot_product_attention(query, key, value, attn_mask=attention_mask)
            out = out.transpose(1, 2).flatten(2, 3)
        else:
            out = self.attention_core_logic(query, key, value, timestep)
        return self.get_o(attn, query, out)

    def attention_core_logic(self, query, key, value, timestep):
        """query/key/value [1, H, S, 128] -> [1, S, H*128] (wan/attention.py:1110-1216)."""
        cfg, H, S, D = query.size()
        assert cfg == 1, "Batch size must be 1 for kmeans block sparse attention"
        cb_step = getattr(self, "_step_from_callback", None)
        self.current_inference_step = cb_step
        assert S == self.context_length + self.num_frame * self.frame_size, (
            f"Query Shape: {S} is not equivalent to {self.context_length} + {self.num_frame} * {self.frame_size}")
        if self._full_attention_flag(timestep):
            if self.zero_step_kmeans_init:
                n_video = self.num_frame * self.frame_size
                self.kmeans_clustering(query[:, :, :n_video].contiguous(), key[:, :, :n_video].contiguous())
            out = self.flash_attention(query, key, value)
        else:
            out = self._sparse(query, key, value)
        return out.transpose(1, 2).flatten(2, 3)


class Hunyuan_SAPAttn_Processor2_0(_SAPBase):
    """Joint-attention core for HunyuanVideo: video tokens are clustered, the text tokens
    that follow them form two dense blocks (prompt, unused prompt)."""
    context_length = 256
    prompt_length = 256

    def attention_core_logic(self, query, key, value, timestep, layer_idx=None, cu_max_seqlens=None):
        """query/key/value [1, H, S, 128] -> [1, H, S, 128] (hunyuan10/attention.py:1031-1110)."""
        cfg, H, S, D = query.size()
        assert cfg == 1, "Batch size must be 1 for kmeans block sparse attention"
        assert S == self.context_length + self.num_frame * self.frame_size, (
            f"Query Shape: {S} is not equivalent to {self.context_length} + {self.num_frame} * {self.frame_size}")
        self.current_inference_step = getattr(self, "_step_from_callback", None)
        if self._full_attention_flag(timestep):
            n_video = self.num_frame * self.frame_size
            if self.zero_step_kmeans_init:
                self.kmeans_clustering(query[:, :, :n_video].contiguous(), key[:, :, :n_video].contiguous())
            # dense: prompt and video attend each other, the unused prompt only itself
            valid = n_video + self.prompt_length
            out = torch.empty_like(query)
            out[:, :, :valid] = self.flash_attention(query[:, :, :valid], key[:, :, :valid], value[:, :, :valid])
            if valid < S:
                out[:, :, valid:] = self.flash_attention(query[:, :, valid:], key[:, :, valid:], value[:, :, valid:])
            return out
        return self._sparse(query, key, value, prompt_length=self.prompt_length)
