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
    # error-aware routing (wan/attention.py:580-581): block selection by estimated error and centroid
    # compensation of the pruned blocks
    use_ear = False
    ear_gamma = 1.0
    # reuse of a clustering across denoising steps
    start_reuse_step = None
    reuse_interval = 1
    # not in the reference (which re-draws random tokens at every clustering call): start a
    # re-clustering from the centroids of the previous one
    warm_start_centroids = False
    # per-(step, layer, head) density from an offline profile
    use_dynamic_min_kc_ratio = False
    sparsity_lookup = None
    dynamic_min_kc_ratio_min = None
    dynamic_min_kc_ratio_max = None

    # scheduler-timestep -> step counter shared by all layers (wan/attention.py:423-444)
    _current_internal_timestep = None
    _inference_step_counter = 0
    _seen_timesteps: set = set()

    def __init__(self, layer_idx):
        self.layer_idx = layer_idx
        self.centroids_init = False
        self.current_inference_step = None
        self._cached_clustering_results = None
        self._last_shape = None
        self.last_block_map = None

    def _get_inference_step(self, timestep):
        """1-based denoising step derived from the scheduler timestep when no pipeline callback
        sets `_step_from_callback`: a new timestep value counts one step, a timestep larger than
        the last one starts a new run (wan/attention.py:423-444)."""
        cls = self.__class__
        t = timestep.flatten()[0].item() if isinstance(timestep, torch.Tensor) else timestep
        if cls._current_internal_timestep is not None and t > cls._current_internal_timestep:
            cls._inference_step_counter = 0
            cls._seen_timesteps.clear()
        if t not in cls._seen_timesteps:
            cls._seen_timesteps.add(t)
            cls._inference_step_counter += 1
            cls._current_internal_timestep = t
        return cls._inference_step_counter

    def check_status(self) -> None:
        """Raises if a tensor-core kernel of this layer's last sparse call gave up on one of its
        bounded waits (its output rows were then left unwritten).  Reads two device words, so it
        synchronises: call it once per denoising step or at the end of a run, not per layer."""
        if self._last_shape is None:
            return
        dev, H, S, n_video, qc_attn, kc_attn = self._last_shape
        attn_status = ops.ear_attention_status if self.use_ear else ops.attention_status
        if attn_status(dev, H, S, qc_attn, kc_attn) != 0:
            raise RuntimeError(f"layer {self.layer_idx}: the attention kernel timed out on a barrier; output incomplete")
        if ops.cluster_status(dev, H, n_video, self.num_q_centroids, self.num_k_centroids) != 0:
            raise RuntimeError(f"layer {self.layer_idx}: the assignment kernel timed out on a barrier; labels incomplete")

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
        q_flat, k_flat = query.reshape(cfg * H, N, D), key.reshape(cfg * H, N, D)
        prev = self._cached_clustering_results if self.centroids_init else None
        if self.use_svoo:
            warm = (prev.qcentroids, prev.kcentroids) if (self.warm_start_centroids and prev is not None) else None
            c = cc.co_cluster(q_flat, k_flat, self.num_q_centroids, self.num_k_centroids, iters, init_centroids=warm,
                              init_indices=self.draw_init_indices(cfg * H, N, query.device))
        else:
            # plain Euclidean k-means per side; later calls continue from the previous centroids
            # (kmeans_init / kmeans_step, wan/attention.py:612-667)
            c = self._euclid_clustering(q_flat, k_flat, iters, prev)
        self.centroids_init = True
        self._cached_clustering_results = c
        return c

    def draw_init_indices(self, BH, N, device):
        """Initial centroid token indices (q [BH,QC], k [BH,KC]) of a fresh clustering, or None to
        let co_cluster draw them on the device in the reference's order (q first, then k,
        svoo/co_clustering.py:2417-2421).  A hook: tests replace it to replay recorded draws."""
        return None

    def _euclid_clustering(self, q_flat, k_flat, iters, prev) -> ops.Clustering:
        out = []
        for x, n_clusters, init in ((q_flat, self.num_q_centroids, None if prev is None else prev.qcentroids),
                                    (k_flat, self.num_k_centroids, None if prev is None else prev.kcentroids)):
            labels, centroids, sizes, _ = cc.batch_kmeans_Euclid(x, n_clusters, max_iters=iters, init_centroids=init)
            idx, off = ops.sort_labels(labels, n_clusters)
            out.append((labels.to(torch.int32), centroids.contiguous(), sizes, idx, off))
        (ql, qc, qs, qi, qo), (kl, kc, ks, ki, ko) = out
        return ops.Clustering(ql, kl, qc, kc, qs, ks, qi, ki, qo, ko)

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
        extra = 2 if self.context_length else 0
        self._last_shape = (query.device, cfg * H, S, n_video, self.num_q_centroids + extra, self.num_k_centroids + extra)
        ratio = self._get_min_kc_ratio_for_heads_from_step(self.current_inference_step, H)
        out, state = sparse_attention_layer(query, key, value, num_q_centroids=self.num_q_centroids,
                                            num_k_centroids=self.num_k_centroids, kmeans_iters=0,
                                            top_p=self.top_p_kmeans, min_kc_ratio=ratio, clustering=c,
                                            context_length=self.context_length, prompt_length=prompt_length,
                                            return_state=True, ear_gamma=self.ear_gamma if self.use_ear else None)
        self.last_block_map = state.block_map              # uint8 [H, QC(+2), KC(+2)] of the last sparse call
        return out


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
        if cb_step is not None:
            self.current_inference_step = cb_step
        elif timestep is not None:
            self.current_inference_step = self._get_inference_step(timestep)
        else:
            self.current_inference_step = None
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


class WanAttn_EARAttn_Processor(WanAttn_SAPAttn_Processor):
    """Wan processor variant with error-aware routing enabled (wan/attention.py:1219-1222)."""

    use_ear = True


class Hunyuan_SAPAttn_Processor2_0(_SAPBase):
    """Joint-attention processor for HunyuanVideo blocks: video tokens are clustered, the text
    tokens that follow them form two dense blocks (prompt, unused prompt)."""
    context_length = 256
    prompt_length = 0                  # as in the reference (hunyuan10/attention.py:368-369); the installer sets it

    # -- call path (hunyuan10/attention.py:460-575) ---------------------------------------------
    def get_qkv(self, attn, hidden_states):
        return attn.to_q(hidden_states), attn.to_k(hidden_states), attn.to_v(hidden_states)

    def get_transpose_qkv(self, attn, query, key, value):
        return tuple(t.unflatten(2, (attn.heads, -1)).transpose(1, 2).contiguous() for t in (query, key, value))

    def get_qk_norm(self, attn, query, key):
        if getattr(attn, "norm_q", None) is not None:
            query = attn.norm_q(query)
        if getattr(attn, "norm_k", None) is not None:
            key = attn.norm_k(key)
        return query, key

    @staticmethod
    def apply_rotary_emb(x, freqs_cis):
        """Interleaved-pair rotation with real tables (cos, sin) [S, D], as diffusers' apply_rotary_emb
        with use_real=True, use_real_unbind_dim=-1, which the reference calls (hunyuan10/attention.py:300-323)."""
        cos, sin = freqs_cis
        cos, sin = cos[None, None].to(x.device), sin[None, None].to(x.device)
        x_real, x_imag = x.reshape(*x.shape[:-1], -1, 2).unbind(-1)
        x_rot = torch.stack([-x_imag, x_real], dim=-1).flatten(3)
        return (x.float() * cos + x_rot.float() * sin).to(x.dtype)

    def get_rotary_emb(self, attn, query, key, image_rotary_emb, encoder_hidden_states):
        if image_rotary_emb is None:
            return query, key
        if getattr(attn, "add_q_proj", None) is None and encoder_hidden_states is not None:
            # single-stream block: text tokens are the tail of the sequence and are not rotated
            txt = encoder_hidden_states.shape[1]
            query = torch.cat([self.apply_rotary_emb(query[:, :, :-txt], image_rotary_emb), query[:, :, -txt:]], dim=2)
            key = torch.cat([self.apply_rotary_emb(key[:, :, :-txt], image_rotary_emb), key[:, :, -txt:]], dim=2)
        else:
            query = self.apply_rotary_emb(query, image_rotary_emb)
            key = self.apply_rotary_emb(key, image_rotary_emb)
        return query, key

    def get_encoder_condition_and_concat(self, attn, query, key, value, encoder_hidden_states):
        if getattr(attn, "add_q_proj", None) is not None and encoder_hidden_states is not None:
            eq, ek, ev = (proj(encoder_hidden_states).unflatten(2, (attn.heads, -1)).transpose(1, 2)
                          for proj in (attn.add_q_proj, attn.add_k_proj, attn.add_v_proj))
            if getattr(attn, "norm_added_q", None) is not None:
                eq = attn.norm_added_q(eq)
            if getattr(attn, "norm_added_k", None) is not None:
                ek = attn.norm_added_k(ek)
            query = torch.cat([query, eq], dim=2)
            key = torch.cat([key, ek], dim=2)
            value = torch.cat([value, ev], dim=2)
        return query, key, value

    @staticmethod
    def get_cu_max_seqlen(attention_mask, device):
        valid = attention_mask.sum()
        cu = torch.stack([torch.zeros_like(valid), valid, torch.full_like(valid, attention_mask.numel())]).to(
            device=device, dtype=torch.int32)
        return cu, cu.clone(), attention_mask.numel(), attention_mask.numel()

    @staticmethod
    def _fused_producer_applies(attn, hidden_states, image_rotary_emb) -> bool:
        """One-pass per-head norm + text-last rotary + head transpose (svoo_b200_qk_prep_heads): one bf16
        CUDA sample, 128-wide heads, weight-only RMS norms over the head dimension, real (cos, sin) tables."""
        if not (hidden_states.is_cuda and hidden_states.dtype == torch.bfloat16 and hidden_states.shape[0] == 1):
            return False
        if hidden_states.shape[-1] != attn.heads * 128 or attn.heads > 128:
            return False
        for name in ("norm_q", "norm_k"):
            n = getattr(attn, name, None)
            if n is None or getattr(n, "weight", None) is None or getattr(n, "bias", None) is not None:
                return False
            if n.weight.numel() != 128 or not hasattr(n, "eps"):
                return False
        for name in ("norm_added_q", "norm_added_k"):
            n = getattr(attn, name, None)
            if n is not None and (getattr(n, "weight", None) is None or n.weight.numel() != 128
                                  or getattr(n, "bias", None) is not None or not hasattr(n, "eps")):
                return False
        if image_rotary_emb is not None:
            if not (isinstance(image_rotary_emb, (tuple, list)) and len(image_rotary_emb) == 2
                    and all(torch.is_tensor(t) and t.shape[-1] == 128 for t in image_rotary_emb)):
                return False
        return True

    def fused_producer(self, attn, hidden_states, encoder_hidden_states, image_rotary_emb):
        """Replaces get_transpose_qkv + apply_qk_norm + apply_qk_rope_single / _double (+ the text
        projections and the concatenation of a double-stream block) of the reference
        (hunyuan10/attention.py:262-290, 460-534) for the case _fused_producer_applies accepts.
        `hidden_states`: video tokens, followed by the text tokens in a single-stream block."""
        H = attn.heads
        cos, sin = (None, None) if image_rotary_emb is None else image_rotary_emb
        query, key, value = self.get_qkv(attn, hidden_states)
        S = hidden_states.shape[1]
        txt = 0 if encoder_hidden_states is None else encoder_hidden_states.shape[1]
        if getattr(attn, "add_q_proj", None) is None or encoder_hidden_states is None:
            rope_rows = S - txt if getattr(attn, "add_q_proj", None) is None else S
            q = ops.qk_prep_heads(query[0].contiguous(), H, attn.norm_q.weight, attn.norm_q.eps, cos, sin, rope_rows)
            k = ops.qk_prep_heads(key[0].contiguous(), H, attn.norm_k.weight, attn.norm_k.eps, cos, sin, rope_rows)
            v = ops.qk_prep_heads(value[0].contiguous(), H)
            return q[None], k[None], v[None]
        # double-stream block: the text tokens have their own projections and norms and follow the video tokens
        outs = [torch.empty(H, S + txt, 128, dtype=hidden_states.dtype, device=hidden_states.device) for _ in range(3)]
        nq, nk = getattr(attn, "norm_added_q", None), getattr(attn, "norm_added_k", None)
        ops.qk_prep_heads(query[0].contiguous(), H, attn.norm_q.weight, attn.norm_q.eps, cos, sin, S, out=outs[0])
        ops.qk_prep_heads(key[0].contiguous(), H, attn.norm_k.weight, attn.norm_k.eps, cos, sin, S, out=outs[1])
        ops.qk_prep_heads(value[0].contiguous(), H, out=outs[2])
        eq, ek, ev = (proj(encoder_hidden_states)[0].contiguous() for proj in (attn.add_q_proj, attn.add_k_proj, attn.add_v_proj))
        ops.qk_prep_heads(eq, H, None if nq is None else nq.weight, 0.0 if nq is None else nq.eps, out=outs[0], out_row0=S)
        ops.qk_prep_heads(ek, H, None if nk is None else nk.weight, 0.0 if nk is None else nk.eps, out=outs[1], out_row0=S)
        ops.qk_prep_heads(ev, H, out=outs[2], out_row0=S)
        return tuple(t[None] for t in outs)

    def get_o(self, attn, hidden_states, encoder_hidden_states):
        if encoder_hidden_states is not None:
            txt = encoder_hidden_states.shape[1]
            hidden_states, encoder_hidden_states = hidden_states[:, :-txt], hidden_states[:, -txt:]
            if getattr(attn, "to_out", None) is not None:
                hidden_states = attn.to_out[1](attn.to_out[0](hidden_states))
            if getattr(attn, "to_add_out", None) is not None:
                encoder_hidden_states = attn.to_add_out(encoder_hidden_states)
        return hidden_states, encoder_hidden_states

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, attention_mask=None, image_rotary_emb=None,
                 timestep=None):
        """Returns (hidden_states, encoder_hidden_states) like the reference (hunyuan10/attention.py:536-575)."""
        if getattr(attn, "add_q_proj", None) is None and encoder_hidden_states is not None:
            hidden_states = torch.cat([hidden_states, encoder_hidden_states], dim=1)
        if self._fused_producer_applies(attn, hidden_states, image_rotary_emb):
            query, key, value = self.fused_producer(attn, hidden_states, encoder_hidden_states, image_rotary_emb)
        else:
            query, key, value = self.get_qkv(attn, hidden_states)
            query, key, value = self.get_transpose_qkv(attn, query, key, value)
            query, key = self.get_qk_norm(attn, query, key)
            query, key = self.get_rotary_emb(attn, query, key, image_rotary_emb, encoder_hidden_states)
            query, key, value = self.get_encoder_condition_and_concat(attn, query, key, value, encoder_hidden_states)
        cu_max_seqlens = None if attention_mask is None else self.get_cu_max_seqlen(attention_mask, query.device)
        hidden_states = self.attention_core_logic(query, key, value, timestep, self.layer_idx, cu_max_seqlens)
        hidden_states = hidden_states.transpose(1, 2).flatten(2, 3).to(query.dtype)
        return self.get_o(attn, hidden_states, encoder_hidden_states)

    def attention_core_logic(self, query, key, value, timestep, layer_idx=None, cu_max_seqlens=None):
        """query/key/value [1, H, S, 128] -> [1, H, S, 128] (hunyuan10/attention.py:1031-1110)."""
        cfg, H, S, D = query.size()
        assert cfg == 1, "Batch size must be 1 for kmeans block sparse attention"
        assert 0 <= self.prompt_length <= self.context_length, "prompt_length must lie in [0, context_length]"
        assert S == self.context_length + self.num_frame * self.frame_size, (
            f"Query Shape: {S} is not equivalent to {self.context_length} + {self.num_frame} * {self.frame_size}")
        self.current_inference_step = getattr(self, "_step_from_callback", None)
        if self._full_attention_flag(timestep):
            n_video = self.num_frame * self.frame_size
            if self.zero_step_kmeans_init:
                self.kmeans_clustering(query[:, :, :n_video].contiguous(), key[:, :, :n_video].contiguous())
            # dense (the reference's flashinfer_varlen_func, :1113-1185): two diagonal blocks, the
            # tokens the attention mask keeps (video + prompt) and the unused prompt
            valid = n_video + self.prompt_length if cu_max_seqlens is None else int(cu_max_seqlens[0][1])
            out = torch.empty_like(query)
            out[:, :, :valid] = self.flash_attention(query[:, :, :valid], key[:, :, :valid], value[:, :, :valid])
            if valid < S:
                out[:, :, valid:] = self.flash_attention(query[:, :, valid:], key[:, :, valid:], value[:, :, valid:])
            return out
        return self._sparse(query, key, value, prompt_length=self.prompt_length)
