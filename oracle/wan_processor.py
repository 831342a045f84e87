"""CPU restatement of the reference's Wan attention processor.  TEST INFRASTRUCTURE ONLY
(like svoo_oracle.py: used by tests/ and by bench.py's CPU legs, never by the product path).

Follows WanAttn_SAPAttn_Processor of the reference: the call path
(svoo/models/wan/attention.py:153-260: projections, QK norm through the block's norm modules,
interleaved-pair rotary embedding, head transpose, output projection), attention_core_logic
(:1110-1216: step index, dense warm-up branch, sparse branch), the clustering reuse schedule
(:682-715, 793-819) and the per-head density lookup with clipping (:931-956).  The sparse
branch is the oracle's co-clustering, map and masked attention.  Pinned by
tests/test_oracle_golden.py against steps recorded from the unmodified reference processor.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import svoo_oracle as O


class OracleWanProcessor:
    context_length = 0
    num_frame = 0
    frame_size = 0
    first_layers_fp = 0
    first_times_fp = 0
    num_q_centroids = 0
    num_k_centroids = 0
    top_p_kmeans = 0
    min_kc_ratio = 0
    kmeans_iter_init = 0
    kmeans_iter_step = 0
    start_reuse_step = None
    reuse_interval = 1
    use_dynamic_min_kc_ratio = False
    sparsity_lookup = None
    dynamic_min_kc_ratio_min = None
    dynamic_min_kc_ratio_max = None

    def __init__(self, layer_idx):
        self.layer_idx = layer_idx
        self.centroids_init = False
        self.cached = None
        self.last_aux = None
        self.current_inference_step = None

    def draw_init_indices(self, BH, N):
        """q indices, then k indices, from the global generator (co_clustering.py:2417-2421)."""
        return torch.randint(0, N, (BH, self.num_q_centroids)), torch.randint(0, N, (BH, self.num_k_centroids))

    def _ratio(self, step, num_heads):
        lk = self.sparsity_lookup
        if self.use_dynamic_min_kc_ratio and lk is not None and step is not None:
            if not lk.has_data_for_step_layer(step, self.layer_idx, num_heads):
                return self.min_kc_ratio
            out = []
            for v in lk.get_sparsity_batch(step, self.layer_idx, num_heads):
                if self.dynamic_min_kc_ratio_min is not None:
                    v = max(v, self.dynamic_min_kc_ratio_min)
                if self.dynamic_min_kc_ratio_max is not None:
                    v = min(v, self.dynamic_min_kc_ratio_max)
                out.append(v)
            return out
        return self.min_kc_ratio

    def _clustering(self, q, k):
        step = self.current_inference_step
        recluster = True
        if step is not None and self.start_reuse_step is not None and self.start_reuse_step > 0 and step >= self.start_reuse_step:
            recluster = (step - self.start_reuse_step) % self.reuse_interval == 0
        if not recluster and self.cached is not None:
            return self.cached
        iters = self.kmeans_iter_step if self.centroids_init else self.kmeans_iter_init
        qi, ki = self.draw_init_indices(q.shape[0], q.shape[1])
        self.cached = O.co_cluster_tokens(q, k, qi, ki, iters)
        self.centroids_init = True
        return self.cached

    def attention_core_logic(self, query, key, value, timestep):
        cfg, H, S, D = query.shape
        assert cfg == 1 and S == self.context_length + self.num_frame * self.frame_size
        self.current_inference_step = getattr(self, "_step_from_callback", None)
        tval = timestep.flatten()[0].item() if isinstance(timestep, torch.Tensor) else timestep
        if self.layer_idx < self.first_layers_fp or (tval is not None and tval > self.first_times_fp):
            self.last_aux = None
            out = F.scaled_dot_product_attention(query, key, value)
        else:
            clustering = self._clustering(query[0], key[0])
            ratio = self._ratio(self.current_inference_step, H)
            out, aux = O.attention_given_clustering(query, key, value, clustering, self.top_p_kmeans, ratio)
            aux["ratio"] = ratio
            self.last_aux = aux
        return out.transpose(1, 2).flatten(2, 3)

    def __call__(self, attn, hidden_states, encoder_hidden_states=None, attention_mask=None, rotary_emb=None, timestep=None):
        enc = hidden_states if encoder_hidden_states is None else encoder_hidden_states
        q, k, v = attn.to_q(hidden_states), attn.to_k(enc), attn.to_v(enc)
        if attn.norm_q is not None:
            q = attn.norm_q(q)
        if attn.norm_k is not None:
            k = attn.norm_k(k)
        q, k, v = (t.unflatten(2, (attn.heads, -1)) for t in (q, k, v))
        if rotary_emb is not None:
            q, k = O.rotary_interleaved(q, *rotary_emb), O.rotary_interleaved(k, *rotary_emb)
        q, k, v = (t.transpose(1, 2).contiguous() for t in (q, k, v))
        if timestep is None:
            out = F.scaled_dot_product_attention(q, k, v, attn_mask=attention_mask).transpose(1, 2).flatten(2, 3)
        else:
            out = self.attention_core_logic(q, k, v, timestep)
        out = attn.to_out[0](out.type_as(q))
        return attn.to_out[1](out)
