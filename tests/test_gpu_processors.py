"""The attention processors (the plug-in boundary) on the GPU against the steps recorded from the
unmodified reference processors (tests/golden/processor_*.npz) and against the oracle.

Bars: labels >= 99.9 % equal, video map equal up to the choice inside an equal-probability group
(the reference's torch.sort is unstable), output rows of comparable tokens within 2e-2."""
import dataclasses
import os

import numpy as np
import pytest
import torch

from oracle import svoo_oracle as O
from svoo_b200 import synth
from tests import golden_util as gu

pytestmark = pytest.mark.gpu

ATOL = 2e-2


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _launches():
    from svoo_b200 import _lib
    return _lib.LIB.svoo_b200_launch_count()


def _fresh(cls):
    """A subclass, so that class attributes set by one test do not leak into the others."""
    return type(cls.__name__, (cls,), {"_seen_timesteps": set()})


def _check_rows(y, want, ok_tokens, min_ok):
    ok = ok_tokens[::gu.PROC_ROWS_KEPT]
    assert ok.float().mean() >= min_ok
    d = (y[::gu.PROC_ROWS_KEPT].float().cpu() - want.float()).abs().amax(-1)
    assert d[ok].max() <= ATOL


@pytest.mark.parametrize("fused_producer", [True, False])
def test_wan_processor_against_reference_steps(dev, fused_producer):
    """WanAttn_SAPAttn_Processor.__call__ over the four recorded denoising steps: dense warm-up,
    first clustering (per-head density from the CSV), reuse of the cached clustering (scalar
    fallback: the CSV has a hole), re-clustering with kmeans_iter_step iterations."""
    from svoo_b200 import processor
    from svoo_b200.sparsity import SparsityLookup
    z = gu.load("processor_wan")
    P = gu.WAN_PROC
    H = P["heads"]
    N = P["grid"][0] * P["grid"][1] * P["grid"][2]
    cls = _fresh(processor.WanAttn_SAPAttn_Processor)
    gu.configure_wan_processor(cls, SparsityLookup(os.path.join(gu.GOLDEN, "processor_wan_density.csv")))
    if not fused_producer:
        cls._fused_producer_applies = staticmethod(lambda *a: False)
    attn = gu.make_attn(31, H).to(dev)
    cos, sin = (t.to(dev) for t in gu.rotary_tables(32, N))
    proc = cls(0)
    deltas, labels_seen = {}, {}
    for step, tval in P["steps"]:
        hidden = gu.wan_step_hidden(step).to(dev)
        proc._step_from_callback = step
        qi = torch.from_numpy(z[f"q_init_{step}"]).long().to(dev)
        ki = torch.from_numpy(z[f"k_init_{step}"]).long().to(dev)
        proc.draw_init_indices = lambda BH, n, d, qi=qi, ki=ki: (qi, ki)
        n0 = _launches()
        with torch.no_grad():
            y = proc(attn, hidden, rotary_emb=(cos, sin), timestep=torch.tensor([tval], device=dev))
        torch.cuda.synchronize()
        deltas[step] = _launches() - n0
        assert y.shape == hidden.shape and y.dtype == hidden.dtype
        want = gu.from_bf16_bits(z[f"out_{step}"])
        if tval > P["first_times_fp"]:                         # dense warm-up step
            assert proc.last_block_map is None
            assert (y[0, ::gu.PROC_ROWS_KEPT].float().cpu() - want.float()).abs().max() <= ATOL
            continue
        proc.check_status()
        assert proc.current_inference_step == step
        c = proc._cached_clustering_results
        labels_seen[step] = c.qlabels
        ql, kl = c.qlabels.cpu().numpy(), c.klabels.cpu().numpy()
        assert (ql == z[f"qlabels_{step}"]).mean() >= 0.999
        assert (kl == z[f"klabels_{step}"]).mean() >= 0.999
        ref_map = gu.unpack_map(z, f"_{step}")[0]
        ratio = [float(r) for r in z[f"ratio_{step}"]]
        ratio = ratio if len(ratio) > 1 else ratio[0]
        got_map = proc.last_block_map.cpu().numpy().astype(bool)
        # bit-exact against the oracle on the processor's own centroids, up to ties against the reference
        m_or = O.identify_dynamic_map(c.qcentroids.cpu()[None], c.kcentroids.cpu()[None], c.qsizes.cpu()[None],
                                      c.ksizes.cpu()[None], P["top_p"], ratio)
        assert (got_map == m_or[0].numpy()).all()
        if (ql == z[f"qlabels_{step}"]).all() and (kl == z[f"klabels_{step}"]).all():
            assert gu.processor_map_ties_ok(c.qcentroids.cpu(), c.kcentroids.cpu(), c.qsizes.cpu(), c.ksizes.cpu(),
                                            P["top_p"], ratio, got_map, ref_map)
        ok = gu.comparable_tokens(ql, z[f"qlabels_{step}"], got_map, ref_map)
        _check_rows(y[0], want, ok, 0.7)
    # the reuse step launched no clustering kernel: the same label tensor, and only the producer (3 when
    # fused), the map (1), the gathers (3) and the attention (3) ran
    assert labels_seen[3] is labels_seen[2] and labels_seen[7] is not labels_seen[2]
    assert deltas[3] == (3 if fused_producer else 0) + 1 + 3 + 3
    assert deltas[2] > deltas[7] > deltas[3]                    # 2 iterations, then 1, then none
    assert deltas[1] == (3 if fused_producer else 0)            # dense step: torch SDPA


def test_wan_processor_step_counter_without_callback(dev):
    """Without a pipeline callback the step index follows the scheduler timesteps (a new value
    counts one step; a larger value than the last one starts a new run)."""
    from svoo_b200 import processor
    cls = _fresh(processor.WanAttn_SAPAttn_Processor)
    a, b = cls(0), cls(1)
    assert [a._get_inference_step(t) for t in (900.0, 900.0, 800.0)] == [1, 1, 2]
    assert b._get_inference_step(torch.tensor([800.0])) == 2     # layers share the counter
    assert a._get_inference_step(999.0) == 1                      # next video


def test_hunyuan_processor_against_reference_step(dev):
    """Hunyuan_SAPAttn_Processor2_0.__call__ on a single-stream block (text after video, prompt 40 of
    64 text tokens, so the unused-prompt block is not empty): returns (hidden, encoder) like the reference."""
    from svoo_b200 import processor
    z = gu.load("processor_hunyuan")
    P = gu.HUN_PROC
    cls = _fresh(processor.Hunyuan_SAPAttn_Processor2_0)
    assert cls.prompt_length == 0 and cls.context_length == 256       # the reference's defaults
    gu.configure_hunyuan_processor(cls)
    attn = gu.make_attn(41, P["heads"], joint=True).to(dev)
    hidden, enc, mask = (t.to(dev) for t in gu.hunyuan_inputs())
    proc = cls(0)
    step, tval = P["steps"][0]
    proc._step_from_callback = step
    qi, ki = torch.from_numpy(z["q_init"]).long().to(dev), torch.from_numpy(z["k_init"]).long().to(dev)
    proc.draw_init_indices = lambda BH, n, d: (qi, ki)
    with torch.no_grad():
        y, y_enc = proc(attn, hidden, encoder_hidden_states=enc, attention_mask=mask, image_rotary_emb=None,
                        timestep=torch.tensor([tval], device=dev))
    proc.check_status()
    assert y.shape == hidden.shape and y_enc.shape == enc.shape
    c = proc._cached_clustering_results
    ql, kl = c.qlabels.cpu().numpy(), c.klabels.cpu().numpy()
    assert (ql == z["qlabels"]).mean() >= 0.999 and (kl == z["klabels"]).mean() >= 0.999
    full = proc.last_block_map.cpu().numpy().astype(bool)
    QC, KC = P["num_q"], P["num_k"]
    assert full.shape == (P["heads"], QC + 2, KC + 2)
    ref_map = gu.unpack_map(z)[0]
    # the text blocks follow the reference's rule
    m2, _, _, _ = O.hunyuan_text_blocks(torch.from_numpy(full[None, :, :QC, :KC]), c.qsizes.cpu()[None], c.ksizes.cpu()[None],
                                        c.q_sorted_idx.cpu(), ql.shape[1], P["context_length"], P["prompt_length"])
    assert (m2[0].numpy() == full).all()
    if (ql == z["qlabels"]).all() and (kl == z["klabels"]).all():
        assert gu.processor_map_ties_ok(c.qcentroids.cpu(), c.kcentroids.cpu(), c.qsizes.cpu(), c.ksizes.cpu(), P["top_p"],
                                        float(P["min_kc_ratio"]), full[:, :QC, :KC], ref_map)
    ok = gu.comparable_tokens(ql, z["qlabels"], full[:, :QC, :KC], ref_map)
    _check_rows(y[0], gu.from_bf16_bits(z["out"]), ok, 0.7)
    assert (y_enc[0].float().cpu() - gu.from_bf16_bits(z["out_enc"]).float()).abs().max() <= ATOL


def test_hunyuan_dense_branch_and_rotary(dev):
    """The dense warm-up branch is two diagonal blocks (tokens the mask keeps, unused prompt), and the
    rotary helper rotates interleaved pairs of the video tokens only."""
    from svoo_b200 import processor
    P = gu.HUN_PROC
    cls = _fresh(processor.Hunyuan_SAPAttn_Processor2_0)
    gu.configure_hunyuan_processor(cls)
    cls.first_times_fp = 100.0                                  # timestep 500 > 100: dense
    attn = gu.make_attn(41, P["heads"], joint=True).to(dev)
    hidden, enc, mask = (t.to(dev) for t in gu.hunyuan_inputs())
    n, ctx = hidden.shape[1], enc.shape[1]
    g = torch.Generator("cpu").manual_seed(2)
    ang = torch.rand(n, 64, generator=g) * 6.2831853
    rot = (torch.cos(ang).repeat_interleave(2, -1).to(dev), torch.sin(ang).repeat_interleave(2, -1).to(dev))
    proc = cls(0)
    with torch.no_grad():
        y, y_enc = proc(attn, hidden, encoder_hidden_states=enc, attention_mask=mask, image_rotary_emb=rot,
                        timestep=torch.tensor([500.0], device=dev))
        # the same with plain torch
        x = torch.cat([hidden, enc], 1)
        q, k, v = (t.unflatten(2, (P["heads"], -1)).transpose(1, 2) for t in (attn.to_q(x), attn.to_k(x), attn.to_v(x)))
        q, k = attn.norm_q(q), attn.norm_k(k)

        def rope(t):
            tv = t[:, :, :n].float()
            x1, x2 = tv[..., 0::2], tv[..., 1::2]
            c, s_ = rot[0][:, 0::2], rot[1][:, 0::2]
            out = torch.stack([x1 * c - x2 * s_, x1 * s_ + x2 * c], -1).flatten(3).to(t.dtype)
            return torch.cat([out, t[:, :, n:]], 2)

        q, k = rope(q), rope(k)
        valid = n + P["prompt_length"]
        o = torch.empty_like(q)
        o[:, :, :valid] = torch.nn.functional.scaled_dot_product_attention(q[:, :, :valid], k[:, :, :valid], v[:, :, :valid])
        o[:, :, valid:] = torch.nn.functional.scaled_dot_product_attention(q[:, :, valid:], k[:, :, valid:], v[:, :, valid:])
        o = o.transpose(1, 2).flatten(2, 3)
        want, want_enc = attn.to_out[0](o[:, :-ctx]), o[:, -ctx:]
    assert (y.float() - want.float()).abs().max() <= ATOL and (y_enc.float() - want_enc.float()).abs().max() <= ATOL


def test_hunyuan_core_at_shipped_cluster_counts(dev):
    """attention_core_logic with the reference's shipped HunyuanVideo setting, 256 query / 1024 key
    clusters plus the two text blocks (258 x 1026 blocks: the attention-side limit), on one head."""
    from svoo_b200 import processor
    cls = _fresh(processor.Hunyuan_SAPAttn_Processor2_0)
    cfg = dataclasses.replace(synth.CONFIGS["cfg1"], heads=1, grid=(4, 30, 40), num_q=256, num_k=1024, text_tokens=256,
                              cfg_id=93)
    cls.num_frame, cls.frame_size, cls.context_length, cls.prompt_length = 4, 1200, 256, 200
    cls.num_q_centroids, cls.num_k_centroids, cls.top_p_kmeans, cls.min_kc_ratio = 256, 1024, 0.9, 0.1
    cls.kmeans_iter_init = cls.kmeans_iter_step = 2
    cls.first_times_fp = 1e9
    q, k, v = synth.make_qkv(cfg)
    proc = cls(0)
    qi, ki = synth.init_indices(cfg)
    proc.draw_init_indices = lambda BH, n, d: (qi.to(d), ki.to(d))
    out = proc.attention_core_logic(q.to(dev), k.to(dev), v.to(dev), torch.tensor([10.0], device=dev))
    proc.check_status()
    assert out.shape == q.shape
    c = proc._cached_clustering_results
    n = cfg.n_video
    clustering = (c.qlabels.cpu().long(), c.qcentroids.cpu(), c.qsizes.cpu(), c.klabels.cpu().long(), c.kcentroids.cpu(),
                  c.ksizes.cpu())
    ref, aux = O.attention_given_clustering(q, k, v, clustering, 0.9, 0.1, 0, 256, 200)
    assert torch.equal(proc.last_block_map.cpu().bool(), aux["map"][0])
    assert (out.cpu().float() - ref.float()).abs().max() <= ATOL
    # prompt rows attend every video and prompt key: exact dense softmax over those keys
    valid = n + 200
    dense = torch.softmax(q[0, 0, n:valid].float() @ k[0, 0, :valid].float().T * 128 ** -0.5, -1) @ v[0, 0, :valid].float()
    assert (out[0, 0, n:valid].cpu().float() - dense).abs().max() <= ATOL


def test_euclidean_mode_processor(dev):
    """use_svoo = False: plain Euclidean k-means per side; later steps continue from the previous
    centroids (kmeans_init / kmeans_step of the reference)."""
    from svoo_b200 import processor
    cls = _fresh(processor.WanAttn_SAPAttn_Processor)
    cfg = dataclasses.replace(gu.TINY_BF16, cfg_id=94)
    cls.num_frame, cls.frame_size, cls.context_length = cfg.grid[0], cfg.grid[1] * cfg.grid[2], 0
    cls.num_q_centroids, cls.num_k_centroids, cls.top_p_kmeans, cls.min_kc_ratio = cfg.num_q, cfg.num_k, 0.9, 0.2
    cls.kmeans_iter_init, cls.kmeans_iter_step, cls.use_svoo, cls.first_times_fp = 3, 1, False, 1e9
    q, k, v = (t.to(dev) for t in synth.make_qkv(cfg))
    proc = cls(0)
    out = proc.attention_core_logic(q, k, v, torch.tensor([5.0], device=dev))
    c1 = proc._cached_clustering_results
    assert out.shape == (1, cfg.n_video, cfg.heads * 128)
    assert int(c1.qsizes.sum()) == cfg.heads * cfg.n_video
    # labels are the nearest centroids of the centroids the last assignment used
    lab = O.euclid_assign(q[0].cpu(), c1.qcentroids.cpu())
    # (the returned centroids are the updated ones unless the loop stopped on tol; check through one more step)
    proc.attention_core_logic(q, k, v, torch.tensor([4.0], device=dev))
    c2 = proc._cached_clustering_results
    lab2 = O.euclid_assign(q[0].cpu(), c1.qcentroids.cpu())
    assert (c2.qlabels.cpu().long() == lab2).float().mean() >= 0.999
    assert lab.shape == lab2.shape
