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


def _record_core_inputs(proc):
    """Wraps attention_core_logic so that the q, k, v it receives are kept (the projections run on
    the GPU here and on the CPU in the reference run: their bf16 roundings differ in a few
    elements, which moves a few labels of a 960-token clustering; the path itself is therefore
    judged on its own inputs)."""
    seen = {}
    inner = proc.attention_core_logic

    def wrapped(query, key, value, *a, **kw):
        seen.update(q=query.detach().cpu(), k=key.detach().cpu(), v=value.detach().cpu())
        return inner(query, key, value, *a, **kw)

    proc.attention_core_logic = wrapped
    return seen


def _oracle_labels_on(seen, qi, ki, iters, n_video=None):
    q, k = seen["q"][0], seen["k"][0]
    if n_video is not None:
        q, k = q[:, :n_video].contiguous(), k[:, :n_video].contiguous()
    return O.co_cluster_tokens(q, k, qi.cpu(), ki.cpu(), iters)


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
    seen = _record_core_inputs(proc)
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
        ratio = [float(r) for r in z[f"ratio_{step}"]]
        ratio = ratio if len(ratio) > 1 else ratio[0]
        # strict: the oracle on the q, k, v this call produced (a clustering step clusters them, the
        # reuse step keeps the oracle's clustering of step 2)
        if step != 3:
            iters = P["iter_init"] if step == 2 else P["iter_step"]
            oracle_clustering = _oracle_labels_on(seen, qi, ki, iters)
        rl = oracle_clustering
        assert (ql == rl[0].numpy()).mean() >= 0.999 and (kl == rl[3].numpy()).mean() >= 0.999
        got_map = proc.last_block_map.cpu().numpy().astype(bool)
        m_or = O.identify_dynamic_map(c.qcentroids.cpu()[None], c.kcentroids.cpu()[None], c.qsizes.cpu()[None],
                                      c.ksizes.cpu()[None], P["top_p"], ratio)
        assert (got_map == m_or[0].numpy()).all()                # bit-exact on the processor's own centroids
        o_ref, aux = O.attention_given_clustering(seen["q"], seen["k"], seen["v"], rl, P["top_p"], ratio)
        with torch.no_grad():
            y_ref = attn.to_out[0](o_ref.transpose(1, 2).flatten(2, 3).to(dev))
        ok = gu.comparable_tokens(ql, rl[0].numpy(), got_map, aux["map"][0].numpy())
        assert ok.float().mean() >= 0.9
        assert (y[0].float() - y_ref[0].float()).abs().amax(-1).cpu()[ok].max() <= ATOL
        # loose: the reference's recorded step.  Its projections ran on the CPU; a few bf16 roundings
        # differ, some labels of this 960-token clustering with them, and then centroids and maps
        assert (ql == z[f"qlabels_{step}"]).mean() >= 0.9 and (kl == z[f"klabels_{step}"]).mean() >= 0.9
        a, b = y[0, ::gu.PROC_ROWS_KEPT].float().cpu().flatten(), want.float().flatten()
        assert float(a @ b / (a.norm() * b.norm())) >= 0.98
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
    seen = _record_core_inputs(proc)
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
    rl = _oracle_labels_on(seen, qi, ki, P["iter_init"], n_video=ql.shape[1])
    assert (ql == rl[0].numpy()).mean() >= 0.999 and (kl == rl[3].numpy()).mean() >= 0.999
    full = proc.last_block_map.cpu().numpy().astype(bool)
    QC, KC = P["num_q"], P["num_k"]
    assert full.shape == (P["heads"], QC + 2, KC + 2)
    # strict: the oracle's joint attention on the q, k, v this call produced
    o_ref, aux = O.attention_given_clustering(seen["q"], seen["k"], seen["v"], rl, P["top_p"], float(P["min_kc_ratio"]), 0,
                                              P["context_length"], P["prompt_length"])
    m_own = O.identify_dynamic_map(c.qcentroids.cpu()[None], c.kcentroids.cpu()[None], c.qsizes.cpu()[None],
                                   c.ksizes.cpu()[None], P["top_p"], float(P["min_kc_ratio"]))
    m2, _, _, _ = O.hunyuan_text_blocks(m_own, c.qsizes.cpu()[None], c.ksizes.cpu()[None], c.q_sorted_idx.cpu(), ql.shape[1],
                                        P["context_length"], P["prompt_length"])
    assert (m2[0].numpy() == full).all()                         # bit-exact, text blocks by the reference's rule
    ctx = P["context_length"]
    y_all = o_ref.transpose(1, 2).flatten(2, 3).to(dev)
    with torch.no_grad():
        y_ref, y_enc_ref = attn.to_out[0](y_all[:, :-ctx]), y_all[:, -ctx:]
    ok = gu.comparable_tokens(ql, rl[0].numpy(), full[:, :QC, :KC], aux["map_video"][0].numpy())
    assert ok.float().mean() >= 0.9
    assert (y[0].float() - y_ref[0].float()).abs().amax(-1).cpu()[ok].max() <= ATOL
    assert (y_enc[0].float() - y_enc_ref[0].float()).abs().max() <= ATOL
    # loose: the reference's recorded step (its projections ran on the CPU)
    assert (ql == z["qlabels"]).mean() >= 0.9 and (kl == z["klabels"]).mean() >= 0.9
    a, b = y[0, ::gu.PROC_ROWS_KEPT].float().cpu().flatten(), gu.from_bf16_bits(z["out"]).float().flatten()
    assert float(a @ b / (a.norm() * b.norm())) >= 0.98
    assert (y_enc[0].float().cpu() - gu.from_bf16_bits(z["out_enc"]).float()).abs().max() <= 2 * ATOL


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


def test_dit_step_two_blocks_against_cpu_oracle(dev):
    """A reduced DiT with the Wan block structure (2 blocks, 4 heads, 960 tokens) over two denoising
    steps (the second one reuses the clustering), density floors read from a CSV through
    SparsityLookup, step index set as the pipeline callback does.  Two copies of the model with the
    same weights run on the GPU: one with WanAttn_SAPAttn_Processor in every block, one with the
    oracle's processor, whose sparse branch is computed on the CPU from the very q, k, v the block
    produced (so that everything outside the path is identical in both)."""
    from oracle.wan_processor import OracleWanProcessor
    from svoo_b200 import processor, wan_dit
    from svoo_b200.sparsity import SparsityLookup

    class OracleOnHost(OracleWanProcessor):
        def attention_core_logic(self, query, key, value, timestep):
            out = super().attention_core_logic(query.cpu(), key.cpu(), value.cpu(), timestep.cpu())
            return out.to(query.device)

    cfg = wan_dit.WanDiTConfig(num_layers=2, dim=512, heads=4, ffn_dim=1024, text_dim=64, text_len=16, latent=(3, 32, 40))
    N = cfg.tokens
    path = os.path.join(os.environ.get("TMPDIR", "/tmp"), "svoo_b200_dit_density.csv")
    wan_dit.write_density_table(path, 2, cfg.num_layers, cfg.heads, 0.1, 0.3, seed=3)
    kw = dict(num_q_centroids=12, num_k_centroids=40, top_p_kmeans=0.9, min_kc_ratio=0.2, kmeans_iter_init=2,
              kmeans_iter_step=1, sparsity_lookup=SparsityLookup(path), dynamic_min_kc_ratio_min=0.05,
              dynamic_min_kc_ratio_max=0.4, start_reuse_step=1, reuse_interval=2)
    ref_model = wan_dit.WanDiT(cfg).init_weights(1).to(device=dev, dtype=torch.bfloat16).eval()
    gpu = wan_dit.WanDiT(cfg).init_weights(1).to(device=dev, dtype=torch.bfloat16).eval()
    ref_procs = wan_dit.install_processors(ref_model, type("OracleCase", (OracleOnHost,), {}), cfg.grid, **kw)
    plain_cls = _fresh(processor.WanAttn_SAPAttn_Processor)
    plain_cls._fused_producer_applies = staticmethod(lambda *a: False)   # q, k, v bit-identical to the oracle model's
    gpu_procs = wan_dit.install_processors(gpu, plain_cls, cfg.grid, **kw)
    fused = wan_dit.WanDiT(cfg).init_weights(1).to(device=dev, dtype=torch.bfloat16).eval()
    fused_procs = wan_dit.install_processors(fused, _fresh(processor.WanAttn_SAPAttn_Processor), cfg.grid, **kw)
    for l, pf in enumerate(fused_procs):
        g = torch.Generator("cpu").manual_seed(50 + l)
        qi, ki = torch.randint(0, N, (cfg.heads, 12), generator=g), torch.randint(0, N, (cfg.heads, 40), generator=g)
        pf.draw_init_indices = lambda BH, n, d, qi=qi, ki=ki: (qi.to(d), ki.to(d))
    for l, (pc, pg) in enumerate(zip(ref_procs, gpu_procs)):
        g = torch.Generator("cpu").manual_seed(50 + l)
        qi, ki = torch.randint(0, N, (cfg.heads, 12), generator=g), torch.randint(0, N, (cfg.heads, 40), generator=g)
        pc.draw_init_indices = lambda BH, n, qi=qi, ki=ki: (qi, ki)
        pg.draw_init_indices = lambda BH, n, d, qi=qi, ki=ki: (qi.to(d), ki.to(d))
    g = torch.Generator("cpu").manual_seed(0)
    lat = torch.randn(1, 16, *cfg.latent, generator=g).bfloat16().to(dev)
    text = torch.randn(1, 16, 64, generator=g).bfloat16().to(dev)
    for step in (1, 2):
        for m in (ref_model, gpu, fused):
            wan_dit.set_attention_step(m, step)
        t = torch.tensor([900.0 - 100 * step], device=dev)
        with torch.no_grad():
            want = ref_model(lat, t, text)
            got = gpu(lat, t, text)
            torch.cuda.synchronize()
            n0 = _launches()
            got_fused = fused(lat, t, text)
        torch.cuda.synchronize()
        launched = _launches() - n0
        for p in gpu_procs:
            p.check_status()
        assert got.shape == want.shape == lat.shape
        for l, (pc, pg) in enumerate(zip(ref_procs, gpu_procs)):
            assert pg.current_inference_step == step
            ql = pg._cached_clustering_results.qlabels.cpu().long()
            assert (ql == pc.cached[0]).float().mean() >= (0.999 if l == 0 else 0.8)    # block 1 sees block 0's output rounding; random-weight activations have no cluster structure
        a, b = got.float().cpu().flatten(), want.float().cpu().flatten()
        assert float(a @ b / (a.norm() * b.norm())) >= 0.999
        # the model with the fused producer (one-ulp differences in q, k; labels of random-weight
        # activations, which have no cluster structure, move with them)
        a = got_fused.float().cpu().flatten()
        assert float(a @ b / (a.norm() * b.norm())) >= 0.98
        if step == 2:
            # reuse step: per block the fused producer (3), the map, three gathers and the attention (3)
            assert launched == cfg.num_layers * 10


@pytest.mark.parametrize("double_stream", [False, True])
def test_hunyuan_fused_producer_equals_module_path(dev, double_stream):
    """The one-pass producer (svoo_b200_qk_prep_heads) hands attention_core_logic the q, k, v that the
    module-by-module path (to_q/k/v, head transpose, norm modules, rotary helper, text projections and
    concatenation) produces: single-stream block (text at the end of the sequence, not rotated) and
    double-stream block (text through add_*_proj and norm_added_*)."""
    from svoo_b200 import processor
    P = gu.HUN_PROC
    hidden, enc, mask = (t.to(dev) for t in gu.hunyuan_inputs())
    n = hidden.shape[1]
    g = torch.Generator("cpu").manual_seed(2)
    ang = torch.rand(n, 64, generator=g) * 6.2831853
    rot = (torch.cos(ang).repeat_interleave(2, -1).to(dev), torch.sin(ang).repeat_interleave(2, -1).to(dev))
    attn = gu.make_attn(41, P["heads"], joint=True)
    if double_stream:
        dim = P["heads"] * 128
        for nm in ("add_q_proj", "add_k_proj", "add_v_proj", "to_add_out"):
            lin = torch.nn.Linear(dim, dim)
            with torch.no_grad():
                lin.weight.copy_(torch.randn(dim, dim, generator=g) / dim ** 0.5)
                lin.bias.copy_(torch.randn(dim, generator=g) * 0.05)
            setattr(attn, nm, lin.bfloat16())
        attn.norm_added_q = gu.RMSNormModule(128, 1e-6, (1.0 + 0.2 * torch.randn(128, generator=g)).bfloat16())
        attn.norm_added_k = gu.RMSNormModule(128, 1e-6, (1.0 + 0.2 * torch.randn(128, generator=g)).bfloat16())
    attn = attn.to(dev)
    results = {}
    for fused in (True, False):
        cls = _fresh(processor.Hunyuan_SAPAttn_Processor2_0)
        gu.configure_hunyuan_processor(cls)
        cls.first_times_fp = 100.0                              # dense branch: the producer is what differs
        if not fused:
            cls._fused_producer_applies = staticmethod(lambda *a: False)
        proc = cls(0)
        seen = _record_core_inputs(proc)
        n0 = _launches()
        with torch.no_grad():
            y, y_enc = proc(attn, hidden, encoder_hidden_states=enc, attention_mask=mask, image_rotary_emb=rot,
                            timestep=torch.tensor([500.0], device=dev))
        results[fused] = (seen, y.cpu(), y_enc.cpu(), _launches() - n0)
    a, b = results[True], results[False]
    assert a[3] == (6 if double_stream else 3) and b[3] == 0       # producer launches of the library
    for t in ("q", "k", "v"):
        x, r = a[0][t].float(), b[0][t].float()
        assert x.shape == r.shape == (1, P["heads"], n + enc.shape[1], 128)
        assert (x == r).float().mean() >= 0.99
        assert (x - r).abs().max() <= 2.0 ** -5 * max(1.0, float(r.abs().max()))
    assert torch.equal(a[0]["v"], b[0]["v"])
    assert (a[1].float() - b[1].float()).abs().max() <= 3e-2 and (a[2].float() - b[2].float()).abs().max() <= 3e-2
