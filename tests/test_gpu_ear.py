"""The error-aware routing (EAR) kernels through the C ABI against the CPU oracle.  Needs a B200.

Bars: centroid logits and the block selection bit-exact (from identical inputs); value centroids
within one bf16 rounding; block scores <= 2e-2 (they are logs of sums whose order differs);
attention max-abs-err <= 2e-2 and cosine >= 0.999 in bf16, log2-sum-exp <= 5e-3.
"""
import dataclasses
import math

import numpy as np
import pytest
import torch

from oracle import ear_oracle as E
from oracle import svoo_oracle as O
from svoo_b200 import synth
from tests import golden_util as gu

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def cosine(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm() + 1e-30))


def clustered_case(dev, H, grid, num_q, num_k, seed, empty_k=()):
    """Seeded bf16 q, k, v, one co-clustering on the GPU, everything permuted on the CPU by the
    stable sort of those labels."""
    from svoo_b200 import ops
    cfg = synth.LayerConfig(f"ear-{seed}", seed, H, grid, torch.bfloat16, num_q, num_k, 2, (0.1, 0.3), 1, True)
    q, k, v = synth.make_qkv(cfg)
    qi, ki = synth.init_indices(cfg)
    c = ops.cocluster(q[0].to(dev), k[0].to(dev), qi.to(dev), ki.to(dev), 2)
    kl = c.klabels.cpu().long()
    for e in empty_k:                                    # force empty key clusters
        kl[kl == e] = (e + 1) % num_k
    ql = c.qlabels.cpu().long()
    q_idx, q_off = O.sort_labels(ql, num_q)
    k_idx, k_off = O.sort_labels(kl, num_k)
    qs, ks = q_off[:, 1:] - q_off[:, :-1], k_off[:, 1:] - k_off[:, :-1]
    t = dict(cfg=cfg, q=q[0], k=k[0], v=v[0], ql=ql, kl=kl, q_idx=q_idx, k_idx=k_idx, q_off=q_off, k_off=k_off, qs=qs, ks=ks,
             qc=c.qcentroids.cpu(), kc=c.kcentroids.cpu(), qp=O.permute(q[0], q_idx), kp=O.permute(k[0], k_idx),
             vp=O.permute(v[0], k_idx))
    return t


def gpu_scores(dev, t, gamma):
    from svoo_b200 import ops
    QC = t["qc"].shape[1]
    vc = ops.ear_value_centroids(t["vp"].to(dev), t["k_off"].int().to(dev), QC)
    clog, sc = ops.ear_block_scores(t["qc"].to(dev), t["kc"].to(dev), t["kp"].to(dev), t["q_off"].int().to(dev),
                                    t["k_off"].int().to(dev), gamma)
    return vc, clog, sc


@pytest.mark.parametrize("H,grid,num_q,num_k,empty", [(3, (4, 16, 32), 20, 70, (0, 5)), (2, (8, 32, 60), 100, 500, ()),
                                                      (2, (3, 16, 20), 100, 500, ()), (1, (2, 16, 16), 5, 9, ()),
                                                      (1, (8, 32, 60), 256, 1024, (7,))])
def test_value_centroids_logits_scores(dev, H, grid, num_q, num_k, empty):
    t = clustered_case(dev, H, grid, num_q, num_k, seed=31 + num_k, empty_k=empty)
    vc, clog, sc = gpu_scores(dev, t, 1.0)
    vc_ref = E.value_centroids(t["v"], t["kl"], t["ks"], num_k)
    assert (vc.cpu().float() - vc_ref.float()).abs().max() <= 2e-2          # one bf16 rounding of a value <= 4
    assert (vc.cpu() == vc_ref).float().mean() >= 0.99
    clog_ref = E.centroid_logits(t["qc"], t["kc"])
    assert np.array_equal(clog.cpu().numpy(), clog_ref)
    vn, cvd, vc_sq = E.value_stats(t["vp"], vc.cpu(), t["k_off"])
    sc_ref = E.error_scores(t["qc"], t["kp"], t["k_off"], t["qs"], t["ks"], clog_ref, vn, cvd, vc_sq, 1.0)
    err = (sc.cpu() - sc_ref).abs()
    assert torch.isfinite(sc).all()
    # a cluster of one or two keys equals its centroid up to rounding: its error is a difference of
    # nearly equal sums, i.e. rounding noise on both sides; the bound is for clusters of >= 8 keys
    big = (t["ks"] >= 8)[:, None, :].expand_as(err)
    if big.any():
        assert err[big].max() <= 2e-2, float(err[big].max())
        assert err[big].mean() <= 1e-3


@pytest.mark.parametrize("H,grid,num_q,num_k,top_p,ratio", [
    (3, (4, 16, 32), 20, 70, 0.9, 0.0), (3, (4, 16, 32), 20, 70, 0.6, 0.1), (3, (4, 16, 32), 20, 70, 0.8, [0.05, 0.0, 0.3]),
    (2, (3, 16, 20), 100, 500, 0.9, [0.07, 0.2]), (1, (4, 16, 32), 64, 1024, 0.5, 0.05), (1, (2, 16, 16), 5, 9, 0.4, 0.2)])
def test_selection_bit_exact(dev, H, grid, num_q, num_k, top_p, ratio):
    """The CUDA selection from the CUDA scores equals the oracle's selection from the same scores."""
    from svoo_b200 import ops
    t = clustered_case(dev, H, grid, num_q, num_k, seed=77 + num_k, empty_k=(1,))
    _, clog, sc = gpu_scores(dev, t, 1.0)
    pres, bud = E.ratio_lengths(num_k, H, ratio)
    got = ops.ear_select_blocks(clog, sc, t["q_off"].int().to(dev), t["k_off"].int().to(dev), top_p, pres, bud)
    ref = E.select_blocks(clog.cpu().numpy(), sc.cpu().numpy(), t["qs"], t["ks"], top_p, ratio, True)
    assert torch.equal(got.cpu().bool(), ref)
    dens = float(ref.float().mean())
    assert 0.0 < dens < 1.0 or top_p >= 0.9


def _ext(dev, perm, cen):
    """[BH*S + BH*KC, 128]: token rows of all heads, then centroid rows of all heads."""
    return torch.cat([perm.reshape(-1, 128), cen.reshape(-1, 128)], 0).contiguous().to(dev)


@pytest.mark.parametrize("H,grid,num_q,num_k,top_p,ratio,empty", [
    (3, (4, 16, 32), 20, 70, 0.5, 0.05, (0, 5)), (2, (3, 16, 20), 100, 500, 0.6, [0.07, 0.2], ()),
    (1, (2, 16, 16), 5, 9, 0.3, 0.0, ()), (2, (5, 16, 24), 7, 300, 0.4, 0.02, (3,)),
    (1, (8, 32, 60), 256, 1024, 0.3, 0.05, ())])
def test_ear_attention_matches_oracle(dev, H, grid, num_q, num_k, top_p, ratio, empty):
    from svoo_b200 import ops
    t = clustered_case(dev, H, grid, num_q, num_k, seed=5 + num_k, empty_k=empty)
    vc, clog, sc = gpu_scores(dev, t, 1.0)
    pres, bud = E.ratio_lengths(num_k, H, ratio)
    m = ops.ear_select_blocks(clog, sc, t["q_off"].int().to(dev), t["k_off"].int().to(dev), top_p, pres, bud)
    S = t["qp"].shape[1]
    k_ext, v_ext = _ext(dev, t["kp"], t["kc"]), _ext(dev, t["vp"], vc.cpu())
    out, lse2 = ops.sparse_attn_ear(t["qp"].to(dev), k_ext, v_ext, m, t["q_off"].int().to(dev), t["k_off"].int().to(dev),
                                    out_row_idx=t["q_idx"].int().to(dev), return_lse=True)
    assert ops.ear_attention_status(dev, H, S, num_q, num_k) == 0
    ref_p, lse_p = E.compensated_attention(t["qp"], t["kp"], t["vp"], t["kc"], vc.cpu(), m.cpu().bool(), t["qs"], t["ks"])
    ref = O.inverse_permute(ref_p, t["q_idx"])
    lse_ref = torch.empty_like(lse_p)
    lse_ref.scatter_(1, t["q_idx"].long(), lse_p)
    assert (out.cpu().float() - ref.float()).abs().max() <= 2e-2
    assert cosine(out.cpu(), ref) >= 0.999
    assert (lse2.cpu() - lse_ref / math.log(2.0)).abs().max() <= 5e-3
    # and the compensation matters: without it the result is further from the oracle
    plain = ops.sparse_attn(t["qp"].to(dev), t["kp"].to(dev), t["vp"].to(dev), m, t["q_off"].int().to(dev),
                            t["k_off"].int().to(dev), out_row_idx=t["q_idx"].int().to(dev))
    assert (plain.cpu().float() - ref.float()).abs().max() > (out.cpu().float() - ref.float()).abs().max()


def test_ear_attention_full_map_equals_plain(dev):
    """Every cluster selected: no centroid key, the EAR kernel gives the plain kernel's bits."""
    from svoo_b200 import ops
    t = clustered_case(dev, 2, (4, 16, 32), 12, 40, seed=3)
    H, S = 2, t["qp"].shape[1]
    m = torch.ones(H, 12, 40, dtype=torch.uint8, device=dev)
    vc = E.value_centroids(t["v"], t["kl"], t["ks"], 40)
    a = ops.sparse_attn_ear(t["qp"].to(dev), _ext(dev, t["kp"], t["kc"]), _ext(dev, t["vp"], vc), m,
                            t["q_off"].int().to(dev), t["k_off"].int().to(dev))
    b = ops.sparse_attn(t["qp"].to(dev), t["kp"].to(dev), t["vp"].to(dev), m, t["q_off"].int().to(dev), t["k_off"].int().to(dev))
    assert torch.equal(a, b)


@pytest.mark.parametrize("name", list(gu.EAR_CASES))
def test_reference_fixture(dev, name):
    """The recorded run of the reference (labels, centroids, maps, compensated output).  The fp32 case
    is computed in bf16 here, so its bounds are the loose ones."""
    from svoo_b200 import ops
    cfg, settings = gu.EAR_CASES[name]
    z = gu.load(name)
    q, k, v = synth.make_qkv(cfg)
    t = gu.ear_inputs(cfg, z, q, k, v)
    b16 = lambda x: x.to(torch.bfloat16)
    H, QC, KC = cfg.heads, cfg.num_q, cfg.num_k
    qo, ko = t["q_off"].int().to(dev), t["k_off"].int().to(dev)
    vc = ops.ear_value_centroids(b16(t["vp"]).to(dev), ko, QC)
    assert (vc.cpu().float() - torch.from_numpy(z["vcentroids"])).abs().max() <= 3e-2
    for n, (top_p, gamma, ratio) in enumerate(settings):
        clog, sc = ops.ear_block_scores(b16(t["qc"]).to(dev), b16(t["kc"]).to(dev), b16(t["kp"]).to(dev), qo, ko, gamma)
        assert (sc.cpu() - torch.from_numpy(z[f"scores_{n}"])).abs().max() <= (3e-2 if cfg.dtype == torch.bfloat16 else 0.15)
        pres, bud = E.ratio_lengths(KC, H, ratio)
        m = ops.ear_select_blocks(clog, sc, qo, ko, top_p, pres, bud)
        agree = float((m.cpu().bool().numpy() == gu.unpack_ear_map(z, n)).mean())
        assert agree >= (0.97 if cfg.dtype == torch.bfloat16 else 0.9), (name, n, agree)
    ref_map = torch.from_numpy(gu.unpack_ear_map(z, len(settings) - 1)).to(torch.uint8).to(dev)
    k_ext = torch.cat([b16(t["kp"]).reshape(-1, 128), b16(t["kc"]).reshape(-1, 128)]).contiguous().to(dev)
    v_ext = torch.cat([b16(t["vp"]).reshape(-1, 128), b16(t["vc"]).reshape(-1, 128)]).contiguous().to(dev)
    out, lse2 = ops.sparse_attn_ear(b16(t["qp"]).to(dev), k_ext, v_ext, ref_map, qo, ko, out_row_idx=t["q_idx"].int().to(dev),
                                    return_lse=True)
    step = int(z["rows_kept"][0])
    ref_rows = torch.from_numpy(z["out_rows"])
    assert (out.cpu()[:, ::step].float() - ref_rows).abs().max() <= 3e-2
    assert cosine(out.cpu()[:, ::step], ref_rows) >= 0.999
    assert (lse2.cpu()[:, ::step] * math.log(2.0) - torch.from_numpy(z["lse_rows"])).abs().max() <= 3e-2


def test_layer_ear_matches_oracle(dev):
    """The whole EAR layer (clustering, permute, value centroids, scores, selection, attention): the
    attention against the oracle on the layer's own clustering and map; the map against the map the
    oracle derives from its own scores."""
    from svoo_b200 import layer
    cfg = synth.LayerConfig("ear-layer", 61, 3, (6, 16, 32), torch.bfloat16, 16, 96, 2, (0.05, 0.2), 1, True)
    q, k, v = synth.make_qkv(cfg)
    qi, ki = synth.init_indices(cfg)
    ratios = synth.head_densities(cfg)
    out, st = layer.sparse_attention_layer(q.to(dev), k.to(dev), v.to(dev), num_q_centroids=cfg.num_q, num_k_centroids=cfg.num_k,
                                           kmeans_iters=2, top_p=0.6, min_kc_ratio=ratios, init_indices=(qi.to(dev), ki.to(dev)),
                                           return_state=True, ear_gamma=1.0)
    c = st.clustering
    ql, kl = c.qlabels.cpu().long(), c.klabels.cpu().long()
    q_idx, q_off = O.sort_labels(ql, cfg.num_q)
    k_idx, k_off = O.sort_labels(kl, cfg.num_k)
    assert torch.equal(q_idx.int(), c.q_sorted_idx.cpu()) and torch.equal(k_off.int(), c.k_offsets.cpu())
    qs, ks = q_off[:, 1:] - q_off[:, :-1], k_off[:, 1:] - k_off[:, :-1]
    qp, kp, vp = O.permute(q[0], q_idx), O.permute(k[0], k_idx), O.permute(v[0], k_idx)
    qc, kc = c.qcentroids.cpu(), c.kcentroids.cpu()
    vc = E.value_centroids(v[0], kl, ks, cfg.num_k)
    m = st.block_map.cpu().bool()
    ref_map = E.identify_dynamic_map_estimated(kp, vp, qs, ks, qc, kc, vc, 0.6, 1.0, ratios)
    assert float((m == ref_map).float().mean()) >= 0.97
    assert 0.05 < float(m.float().mean()) < 0.9
    ref_p, _ = E.compensated_attention(qp, kp, vp, kc, vc, m, qs, ks)
    ref = O.inverse_permute(ref_p, q_idx)
    assert (out[0].cpu().float() - ref.float()).abs().max() <= 2e-2
    assert cosine(out[0].cpu(), ref) >= 0.999


def test_ear_processor(dev, tmp_path):
    """WanAttn_EARAttn_Processor.attention_core_logic: the error-aware branch runs behind the same
    call as the plain one, gives a different map and a result closer to dense attention at the same
    budget (the point of the compensation)."""
    from svoo_b200 import processor as P
    Wp = gu.WAN_PROC
    H, (T, Hh, W) = Wp["heads"], Wp["grid"]
    N = T * Hh * W

    def run(cls):
        gu.configure_wan_processor(cls, None)
        cls.use_dynamic_min_kc_ratio = False
        cls.min_kc_ratio = 0.1
        cls.top_p_kmeans = 0.5
        cls.start_reuse_step = None
        proc = cls(0)
        proc._step_from_callback = 2
        proc.draw_init_indices = lambda BH, n, device: tuple(i.to(device) for i in synth.init_indices(
            synth.LayerConfig("p", 9, BH, (T, Hh, W), torch.bfloat16, Wp["num_q"], Wp["num_k"], 2, (0.1, 0.1), 1, True)))
        return proc, proc.attention_core_logic(q, k, v, torch.tensor([500.0]))

    cfg = synth.LayerConfig("ear-proc", 62, H, (T, Hh, W), torch.bfloat16, Wp["num_q"], Wp["num_k"], 2, (0.1, 0.1), 1, True)
    q, k, v = (t.to(dev) for t in synth.make_qkv(cfg))
    p_ear, y_ear = run(P.WanAttn_EARAttn_Processor)
    p_sap, y_sap = run(P.WanAttn_SAPAttn_Processor)
    assert p_ear.use_ear and not p_sap.use_ear
    p_ear.check_status()
    p_sap.check_status()
    assert y_ear.shape == (1, N, H * 128) and torch.isfinite(y_ear.float()).all()
    dense = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float()).transpose(1, 2).flatten(2, 3)
    e_ear = float((y_ear.float() - dense).abs().mean())
    e_sap = float((y_sap.float() - dense).abs().mean())
    assert not torch.equal(p_ear.last_block_map, p_sap.last_block_map)
    assert e_ear < e_sap, (e_ear, e_sap)


def test_full_size_ear_layer_properties(dev):
    """Two heads of the Wan-14B 720p layer (75,600 tokens, 100 / 500 clusters) through the EAR layer:
    the kernel's status word, the realised density, and three query clusters of head 0 recomputed by
    the oracle's formula from the layer's own clustering and map."""
    from svoo_b200 import layer, ops
    cfg = dataclasses.replace(synth.CONFIGS["cfg2"], heads=2)
    q, k, v = synth.make_qkv(cfg)
    qi, ki = synth.init_indices(cfg)
    ratios = [0.1, 0.2]
    out, st = layer.sparse_attention_layer(q.to(dev), k.to(dev), v.to(dev), num_q_centroids=cfg.num_q, num_k_centroids=cfg.num_k,
                                           kmeans_iters=cfg.iters, top_p=0.0, min_kc_ratio=ratios,
                                           init_indices=(qi.to(dev), ki.to(dev)), return_state=True, ear_gamma=1.0)
    assert ops.ear_attention_status(dev, 2, cfg.n_video, cfg.num_q, cfg.num_k) == 0
    assert torch.isfinite(out.float()).all()
    c = st.clustering
    m = st.block_map.cpu().bool()
    q_off, k_off = c.q_offsets.cpu().long(), c.k_offsets.cpu().long()
    qs, ks = q_off[:, 1:] - q_off[:, :-1], k_off[:, 1:] - k_off[:, :-1]
    rho = O.realised_density(m[None], qs[None], ks[None])[0]
    assert 0.1 < float(rho.min()) and float(rho.max()) < 0.6, rho
    # every query cluster keeps at least its guaranteed clusters
    pres, _ = E.ratio_lengths(cfg.num_k, 2, ratios)
    assert all(int(m[h].sum(-1).min()) >= pres[h] for h in range(2))
    h = 0
    k_idx, q_idx = c.k_sorted_idx[h].cpu().long(), c.q_sorted_idx[h].cpu().long()
    kp, vp = k[0, h][k_idx].float(), v[0, h][k_idx].float()
    kc = c.kcentroids[h].cpu().float()
    vc = E.value_centroids(v[0, h:h + 1], c.klabels[h:h + 1].cpu().long(), ks[h:h + 1], cfg.num_k)[0].float()
    bias = torch.log(ks[h].float() + 1e-6)
    scale = 128 ** -0.5
    for i in (0, 37, 99):
        rows = q_idx[q_off[h, i]:q_off[h, i + 1]]
        if len(rows) == 0:
            continue
        qi_rows = q[0, h][rows].float()
        sel = torch.cat([torch.arange(k_off[h, j], k_off[h, j + 1]) for j in torch.nonzero(m[h, i]).flatten().tolist()])
        rest = torch.nonzero(~m[h, i]).flatten()
        sc = torch.cat([(qi_rows @ kp[sel].T) * scale, (qi_rows @ kc[rest].T) * scale + bias[rest][None, :]], 1)
        ref = torch.softmax(sc, -1) @ torch.cat([vp[sel], vc[rest]], 0)
        got = out[0, h].cpu()[rows].float()
        assert (got - ref).abs().max() <= 2e-2, (i, float((got - ref).abs().max()))
        assert cosine(got, ref) >= 0.999


def test_dit_step_with_ear_pattern(dev):
    """install_processors(pattern="EAR") on a reduced DiT (2 blocks, 4 heads, 3,840 tokens): one
    denoising step runs through WanAttn_SAPAttn_Processor with error-aware routing switched on by the
    installer, stays close to the same model with dense attention, and leaves both status words clear."""
    from svoo_b200 import processor, wan_dit
    cfg = wan_dit.WanDiTConfig(num_layers=2, dim=512, heads=4, ffn_dim=1024, text_dim=64, text_len=16, latent=(3, 32, 40))
    kw = dict(num_q_centroids=12, num_k_centroids=40, top_p_kmeans=0.5, min_kc_ratio=0.15, kmeans_iter_init=2, kmeans_iter_step=1)
    fresh = lambda: type("Case", (processor.WanAttn_SAPAttn_Processor,), {})
    ear = wan_dit.WanDiT(cfg).init_weights(1).to(device=dev, dtype=torch.bfloat16).eval()
    dense = wan_dit.WanDiT(cfg).init_weights(1).to(device=dev, dtype=torch.bfloat16).eval()
    ear_procs = wan_dit.install_processors(ear, fresh(), cfg.grid, pattern="EAR", ear_gamma=1.0, **kw)
    wan_dit.install_processors(dense, fresh(), cfg.grid, first_layers_fp=99, **kw)
    assert all(p.use_ear for p in ear_procs) and not processor.WanAttn_SAPAttn_Processor.use_ear
    g = torch.Generator("cpu").manual_seed(0)
    lat = torch.randn(1, 16, *cfg.latent, generator=g).bfloat16().to(dev)
    text = torch.randn(1, 16, 64, generator=g).bfloat16().to(dev)
    t = torch.tensor([500.0], device=dev)
    for m in (ear, dense):
        wan_dit.set_attention_step(m, 1)
    with torch.no_grad():
        got, want = ear(lat, t, text), dense(lat, t, text)
    for p in ear_procs:
        p.check_status()
        assert p.last_block_map is not None and 0.0 < float(p.last_block_map.float().mean()) < 1.0
    assert got.shape == want.shape and torch.isfinite(got.float()).all()
    assert cosine(got.cpu(), want.cpu()) >= 0.98


@pytest.mark.parametrize("KC,rows_per_cluster", [(32, 128), (1024, 4), (9, 455)])
def test_ear_attention_crafted_maps(dev, KC, rows_per_cluster):
    """Hand-made layouts through the attention entry alone: key clusters of exactly 128 rows (the token
    part ends on a tile boundary), 1024 clusters (the largest centroid run), a query cluster that selects
    nothing (all keys are centroids), one that selects everything (all centroids masked), empty key
    clusters inside and at the end."""
    from svoo_b200 import ops
    H, QC = 2, 4
    N = KC * rows_per_cluster
    g = torch.Generator("cpu").manual_seed(KC)
    q, k, v = (torch.randn(H, N, 128, generator=g).mul(0.7).bfloat16() for _ in range(3))
    ks = torch.full((H, KC), rows_per_cluster, dtype=torch.int64)
    if KC >= 9:                                         # two empty clusters: their rows go to the neighbour
        ks[:, 3] += ks[:, 4]
        ks[:, 4] = 0
        ks[:, KC - 2] += ks[:, KC - 1]
        ks[:, KC - 1] = 0
    qs = torch.tensor([[N // 2, 0, N // 4, N - N // 2 - N // 4]] * H, dtype=torch.int64)
    off = lambda s: torch.cat([torch.zeros(H, 1, dtype=torch.int64), torch.cumsum(s, -1)], 1)
    q_off, k_off = off(qs), off(ks)
    kc = torch.stack([torch.stack([k[h, k_off[h, j]:k_off[h, j + 1]].float().mean(0) if ks[h, j] else torch.zeros(128)
                                   for j in range(KC)]) for h in range(H)]).bfloat16()
    vc = torch.stack([torch.stack([v[h, k_off[h, j]:k_off[h, j + 1]].float().mean(0) if ks[h, j] else torch.zeros(128)
                                   for j in range(KC)]) for h in range(H)]).bfloat16()
    m = torch.rand(H, QC, KC, generator=g) < 0.3
    m[:, 0] = False
    m[:, 2] = True
    m[1, 3, :] = False
    m[1, 3, 4 if KC >= 9 else 0] = True                 # head 1, cluster 3: only an empty cluster selected (or one cluster)
    k_ext = torch.cat([k.reshape(-1, 128), kc.reshape(-1, 128)]).contiguous().to(dev)
    v_ext = torch.cat([v.reshape(-1, 128), vc.reshape(-1, 128)]).contiguous().to(dev)
    out, lse2 = ops.sparse_attn_ear(q.to(dev), k_ext, v_ext, m.to(torch.uint8).to(dev), q_off.int().to(dev), k_off.int().to(dev),
                                    return_lse=True)
    assert ops.ear_attention_status(dev, H, N, QC, KC) == 0
    ref, lse = E.compensated_attention(q, k, v, kc, vc, m, qs, ks)
    assert (out.cpu().float() - ref.float()).abs().max() <= 2e-2
    assert cosine(out.cpu(), ref) >= 0.999
    assert (lse2.cpu() - lse / math.log(2.0)).abs().max() <= 5e-3


def test_reference_named_wrappers(dev):
    """co_clustering.identify_dynamic_map_estimated, error_estimation_triton, compute_value_centroids and
    dynamic_block_sparse_prune_fwd_flashinfer with the reference's signatures (4-D tensors, sizes
    instead of offsets) give what the ops give."""
    from svoo_b200 import co_clustering as cc
    from svoo_b200 import ops
    t = clustered_case(dev, 2, (4, 16, 32), 12, 40, seed=19)
    H, QC, KC = 2, 12, 40
    d4 = lambda x: x[None].to(dev)
    qs4, ks4 = t["qs"][None].int().to(dev), t["ks"][None].int().to(dev)
    vc4 = cc.compute_value_centroids(d4(t["vp"]), ks4)
    vc, clog, sc = gpu_scores(dev, t, 0.7)
    assert torch.equal(vc4[0], vc)
    sc4 = cc.error_estimation_triton(d4(t["qc"]), d4(t["kc"]), vc4, d4(t["kp"]), d4(t["vp"]), qs4, ks4, None, 0.7)
    assert sc4.shape == (1, H, QC, KC) and torch.equal(sc4[0], sc)
    ratio = [0.1, 0.05]
    m4 = cc.identify_dynamic_map_estimated(d4(t["qp"]), d4(t["kp"]), d4(t["vp"]), qs4, ks4, d4(t["qc"]), d4(t["kc"]), vc4,
                                           top_p=0.5, gamma=0.7, min_kc_ratio=ratio)
    pres, bud = cc.ear_limits(KC, H, ratio)
    assert (pres, bud) == E.ratio_lengths(KC, H, ratio)
    m = ops.ear_select_blocks(clog, sc, t["q_off"].int().to(dev), t["k_off"].int().to(dev), 0.5, pres, bud)
    assert m4.dtype == torch.bool and torch.equal(m4[0].to(torch.uint8), m)
    o4 = cc.dynamic_block_sparse_prune_fwd_flashinfer(d4(t["qp"]), d4(t["kp"]), d4(t["vp"]), d4(t["kc"]), vc4, m4, qs4, ks4,
                                                      is_cpu=False)
    k_ext, v_ext = _ext(dev, t["kp"], t["kc"]), _ext(dev, t["vp"], vc.cpu())
    o = ops.sparse_attn_ear(t["qp"].to(dev), k_ext, v_ext, m, t["q_off"].int().to(dev), t["k_off"].int().to(dev))
    assert o4.shape == (1, H, t["qp"].shape[1], 128) and torch.equal(o4[0], o)


def test_ear_attention_first_tile_fully_masked(dev):
    """128 empty key clusters that the map selects, no other cluster selected: the key list has no
    token, its first tile holds 128 masked centroids (bias -inf), the second the 128 pruned ones."""
    from svoo_b200 import ops
    H, QC, KC, rows = 1, 2, 256, 16
    N = 128 * rows
    g = torch.Generator("cpu").manual_seed(5)
    q, k, v = (torch.randn(H, N, 128, generator=g).mul(0.7).bfloat16() for _ in range(3))
    ks = torch.cat([torch.zeros(H, 128, dtype=torch.int64), torch.full((H, 128), rows, dtype=torch.int64)], 1)
    qs = torch.tensor([[N // 2, N // 2]] * H, dtype=torch.int64)
    off = lambda s: torch.cat([torch.zeros(H, 1, dtype=torch.int64), torch.cumsum(s, -1)], 1)
    q_off, k_off = off(qs), off(ks)
    mean = lambda t, j: t[0, k_off[0, j]:k_off[0, j + 1]].float().mean(0) if ks[0, j] else torch.zeros(128)
    kc = torch.stack([mean(k, j) for j in range(KC)])[None].bfloat16()
    vc = torch.stack([mean(v, j) for j in range(KC)])[None].bfloat16()
    m = torch.zeros(H, QC, KC, dtype=torch.bool)
    m[:, 0, :128] = True                               # query cluster 0: the empty clusters only
    m[:, 1, 100:140] = True                            # query cluster 1: some empty, some real ones
    k_ext = torch.cat([k.reshape(-1, 128), kc.reshape(-1, 128)]).contiguous().to(dev)
    v_ext = torch.cat([v.reshape(-1, 128), vc.reshape(-1, 128)]).contiguous().to(dev)
    out, lse2 = ops.sparse_attn_ear(q.to(dev), k_ext, v_ext, m.to(torch.uint8).to(dev), q_off.int().to(dev), k_off.int().to(dev),
                                    return_lse=True)
    assert ops.ear_attention_status(dev, H, N, QC, KC) == 0
    ref, lse = E.compensated_attention(q, k, v, kc, vc, m, qs, ks)
    assert torch.isfinite(out.float()).all()
    assert (out.cpu().float() - ref.float()).abs().max() <= 2e-2
    assert (lse2.cpu() - lse / math.log(2.0)).abs().max() <= 5e-3
