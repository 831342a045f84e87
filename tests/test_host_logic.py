"""Host-side logic of the package that needs no GPU: density limits, profile lookup,
clustering-reuse schedule, synthetic inputs."""
import os

import numpy as np
import pytest
import torch

from oracle import svoo_oracle as O
from svoo_b200 import synth
from svoo_b200.sparsity import SparsityLookup, min_kc_ratio_for_heads
from tests import golden_util as gu


def test_keep_limits_match_oracle():
    from svoo_b200.co_clustering import keep_limits
    H, KC = 4, 500
    cases = [(0, 0), (0.1, 0), (0.1, None), ([0.07, 0.12, 0.2, 0.29], 0), ([0.07, 0.12, 0.2, 0.29], [0.07, 0.12, 0.2, 0.29]),
             ([0.15, 0.2, 0.0, 0.18], 0.1), (0.3, 0.1), (0, 0.001), (torch.tensor([0.1, 0.2, 0.3, 0.4]), 0),
             ([0.0, 0.0, 0.0, 0.0], [0.5, 0.0, 1.0, 2.0])]
    for mn, mx in cases:
        p_ref, c_ref = O.keep_counts(KC, H, mn, mx)
        p, c = keep_limits(KC, H, mn, mx)
        assert p == [min(v, KC) for v in p_ref] and c == [min(v, KC) for v in c_ref], (mn, mx)
    # float32 truncation like the reference's tensor round trip: 0.29 * 500 -> 144, not 145
    assert keep_limits(500, 1, [0.29], 0)[0] == [144]
    assert keep_limits(500, 1, 0.29, 0)[0] == [int(0.29 * 500)]


def test_sparsity_lookup_matches_reference_fixture():
    lk = SparsityLookup(os.path.join(gu.GOLDEN, "density_profile.csv"))
    z = gu.load("density_profile_expected")
    for si, step in enumerate((1, 2)):
        for layer in range(3):
            assert lk.has_data_for_step_layer(step, layer, 4) == bool(z["has"][si, layer])
            np.testing.assert_array_equal(np.array(lk.get_sparsity_batch(step, layer, 4)), z["batch"][si, layer])
    with pytest.raises(FileNotFoundError):
        SparsityLookup("/nonexistent.csv")
    # clipping and fallback
    vals = min_kc_ratio_for_heads(lk, True, 1, 0, 4, 0.1, 0.15, 0.2)
    assert all(0.15 <= v <= 0.2 for v in vals) and len(vals) == 4
    assert min_kc_ratio_for_heads(lk, True, 2, 1, 4, 0.1, 0.15, 0.2) == 0.1      # hole -> scalar fallback
    assert min_kc_ratio_for_heads(lk, False, 1, 0, 4, 0.1, None, None) == 0.1
    assert min_kc_ratio_for_heads(lk, True, None, 0, 4, 0.1, None, None) == 0.1


def test_synth_shapes_and_determinism():
    cfg = synth.CONFIGS["cfg0"]
    q, k, v = synth.make_qkv(cfg)
    assert q.shape == (1, 2, 4096, 128) and q.dtype == torch.float32
    q2, _, _ = synth.make_qkv(cfg, heads=[1])
    assert torch.equal(q2[0, 0], q[0, 1])
    assert synth.CONFIGS["cfg2"].n_video == 75600 and synth.CONFIGS["cfg1"].n_video == 32760
    assert synth.CONFIGS["cfg3"].n_tokens == 118800 + 256
    d = synth.head_densities(synth.CONFIGS["cfg2"])
    assert len(d) == 40 and all(0.05 <= x <= 0.25 for x in d)
    qi, ki = synth.init_indices(cfg)
    assert qi.shape == (2, 32) and ki.shape == (2, 128)


def test_oracle_internal_consistency():
    cfg = gu.TINY_BF16
    q, k, v = synth.make_qkv(cfg)
    qi, ki = synth.init_indices(cfg)
    out, aux = O.sparse_attention_layer(q, k, v, qi, ki, cfg.num_q, cfg.num_k, 2, 1.0)
    assert aux["map"].all()
    dense = torch.softmax((q.float() @ k.float().transpose(-1, -2)) * 128 ** -0.5, -1) @ v.float()
    assert (out.float() - dense).abs().max() < 2e-2          # all-ones map == dense attention
    assert int(aux["qsizes"].sum()) == cfg.heads * cfg.n_video
    assert torch.equal(O.inverse_permute(O.permute(q[0], aux["q_idx"]), aux["q_idx"]), q[0])
    rho = O.realised_density(aux["map"], aux["qsizes"][None], aux["ksizes"][None])
    assert torch.allclose(rho, torch.ones_like(rho))


def test_reuse_schedule():
    pytest.importorskip("svoo_b200._lib")
    from svoo_b200.processor import WanAttn_SAPAttn_Processor
    p = WanAttn_SAPAttn_Processor(layer_idx=3)
    p.start_reuse_step, p.reuse_interval = 11, 40
    got = []
    for step in (1, 10, 11, 12, 50, 51, 52):
        p.current_inference_step = step
        got.append(p._should_recluster())
    assert got == [True, True, True, False, False, True, False]
    p.start_reuse_step = None
    p.current_inference_step = 30
    assert p._should_recluster()
    p.first_layers_fp, p.first_times_fp = 4, 900
    assert p._full_attention_flag(torch.tensor([100]))        # layer 3 < 4
    p.first_layers_fp = 0
    assert p._full_attention_flag(torch.tensor([950])) and not p._full_attention_flag(torch.tensor([100]))
