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
MAP_CASES = ["map_bf16_budget", "map_bf16_topp_floor", "map_bf16_scalar", "map_fp32_topp",
             "map_fp32_cap_scalar", "map_bf16_big", "map_all_ones"]


def load(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def unpack_map(z):
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
