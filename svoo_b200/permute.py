"""Cluster-order permutation of [B, H, S, D] tensors; names and signatures of the
reference's svoo/kernels/triton/permute.py (:68-130)."""
from __future__ import annotations

from typing import Optional

import torch

from . import ops


def permute_tensor_by_labels(tensor: torch.Tensor, labels: Optional[torch.Tensor], dim: int, *,
                             sorted_indices: Optional[torch.Tensor] = None, num_clusters: Optional[int] = None):
    """Returns (permuted [B,H,S,D], sorted_indices int32 [B*H, S]).  The order inside one
    cluster is ascending token index (the reference's torch.argsort leaves it unspecified).
    `num_clusters` saves a device-to-host read of labels.max() when labels are given."""
    assert dim == 2, "permute_tensor_by_labels currently only supports dim==2 (sequence dimension)"
    assert tensor.dim() == 4, "Expected tensor shape [B,H,S,D]"
    assert tensor.is_cuda, "permute_tensor_by_labels requires CUDA tensors"
    B, H, S, D = tensor.shape
    if sorted_indices is not None:
        sorted_indices = sorted_indices.to(torch.int32).contiguous()
    else:
        assert labels is not None, "Either `labels` or `sorted_indices` must be provided."
        labels = labels.to(tensor.device).reshape(B * H, S)
        if num_clusters is None:
            num_clusters = int(labels.max().item()) + 1
        sorted_indices, _ = ops.sort_labels(labels, num_clusters)
    x = tensor.reshape(B * H, S, D)
    x = (x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)).contiguous()
    y = ops.permute(x, sorted_indices.reshape(B * H, S))
    return y.view(B, H, S, D).to(tensor.dtype), sorted_indices


def apply_inverse_permutation(permuted_tensor: torch.Tensor, sorted_indices: torch.Tensor, dim: int):
    """Undo permute_tensor_by_labels for tensors of shape [B, H, S, D]."""
    assert dim == 2, "apply_inverse_permutation currently only supports dim==2"
    assert permuted_tensor.dim() == 4, "Expected tensor shape [B,H,S,D]"
    assert permuted_tensor.is_cuda, "apply_inverse_permutation requires CUDA tensors"
    B, H, S, D = permuted_tensor.shape
    idx = sorted_indices.to(torch.int32).reshape(B * H, S).contiguous()
    x = permuted_tensor.reshape(B * H, S, D)
    x = (x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)).contiguous()
    return ops.inverse_permute(x, idx).view(B, H, S, D).to(permuted_tensor.dtype)


# the reference's names
permute_tensor_by_labels_triton = permute_tensor_by_labels
apply_inverse_permutation_triton = apply_inverse_permutation
