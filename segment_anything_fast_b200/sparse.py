"""2:4 semi-structured sparsity for the encoder's Linear layers, with the reference's entry points
(segment_anything_fast/sparse.py:6-32).

``apply_fake_sparsity(model)`` zeroes, in every group of 4 consecutive in-features of every
``nn.Linear`` weight, the 2 entries of smallest magnitude: what the reference's
``WeightNormSparsifier(sparsity_level=1.0, sparse_block_shape=(1,4), zeros_per_block=2)`` flow leaves
after ``squash_mask``.  ``apply_sparse(model)`` does the same and marks the layers as 2:4 so that the
encoder can pick a sparse kernel for them: in int8 mode (``set_quant("int8")``) the marked ``attn.proj``,
``mlp.lin1`` and ``mlp.lin2`` run compressed on the sparse tensor-core path (``samb_gemm_i8_sp24``); in
bf16 mode, and for ``attn.qkv``, the pruned weights go through the dense GEMMs, which is the identical
arithmetic (a dense product with the masked weight).
"""
from typing import Callable, Optional

import torch


def prune_2_4_(weight: torch.Tensor) -> torch.Tensor:
    """In-place 2:4 magnitude pruning along the in-feature axis of ``weight [N, K]`` (K multiple of 4);
    returns the boolean keep-mask.  Ties keep the lower index."""
    N, K = weight.shape
    if K % 4:
        raise ValueError("in-features must be a multiple of 4 for 2:4 sparsity")
    mag = weight.detach().abs().to(torch.float32).reshape(N, K // 4, 4)
    order = torch.argsort(mag, dim=-1, descending=True, stable=True)
    keep = torch.zeros_like(mag, dtype=torch.bool)
    keep.scatter_(-1, order[..., :2], True)
    keep = keep.reshape(N, K)
    with torch.no_grad():
        weight.mul_(keep.to(weight.dtype))
    return keep


def apply_fake_sparsity(model: torch.nn.Module, filter_fn: Optional[Callable[[str, torch.nn.Module], bool]] = None):
    """Prune every ``nn.Linear`` of ``model`` (optionally only those ``filter_fn(name, module)`` accepts)."""
    for name, mod in model.named_modules():
        if isinstance(mod, torch.nn.Linear) and (filter_fn is None or filter_fn(name, mod)):
            prune_2_4_(mod.weight)
            mod._samb_sparse24 = True
    return model


def apply_sparse(model: torch.nn.Module, mlp_only: bool = False):
    """The reference's ``apply_sparse``: prune all Linear layers (``mlp_only=True``: only ``mlp.lin1`` /
    ``mlp.lin2``, the combination the sparse + int8 benchmark configuration uses)."""
    f = (lambda n, m: ".mlp.lin" in n or n.startswith("mlp.lin")) if mlp_only else None
    return apply_fake_sparsity(model, f)
