"""Un-permute of routed-expert gradients, mirror of linghe/utils/scatter.py (the one entry
point the padded-permute facade needs)."""

from __future__ import annotations

import torch

from linghe_b200 import _lib


def triton_unpermute_with_mask_map(grad: torch.Tensor, row_id_map: torch.Tensor, probs: torch.Tensor):
    """Sum the rows of `grad` that belong to each token (linghe/utils/scatter.py:193).

    grad [num_out_tokens, hidden]; row_id_map [num_tokens, num_experts] int32 (-1 = not routed);
    probs [num_out_tokens] or None.
    Returns (output [num_tokens, hidden] grad.dtype, float32 sums in expert order;
    restore_probs [num_tokens, num_experts] or None)."""
    assert grad.is_contiguous() and row_id_map.is_contiguous()
    assert row_id_map.dtype == torch.int32
    n = grad.shape[1]
    num_tokens, num_experts = row_id_map.shape
    output = torch.empty((num_tokens, n), dtype=grad.dtype, device=grad.device)
    restore_probs = None
    if probs is not None:
        assert probs.is_contiguous()
        restore_probs = torch.zeros((num_tokens, num_experts), dtype=probs.dtype, device=grad.device)
    if num_tokens == 0:
        return output, restore_probs
    _lib.call("lh_unpermute_with_mask_map", grad, _lib.ptr(grad), _lib.dtype_code(grad), _lib.ptr(row_id_map),
              _lib.ptr(probs), _lib.dtype_code(probs) if probs is not None else _lib.F32, num_tokens, num_experts, n,
              _lib.ptr(output), _lib.ptr(restore_probs))
    return output, restore_probs
