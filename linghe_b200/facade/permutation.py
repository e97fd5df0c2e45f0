"""Autograd glue for the padded, blockwise-quantised token permutation, mirror of
`block_padded_permute` / `block_padded_unpermute` (linghe/facade/permutation.py:209, 306).

`cls` is the container the caller wants the quantised tensors wrapped in (TransformerEngine's
Float8BlockwiseQTensor in production); `quantizers[0]` supplies `.force_pow_2_scales` and
`.dtype`."""

from typing import List, Optional

import torch

from linghe_b200.utils.gather import (triton_batch_block_pad_permute_with_indices,
                                      triton_make_row_id_map_and_index)
from linghe_b200.utils.scatter import triton_unpermute_with_mask_map


def _wrap(cls, quantizers, x_q, x_scale, xt_q, xt_scale, dtype, requires_grad):
    return cls(shape=x_q.shape, dtype=dtype, fp8_dtype=quantizers[0].dtype, rowwise_data=x_q,
               rowwise_scale_inv=x_scale, columnwise_data=xt_q, columnwise_scale_inv=xt_scale,
               quantizer=quantizers, requires_grad=requires_grad, is_2D_scaled=False)


class _BlockPaddedPermute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, probs, routing_map, tokens_per_expert_cuda_tensor, tokens_per_expert_list,
                quantizers, cls):
        num_out_tokens = sum((x + 15) // 16 * 16 for x in tokens_per_expert_list)
        row_id_map, row_id_index = triton_make_row_id_map_and_index(routing_map, num_out_tokens, multiple_of=16)
        ctx.shape = tokens.shape
        ctx.prob_shape = probs.shape
        x_q, x_scale, xt_q, xt_scale, permuted_probs = triton_batch_block_pad_permute_with_indices(
            tokens, tokens_per_expert_cuda_tensor, row_id_index, tokens_per_expert_list, probs=probs,
            round_scale=quantizers[0].force_pow_2_scales)
        output = _wrap(cls, quantizers, x_q, x_scale, xt_q, xt_scale, tokens.dtype, tokens.requires_grad)
        ctx.save_for_backward(row_id_map)
        return output, permuted_probs, row_id_map, row_id_index

    @staticmethod
    def backward(ctx, grad_output, grad_prob, grad_map, grad_index):
        (row_id_map,) = ctx.saved_tensors
        output, prob_output = triton_unpermute_with_mask_map(grad_output, row_id_map, grad_prob)
        return output.view(ctx.shape), prob_output.view(ctx.prob_shape), None, None, None, None, None


def block_padded_permute(tokens, routing_map, tokens_per_expert_cuda_tensor, tokens_per_expert_list, quantizers,
                         cls, probs: Optional[torch.Tensor] = None):
    """Group the tokens of each expert together (every expert padded to 16 rows) and quantise
    them on both axes.  Returns (permuted quantised tokens wrapped in `cls`, permuted probs,
    row_id_map, row_id_index)."""
    return _BlockPaddedPermute.apply(tokens, probs, routing_map, tokens_per_expert_cuda_tensor,
                                     tokens_per_expert_list, quantizers, cls)


class _BlockPaddedUnpermute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, permuted_tokens, row_id_map, row_id_index, tokens_per_expert, splits, restore_shape,
                quantizers, cls):
        ctx.save_for_backward(row_id_index)
        ctx.tokens_per_expert = tokens_per_expert
        ctx.splits = splits
        ctx.quantizers = quantizers
        ctx.cls = cls
        output, _ = triton_unpermute_with_mask_map(permuted_tokens, row_id_map, None)
        return output

    @staticmethod
    def backward(ctx, grad_output):
        (row_id_index,) = ctx.saved_tensors
        quantizers = ctx.quantizers
        x_q, x_scale, xt_q, xt_scale, _ = triton_batch_block_pad_permute_with_indices(
            grad_output, ctx.tokens_per_expert, row_id_index, ctx.splits,
            round_scale=quantizers[0].force_pow_2_scales)
        output = _wrap(ctx.cls, quantizers, x_q, x_scale, xt_q, xt_scale, grad_output.dtype, False)
        return output, None, None, None, None, None, None, None


def block_padded_unpermute(permuted_tokens: torch.Tensor, row_id_map: torch.Tensor, row_id_index: torch.Tensor,
                           tokens_per_expert: torch.Tensor, splits: List, restore_shape: torch.Size, quantizers,
                           cls):
    """Inverse of `block_padded_permute` for the expert outputs: every token gets the sum of its
    experts' rows; the backward pass permutes and quantises the incoming gradient again."""
    return _BlockPaddedUnpermute.apply(permuted_tokens, row_id_map, row_id_index, tokens_per_expert, splits,
                                       restore_shape, quantizers, cls)
