"""Autograd entry points for SwiGLU + blockwise FP8 quantisation -- the contract of
linghe/facade/silu.py.  ``cls`` is the injected FP8 tensor container; quantizers need
``force_pow_2_scales`` and ``dtype`` (lists of quantizers on the batched path)."""

from __future__ import annotations

import torch

from linghe_b200.utils.silu import (triton_batch_weighted_silu_and_block_quant_backward,
                                    triton_batch_weighted_silu_and_block_quant_forward,
                                    triton_silu_and_block_quant_backward,
                                    triton_silu_and_block_quant_forward)


def _wrap(cls, shape, dtype, quantizer, fp8_dtype, q, q_scale, qt, qt_scale, requires_grad):
    return cls(
        shape=shape,
        dtype=dtype,
        fp8_dtype=fp8_dtype,
        rowwise_data=q,
        rowwise_scale_inv=q_scale,
        columnwise_data=qt,
        columnwise_scale_inv=qt_scale,
        quantizer=quantizer,
        requires_grad=requires_grad,
        is_2D_scaled=False,
    )


class BlockSiluFunction(torch.autograd.Function):
    """Dense (shared-expert) SwiGLU; forward and backward both return FP8 containers
    (linghe/facade/silu.py:11)."""

    @staticmethod
    def forward(ctx, input, quantizer, grad_quantizer, cls):
        shape = input.shape
        assert len(shape) == 3
        S, B, H2 = shape
        ctx.grad_quantizer = grad_quantizer
        ctx.input_requires_grad = input.requires_grad
        ctx.shape = shape
        ctx.cls = cls
        ctx.save_for_backward(input)
        q, q_scale, qt, qt_scale = triton_silu_and_block_quant_forward(
            input.view(S * B, H2), round_scale=quantizer.force_pow_2_scales)
        H = H2 // 2
        return _wrap(cls, (S, B, H), input.dtype, quantizer, quantizer.dtype, q.view(S, B, H), q_scale,
                     qt.view(H, S, B), qt_scale, input.requires_grad)

    @staticmethod
    def backward(ctx, grad_output):
        S, B, H = grad_output.shape
        (input,) = ctx.saved_tensors
        gq = ctx.grad_quantizer
        q, q_scale, qt, qt_scale = triton_silu_and_block_quant_backward(
            grad_output.view(S * B, H), input.view(S * B, 2 * H), round_scale=gq.force_pow_2_scales)
        out = _wrap(ctx.cls, ctx.shape, grad_output.dtype, gq, gq.dtype, q.view(ctx.shape), q_scale,
                    qt.view(ctx.shape[2], S, B), qt_scale, ctx.input_requires_grad)
        return out, None, None, None


def block_silu_impl(input, quantizer, grad_quantizer, cls):
    """linghe/facade/silu.py:68."""
    return BlockSiluFunction.apply(input, quantizer, grad_quantizer, cls)


class BlockBatchWeightedSiluFunction(torch.autograd.Function):
    """Routed-expert weighted SwiGLU over per-expert row segments
    (linghe/facade/silu.py:73)."""

    @staticmethod
    def forward(ctx, input, weights, counts, splits, quantizers, grad_quantizers, cls, is_recomputing):
        ctx.grad_quantizers = grad_quantizers
        ctx.input_requires_grad = input.requires_grad
        ctx.shape = input.shape
        ctx.splits = splits
        ctx.cls = cls
        ctx.save_for_backward(input, weights, counts)
        mode = 2 if is_recomputing is None else (1 if is_recomputing else 0)
        q, q_scale, qt, qt_scale = triton_batch_weighted_silu_and_block_quant_forward(
            input, weights, counts, splits=splits, round_scale=quantizers[0].force_pow_2_scales,
            output_mode=mode)
        return _wrap(cls, q.shape, input.dtype, quantizers, quantizers[0].dtype, q, q_scale, qt, qt_scale,
                     input.requires_grad)

    @staticmethod
    def backward(ctx, grad_output):
        input, weights, counts = ctx.saved_tensors
        gqs = ctx.grad_quantizers
        q, q_scale, wgrad, qt, qt_scale = triton_batch_weighted_silu_and_block_quant_backward(
            grad_output, input, weights, counts, splits=ctx.splits, round_scale=gqs[0].force_pow_2_scales)
        out = _wrap(ctx.cls, ctx.shape, grad_output.dtype, gqs, gqs[0].dtype, q, q_scale, qt, qt_scale,
                    ctx.input_requires_grad)
        return out, wgrad, None, None, None, None, None, None


def block_batch_weighted_silu_impl(input, weights, counts, splits, quantizers, grad_quantizers, cls,
                                   is_recomputing=None):
    """linghe/facade/silu.py:156."""
    assert input.ndim == 2
    return BlockBatchWeightedSiluFunction.apply(input, weights, counts, splits, quantizers, grad_quantizers,
                                                cls, is_recomputing)
