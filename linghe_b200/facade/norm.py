"""Autograd entry points for RMSNorm -- the contract of linghe/facade/norm.py.

``cls`` is the FP8 tensor container injected by the caller (TransformerEngine's
Float8BlockwiseQTensor in production); it is called with keyword arguments only.
``quantizer`` needs ``force_pow_2_scales`` and ``dtype``."""

from __future__ import annotations

import torch

from linghe_b200.utils.norm import (triton_rms_norm_and_block_quant_forward, triton_rms_norm_backward,
                                    triton_rms_norm_forward)


class RMSNormFunction(torch.autograd.Function):
    """Plain RMSNorm with the fused backward (linghe/facade/norm.py:15)."""

    @staticmethod
    def forward(ctx, x, weight, eps=1e-6):
        y, _ = triton_rms_norm_forward(x, weight, eps)
        ctx.save_for_backward(x, weight)
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dx, dw = triton_rms_norm_backward(dy.contiguous(), x, weight, ctx.eps)
        return dx, dw, None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6):
    """RMSNorm of x with weight (linghe/facade/norm.py:32)."""
    assert x.is_contiguous()
    assert weight.is_contiguous()
    return RMSNormFunction.apply(x, weight, eps)


def _mode_from_recompute(is_recomputing):
    # None: first forward, both layouts; True: recompute pass, column-wise only (reuses
    # the saved 1/rms); False: row-wise only.
    if is_recomputing is None:
        return 2
    return 1 if is_recomputing else 0


class BlockRMSNorm(torch.autograd.Function):
    """RMSNorm feeding a blockwise-FP8 linear (linghe/facade/norm.py:49): the forward
    returns the quantised activation wrapped in ``cls`` plus 1/rms."""

    @staticmethod
    def forward(ctx, input, weight, rms, eps, quantizer, cls, is_recomputing):
        shape = input.shape
        assert len(shape) == 3
        S, B, H = shape
        q, q_scale, out_rms, qt, qt_scale = triton_rms_norm_and_block_quant_forward(
            input.view(S * B, H), weight, rms=rms, eps=eps,
            round_scale=quantizer.force_pow_2_scales, output_mode=_mode_from_recompute(is_recomputing))
        output = cls(
            shape=shape,
            dtype=input.dtype,
            fp8_dtype=quantizer.dtype,
            rowwise_data=None if q is None else q.view(shape),
            rowwise_scale_inv=q_scale,
            columnwise_data=None if qt is None else qt.view(H, S, B),
            columnwise_scale_inv=qt_scale,
            quantizer=quantizer,
            requires_grad=input.requires_grad,
            is_2D_scaled=False,
        )
        ctx.input_requires_grad = input.requires_grad
        ctx.weight_requires_grad = weight.requires_grad
        ctx.shape = shape
        ctx.eps = eps
        ctx.save_for_backward(input, weight)
        return output, out_rms

    @staticmethod
    def backward(ctx, grad_output, grad_rms):
        S, B, H = grad_output.shape
        input, weight = ctx.saved_tensors
        dx, dw = triton_rms_norm_backward(grad_output.contiguous().view(S * B, H), input.view(S * B, H),
                                          weight, eps=ctx.eps)
        return dx.view(S, B, H), dw, None, None, None, None, None


def block_rms_norm(input, weight, rms, quantizer, cls, eps=1e-6, is_recomputing=None):
    """linghe/facade/norm.py:107."""
    output, output_rms = BlockRMSNorm.apply(input, weight, rms, eps, quantizer, cls, is_recomputing)
    return output, output_rms.detach()
