"""RMSNorm kernels -- same entry points as linghe/utils/norm.py (the block-quant and
plain variants), running hand-written sm_100a CUDA through the C ABI."""

from __future__ import annotations

from typing import Optional

import torch

from linghe_b200 import _lib

E4M3 = torch.float8_e4m3fn


def _rows_cols(x):
    shape = x.shape
    assert len(shape) in (2, 3)
    if len(shape) == 3:
        return shape[0] * shape[1], shape[2]
    return shape[0], shape[1]


def triton_rms_norm_forward(x, weight, eps=1e-6, out=None, rms=None):
    """RMSNorm (linghe/utils/norm.py:58).  Returns (out like x, rms float32 [M]);
    a given `rms` (1/rms per row) is reused instead of recomputed."""
    assert x.is_contiguous() and weight.is_contiguous()
    M, n = _rows_cols(x)
    assert n <= 8192
    if out is None:
        out = torch.empty_like(x)
    reuse = rms is not None
    if not reuse:
        rms = torch.empty((M,), device=x.device, dtype=torch.float32)
    _lib.call("lh_rmsnorm_fwd", x, _lib.ptr(x), _lib.ptr(weight), _lib.dtype_code(x), M, n, float(eps),
              _lib.ptr(out), _lib.ptr(rms), int(reuse))
    return out, rms


def triton_rms_norm_backward(grad_output, x, w, eps=1e-6, rms=None):
    """RMSNorm backward (linghe/utils/norm.py:144).  Returns (dx like x, dw float32 [n])."""
    assert grad_output.is_contiguous() and x.is_contiguous()
    M, n = _rows_cols(x)
    assert n <= 8192
    nbytes = _lib.scratch_bytes("rmsnorm_bwd", M, n)
    dx, dw, scratch = _lib.empties(x, (tuple(x.shape), x.dtype), ((n,), torch.float32), ((nbytes,), torch.uint8))
    _lib.call("lh_rmsnorm_bwd", x, _lib.ptr(grad_output), _lib.ptr(x), _lib.ptr(w), _lib.ptr(rms),
              _lib.dtype_code(x), M, n, float(eps), _lib.ptr(dx), _lib.ptr(dw), _lib.ptr(scratch), nbytes)
    return dx, dw


def triton_rms_norm_and_block_quant_forward(
    x: torch.Tensor,
    weight: torch.Tensor,
    eps: float = 1e-6,
    out: Optional[torch.Tensor] = None,
    scale: Optional[torch.Tensor] = None,
    rms: Optional[torch.Tensor] = None,
    round_scale: bool = False,
    output_mode: int = 2,
):
    """Fused RMSNorm + blockwise FP8 quantisation (linghe/utils/norm.py:343).

    Returns (out e4m3 [M,n], scale f32 [n/128,M], rms f32 [M], transpose_output e4m3
    [n,M], transpose_scale f32 [ceil(M/128),n]).  output_mode 0: rows only (`rms` must be
    None); 1: columns only (`rms` required, out/scale are returned as passed); 2: both
    (a passed `rms` is ignored and recomputed)."""
    h = _lib.host()
    if h is not None:   # the same steps in C++ (host/lh_host.cpp): a third of the host time
        return h.rms_norm_and_block_quant_forward(x, weight, eps, out, scale, rms, bool(round_scale), output_mode)
    assert x.is_contiguous() and weight.is_contiguous()
    M, n = x.shape
    assert n <= 8192
    assert output_mode in (0, 1, 2)
    device = x.device
    if out is None and output_mode in (0, 2):
        out = torch.empty((M, n), device=device, dtype=E4M3)
    if scale is None and output_mode in (0, 2):
        scale = torch.empty((n // 128, M), device=device, dtype=torch.float32)
    transpose_output = transpose_scale = None
    if output_mode != 0:
        transpose_output = torch.empty((n, M), device=device, dtype=E4M3)
        transpose_scale = torch.empty(((M + 127) // 128, n), device=device, dtype=torch.float32)
    if output_mode == 0:
        assert rms is None
        rms = torch.empty((M,), dtype=torch.float32, device=device)
    elif output_mode == 1:
        assert rms is not None
    else:
        rms = torch.empty((M,), dtype=torch.float32, device=device)
    _lib.call("lh_rmsnorm_blockquant_fwd", x, _lib.ptr(x), _lib.ptr(weight), _lib.dtype_code(x), M, n,
              float(eps), _lib.ptr(out) if output_mode != 1 else 0,
              _lib.ptr(scale) if output_mode != 1 else 0, _lib.ptr(rms), _lib.ptr(transpose_output),
              _lib.ptr(transpose_scale), int(bool(round_scale)), int(output_mode))
    if transpose_output is None:
        # mode 0 does not write the transposed pair; upstream still returns it (uninitialised), so it is
        # allocated here, after the launch, where the allocator no longer delays the kernel
        transpose_output = torch.empty((n, M), device=device, dtype=E4M3)
        transpose_scale = torch.empty(((M + 127) // 128, n), device=device, dtype=torch.float32)
    return out, scale, rms, transpose_output, transpose_scale


def triton_rms_norm_fp32_gemm_block_quant_forward(
    x: torch.Tensor,
    norm_weight: torch.Tensor,
    route_weight: torch.Tensor,
    rms: Optional[torch.Tensor] = None,
    eps: float = 1e-6,
    output_mode: int = 0,
    round_scale=False,
):
    """RMSNorm + float32 router logits + blockwise quantisation (linghe/utils/norm.py:688).

    y = rms_norm(x); logits = y_f32 @ route_weight.T (float32); quantisation of y_f32.
    output_mode 0 writes y, rms, logits, x_q, x_s (row-wise copy); output_mode 1 needs `rms`
    and writes only the transposed copy xt_q, xt_s.  Returns
    (y [M,K] x.dtype, rms [M], logits [M,N] f32, x_q [M,K], x_s [K/128,M], xt_q [K,M],
    xt_s [M/128,K]); the tensors a mode does not write are allocated and left as they are."""
    assert x.is_contiguous() and norm_weight.is_contiguous() and route_weight.is_contiguous()
    assert output_mode in (0, 1)
    M, K = x.size()
    N, K2 = route_weight.size()
    assert K2 == K
    assert M % 128 == 0 and K % 128 == 0 and N % 128 == 0
    device = x.device
    if rms is None:
        assert output_mode == 0
        rms = torch.empty(M, dtype=torch.float32, device=device)
    nbytes = _lib.scratch_bytes("rmsnorm_gemm", N, K) if output_mode == 0 else 0
    y, logits, x_q, x_s, xt_q, xt_s, scratch = _lib.empties(
        x, ((M, K), x.dtype), ((M, N), torch.float32), ((M, K), E4M3), ((K // 128, M), torch.float32), ((K, M), E4M3),
        ((M // 128, K), torch.float32), ((max(nbytes, 16),), torch.uint8))
    _lib.call("lh_rmsnorm_gemm_blockquant_fwd", x, _lib.ptr(x), _lib.ptr(norm_weight), _lib.ptr(route_weight),
              _lib.dtype_code(x), M, K, N, float(eps), _lib.ptr(y), _lib.ptr(rms), _lib.ptr(logits), _lib.ptr(x_q),
              _lib.ptr(x_s), _lib.ptr(xt_q), _lib.ptr(xt_s), int(bool(round_scale)), int(output_mode),
              _lib.ptr(scratch), nbytes)
    return y, rms, logits, x_q, x_s, xt_q, xt_s


def rms_norm_backward_and_block_quant(grad_output, x, w, eps=1e-6, rms=None, round_scale=False):
    """RMSNorm backward fused with the dual-axis quantisation of `grad_output`.

    Upstream has no single entry point for this: it calls triton_rms_norm_backward
    (linghe/utils/norm.py:144) and triton_blockwise_quant (linghe/quant/block.py:129)
    separately.  Returns (dx, dw, dy_q [M,n], dy_scale [n/128,M], dyT_q [n,M],
    dyT_scale [ceil(M/128),n])."""
    assert grad_output.is_contiguous() and x.is_contiguous()
    M, n = _rows_cols(x)
    assert n <= 8192 and M % 16 == 0
    device = x.device
    nbytes = _lib.scratch_bytes("rmsnorm_bwd_blockquant", M, n)
    dx, dw, dy_q, dy_s, dyt_q, dyt_s, scratch = _lib.empties(
        x, (tuple(x.shape), x.dtype), ((n,), torch.float32), ((M, n), E4M3), ((n // 128, M), torch.float32),
        ((n, M), E4M3), (((M + 127) // 128, n), torch.float32), ((nbytes,), torch.uint8))
    _lib.call("lh_rmsnorm_bwd_blockquant", x, _lib.ptr(grad_output), _lib.ptr(x), _lib.ptr(w), _lib.ptr(rms),
              _lib.dtype_code(x), M, n, float(eps), _lib.ptr(dx), _lib.ptr(dw), _lib.ptr(dy_q), _lib.ptr(dy_s),
              _lib.ptr(dyt_q), _lib.ptr(dyt_s), int(bool(round_scale)), _lib.ptr(scratch), nbytes)
    return dx, dw, dy_q, dy_s, dyt_q, dyt_s


def triton_rms_norm_and_smooth_quant_forward(
    x,
    weight,
    smooth_scale=None,
    eps=1e-6,
    out=None,
    scale=None,
    rms=None,
    calibrate=False,
    output_rms=False,
    round_scale=False,
):
    """RMSNorm + smooth quantisation (linghe/utils/norm.py:557): y = RMSNorm(x) * weight is divided
    by the per-column `smooth_scale` and quantised with ONE scale per row.

    Returns (out e4m3 [M,N], scale f32 [M], maxs f32 [N] or None, rms f32 [M] or None): `maxs`
    (column maxima of |y| before smoothing) only with calibrate=True, `rms` (1/rms per row) only
    with output_rms=True or when a buffer is passed."""
    assert x.is_contiguous() and weight.is_contiguous()
    assert smooth_scale is not None and smooth_scale.is_contiguous()
    M, N = x.shape
    assert N <= 8192 and N % 8 == 0
    device = x.device
    if smooth_scale.dtype != torch.float32:
        smooth_scale = smooth_scale.float()
    if out is None:
        out = torch.empty((M, N), device=device, dtype=E4M3)
    if scale is None:
        scale = torch.empty((M,), device=device, dtype=torch.float32)
    if output_rms and rms is None:
        rms = torch.empty((M,), dtype=torch.float32, device=device)
    maxs = scratch = None
    nbytes = 0
    if calibrate:
        maxs = torch.empty((N,), dtype=torch.float32, device=device)
        nbytes = _lib.scratch_bytes("smooth_quant", M, N)
        scratch = torch.empty((nbytes,), dtype=torch.uint8, device=device)
    _lib.call("lh_rmsnorm_smoothquant_fwd", x, _lib.ptr(x), _lib.ptr(weight), _lib.ptr(smooth_scale), _lib.dtype_code(x),
              M, N, float(eps), _lib.ptr(out), _lib.ptr(scale), _lib.ptr(rms) if output_rms else 0, _lib.ptr(maxs),
              _lib.ptr(scratch), nbytes, int(bool(round_scale)))
    return out, scale, maxs, rms
