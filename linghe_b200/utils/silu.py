"""SwiGLU kernels -- same entry points as linghe/utils/silu.py (plain, block-quant and
per-expert batched block-quant variants), running hand-written sm_100a CUDA through the
C ABI."""

from __future__ import annotations

from typing import Optional

import torch

from linghe_b200 import _lib

E4M3 = torch.float8_e4m3fn


def _cdiv(a, b):
    return (a + b - 1) // b


def triton_weighted_silu_forward(x, weight=None, out=None, asm=False):
    """y = silu(x1) * x2 [* weight] in x.dtype (linghe/utils/silu.py:98).  `asm` selected an
    approximate-exp kernel upstream; here it is accepted and ignored."""
    assert x.is_contiguous()
    M, N = x.shape
    assert N % 256 == 0
    if out is None:
        out = torch.empty((M, N // 2), device=x.device, dtype=x.dtype)
    if weight is not None:
        assert weight.is_contiguous()
    _lib.call("lh_weighted_silu_fwd", x, _lib.ptr(x), _lib.ptr(weight), _lib.dtype_code(x),
              _lib.dtype_code(weight) if weight is not None else _lib.F32, M, N // 2, _lib.ptr(out))
    return out


def triton_weighted_silu_backward(g: torch.Tensor, x: torch.Tensor, weight: Optional[torch.Tensor] = None):
    """Backward of triton_weighted_silu_forward (linghe/utils/silu.py:177).
    Returns (dx [M,2n] x.dtype, dw like weight or None)."""
    assert g.is_contiguous() and x.is_contiguous()
    M, N = x.shape
    assert N % 256 == 0
    dw = None
    if weight is not None:
        assert weight.is_contiguous()
        dx, dw = _lib.empties(x, ((M, N), x.dtype), (tuple(weight.shape), weight.dtype))
    else:
        dx = torch.empty((M, N), device=x.device, dtype=x.dtype)
    _lib.call("lh_weighted_silu_bwd", x, _lib.ptr(g), _lib.ptr(x), _lib.ptr(weight), _lib.dtype_code(x),
              _lib.dtype_code(weight) if weight is not None else _lib.F32, M, N // 2, _lib.ptr(dx), _lib.ptr(dw))
    return dx, dw


def triton_silu_and_block_quant_forward(x, out=None, scale=None, round_scale=False, output_mode=2):
    """Fused SwiGLU + blockwise quantisation (linghe/utils/silu.py:279).
    Returns (out [M,n], scale [n/128,M], transpose_output [n,M], transpose_scale
    [ceil(M/128),n]); outputs a mode skips stay uninitialised."""
    h = _lib.host()
    if h is not None:   # the same steps in C++ (host/lh_host.cpp): a third of the host time
        return h.silu_and_block_quant_forward(x, out, scale, bool(round_scale), output_mode)
    assert x.is_contiguous()
    M, N = x.shape
    n = N // 2
    device = x.device
    # upstream tiles the width by 128 columns, by 64 when only the transposed pair is written
    # (linghe/utils/silu.py:311-317)
    assert n % (64 if output_mode == 1 else 128) == 0
    if out is None:
        out = torch.empty((M, n), device=device, dtype=E4M3)
    if scale is None:
        scale = torch.empty((n // 128, M), device=device, dtype=torch.float32)
    transpose_output = transpose_scale = None
    if output_mode != 0:
        transpose_output = torch.empty((n, M), device=device, dtype=E4M3)
        transpose_scale = torch.empty((_cdiv(M, 128), n), device=device, dtype=torch.float32)
    _lib.call("lh_silu_blockquant_fwd", x, _lib.ptr(x), _lib.dtype_code(x), M, n, _lib.ptr(out), _lib.ptr(scale),
              _lib.ptr(transpose_output), _lib.ptr(transpose_scale), int(bool(round_scale)), int(output_mode))
    if transpose_output is None:
        # mode 0 does not write the transposed pair; upstream still returns it (uninitialised), so it is
        # allocated here, after the launch, where the allocator no longer delays the kernel
        transpose_output = torch.empty((n, M), device=device, dtype=E4M3)
        transpose_scale = torch.empty((_cdiv(M, 128), n), device=device, dtype=torch.float32)
    return out, scale, transpose_output, transpose_scale


def triton_silu_and_block_quant_backward(g, x, round_scale=False, return_bf16=False):
    """Backward of triton_silu_and_block_quant_forward (linghe/utils/silu.py:424).
    Returns (dx e4m3 [M,2n], dx_scale [2n/128,M], transpose_dx [2n,M], transpose_dx_scale
    [M/128,2n]).  With return_bf16=True a fifth element, dx in x.dtype [M,2n], is emitted
    by the same kernel (upstream needs a separate triton_weighted_silu_backward pass)."""
    assert g.is_contiguous() and x.is_contiguous()
    M, N = x.shape
    n = N // 2
    device = x.device
    assert M % 128 == 0 and N % 256 == 0
    specs = [((M, N), E4M3), ((N // 128, M), torch.float32), ((N, M), E4M3), ((_cdiv(M, 128), N), torch.float32)]
    if return_bf16:
        specs.append(((M, N), x.dtype))
    outs = _lib.empties(x, *specs)
    dx, dx_scale, transpose_dx, transpose_dx_scale = outs[:4]
    dx_hp = outs[4] if return_bf16 else None
    _lib.call("lh_silu_blockquant_bwd", x, _lib.ptr(g), _lib.ptr(x), _lib.dtype_code(x), M, n, _lib.ptr(dx),
              _lib.ptr(dx_scale), _lib.ptr(transpose_dx), _lib.ptr(transpose_dx_scale), _lib.ptr(dx_hp),
              int(bool(round_scale)))
    if return_bf16:
        return dx, dx_scale, transpose_dx, transpose_dx_scale, dx_hp
    return dx, dx_scale, transpose_dx, transpose_dx_scale


def triton_batch_weighted_silu_and_block_quant_forward(
    x, weight, counts, splits=None, out=None, scale=None, round_scale=False, output_mode=2
):
    """Per-expert weighted SwiGLU + blockwise quantisation for routed experts
    (linghe/utils/silu.py:797).  `counts` is the device tensor of rows per expert,
    `splits` the same as a host list (only used to size outputs).  Outputs use the
    per-expert packed layouts documented in include/linghe_b200.h."""
    assert splits is not None, "batch mode need splits to launch kernels"
    assert x.is_contiguous() and weight.is_contiguous()
    M, N = x.shape
    n = N // 2
    n_experts = counts.shape[0]
    assert N <= 8192
    device = x.device
    if out is None:
        out = torch.empty((M, n), device=device, dtype=E4M3)
    if scale is None:
        scale = torch.empty((M, n // 128), device=device, dtype=torch.float32)
    blocks = sum([(int(c) + 127) // 128 for c in splits])
    transpose_output, transpose_scale = _lib.empties(x, ((M, n), E4M3), ((blocks, n), torch.float32))
    if M == 0:
        return out, scale, transpose_output, transpose_scale
    assert counts.is_cuda and counts.is_contiguous()
    _lib.call("lh_batch_silu_blockquant_fwd", x, _lib.ptr(x), _lib.ptr(weight), _lib.dtype_code(x),
              _lib.dtype_code(weight), _lib.ptr(counts), _lib.itype_code(counts), n_experts, M, n, _lib.ptr(out),
              _lib.ptr(scale), _lib.ptr(transpose_output), _lib.ptr(transpose_scale), int(bool(round_scale)),
              int(output_mode))
    return out, scale, transpose_output, transpose_scale


def triton_batch_weighted_silu_and_block_quant_backward(g, x, weight, counts, splits=None, round_scale=False):
    """Backward of the per-expert forward (linghe/utils/silu.py:1293).  Returns
    (dx e4m3 [R,2n], dx_scale, dw like weight, transpose_dx, transpose_dx_scale)."""
    M, N = x.shape
    n = N // 2
    n_expert = counts.shape[0]
    assert n % 128 == 0
    assert g.is_contiguous() and x.is_contiguous() and weight.is_contiguous()
    assert splits is not None, "batch mode need splits to launch kernels"
    device = x.device
    s = sum([(int(c) + 127) // 128 for c in splits])
    nbytes = M * (n // 128) * 4          # lh_scratch_bytes("batch_silu_bwd", M, n): the per-block dw partials
    dx, dx_scale, transpose_dx, transpose_dx_scale, dw, scratch = _lib.empties(
        x, ((M, N), E4M3), ((M, N // 128), torch.float32), ((M, N), E4M3), ((s, N), torch.float32),
        (tuple(weight.shape), weight.dtype), ((nbytes,), torch.uint8))
    if s == 0:
        return dx, dx_scale, dw, transpose_dx, transpose_dx_scale
    assert counts.is_cuda and counts.is_contiguous()
    _lib.call("lh_batch_silu_blockquant_bwd", x, _lib.ptr(g), _lib.ptr(x), _lib.ptr(weight), _lib.dtype_code(x),
              _lib.dtype_code(weight), _lib.ptr(counts), _lib.itype_code(counts), n_expert, M, n, _lib.ptr(dx),
              _lib.ptr(dx_scale), _lib.ptr(dw), _lib.ptr(transpose_dx), _lib.ptr(transpose_dx_scale),
              int(bool(round_scale)), _lib.ptr(scratch), nbytes)
    return dx, dx_scale, dw, transpose_dx, transpose_dx_scale


def triton_silu_and_smooth_quant_forward(x, smooth_scale=None, out=None, scale=None, maxs=None, round_scale=False,
                                         calibrate=False):
    """SwiGLU + smooth quantisation (linghe/utils/silu.py:1498): y = silu(x1) * x2 is divided by
    the per-column `smooth_scale` and quantised with ONE scale per row.

    Returns (out e4m3 [M,n], scale f32 [M], maxs f32 [n] or None); `maxs` (column maxima of |y|
    before smoothing) only with calibrate=True."""
    assert x.is_contiguous()
    assert smooth_scale is not None and smooth_scale.is_contiguous()
    M, N = x.shape
    n = N // 2
    assert N % 16 == 0 and n <= 8192
    device = x.device
    if smooth_scale.dtype != torch.float32:
        smooth_scale = smooth_scale.float()
    if out is None:
        out = torch.empty((M, n), device=device, dtype=E4M3)
    if scale is None:
        scale = torch.empty((M,), device=device, dtype=torch.float32)
    scratch = None
    nbytes = 0
    cmax = None
    if calibrate:
        cmax = torch.empty((n,), dtype=torch.float32, device=device)
        nbytes = _lib.scratch_bytes("smooth_quant", M, n)
        scratch = torch.empty((nbytes,), dtype=torch.uint8, device=device)
    _lib.call("lh_silu_smoothquant_fwd", x, _lib.ptr(x), _lib.ptr(smooth_scale), _lib.dtype_code(x), M, n,
              _lib.ptr(out), _lib.ptr(scale), _lib.ptr(cmax), _lib.ptr(scratch), nbytes, int(bool(round_scale)))
    return out, scale, cmax


def triton_batch_weighted_silu_and_smooth_quant_forward(x, weight, counts, smooth_scale=None, splits=None, out=None,
                                                        scale=None, round_scale=False, reverse=False, calibrate=False):
    """Per-expert weighted SwiGLU + smooth quantisation (linghe/utils/silu.py:1821): rows grouped by
    expert (`counts[e]` rows each), expert e smoothed by `smooth_scale[e]` ([E, n]; multiplied when
    `reverse`), one scale per row.

    Returns (out e4m3 [M,n], scale f32 [M], maxs f32 [E,n] or None); `maxs` (per-expert column
    maxima of |silu(x1) * x2|, before the row weight) with calibrate=True, zeros when M == 0."""
    assert x.is_contiguous() and weight.is_contiguous()
    assert smooth_scale is not None and smooth_scale.is_contiguous()
    M, N = x.shape
    n = N // 2
    n_experts = counts.shape[0]
    assert N <= 16384 and N % 16 == 0
    assert smooth_scale.numel() == n_experts * n and weight.numel() == M
    device = x.device
    if smooth_scale.dtype != torch.float32:
        smooth_scale = smooth_scale.float()
    if out is None:
        out = torch.empty((M, n), device=device, dtype=E4M3)
    if scale is None:
        scale = torch.empty((M,), device=device, dtype=torch.float32)
    maxs = None
    if M == 0:
        return out, scale, torch.zeros((n_experts, n), device=device, dtype=torch.float32)
    if calibrate:
        maxs = torch.empty((n_experts, n), device=device, dtype=torch.float32)
    _lib.call("lh_batch_silu_smoothquant_fwd", x, _lib.ptr(x), _lib.ptr(weight), _lib.dtype_code(x), _lib.dtype_code(weight),
              _lib.ptr(smooth_scale), _lib.ptr(counts), _lib.itype_code(counts), n_experts, M, n, _lib.ptr(out),
              _lib.ptr(scale), _lib.ptr(maxs), int(bool(round_scale)), int(bool(reverse)))
    return out, scale, maxs


def triton_silu_and_smooth_quant_backward(g, x, smooth_scale=None, transpose_smooth_scale=None, reverse=True,
                                          round_scale=False):
    """SwiGLU backward + smooth quantisation on both axes (linghe/utils/silu.py:1705).

    dx = [dx1 | dx2] is smoothed by `smooth_scale` [2n] along the row (multiplied when `reverse`,
    else divided) and quantised with one scale per row; the transposed copy is smoothed by
    `transpose_smooth_scale` [M] and quantised with one scale per column of dx (over all rows).
    Returns (dx e4m3 [M,2n], dx_scale [M], transpose_dx e4m3 [2n,M], transpose_dx_scale [2n]).
    Upstream asserts `round_scale` (its requantisation pass needs power-of-two scales); here both
    settings work, the values being quantised once with the final column scale."""
    assert g.is_contiguous() and x.is_contiguous()
    assert smooth_scale is not None and transpose_smooth_scale is not None
    assert smooth_scale.is_contiguous() and transpose_smooth_scale.is_contiguous()
    M, N = x.shape
    n = N // 2
    assert N % 16 == 0 and n <= 4096
    assert smooth_scale.numel() == N and transpose_smooth_scale.numel() == M
    device = x.device
    if smooth_scale.dtype != torch.float32:
        smooth_scale = smooth_scale.float()
    if transpose_smooth_scale.dtype != torch.float32:
        transpose_smooth_scale = transpose_smooth_scale.float()
    dx = torch.empty((M, N), device=device, dtype=E4M3)
    dx_scale = torch.empty((M,), device=device, dtype=torch.float32)
    transpose_dx = torch.empty((N, M), device=device, dtype=E4M3)
    transpose_dx_scale = torch.empty((N,), device=device, dtype=torch.float32)
    nbytes = _lib.scratch_bytes("smooth_quant_bwd", M, n)
    scratch = torch.empty((nbytes,), dtype=torch.uint8, device=device)
    _lib.call("lh_silu_smoothquant_bwd", x, _lib.ptr(g), _lib.ptr(x), _lib.ptr(smooth_scale),
              _lib.ptr(transpose_smooth_scale), _lib.dtype_code(x), M, n, _lib.ptr(dx), _lib.ptr(dx_scale),
              _lib.ptr(transpose_dx), _lib.ptr(transpose_dx_scale), _lib.ptr(scratch), nbytes, int(bool(round_scale)),
              int(bool(reverse)))
    return dx, dx_scale, transpose_dx, transpose_dx_scale


def triton_batch_weighted_silu_and_smooth_quant_backward(g, x, weight, counts, smooth_scale=None,
                                                         transpose_smooth_scale=None, splits=None, reverse=True,
                                                         round_scale=False):
    """Per-expert weighted SwiGLU backward + smooth quantisation on both axes
    (linghe/utils/silu.py:2126).

    Returns (dx e4m3 [M,2n], dx_scale f32 [M], dw like weight, transpose_dx e4m3 flat
    [2n * sum_e pad32(splits[e])] -- expert e's [2n, pad32(c_e)] block after those before it, zero
    codes in the padding --, transpose_dx_scale f32 [E, 2n]).  `splits` (host list of the counts)
    sizes the flat buffer.  Upstream asserts `round_scale`; both settings work here."""
    assert g.is_contiguous() and x.is_contiguous() and weight.is_contiguous()
    assert smooth_scale is not None and transpose_smooth_scale is not None
    assert smooth_scale.is_contiguous() and transpose_smooth_scale.is_contiguous()
    assert splits is not None, "batch mode need splits to launch kernels"
    M, N = x.shape
    n = N // 2
    n_expert = counts.shape[0]
    assert N % 16 == 0 and n <= 4096
    assert smooth_scale.numel() == n_expert * N and transpose_smooth_scale.numel() == M and weight.numel() == M
    device = x.device
    if smooth_scale.dtype != torch.float32:
        smooth_scale = smooth_scale.float()
    if transpose_smooth_scale.dtype != torch.float32:
        transpose_smooth_scale = transpose_smooth_scale.float()
    dx = torch.empty((M, N), device=device, dtype=E4M3)
    dx_scale = torch.empty((M,), device=device, dtype=torch.float32)
    dw = torch.empty_like(weight)
    s = sum((int(c) + 31) // 32 for c in splits) * 32
    transpose_dx = torch.empty((N * s,), device=device, dtype=E4M3)
    transpose_dx_scale = torch.empty((n_expert, N), device=device, dtype=torch.float32)
    _lib.call("lh_batch_silu_smoothquant_bwd", x, _lib.ptr(g), _lib.ptr(x), _lib.ptr(weight), _lib.dtype_code(x),
              _lib.dtype_code(weight), _lib.ptr(smooth_scale), _lib.ptr(transpose_smooth_scale), _lib.ptr(counts),
              _lib.itype_code(counts), n_expert, M, n, s, _lib.ptr(dx), _lib.ptr(dx_scale), _lib.ptr(dw),
              _lib.ptr(transpose_dx), _lib.ptr(transpose_dx_scale), int(bool(round_scale)), int(bool(reverse)))
    return dx, dx_scale, dw, transpose_dx, transpose_dx_scale
