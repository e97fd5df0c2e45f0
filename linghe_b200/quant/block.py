"""Blockwise FP8 quantisers -- same entry points as linghe/quant/block.py, running
hand-written sm_100a CUDA (csrc/lh_tile.cu) through the C ABI."""

from __future__ import annotations

import torch

from linghe_b200 import _lib

E4M3 = torch.float8_e4m3fn


def _cdiv(a, b):
    return (a + b - 1) // b


def triton_block_quant(x, block_size=128, round_scale=False):
    """128x128 2-D block quantisation of a weight matrix (linghe/quant/block.py:32).

    Returns (y e4m3 [M,N], s float32 [M/128, N/128])."""
    assert x.is_contiguous()
    assert block_size == 128, "only 128x128 blocks are implemented"
    M, N = x.size()
    y, s = _lib.empties(x, ((M, N), E4M3), ((M // block_size, N // block_size), torch.float32))
    _lib.call("lh_block_quant", x, _lib.ptr(x), _lib.dtype_code(x), M, N, _lib.ptr(y), _lib.ptr(s),
              int(bool(round_scale)))
    return y, s


def triton_blockwise_quant(x, round_scale=False, output_mode=2):
    """Dual-axis activation quantisation, 1x128 rows and 128x1 columns
    (linghe/quant/block.py:129).

    Returns (x_q [M,N], x_scale [N/128,M], xt_q [N,M], xt_scale [ceil(M/128),N]); all four
    are allocated, the ones `output_mode` (0 rows / 1 columns / 2 both) skips stay
    uninitialised, as upstream."""
    M, N = x.shape
    assert M % 16 == 0 and x.is_contiguous()
    x_q, x_scale, xt_q, xt_scale = _lib.empties(x, ((M, N), E4M3), ((N // 128, M), torch.float32), ((N, M), E4M3),
                                               ((_cdiv(M, 128), N), torch.float32))
    _lib.call("lh_blockwise_quant", x, _lib.ptr(x), _lib.dtype_code(x), M, N, _lib.ptr(x_q),
              _lib.ptr(x_scale), _lib.ptr(xt_q), _lib.ptr(xt_scale), int(bool(round_scale)), int(output_mode))
    return x_q, x_scale, xt_q, xt_scale


def triton_batch_blockwise_quant(xs, token_count_per_expert, splits, round_scale=False):
    """Per-expert dual-axis quantisation with flat packed outputs
    (linghe/quant/block.py:251).  `splits` (host list) only sizes the outputs."""
    assert xs.is_contiguous()
    M, N = xs.shape
    n_experts = token_count_per_expert.size(0)
    device = xs.device
    blocks = sum([(int(c) + 127) // 128 for c in splits])
    x_q, x_scale, xt_q, xt_scale = _lib.empties(xs, ((M, N), E4M3), ((M * N // 128,), torch.float32), ((M * N,), E4M3),
                                               ((blocks * N,), torch.float32))
    if M == 0:
        return x_q, x_scale, xt_q, xt_scale
    assert token_count_per_expert.is_cuda and token_count_per_expert.is_contiguous()
    _lib.call("lh_batch_blockwise_quant", xs, _lib.ptr(xs), _lib.dtype_code(xs),
              _lib.ptr(token_count_per_expert), _lib.itype_code(token_count_per_expert), n_experts, M, N,
              _lib.ptr(x_q), _lib.ptr(x_scale), _lib.ptr(xt_q), _lib.ptr(xt_scale), int(bool(round_scale)))
    return x_q, x_scale, xt_q, xt_scale
