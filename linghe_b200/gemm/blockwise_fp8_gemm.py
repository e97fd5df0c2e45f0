"""Blockwise-scaled FP8 GEMM, mirror of linghe/gemm/blockwise_fp8_gemm.py.

`triton_tt_fp8_gemm` (linghe/gemm/blockwise_fp8_gemm.py:152) takes one scale per 1 x block run
along K on both operands -- the activations' wire format; `triton_bb_fp8_gemm`
(linghe/gemm/blockwise_fp8_gemm.py:59) one scale per block x block sub-matrix, the format of
`triton_block_quant`.  Both run the same tcgen05 kernel."""

import torch

from linghe_b200 import _lib

_OUT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def triton_tt_fp8_gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_s: torch.Tensor,
    b_s: torch.Tensor,
    out_dtype=torch.bfloat16,
    block_size=128,
    scales_transposed=False,
):
    """c = dequant(a) @ dequant(b).T for e4m3 `a` [..., K], `b` [N, K] with one float32 scale
    per 1 x block_size run along K: a_s [M, K/block_size], b_s [N, K/block_size] as upstream
    stores them.  With scales_transposed=True the scales are taken as the quantisers of this
    package write them ([K/block_size, M] and [K/block_size, N]), so the row-wise outputs of
    `triton_blockwise_quant` / `triton_rms_norm_and_block_quant_forward` feed it directly."""
    assert a.is_contiguous() and b.is_contiguous()
    assert a_s.is_contiguous() and b_s.is_contiguous()
    assert a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn
    assert a_s.dtype == torch.float32 and b_s.dtype == torch.float32
    assert out_dtype in _OUT
    K = a.size(-1)
    M = a.numel() // K
    N = b.size(0)
    assert b.size(1) == K and K % block_size == 0
    assert a_s.numel() == M * (K // block_size) and b_s.numel() == N * (K // block_size)
    c = torch.empty(*a.size()[:-1], N, dtype=out_dtype, device=a.device)
    t = int(bool(scales_transposed))
    _lib.call("lh_fp8_gemm", a, _lib.ptr(a), _lib.ptr(b), _lib.ptr(a_s), _lib.ptr(b_s), _lib.ptr(c), M, N, K,
              int(block_size), t, t, _OUT[out_dtype])
    return c


def triton_bb_fp8_gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_s: torch.Tensor,
    b_s: torch.Tensor,
    out_dtype=torch.bfloat16,
    block_size=128,
):
    """c = dequant(a) @ dequant(b).T for e4m3 `a` [..., K], `b` [N, K] with one float32 scale per
    block_size x block_size sub-matrix: a_s [ceil(M/block_size), K/block_size],
    b_s [ceil(N/block_size), K/block_size] (linghe/gemm/blockwise_fp8_gemm.py:59-97).  Returns
    c [M, N] as upstream does."""
    assert a.is_contiguous() and b.is_contiguous()
    assert a_s.is_contiguous() and b_s.is_contiguous()
    assert a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn
    assert a_s.dtype == torch.float32 and b_s.dtype == torch.float32
    assert out_dtype in _OUT
    K = a.size(-1)
    M = a.numel() // K
    N = b.size(0)
    assert b.size(1) == K and K % block_size == 0
    nb = K // block_size
    assert a_s.numel() == -(-M // block_size) * nb and b_s.numel() == -(-N // block_size) * nb
    c = torch.empty(M, N, dtype=out_dtype, device=a.device)
    _lib.call("lh_fp8_gemm_bb", a, _lib.ptr(a), _lib.ptr(b), _lib.ptr(a_s), _lib.ptr(b_s), _lib.ptr(c), M, N, K,
              int(block_size), _OUT[out_dtype])
    return c
