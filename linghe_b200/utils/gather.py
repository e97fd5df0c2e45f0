"""Permute + pad + blockwise quantisation for routed experts -- the entry point of
linghe/utils/gather.py that feeds the per-expert SwiGLU path, on hand-written sm_100a
CUDA through the C ABI."""

from __future__ import annotations

import torch

from linghe_b200 import _lib

E4M3 = torch.float8_e4m3fn


def triton_batch_block_pad_permute_with_indices(xs, token_count_per_expert, indices, splits, probs=None,
                                                round_scale=False):
    """Gather token rows per expert, pad every expert to a multiple of 16 rows and quantise
    on both axes (linghe/utils/gather.py:1049).

    xs [m, N]; token_count_per_expert [E] (device); indices [M] = source row of every padded
    output position, M = sum of the counts rounded up to 16; splits = the counts as a host
    list (sizes the outputs); probs optional [m, E].
    Returns (x_q [M,N], x_scale buffer (M, N/128) packed per expert as [N/128, padded c],
    xt_q buffer (M,N) packed per expert as [N, padded c], xt_scale [sum ceil(c/128), N],
    prob_output [M] or None)."""
    assert xs.is_contiguous()
    m, N = xs.shape
    assert N % 128 == 0
    n_experts = token_count_per_expert.size(0)
    M = indices.shape[0]
    device = xs.device
    blocks = sum([(int(c) + 127) // 128 for c in splits])
    specs = [((M, N), E4M3), ((M, N // 128), torch.float32), ((M, N), E4M3), ((blocks, N), torch.float32)]
    if probs is not None:
        specs.append(((M,), probs.dtype))
    outs = _lib.empties(xs, *specs)
    x_q, x_scale, xt_q, xt_scale = outs[:4]
    prob_output = outs[4] if probs is not None else None
    if m == 0:
        return x_q, x_scale, xt_q, xt_scale, prob_output
    assert indices.is_contiguous() and token_count_per_expert.is_contiguous()
    if probs is not None:
        assert probs.is_contiguous() and probs.shape == (m, n_experts)
    _lib.call("lh_batch_block_pad_permute", xs, _lib.ptr(xs), _lib.dtype_code(xs), _lib.ptr(probs),
              _lib.dtype_code(probs) if probs is not None else _lib.F32, _lib.ptr(indices), _lib.itype_code(indices),
              _lib.ptr(token_count_per_expert), _lib.itype_code(token_count_per_expert), n_experts, m, M, N,
              _lib.ptr(x_q), _lib.ptr(x_scale), _lib.ptr(xt_q), _lib.ptr(xt_scale), _lib.ptr(prob_output),
              int(bool(round_scale)))
    return x_q, x_scale, xt_q, xt_scale, prob_output


def triton_make_row_id_map_and_index(routing_map: torch.Tensor, num_out_tokens: int, multiple_of: int = 1):
    """Destination rows of a routing map with per-expert padding (linghe/utils/gather.py:161).

    routing_map [n_tokens, n_experts] (bool / uint8 / int32); num_out_tokens = sum over experts
    of the token count rounded up to `multiple_of`.
    Returns (row_id_map [n_tokens, n_experts] int32: row of the token in the permuted output or
    -1; row_indices [num_out_tokens] int32: source token of every output row, 0 in padding rows)."""
    assert routing_map.is_contiguous()
    n_tokens, n_experts = routing_map.shape
    device = routing_map.device
    if routing_map.dtype in (torch.bool, torch.uint8, torch.int8):
        is_i32 = 0
    else:
        assert routing_map.dtype == torch.int32, f"unsupported routing map dtype {routing_map.dtype}"
        is_i32 = 1
    row_id_map = torch.empty((n_tokens, n_experts), dtype=torch.int32, device=device)
    row_id_indices = torch.zeros((num_out_tokens,), dtype=torch.int32, device=device)
    if n_tokens == 0:
        return row_id_map, row_id_indices
    nbytes = _lib.scratch_bytes("row_id_map", n_tokens, n_experts)
    scratch = torch.empty((nbytes,), dtype=torch.uint8, device=device)
    _lib.call("lh_make_row_id_map_and_index", routing_map, _lib.ptr(routing_map), is_i32, n_tokens, n_experts,
              int(multiple_of), _lib.ptr(row_id_map), _lib.ptr(row_id_indices), _lib.ptr(scratch), nbytes)
    return row_id_map, row_id_indices
