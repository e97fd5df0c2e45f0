"""Row-wise 1x128 group quantiser -- same entry point as linghe/quant/group.py."""

from __future__ import annotations

import torch

from linghe_b200 import _lib


def triton_group_quant(x, dtype=torch.float8_e4m3fn, group_size=128, round_scale=False):
    """1x128 groups along rows (linghe/quant/group.py:40).

    Returns (y e4m3 [M,N], s float32 [M, N/128]) -- scales are NOT transposed here."""
    M, N = x.shape
    assert group_size == 128 and dtype == torch.float8_e4m3fn
    assert N % group_size == 0
    assert x.is_contiguous()
    y, s = _lib.empties(x, ((M, N), dtype), ((M, N // group_size), torch.float32))
    _lib.call("lh_group_quant", x, _lib.ptr(x), _lib.dtype_code(x), M, N, _lib.ptr(y), _lib.ptr(s),
              int(bool(round_scale)))
    return y, s
