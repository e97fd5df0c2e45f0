"""lh_rmsnorm_bwd_static -- the RMSNorm backward for callers that cannot allocate.

Some users of the C ABI have no way to obtain scratch memory: a C/C++ host that lives
outside PyTorch's caching allocator, or a job whose pool already owns all free device
memory so that a raw cudaMalloc would fail (and cudaMalloc / cudaFree would stall the GPU
anyway).  For them the library carries its own dgamma scratch, a fixed device array of
148 x 8192 floats.  This test drives that entry point through the C ABI with raw pointers
and checks dx and dgamma against the scratch-taking lh_rmsnorm_bwd on two calls in a row;
the second call is smaller, so it runs on top of whatever the first left in the array.

Collected last on purpose: a run that stops at the first failure has by then run every
other test."""

import ctypes

import pytest
import torch

from linghe_b200 import _lib
from tests.common import assert_rel_close

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
BF16 = 0


def _inputs(M, n, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, n), generator=g).to(torch.bfloat16).to(DEV)
    gamma = (1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).to(DEV)
    dy = (0.01 * torch.randn((M, n), generator=g)).to(torch.bfloat16).to(DEV)
    return x, gamma, dy


def _call_pair(lib, M, n, seed):
    x, gamma, dy = _inputs(M, n, seed)
    stream = torch.cuda.current_stream().cuda_stream
    nbytes = _lib.scratch_bytes("rmsnorm_bwd", M, n)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    dx_ref = torch.empty_like(x)
    dg_ref = torch.empty(n, dtype=torch.float32, device=DEV)
    rc = lib.lh_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), None, BF16, M, n, 1e-6,
                            dx_ref.data_ptr(), dg_ref.data_ptr(), scratch.data_ptr(), nbytes, stream)
    assert rc == 0, lib.lh_last_error()
    dx = torch.full_like(x, float("nan"))
    dg = torch.full((n,), float("nan"), dtype=torch.float32, device=DEV)
    before = torch.cuda.memory_allocated()
    rc = lib.lh_rmsnorm_bwd_static(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), None, BF16, M, n, 1e-6,
                                   dx.data_ptr(), dg.data_ptr(), stream)
    assert rc == 0, lib.lh_last_error()
    assert torch.cuda.memory_allocated() == before   # nothing came from torch's allocator either
    torch.cuda.synchronize()
    assert_rel_close(dx, dx_ref, f"dx M={M} n={n}", 1e-2)
    assert_rel_close(dg, dg_ref, f"dgamma M={M} n={n}", 1e-3, 1e-5)
    return dx, dx_ref, dg, dg_ref


def test_static_scratch_matches_scratch_taking_entry_point():
    lib = _lib.load()
    torch.cuda.set_device(0)
    # the first call on the device also resolves the array's address: no capture is active
    _call_pair(lib, 4096, 4096, 1)
    # second call in a row, fewer CTAs and narrower rows: runs over the first call's leftovers
    _call_pair(lib, 300, 1536, 2)
    # widest supported row, and 1/rms handed in instead of recomputed
    x, gamma, dy = _inputs(520, 8192, 3)
    r = torch.rsqrt(x.float().pow(2).mean(1) + 1e-6).contiguous()
    stream = torch.cuda.current_stream().cuda_stream
    nbytes = _lib.scratch_bytes("rmsnorm_bwd", 520, 8192)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    outs = []
    for static in (False, True):
        dx = torch.empty_like(x)
        dg = torch.empty(8192, dtype=torch.float32, device=DEV)
        if static:
            rc = lib.lh_rmsnorm_bwd_static(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), r.data_ptr(), BF16, 520,
                                           8192, 1e-6, dx.data_ptr(), dg.data_ptr(), stream)
        else:
            rc = lib.lh_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), r.data_ptr(), BF16, 520, 8192,
                                    1e-6, dx.data_ptr(), dg.data_ptr(), scratch.data_ptr(), nbytes, stream)
        assert rc == 0, lib.lh_last_error()
        outs.append((dx, dg))
    torch.cuda.synchronize()
    assert_rel_close(outs[1][0], outs[0][0], "dx with given rms", 1e-2)
    assert_rel_close(outs[1][1], outs[0][1], "dgamma with given rms", 1e-3, 1e-5)
    assert _lib.device_status(0) == 0


def test_static_scratch_rejects_rows_wider_than_its_array():
    lib = _lib.load()
    null = ctypes.c_void_p(0)
    rc = lib.lh_rmsnorm_bwd_static(null, null, null, null, BF16, 128, 8192 + 128, 1e-6, null, null, null)
    assert rc == _lib.LH_ERR_ARG
    assert b"8192" in lib.lh_last_error()
