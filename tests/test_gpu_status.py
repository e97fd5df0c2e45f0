"""The give-up path of the kernels' bounded waits, exercised without making any production
kernel fail: a one-warp self-test kernel waits a few thousand polls on a barrier nobody
arrives at, records the status code and returns normally."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_timeout_sets_and_clears_status():
    from linghe_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.lh_selftest_wait_timeout(4096, stream) == 0
    torch.cuda.synchronize()                     # the kernel returned by itself
    assert _lib.device_status(0) == 1            # DEVERR_FULL_WAIT, recorded once
    assert _lib.device_status(0) == 0            # read-and-clear
    # the context is still usable and production kernels still run clean
    from linghe_b200.quant.group import triton_group_quant
    x = torch.randn((256, 256), device="cuda:0").to(torch.bfloat16)
    q, s = triton_group_quant(x)
    torch.cuda.synchronize()
    assert _lib.device_status(0) == 0
    assert lib.lh_selftest_wait_timeout(0, stream) == _lib.LH_ERR_ARG
