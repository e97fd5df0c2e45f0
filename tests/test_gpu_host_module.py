"""The two hottest wrappers have their argument handling in C++ (linghe_b200/host/lh_host.cpp)
with the Python/ctypes version behind it as the fallback of a failed host build.  Both are
product paths to the same entry points; they must return the same tensors, the same None
entries and raise the same exception types."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both_paths(fn):
    from linghe_b200 import _lib
    assert _lib.host() is not None, "host module was not built"
    fast = fn()
    saved = _lib._host
    _lib._host = None
    try:
        slow = fn()
    finally:
        _lib._host = saved
    return fast, slow


def _same(a, b):
    assert len(a) == len(b)
    for u, v in zip(a, b):
        assert (u is None) == (v is None)
        if u is not None:
            assert u.shape == v.shape and u.dtype == v.dtype and u.device == v.device


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,n", [(512, 2048), (130, 4096)])
def test_rms_wrapper_paths_agree(M, n, dtype):
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward as f
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((M, n), device="cuda", generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn((n,), device="cuda", generator=g)).to(dtype)
    for rs in (False, True):
        a, b = _both_paths(lambda: f(x, w, round_scale=rs, output_mode=0))
        _same(a, b)
        for i in (0, 1, 2):           # written outputs agree bit for bit; the transposed pair is unwritten in mode 0
            assert torch.equal(a[i].view(torch.uint8) if i == 0 else a[i], b[i].view(torch.uint8) if i == 0 else b[i])
        rms = a[2]
        a, b = _both_paths(lambda: f(x, w, rms=rms, round_scale=rs, output_mode=1))
        _same(a, b)
        assert a[0] is None and a[1] is None and a[2] is rms and b[2] is rms
        assert torch.equal(a[3].view(torch.uint8), b[3].view(torch.uint8)) and torch.equal(a[4], b[4])
        a, b = _both_paths(lambda: f(x, w, round_scale=rs, output_mode=2))
        _same(a, b)
        for i in range(5):
            assert torch.equal(a[i].view(torch.uint8) if a[i].dtype == torch.float8_e4m3fn else a[i],
                               b[i].view(torch.uint8) if b[i].dtype == torch.float8_e4m3fn else b[i])
    # caller-provided out / scale are written in place and returned
    out = torch.empty((M, n), device="cuda", dtype=torch.float8_e4m3fn)
    scale = torch.empty((n // 128, M), device="cuda", dtype=torch.float32)
    r = f(x, w, out=out, scale=scale, output_mode=0)
    assert r[0] is out and r[1] is scale


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,n", [(512, 1408), (130, 2048)])
def test_silu_wrapper_paths_agree(M, n, dtype):
    from linghe_b200.utils.silu import triton_silu_and_block_quant_forward as f
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn((M, 2 * n), device="cuda", generator=g).to(dtype)
    for mode in (0, 1, 2):
        a, b = _both_paths(lambda: f(x, round_scale=False, output_mode=mode))
        _same(a, b)
        written = {0: (0, 1), 1: (2, 3), 2: (0, 1, 2, 3)}[mode]
        for i in written:
            assert torch.equal(a[i].view(torch.uint8) if a[i].dtype == torch.float8_e4m3fn else a[i],
                               b[i].view(torch.uint8) if b[i].dtype == torch.float8_e4m3fn else b[i])
    with pytest.raises(AssertionError):
        f(x[:, : 2 * 200].contiguous(), output_mode=0)


def test_wrapper_uses_the_tensor_device_and_stream():
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward as f
    x = torch.randn((256, 1024), device="cuda").to(torch.bfloat16)
    w = torch.ones((1024,), device="cuda", dtype=torch.bfloat16)
    ref = f(x, w, output_mode=0)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        got = f(x, w, output_mode=0)
    s.synchronize()
    assert torch.equal(got[0].view(torch.uint8), ref[0].view(torch.uint8)) and torch.equal(got[1], ref[1])
