"""The C ABI without a GPU: the library builds and loads, exports every symbol the header
declares, the ctypes signature table matches the header, and argument validation rejects
bad sizes before anything is launched."""

import ctypes
import os
import re

from linghe_b200 import _lib
from linghe_b200 import build as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_decls():
    txt = open(os.path.join(ROOT, "include", "linghe_b200.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    decls = {}
    for m in re.finditer(r"(?:int|int64_t|const char\*)\s+(lh_\w+)\s*\(([^)]*)\)\s*;", txt):
        args = m.group(2).strip()
        n = 0 if args in ("", "void") else len(args.split(","))
        decls[m.group(1)] = n
    return decls


def test_library_builds_and_exports_header_symbols():
    # a real compile of every translation unit (not the stamp-matched prebuilt file), unless an
    # earlier test of this process already mapped the library
    path = B.build(force=_lib._lib is None)
    assert os.path.exists(path)
    lib = _lib.load()
    decls = _header_decls()
    assert len(decls) >= 19
    for name, nargs in decls.items():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} missing from the ctypes signature table"
        assert len(_lib.SIGNATURES[name][1]) == nargs, f"{name}: header has {nargs} args"
    for name in _lib.SIGNATURES:
        assert name in decls, f"{name} bound but not declared in the header"


def test_host_only_entry_points():
    lib = _lib.load()
    assert lib.lh_version() == 100
    assert _lib.scratch_bytes("rmsnorm_bwd", 16384, 4096) > 0
    assert _lib.scratch_bytes("batch_silu_bwd", 83328, 512) == 83328 * 4 * 4
    assert lib.lh_scratch_bytes(b"nope", 1, 1) < 0


def test_argument_validation_needs_no_gpu():
    lib = _lib.load()
    null = ctypes.c_void_p(0)
    rc = lib.lh_blockwise_quant(null, 0, 128, 100, null, null, null, null, 0, 2, null)
    assert rc == _lib.LH_ERR_ARG and b"128" in lib.lh_last_error()
    rc = lib.lh_blockwise_quant(null, 0, 128, 128, null, null, null, null, 0, 7, null)
    assert rc == _lib.LH_ERR_ARG
    rc = lib.lh_silu_blockquant_fwd(null, 3, 128, 128, null, null, null, null, 0, 0, null)
    assert rc == _lib.LH_ERR_ARG and b"dtype" in lib.lh_last_error()     # raw bytes are not a float type
    rc = lib.lh_silu_blockquant_fwd(null, 2, 128, 128, null, null, null, null, 0, 0, null)
    assert rc == _lib.LH_ERR_ARG and b"NULL" in lib.lh_last_error()      # float32 is accepted, NULL x is not
    rc = lib.lh_rmsnorm_blockquant_fwd(null, null, 0, 16, 16384, 1e-6, null, null, null, null, null, 0, 0, null)
    assert rc == _lib.LH_ERR_ARG


def test_no_cpu_fallback():
    import pytest
    import torch
    from linghe_b200.quant.block import triton_blockwise_quant
    with pytest.raises(RuntimeError):
        triton_blockwise_quant(torch.zeros((128, 128), dtype=torch.bfloat16))


def test_host_module_loads_and_has_no_cpu_fallback():
    # the C++ argument handling in front of the two hottest entry points (host/lh_host.cpp)
    import pytest
    import torch
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward
    from linghe_b200.utils.silu import triton_silu_and_block_quant_forward
    B.build()
    h = _lib.host()
    assert h is not None, "host module was not built"
    with pytest.raises(RuntimeError):
        triton_rms_norm_and_block_quant_forward(torch.zeros((128, 128), dtype=torch.bfloat16),
                                                torch.ones((128,), dtype=torch.bfloat16), output_mode=0)
    with pytest.raises(AssertionError):     # n % 128 in the row-wise modes, as upstream asserts
        triton_silu_and_block_quant_forward(torch.zeros((128, 200), dtype=torch.bfloat16), output_mode=0)
    with pytest.raises(AssertionError):     # rms is an output in mode 0
        triton_rms_norm_and_block_quant_forward(torch.zeros((128, 128), dtype=torch.bfloat16),
                                                torch.ones((128,), dtype=torch.bfloat16), rms=torch.zeros(128),
                                                output_mode=0)
