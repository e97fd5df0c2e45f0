"""ctypes binding of the C ABI declared in include/linghe_b200.h.

The shared library is built in-tree by ``python -m linghe_b200.build``.  Loading fails
loudly when it is missing: there is no CPU or PyTorch fallback behind these entry points.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("LINGHE_B200_LIB", os.path.join(_HERE, "lib", "liblinghe_b200.so"))

LH_ERR_ARG = -1
BF16, F16, F32 = 0, 1, 2
I32, I64 = 0, 1

_DTYPES = {torch.bfloat16: BF16, torch.float16: F16, torch.float32: F32}
_ITYPES = {torch.int32: I32, torch.int64: I64}

_p = ctypes.c_void_p
_i = ctypes.c_int
_l = ctypes.c_int64
_f = ctypes.c_float

# name -> (restype, argtypes); mirrors include/linghe_b200.h one to one
SIGNATURES = {
    "lh_version": (_i, []),
    "lh_last_error": (ctypes.c_char_p, []),
    "lh_device_check": (_i, [_i]),
    "lh_device_status": (_i, [ctypes.POINTER(_i)]),
    "lh_selftest_wait_timeout": (_i, [_i, _p]),
    "lh_tuning": (_i, [ctypes.c_char_p, _i]),
    "lh_scratch_bytes": (_l, [ctypes.c_char_p, _l, _l]),
    "lh_blockwise_quant": (_i, [_p, _i, _l, _l, _p, _p, _p, _p, _i, _i, _p]),
    "lh_group_quant": (_i, [_p, _i, _l, _l, _p, _p, _i, _p]),
    "lh_block_quant": (_i, [_p, _i, _l, _l, _p, _p, _i, _p]),
    "lh_batch_blockwise_quant": (_i, [_p, _i, _p, _i, _i, _l, _l, _p, _p, _p, _p, _i, _p]),
    "lh_batch_block_pad_permute": (_i, [_p, _i, _p, _i, _p, _i, _p, _i, _i, _l, _l, _l, _p, _p, _p, _p, _p, _i, _p]),
    "lh_rmsnorm_fwd": (_i, [_p, _p, _i, _l, _l, _f, _p, _p, _i, _p]),
    "lh_rmsnorm_blockquant_fwd": (_i, [_p, _p, _i, _l, _l, _f, _p, _p, _p, _p, _p, _i, _i, _p]),
    "lh_rmsnorm_gemm_blockquant_fwd": (_i, [_p, _p, _p, _i, _l, _l, _l, _f, _p, _p, _p, _p, _p, _p, _p, _i, _i, _p, _l, _p]),
    "lh_make_row_id_map_and_index": (_i, [_p, _i, _l, _l, _i, _p, _p, _p, _l, _p]),
    "lh_unpermute_with_mask_map": (_i, [_p, _i, _p, _p, _i, _l, _l, _l, _p, _p, _p]),
    "lh_fp8_gemm": (_i, [_p, _p, _p, _p, _p, _l, _l, _l, _i, _i, _i, _i, _p]),
    "lh_fp8_gemm_bb": (_i, [_p, _p, _p, _p, _p, _l, _l, _l, _i, _i, _p]),
    "lh_rmsnorm_smoothquant_fwd": (_i, [_p, _p, _p, _i, _l, _l, _f, _p, _p, _p, _p, _p, _l, _i, _p]),
    "lh_silu_smoothquant_fwd": (_i, [_p, _p, _i, _l, _l, _p, _p, _p, _p, _l, _i, _p]),
    "lh_silu_smoothquant_bwd": (_i, [_p, _p, _p, _p, _i, _l, _l, _p, _p, _p, _p, _p, _l, _i, _i, _p]),
    "lh_batch_silu_smoothquant_bwd": (_i, [_p, _p, _p, _i, _i, _p, _p, _p, _i, _i, _l, _l, _l, _p, _p, _p, _p, _p, _i, _i, _p]),
    "lh_batch_silu_smoothquant_fwd": (_i, [_p, _p, _i, _i, _p, _p, _i, _i, _l, _l, _p, _p, _p, _i, _i, _p]),
    "lh_rmsnorm_bwd": (_i, [_p, _p, _p, _p, _i, _l, _l, _f, _p, _p, _p, _l, _p]),
    "lh_rmsnorm_bwd_static": (_i, [_p, _p, _p, _p, _i, _l, _l, _f, _p, _p, _p]),
    "lh_rmsnorm_bwd_blockquant": (_i, [_p, _p, _p, _p, _i, _l, _l, _f, _p, _p, _p, _p, _p, _p, _i, _p, _l, _p]),
    "lh_weighted_silu_fwd": (_i, [_p, _p, _i, _i, _l, _l, _p, _p]),
    "lh_weighted_silu_bwd": (_i, [_p, _p, _p, _i, _i, _l, _l, _p, _p, _p]),
    "lh_silu_blockquant_fwd": (_i, [_p, _i, _l, _l, _p, _p, _p, _p, _i, _i, _p]),
    "lh_silu_blockquant_bwd": (_i, [_p, _p, _i, _l, _l, _p, _p, _p, _p, _p, _i, _p]),
    "lh_batch_silu_blockquant_fwd": (_i, [_p, _p, _i, _i, _p, _i, _i, _l, _l, _p, _p, _p, _p, _i, _i, _p]),
    "lh_batch_silu_blockquant_bwd": (_i, [_p, _p, _p, _i, _i, _p, _i, _i, _l, _l, _p, _p, _p, _p, _p, _i, _p, _l, _p]),
}

_lock = threading.Lock()
_lib = None
_checked_devices = set()


def load() -> ctypes.CDLL:
    """Load (once) and return the shared library with argument types declared."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"linghe_b200: CUDA library not found at {LIB_PATH}. Build it with "
                "`python -m linghe_b200.build` (needs nvcc; targets sm_100a only). "
                "There is no CPU fallback.")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the header and the build disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


_host = False


def host():
    """The C++ argument handling of the hottest wrappers (host/lh_host.cpp), or None when it was
    not built; the callers then take the ctypes path to the same entry points."""
    global _host
    if _host is False:
        load()
        path = os.path.join(os.path.dirname(LIB_PATH), "_lh_host.so")
        mod = None
        if os.path.exists(path) and os.environ.get("LINGHE_B200_NO_HOST_MODULE") is None:
            try:
                import importlib.util
                spec = importlib.util.spec_from_file_location("_lh_host", path)
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
            except Exception:  # noqa: BLE001 -- optional accelerator of the host side only
                mod = None
        _host = mod
    return _host


_DT_CODE = {torch.float8_e4m3fn: 0, torch.float32: 1, torch.bfloat16: 2, torch.float16: 3, torch.uint8: 4,
            torch.int32: 5, torch.int64: 6}


def empties(ref: torch.Tensor, *specs):
    """Uninitialised tensors on the device of `ref`, one per (shape, dtype) in `specs`.  With the
    host module they come from ONE call into C++ (a torch.empty from Python costs about 2.4 us, which
    for the four or five outputs of a wrapper is more than a small kernel takes)."""
    h = host()
    if h is not None:
        return h.empty_many(ref, [(shape, _DT_CODE[dt]) for shape, dt in specs])
    dev = ref.device
    return [torch.empty(shape, device=dev, dtype=dt) for shape, dt in specs]


def last_error() -> str:
    return load().lh_last_error().decode()


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise AssertionError(f"unsupported dtype {t.dtype}") from None


def itype_code(t: torch.Tensor) -> int:
    try:
        return _ITYPES[t.dtype]
    except KeyError:
        raise AssertionError(f"counts must be int32 or int64, got {t.dtype}") from None


def ptr(t):
    """device address of a tensor, 0 for None (a NULL pointer at the C ABI)"""
    return 0 if t is None else t.data_ptr()


def _check_device(idx: int):
    rc = load().lh_device_check(idx)
    if rc != 0:
        raise RuntimeError(f"linghe_b200: {last_error()}")
    _checked_devices.add(idx)


_fn_cache = {}
# raw cudaStream_t of torch's current stream on a device, without building a Stream object
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_of(idx: int) -> int:
    if _raw_stream is not None:
        return _raw_stream(idx)
    return torch.cuda.current_stream(idx).cuda_stream


def call(name: str, ref: torch.Tensor, *args):
    """Invoke entry point `name` on the device and current stream of tensor `ref`.

    Argument errors raise AssertionError (the upstream wrappers use bare asserts);
    CUDA launch errors raise RuntimeError.  The host cost of a call is part of the
    product (a training step is not graph-captured), so the common case -- tensor on the
    current device -- takes no context manager and builds no stream object."""
    dev = ref.device
    if dev.type != "cuda":
        raise RuntimeError("linghe_b200 runs on CUDA tensors only (no CPU fallback)")
    fn = _fn_cache.get(name)
    if fn is None:
        # the generated pybind11 binding of the same C function when the host module is there
        # (about 1 us per call), the ctypes one otherwise (about 4 us)
        h = host()
        fn = _fn_cache[name] = getattr(h, name, None) if h is not None else None
        if fn is None:
            fn = _fn_cache[name] = getattr(load(), name)
    idx = dev.index
    if idx not in _checked_devices:
        _check_device(idx)
    if idx == torch.cuda.current_device():
        rc = fn(*args, _stream_of(idx))
    else:
        with torch.cuda.device(idx):
            rc = fn(*args, _stream_of(idx))
    if rc == 0:
        return
    msg = load().lh_last_error().decode()
    if rc == LH_ERR_ARG:
        raise AssertionError(msg)
    raise RuntimeError(f"linghe_b200 {name}: CUDA error {rc}: {msg}")


def scratch_bytes(what: str, rows: int, cols: int) -> int:
    h = host()
    v = h.lh_scratch_bytes(what, rows, cols) if h is not None else load().lh_scratch_bytes(what.encode(), rows, cols)
    if v < 0:
        raise RuntimeError(f"unknown scratch kind {what}")
    return v


def device_status(device=None) -> int:
    """Read-and-clear the device status word (synchronises).  0 = no kernel gave up a wait."""
    out = ctypes.c_int(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        rc = load().lh_device_status(ctypes.byref(out))
    if rc != 0:
        raise RuntimeError(last_error())
    return out.value
