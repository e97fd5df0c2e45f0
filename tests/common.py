"""Shared helpers for the parity tests: golden-file access, bit views, and the
tolerance checks stated by the benchmark contract."""

import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# one e4m3 ulp of slack on at most this fraction of codes for fused variants
MAX_CODE_MISMATCH_FRAC = 1e-3
SCALE_RTOL = 1e-6
GRAD_RTOL = 1e-2


def golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def bf16(a):
    """uint16 raw bits -> bf16 tensor"""
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def fp8(a):
    """uint8 raw bits -> float8_e4m3fn tensor"""
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.float8_e4m3fn)


def bits(t):
    """raw bytes of an fp8 tensor as a flat uint8 cpu tensor"""
    return t.detach().contiguous().view(torch.uint8).cpu().reshape(-1)


def assert_bits_equal(got, ref, what):
    g, r = bits(got), bits(ref)
    assert g.numel() == r.numel(), f"{what}: size {g.numel()} vs {r.numel()}"
    bad = (g != r).sum().item()
    assert bad == 0, f"{what}: {bad} of {g.numel()} fp8 codes differ"


def assert_f32_equal(got, ref, what):
    g = got.detach().float().cpu().reshape(-1)
    r = ref.detach().float().cpu().reshape(-1)
    assert g.numel() == r.numel(), f"{what}: size {g.numel()} vs {r.numel()}"
    bad = (g.view(torch.int32) != r.view(torch.int32)).sum().item()
    assert bad == 0, f"{what}: {bad} of {g.numel()} float32 values differ bitwise"


def e4m3_ulp_distance(got, ref):
    """distance in e4m3 code steps between two code tensors (sign-magnitude order)."""
    g = bits(got).to(torch.int32)
    r = bits(ref).to(torch.int32)

    def order(c):
        mag = c & 0x7F
        return torch.where((c & 0x80) != 0, -mag, mag)

    return (order(g) - order(r)).abs()


def assert_codes_close(got, ref, what, frac=MAX_CODE_MISMATCH_FRAC):
    """fused-variant rule: at most `frac` of the codes differ, each by one e4m3 ulp."""
    d = e4m3_ulp_distance(got, ref)
    assert d.numel() > 0 or bits(ref).numel() == 0
    if d.numel() == 0:
        return 0.0
    assert d.max().item() <= 1, f"{what}: a code differs by {d.max().item()} ulps"
    f = (d != 0).float().mean().item()
    assert f <= frac, f"{what}: {f:.2e} of codes differ (limit {frac:.1e})"
    return f


def assert_scales_close(got, ref, what, rtol=SCALE_RTOL):
    g = got.detach().float().cpu().reshape(-1).double()
    r = ref.detach().float().cpu().reshape(-1).double()
    assert g.numel() == r.numel(), f"{what}: size {g.numel()} vs {r.numel()}"
    if g.numel() == 0:
        return 0.0
    rel = ((g - r).abs() / r.abs().clamp_min(1e-300)).max().item()
    assert rel <= rtol, f"{what}: max relative error {rel:.3e} > {rtol:.1e}"
    return rel


def assert_rel_close(got, ref, what, rtol, atol=0.0):
    """|got-ref| <= rtol*max|ref| + atol: relative to the tensor's scale, the sense
    in which 'bf16 gradients within 1e-2 relative' is checked."""
    g = got.detach().float().cpu().double()
    r = ref.detach().float().cpu().double()
    assert g.shape == r.shape, f"{what}: shape {tuple(g.shape)} vs {tuple(r.shape)}"
    if g.numel() == 0:
        return 0.0
    err = (g - r).abs()
    lim = rtol * r.abs() + atol + rtol * 1e-3 * r.abs().max()
    worst = (err - lim).max().item()
    assert worst <= 0, f"{what}: max abs err {err.max().item():.3e} exceeds rtol {rtol}"
    return err.max().item()
