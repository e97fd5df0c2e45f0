"""Tolerance checker in the spirit of linghe/tools/check.py: element-wise
|out - ref| < rtol*|ref| + atol with dtype-dependent defaults, plus a summary line."""

from __future__ import annotations

import torch

_DEFAULTS = {
    torch.float32: (1e-4, 1e-6),
    torch.bfloat16: (2e-2, 1e-3),
    torch.float16: (2e-3, 1e-4),
    torch.float8_e4m3fn: (0.125, 0.125),
}


def output_check(org_out, opt_out, name="", rtol=None, atol=None, raise_error=True, quiet=False):
    """Compare `opt_out` with the reference `org_out` (linghe/tools/check.py:11)."""
    assert org_out.shape == opt_out.shape, f"{name}: shape {tuple(org_out.shape)} vs {tuple(opt_out.shape)}"
    assert org_out.dtype == opt_out.dtype, f"{name}: dtype {org_out.dtype} vs {opt_out.dtype}"
    d_rtol, d_atol = _DEFAULTS.get(org_out.dtype, (1e-4, 1e-6))
    rtol = d_rtol if rtol is None else rtol
    atol = d_atol if atol is None else atol
    ref = org_out.detach().float().cpu()
    out = opt_out.detach().float().cpu()
    if ref.numel() == 0:
        return True
    err = (out - ref).abs()
    ok = bool((err <= rtol * ref.abs() + atol).all())
    if not quiet:
        rel = (err.mean() / ref.abs().mean().clamp_min(1e-30)).item()
        print(f"{name:<24} max_abs_err {err.max().item():.3e}  mean_rel_err {rel:.3e}  {'ok' if ok else 'MISMATCH'}")
    if raise_error and not ok:
        raise AssertionError(f"{name}: output differs beyond rtol={rtol} atol={atol}")
    return ok


def quant_check(org_out, xq, wq, opt_out, mode):
    """Print the fraction of saturated / flushed-to-zero codes (linghe/tools/check.py:132)."""
    xf, wf = xq.float().abs(), wq.float().abs()
    print(f"{mode}: x sat {(xf >= 448).float().mean().item():.2e} zero {(xf == 0).float().mean().item():.2e} | "
          f"w sat {(wf >= 448).float().mean().item():.2e} zero {(wf == 0).float().mean().item():.2e}")
    return output_check(org_out, opt_out, mode, raise_error=False)
