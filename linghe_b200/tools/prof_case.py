"""Run one entry point a few times on seeded synthetic inputs -- the small, fixed program that
profiler captures of a single kernel are taken from.

    python -m linghe_b200.tools.prof_case --case swiglu_rows --rows 32768 --cols 8192 --iters 2

`--cols` is the OUTPUT width n (SwiGLU inputs are [rows, 2n]).  Cases:
  norm_rows / norm_col / norm_both   RMSNorm + blockwise quant, output_mode 0 / 1 / 2
  swiglu_rows / swiglu_both          SwiGLU + blockwise quant, output_mode 0 / 2
  swiglu_bwd                         SwiGLU backward + dual quant (+ bf16 dx)
  quant_rows / quant_col / quant_both  pure blockwise quantiser, output_mode 0 / 1 / 2
  group_quant                        1x128 group quantiser
  norm_fwd / norm_bwd                plain RMSNorm forward / backward
  norm_bwd_quant                     RMSNorm backward fused with the dual-axis quantisation of dy
  fp8_gemm                           blockwise-scaled FP8 GEMM, [rows, k] x [cols, k]^T with 1 x 128 scales (`--k`)
`--tuning key=value` (repeatable) sets a dispatch option through lh_tuning() first, e.g.
`--tuning rmsnorm_bwd_quant_two_role_min_n=128` to capture the two-role backward kernel.
"""

from __future__ import annotations

import argparse

import torch


def bf16_randn(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = torch.empty(shape, device="cuda", dtype=torch.bfloat16)
    step = max(1, (1 << 26) // shape[1])
    for r0 in range(0, shape[0], step):
        r1 = min(shape[0], r0 + step)
        out[r0:r1] = (torch.randn((r1 - r0, shape[1]), generator=g, device="cuda") * scale).to(torch.bfloat16)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--k", type=int, default=4096, help="contraction length of the fp8_gemm case")
    ap.add_argument("--tuning", action="append", default=[])
    a = ap.parse_args()
    torch.cuda.set_device(0)
    if a.tuning:
        from linghe_b200 import _lib
        lib = _lib.load()
        for kv in a.tuning:
            key, val = kv.split("=")
            assert lib.lh_tuning(key.encode(), int(val)) >= 0, f"unknown tuning key {key}"
    from linghe_b200.quant.block import triton_blockwise_quant
    from linghe_b200.quant.group import triton_group_quant
    from linghe_b200.utils.norm import (rms_norm_backward_and_block_quant, triton_rms_norm_and_block_quant_forward,
                                        triton_rms_norm_backward, triton_rms_norm_forward)
    from linghe_b200.utils.silu import triton_silu_and_block_quant_backward, triton_silu_and_block_quant_forward
    M, n = a.rows, a.cols
    gam = (1 + 0.1 * torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(3))).to(torch.bfloat16)
    c = a.case
    if c.startswith("norm_") and c not in ("norm_bwd", "norm_bwd_quant", "norm_fwd"):
        x = bf16_randn((M, n), 1)
        mode = {"norm_rows": 0, "norm_col": 1, "norm_both": 2}[c]
        rms = triton_rms_norm_and_block_quant_forward(x, gam, output_mode=0)[2] if mode == 1 else None
        fn = lambda: triton_rms_norm_and_block_quant_forward(x, gam, rms=rms, output_mode=mode)
    elif c in ("swiglu_rows", "swiglu_both"):
        x = bf16_randn((M, 2 * n), 1)
        fn = lambda: triton_silu_and_block_quant_forward(x, output_mode=0 if c == "swiglu_rows" else 2)
    elif c == "swiglu_bwd":
        x, g = bf16_randn((M, 2 * n), 1), bf16_randn((M, n), 2, 0.01)
        fn = lambda: triton_silu_and_block_quant_backward(g, x, return_bf16=True)
    elif c in ("quant_rows", "quant_col", "quant_both"):
        x = bf16_randn((M, n), 2, 0.01)
        fn = lambda: triton_blockwise_quant(x, output_mode={"quant_rows": 0, "quant_col": 1, "quant_both": 2}[c])
    elif c == "group_quant":
        x = bf16_randn((M, n), 2)
        fn = lambda: triton_group_quant(x)
    elif c == "norm_fwd":
        x = bf16_randn((M, n), 1)
        fn = lambda: triton_rms_norm_forward(x, gam)
    elif c in ("norm_bwd", "norm_bwd_quant"):
        x, dy = bf16_randn((M, n), 1), bf16_randn((M, n), 2, 0.01)
        fn = (lambda: triton_rms_norm_backward(dy, x, gam)) if c == "norm_bwd" else \
             (lambda: rms_norm_backward_and_block_quant(dy, x, gam))
    elif c == "fp8_gemm":
        from linghe_b200.gemm.blockwise_fp8_gemm import triton_tt_fp8_gemm
        g = torch.Generator(device="cuda").manual_seed(5)
        qa = torch.randn((M, a.k), device="cuda", generator=g).to(torch.float8_e4m3fn)
        qb = torch.randn((n, a.k), device="cuda", generator=g).to(torch.float8_e4m3fn)
        sa = torch.rand((M, a.k // 128), device="cuda", generator=g) + 0.1
        sb = torch.rand((n, a.k // 128), device="cuda", generator=g) + 0.1
        fn = lambda: triton_tt_fp8_gemm(qa, qb, sa, sb)
    else:
        raise SystemExit(f"unknown case {c}")
    keep = None
    for _ in range(a.iters):
        keep = fn()
    torch.cuda.synchronize()
    del keep
    print(f"{c} {M}x{n}: {a.iters} calls done")


if __name__ == "__main__":
    main()
