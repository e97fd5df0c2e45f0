"""Per-kernel timing of every benchmark configuration of the fused norm / SwiGLU + FP8
blockwise-quant path, with the achieved fraction of the HBM roofline.

    python -m linghe_b200.tools.bench_configs [--upstream PATH] [--only cfg1,cfg5] [--json out.json]

For each configuration the call is timed two ways on the current CUDA device:
  * "event"  median CUDA-event time around single calls (as linghe/tools/benchmark.py does);
  * "graph"  steady-state time per call when a ring of calls is replayed from a CUDA graph
             (no host launch gaps) -- this is the number used for GB/s.
Inputs AND outputs rotate through a ring whose footprint exceeds twice the L2 size, so
every call streams from and to HBM.  Algorithmic bytes count each tensor once.

With --upstream (a directory containing the upstream `linghe` package, e.g. a
`pip install --target` of it) the upstream Triton kernels are timed in the same run with
the same inputs and the same harness.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

import numpy as np
import torch

NOMINAL = 8000.0
L2_BYTES = 126 * 1024 * 1024


def measured_peak():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["hbm_gbs"])
    except Exception:
        return 6650.0


def bf16_randn(shape, seed, scale=1.0, device="cuda"):
    g = torch.Generator(device=device).manual_seed(seed)
    rows = shape[0]
    out = torch.empty(shape, device=device, dtype=torch.bfloat16)
    step = max(1, (1 << 26) // max(1, int(np.prod(shape[1:]))))
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        out[r0:r1] = (torch.randn((r1 - r0, *shape[1:]), generator=g, device=device) * scale).to(torch.bfloat16)
    return out


def moe_counts(seed=0, experts=256, tokens=65536, alpha=0.3):
    rng = np.random.default_rng(seed)
    p = rng.dirichlet(np.full(experts, alpha))
    c = rng.multinomial(tokens, p)
    return ((c + 127) // 128 * 128).astype(np.int64)


def time_call(make_args, fn, nbytes_set, iters=50):
    """make_args(i) -> args for ring slot i; fn(*args) -> outputs (kept alive in a ring)."""
    nsets = int(min(16, max(2, math.ceil(2.2 * L2_BYTES / max(1, nbytes_set)))))
    args = [make_args(i) for i in range(nsets)]
    keep = [None] * nsets
    for i in range(nsets):  # warm-up, also fills the output ring
        keep[i] = fn(*args[i])
    for i in range(3 * nsets):
        keep[i % nsets] = fn(*args[i % nsets])
    torch.cuda.synchronize()
    ev = []
    for i in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        keep[i % nsets] = fn(*args[i % nsets])
        b.record()
        ev.append((a, b))
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) * 1e3 for a, b in ev)
    event_us = ts[len(ts) // 2]
    graph_us = None
    try:
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                for i in range(nsets):
                    keep[i] = fn(*args[i])
        torch.cuda.synchronize()
        reps = max(3, iters // nsets)
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        graph_us = a.elapsed_time(b) * 1e3 / (reps * nsets)
        del g
    except Exception as e:  # graph capture is a convenience; fall back to event timing
        print(f"  (graph timing unavailable: {type(e).__name__}: {e})", file=sys.stderr)
    del keep, args
    torch.cuda.empty_cache()
    return event_us, graph_us, nsets


FLOPS = {}   # case name -> floating-point operations, for the GEMM rows


def build_cases(mods):
    """name -> (make_args, callable, algorithmic bytes, ring bytes per set)"""
    norm_q, rms_bwd, bq, silu_f, silu_b, wsilu_b, bsilu_f, bsilu_b, fused_bwd, permute, router, gemm, route = mods
    cases = {}

    def add(name, make_args, fn, nbytes, set_bytes=None):
        cases[name] = (make_args, fn, nbytes, set_bytes or nbytes)

    # cfg1: RMSNorm + quant 8192 x 2048
    M, n = 8192, 2048
    gam = (1 + 0.1 * torch.randn(8192, device="cuda")).to(torch.bfloat16)
    b0 = M * n * 3 + M * (n // 128) * 4 + M * 4 + n * 2
    add("cfg1 rmsnorm+quant 8192x2048 rows", lambda i: (bf16_randn((8192, 2048), i), gam[:2048].contiguous()),
        lambda x, g: norm_q(x, g, output_mode=0), b0)
    add("cfg1 rmsnorm+quant 8192x2048 both", lambda i: (bf16_randn((8192, 2048), i), gam[:2048].contiguous()),
        lambda x, g: norm_q(x, g, output_mode=2), b0 + M * n + (M // 128) * n * 4)
    # cfg2: SwiGLU fwd / bwd 8192 x 2816
    M, n = 8192, 1408
    f0 = M * 2 * n * 2 + M * n + M * (n // 128) * 4
    add("cfg2 swiglu+quant fwd 8192x2816 rows", lambda i: (bf16_randn((8192, 2816), i),),
        lambda x: silu_f(x, output_mode=0), f0)
    add("cfg2 swiglu+quant fwd 8192x2816 both", lambda i: (bf16_randn((8192, 2816), i),),
        lambda x: silu_f(x, output_mode=2), f0 + M * n + (M // 128) * n * 4)
    bw = M * n * 2 + M * 2 * n * 2 + M * 2 * n * 2 + 2 * (M * 2 * n) + M * (2 * n // 128) * 4 + (M // 128) * 2 * n * 4
    if silu_b is not None:
        add("cfg2 swiglu+quant bwd 8192x2816 (+bf16 dx)",
            lambda i: (bf16_randn((8192, 1408), 100 + i, 0.01), bf16_randn((8192, 2816), i)), silu_b, bw)
    # a7: the plain (unquantised) weighted SwiGLU forward / backward at the cfg2 shape
    if wsilu_b is not None:
        wsf, wsb = wsilu_b
        wrow2 = torch.randn((8192, 1), device="cuda")
        add("cfg2 weighted swiglu fwd 8192x2816 (bf16 out)", lambda i: (bf16_randn((8192, 2816), i),),
            lambda x: wsf(x, wrow2), M * 2 * n * 2 + M * n * 2 + M * 4)
        add("cfg2 weighted swiglu bwd 8192x2816 (bf16 dx)",
            lambda i: (bf16_randn((8192, 1408), 100 + i, 0.01), bf16_randn((8192, 2816), i)),
            lambda g, x: wsb(g, x, wrow2), M * n * 2 + 2 * (M * 2 * n * 2) + 2 * M * 4)
    # cfg3: per-expert batched
    counts = moe_counts()
    R = int(counts.sum())
    n = 512
    ct = torch.tensor(counts, dtype=torch.int32, device="cuda")
    splits = counts.tolist()
    wrow = torch.randn((R, 1), device="cuda")
    add(f"cfg3 batched swiglu+quant fwd R={R} both", lambda i: (bf16_randn((R, 1024), i),),
        lambda x: bsilu_f(x, wrow, ct, splits, output_mode=2), R * 3108 + 1024)
    add(f"cfg3 batched swiglu+quant bwd R={R}",
        lambda i: (bf16_randn((R, 512), 100 + i, 0.01), bf16_randn((R, 1024), i)),
        lambda g, x: bsilu_b(g, x, wrow, ct, splits), R * 5192)
    # the step before cfg3: gather 8192 tokens x hidden 2048 into 256 experts (top-8), pad to 16, dual quant
    if permute is not None:
        rng = np.random.default_rng(0)
        pe = rng.dirichlet(np.full(256, 0.3))
        gum = -np.log(-np.log(rng.random((8192, 256))))
        top = np.argsort(-(np.log(pe + 1e-30)[None, :] + gum), axis=1)[:, :8]
        route_np = np.zeros((8192, 256), dtype=bool)
        np.put_along_axis(route_np, top, True, axis=1)
        pcounts = route_np.sum(0)
        idx_parts = []
        for e in range(256):
            rows_e = np.nonzero(route_np[:, e])[0]
            padn = (-len(rows_e)) % 16
            idx_parts.append(np.concatenate([rows_e, np.zeros(padn, dtype=rows_e.dtype)]))
        pidx = torch.tensor(np.concatenate(idx_parts), dtype=torch.int32, device="cuda")
        pct = torch.tensor(pcounts, dtype=torch.int32, device="cuda")
        Mp = int(pidx.numel())
        add(f"next pad-permute+quant 8192x2048 -> {Mp} rows both", lambda i: (bf16_randn((8192, 2048), i),),
            lambda x: permute(x, pct, pidx, pcounts.tolist()), Mp * 2048 * 4 + 2 * Mp * 2048 * 4 // 128)
        if route is not None:
            make_map, unpermute = route
            rmap = torch.from_numpy(route_np).to("cuda")
            add("next row-id map + index 8192 tokens x 256 experts", lambda i: (rmap,),
                lambda m: make_map(m, Mp, multiple_of=16), 8192 * 256 * 5 + Mp * 4)
            rid, _ = make_map(rmap, Mp, multiple_of=16)
            add(f"next un-permute {Mp} rows -> 8192x2048", lambda i: (bf16_randn((Mp, 2048), i),),
                lambda g: unpermute(g, rid, None), Mp * 2048 * 2 + 8192 * 2048 * 2 + 8192 * 256 * 4)
    # the step beside cfg1 in the MoE block: RMSNorm + float32 router logits (256 experts) + row quant
    if router is not None:
        M, K, N = 8192, 2048, 256
        rw = torch.randn((N, K), device="cuda").to(torch.bfloat16)
        add("next rmsnorm+router gemm+quant 8192x2048 N=256 rows",
            lambda i: (bf16_randn((8192, 2048), i), gam[:2048].contiguous()),
            lambda x, g: router(x, g, rw, output_mode=0),
            M * K * 5 + M * (K // 128) * 4 + M * 4 + M * N * 4 + N * K * 2 + K * 2)
    # consumer of the wire format: blockwise-scaled FP8 GEMM (upstream test shape 4096^3, blocks of 128)
    if gemm is not None:
        for (M, N, K) in ((4096, 4096, 4096), (8192, 2816, 2048)):
            FLOPS[f"next fp8 gemm tt {M}x{N}x{K} block 128"] = 2 * M * N * K
            add(f"next fp8 gemm tt {M}x{N}x{K} block 128",
                lambda i, M=M, N=N, K=K: (torch.randn((M, K), device="cuda").to(torch.float8_e4m3fn),
                                          torch.randn((N, K), device="cuda").to(torch.float8_e4m3fn),
                                          torch.rand((M, K // 128), device="cuda") + 0.01,
                                          torch.rand((N, K // 128), device="cuda") + 0.01),
                lambda a, b, sa, sb: gemm(a, b, sa, sb, out_dtype=torch.bfloat16, block_size=128),
                M * K + N * K + 2 * M * N + (M + N) * (K // 128) * 4)
    # cfg4: RMSNorm bwd + dual-axis dy quant 16384 x 4096
    M, n = 16384, 4096
    c4 = 3 * M * n * 2 + 2 * M * n + 2 * M * n * 4 // 128 + n * 2 + n * 4
    add("cfg4 rmsnorm bwd + dy dual quant 16384x4096",
        lambda i: (bf16_randn((16384, 4096), 100 + i, 0.01), bf16_randn((16384, 4096), i), gam[:4096].contiguous()),
        fused_bwd, c4)
    add("cfg4a rmsnorm bwd alone 16384x4096",
        lambda i: (bf16_randn((16384, 4096), 100 + i, 0.01), bf16_randn((16384, 4096), i), gam[:4096].contiguous()),
        rms_bwd, 3 * M * n * 2 + n * 6)
    add("cfg4b blockwise_quant dy 16384x4096 both", lambda i: (bf16_randn((16384, 4096), 100 + i, 0.01),),
        lambda x: bq(x), M * n * 4 + 2 * M * n * 4 // 128)
    # cfg5: scale-out shapes, one GPU's shard
    M, n = 65536, 8192
    add("cfg5 rmsnorm+quant 65536x8192 rows", lambda i: (bf16_randn((65536, 8192), i), gam),
        lambda x, g: norm_q(x, g, output_mode=0), M * n * 3 + M * (n // 128) * 4 + M * 4 + n * 2)
    add("cfg5 swiglu+quant 65536x16384 rows", lambda i: (bf16_randn((65536, 16384), i),),
        lambda x: silu_f(x, output_mode=0), M * 2 * n * 2 + M * n + M * (n // 128) * 4)
    add("cfg5 rmsnorm+quant 65536x8192 both", lambda i: (bf16_randn((65536, 8192), i), gam),
        lambda x, g: norm_q(x, g, output_mode=2), M * n * 4 + M * (n // 128) * 4 + M * 4 + n * 2 + (M // 128) * n * 4)
    add("cfg5 swiglu+quant 65536x16384 both", lambda i: (bf16_randn((65536, 16384), i),),
        lambda x: silu_f(x, output_mode=2), M * 2 * n * 2 + 2 * M * n + M * (n // 128) * 4 + (M // 128) * n * 4)
    return cases


def ours():
    from linghe_b200.quant.block import triton_blockwise_quant
    from linghe_b200.utils.norm import (rms_norm_backward_and_block_quant, triton_rms_norm_and_block_quant_forward,
                                        triton_rms_norm_backward)
    from linghe_b200.utils.silu import (triton_batch_weighted_silu_and_block_quant_backward,
                                        triton_batch_weighted_silu_and_block_quant_forward,
                                        triton_silu_and_block_quant_backward, triton_silu_and_block_quant_forward,
                                        triton_weighted_silu_backward, triton_weighted_silu_forward)
    return (triton_rms_norm_and_block_quant_forward, triton_rms_norm_backward, triton_blockwise_quant,
            triton_silu_and_block_quant_forward,
            lambda g, x: triton_silu_and_block_quant_backward(g, x, return_bf16=True),
            (triton_weighted_silu_forward, triton_weighted_silu_backward),
            triton_batch_weighted_silu_and_block_quant_forward,
            triton_batch_weighted_silu_and_block_quant_backward, rms_norm_backward_and_block_quant,
            _ours_permute(), _ours_router(), _ours_gemm(), _ours_route())


def _ours_route():
    from linghe_b200.utils.gather import triton_make_row_id_map_and_index
    from linghe_b200.utils.scatter import triton_unpermute_with_mask_map
    return triton_make_row_id_map_and_index, triton_unpermute_with_mask_map


def _upstream_route():
    from linghe.utils.gather import triton_make_row_id_map_and_index
    from linghe.utils.scatter import triton_unpermute_with_mask_map
    return triton_make_row_id_map_and_index, triton_unpermute_with_mask_map


def _ours_gemm():
    from linghe_b200.gemm.blockwise_fp8_gemm import triton_tt_fp8_gemm
    return triton_tt_fp8_gemm


def _ours_router():
    from linghe_b200.utils.norm import triton_rms_norm_fp32_gemm_block_quant_forward
    return triton_rms_norm_fp32_gemm_block_quant_forward


def _ours_permute():
    from linghe_b200.utils.gather import triton_batch_block_pad_permute_with_indices
    return triton_batch_block_pad_permute_with_indices


def upstream(path):
    sys.path.insert(0, path)
    from linghe.quant.block import triton_blockwise_quant
    from linghe.utils.norm import triton_rms_norm_and_block_quant_forward, triton_rms_norm_backward
    from linghe.utils.silu import (triton_batch_weighted_silu_and_block_quant_backward,
                                   triton_batch_weighted_silu_and_block_quant_forward,
                                   triton_silu_and_block_quant_backward, triton_silu_and_block_quant_forward,
                                   triton_weighted_silu_backward, triton_weighted_silu_forward)

    def silu_b(g, x):  # upstream needs two passes for fp8 + bf16 dx
        return triton_silu_and_block_quant_backward(g, x), triton_weighted_silu_backward(g, x)

    def fused_bwd(dy, x, w):  # upstream: backward pass + separate dual-axis quant of dy
        return triton_rms_norm_backward(dy, x, w), triton_blockwise_quant(dy)

    return (triton_rms_norm_and_block_quant_forward, triton_rms_norm_backward, triton_blockwise_quant,
            triton_silu_and_block_quant_forward, silu_b, (triton_weighted_silu_forward, triton_weighted_silu_backward),
            triton_batch_weighted_silu_and_block_quant_forward,
            triton_batch_weighted_silu_and_block_quant_backward, fused_bwd, _upstream_permute(),
            _upstream_router(), _upstream_gemm(), _upstream_route())


def _upstream_gemm():
    from linghe.gemm.blockwise_fp8_gemm import triton_tt_fp8_gemm
    return triton_tt_fp8_gemm


def _upstream_router():
    from linghe.utils.norm import triton_rms_norm_fp32_gemm_block_quant_forward
    return triton_rms_norm_fp32_gemm_block_quant_forward


def _upstream_permute():
    from linghe.utils.gather import triton_batch_block_pad_permute_with_indices
    return triton_batch_block_pad_permute_with_indices


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--upstream", default=None, help="directory holding the upstream `linghe` package")
    ap.add_argument("--only", default=None, help="comma-separated substrings of case names")
    ap.add_argument("--json", default=None)
    ap.add_argument("--iters", type=int, default=50)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    peak = measured_peak()
    impls = [("cuda sm_100a", ours())]
    if a.upstream:
        impls.append(("upstream triton", upstream(a.upstream)))
    rows = []
    for impl_name, mods in impls:
        torch.manual_seed(0)
        for name, (make_args, fn, nbytes, set_bytes) in build_cases(mods).items():
            if a.only and not any(k in name for k in a.only.split(",")):
                continue
            if set_bytes > 6e9:
                continue
            try:
                ev_us, gr_us, nsets = time_call(make_args, fn, set_bytes, a.iters if nbytes < 1e9 else 12)
            except Exception as e:
                print(f"{impl_name:16} {name:52} FAILED {type(e).__name__}: {e}")
                continue
            us = gr_us if gr_us is not None else ev_us
            gbs = nbytes / us / 1e3
            rows.append({"impl": impl_name, "case": name, "bytes": nbytes, "event_us": round(ev_us, 2),
                         "graph_us": None if gr_us is None else round(gr_us, 2), "gbs": round(gbs, 1),
                         "pct_nominal": round(100 * gbs / NOMINAL, 1), "pct_measured": round(100 * gbs / peak, 1),
                         "ring": nsets})
            print(f"{impl_name:16} {name:52} event {ev_us:9.1f} us  graph {us:9.1f} us  {gbs:8.1f} GB/s  "
                  f"{100 * gbs / NOMINAL:5.1f}% of 8 TB/s  {100 * gbs / peak:5.1f}% of measured {peak:.0f}", flush=True)
            if name in FLOPS:
                rows[-1]["tflops"] = round(FLOPS[name] / us / 1e6, 1)
                print(f"{'':16} {'':52} {FLOPS[name] / us / 1e6:9.1f} TFLOP/s", flush=True)
    if a.json:
        with open(a.json, "w") as fh:
            json.dump(rows, fh, indent=1)


if __name__ == "__main__":
    main()
