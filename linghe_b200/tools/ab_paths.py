"""A/B timing of the selectable implementations behind two entry points (CUDA-graph replay over
rotating buffers, the harness of bench_configs):

    python -m linghe_b200.tools.ab_paths --what fwd     both-axes RMSNorm + quant: row kernel then column
                                                        kernel ("two") against the single-pass cluster kernel
    python -m linghe_b200.tools.ab_paths --what bwd     RMSNorm backward + dy dual quant: two launches against
                                                        the single-pass cluster kernel ("band") and the
                                                        streaming kernel with a second, tile-quantising role per CTA
    python -m linghe_b200.tools.ab_paths --what fwd_clusters   the single-pass forward kernel at each forced
                                                        cluster size (1, 2, 4, 8) beside the two launches

The paths are switched with lh_tuning(); the defaults are restored at the end.
"""

from __future__ import annotations

import argparse
import json

import torch

from linghe_b200 import _lib
from linghe_b200.tools import bench_configs as BC
from linghe_b200.utils.norm import rms_norm_backward_and_block_quant, triton_rms_norm_and_block_quant_forward


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", choices=["fwd", "bwd", "fwd_clusters"], required=True)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    lib = _lib.load()
    gam = (1 + 0.1 * torch.randn(8192, device="cuda")).to(torch.bfloat16)
    rows = []
    if a.what == "fwd":
        for n in (1024, 1280, 1536, 1792, 2048, 2304, 2560, 3072, 3584, 4096, 5120, 6144, 7168, 8192):
            for M in (4096, 16384, 65536):
                if M * n > 300e6:
                    continue
                g = gam[:n].contiguous()
                nbytes = M * n * 4
                row = {"n": n, "M": M}
                for name, mode in (("two_launch_us", 0), ("single_pass_us", 2)):
                    lib.lh_tuning(b"rmsnorm_both_single_pass", mode)
                    ev, gr, _ = BC.time_call(lambda i: (BC.bf16_randn((M, n), i), g),
                                             lambda x, w: triton_rms_norm_and_block_quant_forward(x, w, output_mode=2),
                                             nbytes, 40 if nbytes < 1e9 else 12)
                    row[name] = round(gr if gr else ev, 2)
                row["two_over_single"] = round(row["two_launch_us"] / row["single_pass_us"], 3)
                print(row, flush=True)
                rows.append(row)
        lib.lh_tuning(b"rmsnorm_both_single_pass", 1)
    elif a.what == "fwd_clusters":
        for n in (1024, 2048, 3072, 4096, 5120, 6144, 8192):
            for M in (4096, 16384, 65536):
                if M * n > 600e6:
                    continue
                g = gam[:n].contiguous()
                nbytes = M * n * 4
                row = {"n": n, "M": M}
                for name, mode, C in (("C1_us", 2, 1), ("C2_us", 2, 2), ("C4_us", 2, 4), ("C8_us", 2, 8),
                                      ("chosen_us", 2, 0), ("two_launch_us", 0, 0)):
                    lib.lh_tuning(b"rmsnorm_both_single_pass", mode)
                    lib.lh_tuning(b"band_cluster", C)
                    ev, gr, _ = BC.time_call(lambda i: (BC.bf16_randn((M, n), i), g),
                                             lambda x, w: triton_rms_norm_and_block_quant_forward(x, w, output_mode=2),
                                             nbytes, 30 if nbytes < 1e9 else 10)
                    row[name] = round(gr if gr else ev, 1)
                print(row, flush=True)
                rows.append(row)
        lib.lh_tuning(b"rmsnorm_both_single_pass", 1)
        lib.lh_tuning(b"band_cluster", 0)
    else:
        for (M, n) in ((16384, 4096), (8192, 2048), (65536, 2048), (16384, 8192), (32768, 4096), (4096, 4096),
                       (16384, 1536), (8192, 5120)):
            g = gam[:n].contiguous()
            nbytes = 3 * M * n * 2 + 2 * M * n + 2 * M * n * 4 // 128 + n * 6
            row = {"M": M, "n": n}
            for name, band, il in (("two_launch_us", 0, 1 << 30), ("two_role_us", 0, 128), ("band_us", 1, 1 << 30)):
                lib.lh_tuning(b"rmsnorm_bwd_quant_single_pass", band)
                lib.lh_tuning(b"rmsnorm_bwd_quant_two_role_min_n", il)
                ev, gr, _ = BC.time_call(lambda i: (BC.bf16_randn((M, n), 100 + i, 0.01), BC.bf16_randn((M, n), i), g),
                                         rms_norm_backward_and_block_quant, nbytes, 50 if nbytes < 1e9 else 12)
                row[name] = round(gr if gr else ev, 2)
            print(row, flush=True)
            rows.append(row)
        lib.lh_tuning(b"rmsnorm_bwd_quant_single_pass", 0)
        lib.lh_tuning(b"rmsnorm_bwd_quant_two_role_min_n", 1 << 30)
    assert _lib.device_status(0) == 0
    if a.json:
        with open(a.json, "w") as fh:
            json.dump(rows, fh, indent=1)


if __name__ == "__main__":
    main()
