"""How the time of the RMSNorm + 1x128 quant call at the benchmark shape depends on the SM clock and
on where the input sits in memory.

    python -m linghe_b200.tools.clock_probe [--rows 65536] [--cols 8192] [--calls 200]

The call is timed `--calls` times with CUDA events at eight input offsets 2 MiB apart while a thread
samples the SM and memory clocks through NVML (read-only queries).  A long run heats the GPU into its
power cap, so later offsets see lower clocks: time x clock staying constant across the rows of the
table means the kernel is bound by instruction issue / on-chip latency, not by HBM.
"""

from __future__ import annotations

import argparse
import json
import threading
import time

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--cols", type=int, default=8192)
    ap.add_argument("--calls", type=int, default=200)
    ap.add_argument("--json", default=None)
    a = ap.parse_args()
    import pynvml
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward as norm_q
    torch.cuda.set_device(0)
    pynvml.nvmlInit()
    props = torch.cuda.get_device_properties(0)
    try:
        h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(props.uuid)).encode())
    except Exception:
        h = pynvml.nvmlDeviceGetHandleByIndex(0)
    M, n = a.rows, a.cols
    buf = torch.empty(M * n + 8 * (1 << 20), dtype=torch.bfloat16, device="cuda")
    buf.normal_()
    gam = (1 + 0.1 * torch.randn(n, device="cuda")).to(torch.bfloat16)
    q = torch.empty((M, n), device="cuda", dtype=torch.float8_e4m3fn)
    s = torch.empty((n // 128, M), device="cuda", dtype=torch.float32)
    clk, stop = [], [False]

    def pump():
        while not stop[0]:
            clk.append((time.perf_counter(), pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM),
                        pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_MEM)))
            time.sleep(0.005)

    th = threading.Thread(target=pump, daemon=True)
    th.start()
    res = []
    for k in range(8):
        off = k * (1 << 20)          # elements: steps of 2 MiB
        x = buf[off:off + M * n].view(M, n)
        for _ in range(5):
            norm_q(x, gam, out=q, scale=s, output_mode=0)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        evs = []
        for _ in range(a.calls):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            norm_q(x, gam, out=q, scale=s, output_mode=0)
            e1.record()
            evs.append((e0, e1))
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        ts = sorted(e0.elapsed_time(e1) * 1e3 for e0, e1 in evs)
        c = sorted(v[1] for v in clk if t0 <= v[0] <= t1)
        m = sorted(v[2] for v in clk if t0 <= v[0] <= t1)
        row = {"offset_MiB": 2 * k, "min_us": round(ts[0], 1), "median_us": round(ts[len(ts) // 2], 1),
               "max_us": round(ts[-1], 1), "sm_mhz_median": c[len(c) // 2] if c else None,
               "sm_mhz_min": c[0] if c else None, "mem_mhz": m[len(m) // 2] if m else None}
        if row["sm_mhz_median"]:
            row["median_us_x_ghz"] = round(row["median_us"] * row["sm_mhz_median"] / 1e3, 1)
        print(row, flush=True)
        res.append(row)
    stop[0] = True
    if a.json:
        with open(a.json, "w") as fh:
            json.dump(res, fh, indent=1)


if __name__ == "__main__":
    main()
