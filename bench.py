#!/usr/bin/env python
"""Benchmark of the fused norm / SwiGLU + FP8 blockwise-quant hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    torchrun ... bench.py --gpus N ...           (one rank per GPU, N > 1)

Workload ("scaleout-65536x8192"): per GPU, one step is
  (1) RMSNorm + 1x128 FP8 quantisation of x bf16 [65536, 8192]   (row-wise outputs)
  (2) SwiGLU  + 1x128 FP8 quantisation of x bf16 [65536, 16384] -> [65536, 8192]
on seeded synthetic N(0,1) inputs; token rows are sharded across ranks with no
data-path collective (weak scaling: every rank owns 65536 rows).  Inputs (1 GiB and
2 GiB) are far larger than L2, so no L2 flush is needed between iterations.

`value` is the aggregate algorithmic GB/s (each tensor counted once) over all ranks,
timed on the device with CUDA events, max over ranks.  `e2e` is the same metric through
the public Python API with HOST (pinned) inputs and outputs: host->device copies of both
inputs and device->host copies of every output are inside the timed region.
`--impl reference` times the CPU oracle (the reference's PyTorch math restated) on the
host cores for a bounded row sample of the same workload.

One JSON line is printed by rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

ROWS = 65536
HIDDEN = 8192
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0


def norm_bytes(M, n):  # x bf16 + q fp8 + scales + rms + gamma
    return M * n * 3 + M * (n // 128) * 4 + M * 4 + n * 2


def silu_bytes(M, n):  # x bf16 [M,2n] + q fp8 [M,n] + scales
    return M * 2 * n * 2 + M * n + M * (n // 128) * 4


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """SM clock / throttle-reason samples (read-only NVML queries from a thread, every few
    milliseconds, each with a time stamp so that a phase of the run can be summarised by itself).
    Falls back to an `nvidia-smi -lms` child process when NVML cannot be loaded."""

    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, cuda_index):
        self.cuda_index = cuda_index
        self.samples = []          # (t, sm_mhz, max_mhz, power_w, reasons bitmask)
        self.stop_flag = threading.Event()
        self.thread = None
        self.nv = None
        self.handle = None
        self.smi = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            props = torch.cuda.get_device_properties(self.cuda_index)
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(props.uuid)).encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index())
            self.nv = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._pump_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nv = None
        try:
            q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
                 "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
            self.smi = subprocess.Popen(
                ["nvidia-smi", f"--id={gpu_index()}", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump_smi, daemon=True)
            self.thread.start()
        except Exception:
            self.smi = None

    def _pump_nvml(self):
        nv = self.nv
        bits = [(getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8), 0),
                (getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40), 1),
                (getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20), 2),
                (getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4), 3)]
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons",
                              getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons", None))
        while not self.stop_flag.is_set():
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                raw = int(get_reasons(self.handle)) if get_reasons else 0
                mask = 0
                for bit, i in bits:
                    if raw & bit:
                        mask |= 1 << i
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                except Exception:
                    watts = None
                self.samples.append((time.perf_counter(), mhz, self.max_mhz, watts, mask))
            except Exception:
                pass
            time.sleep(0.004)

    def _pump_smi(self):
        for line in self.smi.stdout:
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                mask = 0
                for i, v in enumerate(f[5:9]):
                    if v.lower().startswith("active"):
                        mask |= 1 << i
                self.samples.append((time.perf_counter(), float(f[1]), float(f[2]), float(f[3]), mask))
            except ValueError:
                continue

    def stop(self):
        self.stop_flag.set()
        if self.smi is not None:
            time.sleep(0.15)
            self.smi.terminate()
            try:
                self.smi.wait(timeout=5)
            except Exception:
                self.smi.kill()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self, t0=None, t1=None):
        """median SM clock and the throttle reasons seen among the samples taken in [t0, t1]"""
        if self.nv is None and self.smi is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML and no nvidia-smi"], "samples": 0}
        rows = [r for r in self.samples if (t0 is None or r[0] >= t0) and (t1 is None or r[0] <= t1)]
        sm = sorted(r[1] for r in rows)
        mask = 0
        for r in rows:
            mask |= r[4]
        watts = [r[3] for r in rows if r[3] is not None]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max((r[2] for r in rows), default=None),
                "reasons": [n for i, n in enumerate(self.NAMES) if mask & (1 << i)], "samples": len(sm),
                "power_w_max": round(max(watts), 1) if watts else None,
                "source": "nvml" if self.nv is not None else "nvidia-smi"}


def gpu_index():
    """Physical index nvidia-smi knows this process's current device by."""
    cur = torch.cuda.current_device()
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[cur])
        except (ValueError, IndexError):
            return cur
    return cur


def make_inputs(rank, device, rows):
    g = torch.Generator(device=device).manual_seed(1000 + rank)
    xn = torch.randn((rows, HIDDEN), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn((HIDDEN,), generator=g, device=device)).to(torch.bfloat16)
    xs = torch.empty((rows, 2 * HIDDEN), device=device, dtype=torch.bfloat16)
    half = rows // 2
    for r0 in (0, half):  # generate in two pieces to bound the float32 temporary
        xs[r0:r0 + half] = torch.randn((half, 2 * HIDDEN), generator=g, device=device).to(torch.bfloat16)
    return xn, gamma, xs


def run_ours(args, rank, world, device):
    from linghe_b200 import _lib
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward as norm_q
    from linghe_b200.utils.silu import triton_silu_and_block_quant_forward as silu_q

    _lib.load()
    rows = args.rows
    xn, gamma, xs = make_inputs(rank, device, rows)
    # preallocated outputs: the timed region measures the kernels, not the allocator
    q1 = torch.empty((rows, HIDDEN), device=device, dtype=torch.float8_e4m3fn)
    s1 = torch.empty((HIDDEN // 128, rows), device=device, dtype=torch.float32)
    q2 = torch.empty_like(q1)
    s2 = torch.empty_like(s1)

    def step():
        norm_q(xn, gamma, out=q1, scale=s1, output_mode=0)
        silu_q(xs, out=q2, scale=s2, output_mode=0)

    bytes_norm, bytes_silu = norm_bytes(rows, HIDDEN), silu_bytes(rows, HIDDEN)
    step_bytes = bytes_norm + bytes_silu

    sampler = ClockSampler(gpu_index())
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            torch.distributed.barrier()

    K = args.steps
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    barrier()
    torch.cuda.synchronize()
    t_start = torch.cuda.Event(enable_timing=True)
    t_stop = torch.cuda.Event(enable_timing=True)
    t_timed0 = time.perf_counter()
    t_start.record()
    for i in range(K):
        ev[i][0].record()
        norm_q(xn, gamma, out=q1, scale=s1, output_mode=0)
        ev[i][1].record()
        silu_q(xs, out=q2, scale=s2, output_mode=0)
        ev[i][2].record()
    t_stop.record()
    torch.cuda.synchronize()
    t_timed1 = time.perf_counter()
    barrier()
    total_ms = t_start.elapsed_time(t_stop)
    norm_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / K
    silu_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / K

    # ---- sustained: the same step back to back for about two seconds, with the clocks sampled
    # over exactly that window (the K-step region above is shorter than most sampling periods)
    n_sus = max(K, int(args.sustained_s * 1e3 / max(total_ms / K, 1e-3)) + 1) if args.sustained_s > 0 else 0
    sus_ms, sus_t0, sus_t1 = 0.0, None, None
    if n_sus:
        u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        sus_t0 = time.perf_counter()
        u0.record()
        for _ in range(n_sus):
            step()
        u1.record()
        # the split between the two kernels at the clocks the long loop settles at: the last 16 steps
        # again with an event between the launches (outside the sustained window)
        sev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(16)]
        for e in sev:
            e[0].record()
            norm_q(xn, gamma, out=q1, scale=s1, output_mode=0)
            e[1].record()
            silu_q(xs, out=q2, scale=s2, output_mode=0)
            e[2].record()
        torch.cuda.synchronize()
        sus_t1 = time.perf_counter()
        sus_ms = u0.elapsed_time(u1)
        sus_split = (sum(e[0].elapsed_time(e[1]) for e in sev) / 16 * 1e3, sum(e[1].elapsed_time(e[2]) for e in sev) / 16 * 1e3)
    barrier()

    # ---- end to end through the public API with host buffers --------------------------
    Ke = min(K, args.e2e_steps)
    h_xn = torch.empty(xn.shape, dtype=xn.dtype, pin_memory=True).copy_(xn)
    h_xs = torch.empty(xs.shape, dtype=xs.dtype, pin_memory=True).copy_(xs)
    h_out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in (q1, s1, q2, s2)]
    h_rms = torch.empty((rows,), dtype=torch.float32, pin_memory=True)
    NCH = 16 if rows % (16 * 128) == 0 else (8 if rows % (8 * 128) == 0 else 1)
    h_s1 = [torch.empty((HIDDEN // 128, rows // NCH), dtype=torch.float32, pin_memory=True) for _ in range(NCH)]
    h_s2 = [torch.empty((HIDDEN // 128, rows // NCH), dtype=torch.float32, pin_memory=True) for _ in range(NCH)]
    h2d = h_xn.numel() * 2 + h_xs.numel() * 2
    d2h = sum(t.numel() * t.element_size() for t in h_out) + h_rms.numel() * 4

    # Rows are independent, so the end-to-end path pipelines row chunks over three streams:
    # host->device copies, kernels, device->host copies (PCIe is full duplex).  Consecutive steps are
    # not separated by a stream join: step k+1's first copy in may start while step k's last results
    # are still on their way out (stream order alone keeps every buffer's writes in sequence).
    NCHUNK = NCH
    crow = rows // NCHUNK
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    s_main = torch.cuda.current_stream()

    s_in.wait_stream(s_main)
    s_out.wait_stream(s_main)

    def e2e_step():
        keep = []
        for c in range(NCHUNK):
            r0, r1 = c * crow, (c + 1) * crow
            with torch.cuda.stream(s_in):
                dxn = h_xn[r0:r1].to(device, non_blocking=True)
                dxs = h_xs[r0:r1].to(device, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            s_main.wait_event(ready)
            a, b, r, _, _ = norm_q(dxn, gamma, output_mode=0)
            cq, d, _, _ = silu_q(dxs, output_mode=0)
            done = torch.cuda.Event()
            done.record(s_main)
            dxn.record_stream(s_main)
            dxs.record_stream(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                h_out[0][r0:r1].copy_(a, non_blocking=True)
                h_out[2][r0:r1].copy_(cq, non_blocking=True)
                h_s1[c].copy_(b, non_blocking=True)     # [n/128, chunk rows] column slice of the scales
                h_s2[c].copy_(d, non_blocking=True)
                h_rms[r0:r1].copy_(r, non_blocking=True)
                for t_ in (a, b, cq, d, r):
                    t_.record_stream(s_out)
            keep.append((a, b, cq, d, r))

    del xn, xs
    e2e_step()
    s_main.wait_stream(s_out)
    torch.cuda.synchronize()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(Ke):
        e2e_step()
    s_main.wait_stream(s_out)     # the last results have reached the host before the closing event
    e1.record()
    torch.cuda.synchronize()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    sampler.stop()
    # the K-step region and the sustained loop run the same two kernels back to back: their
    # samples together describe the clocks the reported numbers were taken at
    clocks = sampler.summary(t_timed0, sus_t1 if sus_t1 is not None else t_timed1)
    clocks["window"] = "timed K steps + sustained loop"
    clocks["whole_run"] = sampler.summary()

    times = torch.tensor([total_ms, e2e_ms, norm_ms, silu_ms, sus_ms], device=device, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
    total_ms, e2e_ms, norm_ms, silu_ms, sus_ms = times.tolist()

    validated = validate_sharding(rank, world, device)

    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    value = world * step_bytes * K / (total_ms * 1e-3) / 1e9
    e2e_value = world * step_bytes * Ke / (e2e_ms * 1e-3) / 1e9
    achieved = bytes_silu / (silu_ms * 1e-3) / 1e9
    line = {
        "metric": "achieved HBM GB/s, fused RMSNorm+FP8 quant and SwiGLU+FP8 quant (algorithmic bytes / device time)",
        "value": round(value, 1),
        "unit": "GB/s",
        "n_gpus": world,
        "steps": K,
        "warmup": max(args.warmup, 3),
        "ms_per_step": round(total_ms / K, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32 math, bf16 in, e4m3 out",
        "data": "synthetic",
        "config": {"workload": f"scaleout-{rows}x{HIDDEN}: RMSNorm+quant [{rows},{HIDDEN}] and SwiGLU+quant "
                               f"[{rows},{2 * HIDDEN}]->[{rows},{HIDDEN}] per GPU, row-wise 1x128 outputs",
                   "rows_per_gpu": rows, "hidden": HIDDEN, "sharding": f"rows x{world}, no collective",
                   "l2": "inputs (1 GiB, 2 GiB) larger than L2; no flush needed",
                   "bytes_per_step_per_gpu": step_bytes},
        "pct_of_nominal_8TBs_per_gpu": round(100 * value / world / NOMINAL_HBM_GBS, 1),
        "us_per_call": {"rmsnorm_quant": round(norm_ms * 1e3, 1), "swiglu_quant": round(silu_ms * 1e3, 1)},
        "gbs_per_call": {"rmsnorm_quant": round(bytes_norm / norm_ms / 1e6, 1),
                         "swiglu_quant": round(bytes_silu / silu_ms / 1e6, 1)},
        "roofline": {"bound": "hbm", "kernel": "small_units_kernel<SILU, 2> (SwiGLU + 1x128 quant, dominant launch of the step)",
                     "achieved": round(achieved, 1), "peak": peak, "peak_kind": f"of {peak_kind}",
                     "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": int(TRAFFIC_SWIGLU_BYTES * rows / TRAFFIC_CAPTURE_ROWS),
                     "traffic_note": TRAFFIC_NOTE,
                     "second_kernel": {"kernel": "RMSNorm + 1x128 quant launch of the step",
                                       "achieved": round(bytes_norm / norm_ms / 1e6, 1),
                                       "frac": round(bytes_norm / norm_ms / 1e6 / peak, 4),
                                       "frac_of_nominal_8TBs": round(bytes_norm / norm_ms / 1e6 / NOMINAL_HBM_GBS, 4)}},
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": Ke},
        "gpu_launches": 2 * K,
        "clocks": clocks,
        "validated": validated,
    }
    if n_sus:
        sus_value = world * step_bytes * n_sus / (sus_ms * 1e-3) / 1e9
        line["sustained"] = {"gbs": round(sus_value, 1), "seconds": round(sus_ms * 1e-3, 2), "steps": n_sus,
                             "ms_per_step": round(sus_ms / n_sus, 4),
                             "us_per_call": {"rmsnorm_quant": round(sus_split[0], 1), "swiglu_quant": round(sus_split[1], 1)},
                             "pct_of_nominal_8TBs_per_gpu": round(100 * sus_value / world / NOMINAL_HBM_GBS, 1),
                             "clocks": sampler.summary(sus_t0, sus_t1)}
    if world == 1 and not args.no_configs:
        line.update(other_configs(args, peak))
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.cpu_rows, repeats=1)
    return line


def validate_sharding(rank, world, device):
    """Outside every timed region: both kernels (row-wise and transposed outputs) on this rank's
    128-aligned row slice of one seeded 4096-row tensor; the slices are all-gathered over NCCL and
    rank 0 compares the assembled tensors bit for bit with its own single-GPU run on all 4096
    rows.  With one GPU the same code runs as two virtual shards, one after the other."""
    from linghe_b200.tools import shard as S
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward as norm_q
    from linghe_b200.utils.silu import triton_silu_and_block_quant_forward as silu_q
    rows = 4096
    try:
        g = torch.Generator().manual_seed(4242)          # the same tensors on every rank
        x = torch.randn((rows, HIDDEN), generator=g).to(torch.bfloat16)
        xs = torch.randn((rows, 2 * HIDDEN), generator=g).to(torch.bfloat16)
        gamma = (1 + 0.1 * torch.randn((HIDDEN,), generator=g)).to(torch.bfloat16).to(device)

        def f_norm(xl):
            q, s_, _, qt, st = norm_q(xl, gamma, output_mode=2)
            return q, s_, qt, st

        def f_silu(xl):
            return silu_q(xl, output_mode=2)

        def u8(t):
            return t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t

        if world > 1:
            got = [S.run_sharded(f, t, world, rank, device) for f, t in ((f_norm, x), (f_silu, xs))]
        else:
            got = []
            for f, t in ((f_norm, x), (f_silu, xs)):
                parts = [f(t[a:b].contiguous().to(device)) for a, b in (S.shard_rows(rows, 2, 0), S.shard_rows(rows, 2, 1))]
                got.append((torch.cat([u8(p[0]) for p in parts], 0), torch.cat([p[1] for p in parts], 1),
                            torch.cat([u8(p[2]) for p in parts], 1), torch.cat([p[3] for p in parts], 0)))
        ok = True
        differing = []
        if rank == 0:
            ref = [f_norm(x.to(device)), f_silu(xs.to(device))]
            for kname, gt, rf in zip(("rmsnorm", "swiglu"), got, ref):
                for tname, a, b in zip(("q", "s", "qT", "sT"), gt, rf):
                    if not bool(torch.equal(u8(a), u8(b))):
                        ok = False
                        differing.append(f"{kname}.{tname}: {int((u8(a) != u8(b)).sum())} of {a.numel()}")
        torch.cuda.synchronize()
        return {"ranks": world, "shards": max(world, 2), "rows": rows, "ok": ok, "differing": differing,
                "what": "RMSNorm+quant and SwiGLU+quant, codes + scales on both axes, sharded == single GPU bit for bit",
                "gather": "NCCL all_gather" if world > 1 else "none (two virtual shards on one GPU)"}
    except Exception as e:  # validation must not lose the measurement
        return {"ranks": world, "ok": False, "error": f"{type(e).__name__}: {e}"}


def other_configs(args, peak):
    """Per-call times of the remaining benchmark configurations (cfg1-cfg4: the other shapes the
    metric names) with the same harness as linghe_b200/tools/bench_configs.py: CUDA-graph replay
    over rotating input/output sets larger than twice L2, plus the un-graphed CUDA-event time of
    a single call through the Python API.  With the upstream package installed under
    baseline/_ref its Triton kernels are timed in the same process on the same tensors, for the
    two calls of the benchmark step and for every configuration."""
    out = {}
    t_begin = time.perf_counter()
    try:
        from linghe_b200.tools import bench_configs as BC
    except Exception as e:
        return {"configs": {"error": f"{type(e).__name__}: {e}"}}

    def run_cases(mods, only_prefix, budget_s, suffix=""):
        res = {}
        for name, (make_args, fn, nbytes, set_bytes) in BC.build_cases(mods).items():
            if not (name.startswith(only_prefix) and name.endswith(suffix)):
                continue
            if time.perf_counter() - t_begin > budget_s:
                res[name] = {"skipped": "time budget of the default run"}
                continue
            try:
                ev_us, gr_us, nsets = BC.time_call(make_args, fn, set_bytes, 50 if nbytes < 1e9 else 12)
            except Exception as e:
                res[name] = {"error": f"{type(e).__name__}: {e}"[:200]}
                continue
            us = gr_us if gr_us is not None else ev_us
            gbs = nbytes / us / 1e3
            res[name] = {"us": round(us, 2), "event_us": round(ev_us, 2), "gbs": round(gbs, 1),
                         "frac_nominal": round(gbs / NOMINAL_HBM_GBS, 4), "frac_measured": round(gbs / peak, 4)}
        return res

    prefixes = ("cfg1", "cfg2", "cfg3", "cfg4")
    mine = {}
    for pfx in prefixes:
        mine.update(run_cases(BC.ours(), pfx, args.configs_budget_s))
    out["configs"] = mine
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if args.no_upstream:
        out["upstream_triton"] = {"unavailable": "--no-upstream"}
        return out
    try:
        ups = BC.upstream(ref_dir)
    except Exception as e:
        out["upstream_triton"] = {"unavailable": f"cannot import upstream from baseline/_ref: {type(e).__name__}: {e}"[:240]}
        return out
    try:
        rows_case = run_cases(ups, "cfg5", args.configs_budget_s * 2, " rows")   # the two calls of the benchmark step first
        mine5 = run_cases(BC.ours(), "cfg5", args.configs_budget_s * 2, " rows")
        up = {"source": "baseline/_ref (pip --target install of the unmodified reference), same process, same harness",
              "us_per_call": {}, "gbs": {}, "speedup": {}}
        for k, v in rows_case.items():
            short = "rmsnorm_quant" if "rmsnorm" in k else "swiglu_quant"
            if "us" in v and "us" in mine5.get(k, {}):
                up["us_per_call"][short] = v["us"]
                up["gbs"][short] = v["gbs"]
                up["speedup"][short] = round(v["us"] / mine5[k]["us"], 3)
                up.setdefault("ours_us_per_call", {})[short] = mine5[k]["us"]
            else:
                up["us_per_call"][short] = v
        for pfx in prefixes:
            for k, v in run_cases(ups, pfx, args.configs_budget_s * 3).items():
                if k in mine and "us" in v and "us" in mine[k]:
                    mine[k]["upstream_us"] = v["us"]
                    mine[k]["upstream_event_us"] = v["event_us"]
                    mine[k]["speedup"] = round(v["us"] / mine[k]["us"], 3)
                elif k in mine:
                    mine[k]["upstream"] = v
        out["upstream_triton"] = up
    except Exception as e:
        out["upstream_triton"] = {"unavailable": f"{type(e).__name__}: {e}"[:240]}
    return out


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the SwiGLU+quant kernel in an ncu
# capture at TRAFFIC_CAPTURE_ROWS rows (profiles/); traffic grows in proportion to the rows, so the
# bench line scales it by rows / TRAFFIC_CAPTURE_ROWS.
TRAFFIC_SWIGLU_BYTES = 1073767680 + 258864640     # dram__bytes_read.sum + dram__bytes_write.sum
TRAFFIC_CAPTURE_ROWS = 32768
TRAFFIC_NOTE = ("one launch captured at 32768 rows (profiles/), scaled by rows; reads equal the algorithmic input "
                "bytes, writes read 7 % low because the tail of the output is still dirty in L2 when the kernel "
                "ends (not a saving)")


def cpu_baseline(rows, repeats=1):
    """The CPU oracle (PyTorch reference math restated) on `rows` rows of the workload."""
    from oracle import oracle as O
    g = torch.Generator().manual_seed(7)
    xn = torch.randn((rows, HIDDEN), generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn((HIDDEN,), generator=g)).to(torch.bfloat16)
    xs = torch.randn((rows, 2 * HIDDEN), generator=g).to(torch.bfloat16)
    best = None
    for _ in range(repeats + 1):  # first pass warms the allocator
        t0 = time.perf_counter()
        y = torch.nn.functional.rms_norm(xn.float(), (HIDDEN,), gamma.float(), 1e-6)
        O.quant_rows_1x128(y)
        O.rms_recip(xn)
        O.quant_rows_1x128(O._swiglu_f32(xs))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    nbytes = norm_bytes(rows, HIDDEN) + silu_bytes(rows, HIDDEN)
    return {"value": round(nbytes / best / 1e9, 3), "unit": "GB/s", "cores": torch.get_num_threads(),
            "kind": "port", "sample": f"{rows} of {ROWS} rows of each tensor, {best:.2f} s per pass, "
                                      "torch CPU float32 oracle (oracle/oracle.py)"}


def run_reference(args, rank, world):
    """Reference arm: the reference's own CPU math (oracle port) on the host cores."""
    if rank != 0:
        return None
    # torchrun sets OMP_NUM_THREADS=1 for multi-rank launches; the CPU arm uses every core it may run on
    try:
        ncores = len(os.sched_getaffinity(0))
    except AttributeError:
        ncores = os.cpu_count() or 1
    torch.set_num_threads(max(ncores, 1))
    rows = args.cpu_rows
    from oracle import oracle as O  # noqa: F401
    res = []
    for i in range(max(args.warmup, 1) + args.steps):
        t0 = time.perf_counter()
        cb = cpu_baseline(rows, repeats=0)
        res.append((time.perf_counter() - t0, cb))
    timed = res[max(args.warmup, 1):]
    nbytes = norm_bytes(rows, HIDDEN) + silu_bytes(rows, HIDDEN)
    tot = sum(float(cb["sample"].split(" rows of each tensor, ")[1].split(" s")[0]) for _, cb in timed)
    value = nbytes * len(timed) / tot / 1e9
    cb = dict(timed[-1][1])
    cb["value"] = round(value, 3)
    return {
        "impl": "reference",
        "metric": "achieved HBM GB/s, fused RMSNorm+FP8 quant and SwiGLU+FP8 quant (algorithmic bytes / device time)",
        "value": round(value, 3), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 1), "ms_per_step": round(1e3 * tot / len(timed), 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 math, bf16 in, e4m3 out", "data": "synthetic",
        "config": {"workload": f"scaleout-{ROWS}x{HIDDEN} (bounded sample: {rows} rows per step on host CPU)"},
        "cpu_baseline": cb,
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS, help="rows per GPU (default: the benchmark size)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--cpu-rows", type=int, default=4096)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sustained-s", type=float, default=2.0, help="length of the back-to-back loop (0: skip)")
    ap.add_argument("--no-configs", action="store_true", help="skip the cfg1-cfg4 rows and the upstream column")
    ap.add_argument("--no-upstream", action="store_true", help="do not time the upstream Triton kernels")
    ap.add_argument("--configs-budget-s", type=float, default=60.0)
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        line = run_reference(args, rank, world)
        if line is not None:
            print(json.dumps(line), flush=True)
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; this benchmark has no CPU path (use --impl reference)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL prints a version banner on stdout when its first communicator comes up; stdout should
        # carry the JSON line only, so file descriptor 1 points at stderr until that has happened
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            torch.distributed.init_process_group("nccl", device_id=device)
            torch.distributed.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    try:
        line = run_ours(args, rank, world, device)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
