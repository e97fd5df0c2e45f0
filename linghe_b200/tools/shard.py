"""Row sharding of the fused norm / SwiGLU + FP8 quant path across ranks, and the
validation gather.

The path has no exchange step: every output depends only on its own row (1x128 row
blocks), its own 128-row block (128x1 column blocks) or its own expert segment.  Ranks
therefore own contiguous row slices whose boundaries are multiples of 128 rows and run
the single-GPU entry points unchanged.  The only collective is the all-gather used to
*validate* a sharded run against a single-rank computation:

    torchrun --nproc-per-node N -m linghe_b200.tools.shard --rows 4096 --hidden 2048
"""

from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

BLOCK = 128


def shard_rows(M: int, world: int, rank: int):
    """[r0, r1) of `rank`: contiguous, 128-row aligned, balanced to within one block."""
    blocks = (M + BLOCK - 1) // BLOCK
    b0 = blocks * rank // world
    b1 = blocks * (rank + 1) // world
    return min(M, b0 * BLOCK), min(M, b1 * BLOCK)


def gather_outputs(local, world: int, rank: int, rows_per_rank, device):
    """All-gather per-rank (q [m,n], s [nb,m], qT [n,m], sT [m/128,n]) and assemble the global
    tensors on every rank.  Row-sharded `s` and `qT` are column slices of the global arrays."""
    q, s, qt, st = local
    max_rows = max(rows_per_rank)

    def pad_rows(t, dim, to):
        if t.shape[dim] == to:
            return t.contiguous()
        shape = list(t.shape)
        shape[dim] = to - t.shape[dim]
        return torch.cat([t, torch.zeros(shape, dtype=t.dtype, device=t.device)], dim).contiguous()

    def gather(t):
        bufs = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(bufs, t)
        return bufs

    q_all = gather(pad_rows(q.view(torch.uint8), 0, max_rows))
    s_all = gather(pad_rows(s, 1, max_rows))
    qt_all = gather(pad_rows(qt.view(torch.uint8), 1, max_rows))
    st_all = gather(pad_rows(st, 0, (max_rows + BLOCK - 1) // BLOCK))
    Q = torch.cat([t[:m] for t, m in zip(q_all, rows_per_rank)], 0).view(torch.float8_e4m3fn)
    S = torch.cat([t[:, :m] for t, m in zip(s_all, rows_per_rank)], 1)
    QT = torch.cat([t[:, :m] for t, m in zip(qt_all, rows_per_rank)], 1).view(torch.float8_e4m3fn)
    ST = torch.cat([t[:(m + BLOCK - 1) // BLOCK] for t, m in zip(st_all, rows_per_rank)], 0)
    return Q, S, QT, ST


def run_sharded(fn, x_global: torch.Tensor, world: int, rank: int, device):
    """Run `fn(x_shard) -> (q, s, qT, sT)` on this rank's rows of `x_global` and return the
    assembled global outputs (validation path: uses one all-gather per output)."""
    M = x_global.shape[0]
    spans = [shard_rows(M, world, r) for r in range(world)]
    r0, r1 = spans[rank]
    local = fn(x_global[r0:r1].contiguous().to(device))
    return gather_outputs(local, world, rank, [b - a for a, b in spans], device)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=2048)
    a = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    from linghe_b200.utils.norm import triton_rms_norm_and_block_quant_forward as norm_q
    from linghe_b200.utils.silu import triton_silu_and_block_quant_forward as silu_q
    g = torch.Generator().manual_seed(0)
    x = torch.randn((a.rows, a.hidden), generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(a.hidden, generator=g)).to(torch.bfloat16)
    xs = torch.randn((a.rows, 2 * a.hidden), generator=g).to(torch.bfloat16)
    gd = gamma.to(device)

    def f_norm(xl):
        q, s, _, qt, st = norm_q(xl, gd, output_mode=2)
        return q, s, qt, st

    outs_n = run_sharded(f_norm, x, world, rank, device)
    outs_s = run_sharded(lambda xl: silu_q(xl, output_mode=2), xs, world, rank, device)
    ok = True
    if rank == 0:
        ref_n = norm_q(x.to(device), gd, output_mode=2)
        ref_n = (ref_n[0], ref_n[1], ref_n[3], ref_n[4])
        ref_s = silu_q(xs.to(device), output_mode=2)
        for name, got, ref in (("rmsnorm", outs_n, ref_n), ("swiglu", outs_s, ref_s)):
            for g_, r_ in zip(got, ref):
                same = torch.equal(g_.view(torch.uint8) if g_.dtype == torch.float8_e4m3fn else g_,
                                   r_.view(torch.uint8) if r_.dtype == torch.float8_e4m3fn else r_)
                ok = ok and same
            print(f"{name}: sharded x{world} == single-GPU: {ok}")
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0 and not ok:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
