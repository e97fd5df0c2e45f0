"""Row sharding across ranks, exercised on CPU with the gloo backend and world size 2:
the oracle stands in for the kernels, the sharding / gather code is the product's."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from linghe_b200.tools.shard import shard_rows, run_sharded
from oracle import oracle as O


def test_shard_rows_aligned():
    for M in (128, 1000, 4096, 65536, 130):
        for world in (1, 2, 3, 8):
            spans = [shard_rows(M, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == M
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a1 % 128 == 0
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(s for s in sizes) <= 128 + 127


def _worker(rank, world, port, M, n, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    g = torch.Generator().manual_seed(3)
    x = torch.randn((M, 2 * n), generator=g).to(torch.bfloat16)
    got = run_sharded(lambda xl: O.silu_and_block_quant_forward(xl, False), x, world, rank, "cpu")
    if rank == 0:
        ref = O.silu_and_block_quant_forward(x, False)
        ok = all(torch.equal(a.view(torch.uint8) if a.dtype == torch.float8_e4m3fn else a,
                             b.view(torch.uint8) if b.dtype == torch.float8_e4m3fn else b)
                 for a, b in zip(got, ref))
        ret.put(ok)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("M", [512, 1000])
def test_sharded_equals_single_rank_gloo(M):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = 29611 + (M % 7)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, M, 256, ret)) for r in range(2)]
    for p in procs:
        p.start()
    ok = ret.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok
