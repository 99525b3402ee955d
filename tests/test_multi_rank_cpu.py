"""World-size-2 tests of the multi-GPU host logic on CPU ranks (gloo): unit sharding and the banded
all-gather of the column-parallel matmul.  The local matmul is a stand-in here (the CUDA kernel needs
a GPU); what is under test is the exchange and the layout."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_round_robin_units_cover_everything_once():
    from pybuda.sharding import band_slices, column_shard, units_of_rank

    for n, world in ((64, 1), (64, 2), (64, 8), (24, 8), (5, 4)):
        seen = sorted(u for r in range(world) for u in units_of_rank(n, r, world))
        assert seen == list(range(n))
    assert units_of_rank(24, 3, 8) == [3, 11, 19]                   # 3 layers per GPU at g = 8
    assert band_slices(8192, 8, 256) == [(i * 1024, (i + 1) * 1024) for i in range(8)]
    assert band_slices(300, 4, 32) == [(0, 96), (96, 192), (192, 288), (288, 300)]
    assert column_shard(16384, 3, 8) == (6144, 8192)
    with pytest.raises(ValueError):
        column_shard(1000, 0, 8)
    with pytest.raises(ValueError):
        units_of_rank(4, 4, 4)


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.join(ROOT, "tt-buda_b200"))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pybuda.parallel_matmul import ColumnParallelBfp8Matmul

        m, k, n = 96, 64, 512
        g = torch.Generator().manual_seed(0)
        a = torch.randn(m, k, generator=g)
        w = torch.randn(k, n, generator=g)
        # stand-in for the device kernel: the "weight image" is simply the float shard
        op = ColumnParallelBfp8Matmul(k, n, bands=3, local_matmul=lambda a_, w_, nl, out: out.copy_(a_ @ w_))
        op.weight_image = w[:, op.col0:op.col1].contiguous()
        c = op(a)
        ok = torch.allclose(c, a @ w, atol=1e-5) and c.shape == (m, n)
        only_local = op(a, gather=False)
        ok = ok and torch.allclose(only_local, (a @ w)[:, op.col0:op.col1], atol=1e-5)
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_banded_all_gather_two_ranks_gloo():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29500 + (os.getpid() % 500)
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}
