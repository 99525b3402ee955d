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
    from pybuda.sharding import band_record_slice, bands_of_rank
    for rows, world in ((32, 8), (32, 3), (5, 8), (1, 2)):
        owned = sorted(b for r in range(world) for b in range(*(lambda f, s, c: (f, f + s * c, s))(*bands_of_rank(rows, r, world))))
        assert owned == list(range(rows))
    assert bands_of_rank(32, 5, 8) == (5, 8, 4) and bands_of_rank(5, 7, 8) == (7, 8, 0)
    # config 1: [1,1,1024,1024] -> 32 bands of 32 Bfp8_b records; band 3 is bytes [3*32*1088, 4*32*1088)
    assert band_record_slice(3, 32, 32, 1088) == (3 * 32 * 1088, 32 * 1088)
    assert band_record_slice(0, 4, 2, 1088, z=1, entry=2, t=3) == (((2 * 3 + 1) * 4 * 2) * 1088, 2 * 1088)
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


def _scatter_worker(rank, world, port, outs, results):
    """The fused exchange with stand-ins: "peer memory" is shared host memory, the "kernel" a thread that stores this
    rank's column block into every rank's output some time after the call returned."""
    import threading
    import time
    from types import SimpleNamespace

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, os.path.join(ROOT, "tt-buda_b200"))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pybuda.parallel_matmul import ColumnParallelBfp8Matmul

        m, k, n = 64, 32, 512
        g = torch.Generator().manual_seed(1)
        a = torch.randn(m, k, generator=g)
        w = torch.randn(k, n, generator=g)
        pending = []

        def scatter(a_):
            def run():
                time.sleep(0.4 if rank == 0 else 0.05)          # rank 0's "kernel" is the slow one
                block = a_ @ w[:, op.col0:op.col1]
                for o in outs:
                    o[:, op.col0:op.col1] = block
            t = threading.Thread(target=run)
            t.start()
            pending.append(t)

        def wait_local():
            while pending:
                pending.pop().join()

        op = ColumnParallelBfp8Matmul(k, n, scatter=scatter, wait_local=wait_local)
        op.weight_image = w[:, op.col0:op.col1].contiguous()
        op._shared = SimpleNamespace(rows=m, tensor=outs[rank])
        c = op.fused(a)
        # complete everywhere the moment fused() returns: the fast rank must have waited for the slow rank's stores
        ok = torch.allclose(c, a @ w, atol=1e-5)
        # without the completion step the result must NOT be claimed: the call returns with stores still pending
        dist.barrier()
        for o in outs[rank:rank + 1]:
            o.zero_()
        dist.barrier()
        op.fused(a, sync=False)
        still_pending = len(pending) == 1
        op.complete()
        ok = ok and still_pending and torch.allclose(outs[rank], a @ w, atol=1e-5)
        results[rank] = bool(ok)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_fused_exchange_is_complete_when_the_call_returns_two_ranks_gloo():
    world = 2
    outs = [torch.zeros(64, 512).share_memory_() for _ in range(world)]
    mgr = mp.Manager()
    results = mgr.dict()
    port = 30100 + (os.getpid() % 500)
    mp.spawn(_scatter_worker, args=(world, port, outs, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def _band_worker(rank, world, port, image, results):
    """Tile-row bands of one tensor dealt to the ranks (band b -> rank b % world).  On CPU ranks the conversion of a
    band is done by the oracle (the CUDA kernel needs a GPU); what is under test is who owns which band and where its
    records land in the shared image."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    for p in (ROOT, os.path.join(ROOT, "tt-buda_b200")):
        sys.path.insert(0, p)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import numpy as np
        from oracle import budaref as R
        from pybuda.sharding import band_record_slice, bands_of_rank

        R.build()
        x = torch.randn(1, 1, 1024, 1024, generator=torch.Generator().manual_seed(0)).numpy()      # config 1
        rt, ct = 32, 32
        first, step, count = bands_of_rank(rt, rank, world)
        img = image.numpy()
        for b in range(first, first + step * count, step):
            off, n = band_record_slice(b, rt, ct, 1088)
            img[off:off + n] = R.tilize_pack(x[:, :, b * 32:(b + 1) * 32, :], R.Bfp8_b)
        dist.barrier()
        results[rank] = bool(np.array_equal(img, R.tilize_pack(x, R.Bfp8_b)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_tile_row_bands_two_ranks_gloo():
    world = 2
    image = torch.zeros(1114112, dtype=torch.uint8).share_memory_()
    mgr = mp.Manager()
    results = mgr.dict()
    port = 30700 + (os.getpid() % 500)
    mp.spawn(_band_worker, args=(world, port, image, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}
