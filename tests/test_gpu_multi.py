"""Two-GPU tests (skipped on a one-GPU box): tensors sharded round-robin with no collective, and the
column-parallel Bfp8_b matmul whose output slices are exchanged by an NCCL all-gather."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    for p in (ROOT, os.path.join(ROOT, "tt-buda_b200")):
        sys.path.insert(0, p)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import numpy as np
        from oracle import budaref as R
        from pybuda import cuda_ops
        from pybuda.parallel_matmul import ColumnParallelBfp8Matmul
        from pybuda.sharding import units_of_rank

        torch.backends.cuda.matmul.allow_tf32 = False
        ok = True
        # independent tensors: tensor i -> rank i % world, packed on that rank's GPU, checked against the oracle
        for i in units_of_rank(6, rank, world):
            x = torch.randn(1, 1, 256, 512, generator=torch.Generator().manual_seed(1000 + i))
            img = cuda_ops.tilize_pack(x.cuda(), cuda_ops.DF.Bfp8_b)
            ok = ok and np.array_equal(img.cpu().numpy(), R.tilize_pack(x.numpy(), R.Bfp8_b))
        # column-parallel matmul: every rank ends with the full [M, N] product
        m, k, n = 1024, 512, 1024
        g = torch.Generator().manual_seed(6)
        a = torch.randn(m, k, generator=g).bfloat16().cuda()
        w = torch.randn(k, n, generator=g) * 0.02
        op = ColumnParallelBfp8Matmul(k, n, bands=4)
        op.load_weight_shard(w)
        c = op(a)
        full_img = cuda_ops.tilize_pack(w.reshape(1, 1, k, n).cuda(), cuda_ops.DF.Bfp8_b)
        wd = cuda_ops.unpack_untilize(full_img, cuda_ops.DF.Bfp8_b, (1, 1, k, n))[0, 0]
        ref = a.float() @ wd
        rel = ((c.float() - ref.bfloat16().float()).norm() / ref.norm()).item()
        ok = ok and rel <= 1e-3 and c.shape == (m, n)
        single = cuda_ops.bfp8b_matmul(a, full_img, n)
        ok = ok and torch.equal(single, c)            # same kernel, same k order: identical bits
        # the same product with the exchange fused into the kernel: each rank's epilogue stores its column
        # block into every rank's output through peer-mapped memory
        fused_equal, routes = True, []
        for multicast in (False, True):                 # one store per peer; then the switch's multicast where there is one
            try:
                out = op.enable_fused_scatter(m, multicast=multicast)
            except RuntimeError:
                routes.append("no multicast on this system")
                continue
            routes.append(op.exchange)
            out.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            for _ in range(2):
                cf = op.fused(a)
            torch.cuda.synchronize()
            fused_equal = fused_equal and torch.equal(cf, single)
            op.disable_fused_scatter()
        ok = ok and fused_equal and routes[0] == "peer stores"
        # tile-row bands of ONE tensor dealt to the ranks (band b -> rank b % world): every rank packs its bands into
        # its own copy of the image; merged by ownership on rank 0 they are the oracle's image of the whole tensor
        from pybuda.sharding import band_record_slice, bands_of_rank
        x1 = torch.randn(1, 1, 1024, 1024, generator=torch.Generator().manual_seed(0))
        ref1 = R.tilize_pack(x1.numpy(), R.Bfp8_b)
        mine = torch.full((ref1.size,), 0xAB, dtype=torch.uint8, device="cuda")
        cuda_ops.tilize_pack_jobs([x1.cuda()], cuda_ops.DF.Bfp8_b, outs=[mine], bands=[bands_of_rank(32, rank, world)])
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        merged = np.empty(ref1.size, np.uint8)
        for b in range(32):
            off, nb = band_record_slice(b, 32, 32, 1088)
            merged[off:off + nb] = gathered[b % world][off:off + nb].cpu().numpy()
            other = gathered[(b + 1) % world][off:off + nb].cpu().numpy()
            ok = ok and bool((other == 0xAB).all())               # nobody touches a band it does not own
        bands_equal = bool(np.array_equal(merged, ref1))
        ok = ok and bands_equal
        results[rank] = (bool(ok), rel, bool(fused_equal), bands_equal, routes)
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharding_and_column_parallel_matmul():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29700 + (os.getpid() % 200)
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert all(v[0] for v in results.values()), dict(results)
