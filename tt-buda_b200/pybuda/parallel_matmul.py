"""Column-parallel matmul with Bfp8_b weights over the GPUs of one box.

Rank r holds columns [r*N/g, (r+1)*N/g) of the weight as a Bfp8_b queue image and all of the
activations; it computes its [M, N/g] slice with the tcgen05 kernel, and the slices are exchanged
with an NCCL all-gather over NVLink.  At 8 GPUs the gather of the 256 MiB output takes longer than
the 1/8-size matmul, so the rows are cut into bands: while band k is gathered on a side stream,
band k+1 is computed.
"""
from typing import Callable, Optional

import torch
import torch.distributed as dist

from .sharding import band_slices, column_shard, gather_layout_to_row_major


class ColumnParallelBfp8Matmul:
    def __init__(self, k: int, n: int, group=None, bands: int = 8,
                 local_matmul: Optional[Callable[[torch.Tensor, torch.Tensor, int, torch.Tensor], torch.Tensor]] = None):
        """local_matmul(a, weight_image, n_local, out) -> out.  The default is the CUDA kernel; tests of the
        exchange logic on CPU ranks (gloo) pass a stand-in."""
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.k, self.n, self.bands = k, n, bands
        self.col0, self.col1 = column_shard(n, self.rank, self.world)
        self.n_local = self.col1 - self.col0
        if local_matmul is None:
            from . import cuda_ops

            local_matmul = lambda a, w, nl, out: cuda_ops.bfp8b_matmul(a, w, nl, out=out)
        self._mm = local_matmul
        self.weight_image = None

    def load_weight_shard(self, w_full_or_shard: torch.Tensor, already_sharded: bool = False):
        """Pack this rank's columns of a [K, N] float weight to a Bfp8_b queue image on its device."""
        from . import cuda_ops

        w = w_full_or_shard if already_sharded else w_full_or_shard[..., self.col0:self.col1]
        w = w.reshape(1, 1, self.k, self.n_local).contiguous()
        self.weight_image = cuda_ops.tilize_pack(w.cuda() if not w.is_cuda else w, cuda_ops.DF.Bfp8_b)
        return self.weight_image

    def __call__(self, a: torch.Tensor, out: Optional[torch.Tensor] = None, gather: bool = True) -> torch.Tensor:
        m = a.shape[0]
        if self.weight_image is None:
            raise RuntimeError("load_weight_shard() first")
        local = torch.empty((m, self.n_local), dtype=a.dtype, device=a.device)
        if self.world == 1 or not gather:
            self._mm(a, self.weight_image, self.n_local, local)
            return local
        if out is None:
            out = torch.empty((m, self.n), dtype=a.dtype, device=a.device)
        on_gpu = a.is_cuda
        comm = torch.cuda.Stream(device=a.device) if on_gpu else None
        slices = band_slices(m, self.bands, 256 if on_gpu else 1)
        band_rows = slices[0][1] - slices[0][0]
        staging = torch.empty(self.world * band_rows * self.n_local, dtype=a.dtype, device=a.device)
        for (r0, r1) in slices:
            rows = r1 - r0
            self._mm(a[r0:r1], self.weight_image, self.n_local, local[r0:r1])
            # the gather concatenates the ranks' [rows, n_local] slices along dim 0
            stage = staging[: self.world * rows * self.n_local].view(self.world * rows, self.n_local)
            if on_gpu:
                done = torch.cuda.Event()
                done.record()
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    dist.all_gather_into_tensor(stage, local[r0:r1], group=self.group)
                    gather_layout_to_row_major(stage.view(self.world, rows, self.n_local), out[r0:r1])
            else:
                dist.all_gather_into_tensor(stage, local[r0:r1], group=self.group)
                gather_layout_to_row_major(stage.view(self.world, rows, self.n_local), out[r0:r1])
        if on_gpu:
            torch.cuda.current_stream().wait_stream(comm)
        return out
