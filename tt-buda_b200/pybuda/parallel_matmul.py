"""Column-parallel matmul with Bfp8_b weights over the GPUs of one box.

Rank r holds columns [r*N/g, (r+1)*N/g) of the weight as a Bfp8_b queue image and all of the
activations; it computes its [M, N/g] slice with the tcgen05 kernel, and the slices are exchanged
in one of two ways:

  * fused (`enable_fused_scatter`, the fast path on GPUs): every rank keeps the full [M, N] output in
    device memory its peers can reach, and the matmul kernel's epilogue stores each finished tile
    into its own copy AND into every peer's copy over NVLink, while the tensor cores work on
    the next tile -- through the NVSwitch's multicast where the system offers it (one multimem store
    per value, replicated by the switch), else with one plain store per peer.  No all-gather, no
    staging, no permute pass: a barrier after the kernel is the only host-visible exchange step.
  * library all-gather (the baseline, and what CPU ranks test): the rows are cut into bands and band k
    is gathered with NCCL on a side stream while band k+1 is computed.
"""
from typing import Callable, Optional

import torch
import torch.distributed as dist

from .sharding import band_slices, column_shard, gather_layout_to_row_major


class ColumnParallelBfp8Matmul:
    def __init__(self, k: int, n: int, group=None, bands: int = 8,
                 local_matmul: Optional[Callable[[torch.Tensor, torch.Tensor, int, torch.Tensor], torch.Tensor]] = None,
                 scatter: Optional[Callable[[torch.Tensor], None]] = None, wait_local: Optional[Callable[[], None]] = None):
        """local_matmul(a, weight_image, n_local, out) -> out.  The default is the CUDA kernel; tests of the
        exchange logic on CPU ranks (gloo) pass a stand-in.  scatter(a) starts this rank's stores into every rank's
        output and wait_local() returns when they are done (defaults: the fused kernel on the current CUDA stream and
        a synchronisation of that stream)."""
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
        self._shared = None        # this rank's full output where the peers can reach it
        self._dst_ptrs = None
        self._mc = None            # set when the output lives in symmetric memory with a multicast mapping
        self._scatter = scatter if scatter is not None else self._scatter_kernel
        self._wait_local = wait_local if wait_local is not None else (lambda: torch.cuda.current_stream().synchronize())

    def enable_fused_scatter(self, m: int, multicast: Optional[bool] = None):
        """Allocate this rank's full [m, n] output where the peers can reach it.  Collective: every rank of the group
        calls it with the same arguments.  Two routes.  multicast=False: peer-mapped memory, one store per peer.
        multicast=True: the matrix in symmetric memory bound to one NVSwitch multicast object, so a rank's epilogue sends
        each value once and the switch replicates it (RuntimeError where the system has no such mapping).  Default
        (None): by measurement on B200 boxes -- peer stores up to 4 GPUs (0.405 against 0.445 ms at 4, where every GPU
        also gets its own block back through the switch), multicast from 8 GPUs on, where a rank would otherwise send
        its block seven times (0.439 against 0.457 ms), falling back to peer stores where there is no multicast."""
        from . import cuda_ops

        self.disable_fused_scatter()
        self._mc = None
        want = (self.world >= 8) if multicast is None else bool(multicast)
        if want and self.world > 1:
            self._mc = self._try_multicast(m)
            if self._mc is None and multicast:
                raise RuntimeError("no multicast (NVSwitch) mapping of symmetric memory on this system")
        if self._mc is not None:
            self._shared = self._mc
            return self._shared.tensor
        self._shared = cuda_ops.SharedDeviceMatrix(m, self.n)
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, self._shared.handle(), group=self.group)
        col_bytes = self.col0 * 2
        ptrs = [self._shared.ptr + col_bytes]
        for r in range(self.world):
            if r != self.rank:
                ptrs.append(self._shared.open_peer(handles[r]) + col_bytes)
        self._dst_ptrs = ptrs
        if self.world > 1:
            dist.barrier(group=self.group)
        return self._shared.tensor

    def _try_multicast(self, m: int):
        """The [m, n] output in torch's symmetric memory with a multicast mapping, or None when the system has none
        (every rank answers alike: the decision is agreed on with an all-reduce)."""
        from types import SimpleNamespace

        hdl = tensor = None
        try:
            import torch.distributed._symmetric_memory as symm_mem

            tensor = symm_mem.empty((m, self.n), dtype=torch.bfloat16, device=torch.device("cuda", torch.cuda.current_device()))
            hdl = symm_mem.rendezvous(tensor, self.group if self.group is not None else dist.group.WORLD)
            ok = int(hdl.multicast_ptr != 0)
        except Exception:   # noqa: BLE001  no symmetric memory / no fabric: the peer-mapped route still works
            ok = 0
        agreed = torch.tensor([ok], device="cuda")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=self.group)
        if int(agreed.item()) == 0:
            return None
        return SimpleNamespace(rows=m, tensor=tensor, handle=hdl, local_ptr=tensor.data_ptr(), mc_ptr=int(hdl.multicast_ptr),
                               close=lambda: None)

    @property
    def block_pointers(self):
        """Device addresses of this rank's block of columns in every copy of the output (this rank's own first), as the
        peer-store route uses them; None under the multicast route or before enable_fused_scatter."""
        return None if self._dst_ptrs is None else list(self._dst_ptrs)

    def disable_fused_scatter(self):
        if self._shared is not None:
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.group)   # nobody unmaps while a peer may still be storing
            self._shared.close()
            self._shared, self._dst_ptrs, self._mc = None, None, None

    @property
    def exchange(self) -> str:
        """How fused() reaches the peers: "multicast" (NVSwitch replication), "peer stores" or "off"."""
        if self._shared is None:
            return "off"
        return "multicast" if getattr(self, "_mc", None) is not None else "peer stores"

    def _scatter_kernel(self, a: torch.Tensor):
        from . import cuda_ops

        if getattr(self, "_mc", None) is not None:
            col_bytes = self.col0 * 2
            cuda_ops.bfp8b_matmul_multicast(a, self.weight_image, self.n_local, self._mc.local_ptr + col_bytes,
                                            self._mc.mc_ptr + col_bytes, self.n)
        else:
            cuda_ops.bfp8b_matmul_scatter(a, self.weight_image, self.n_local, self._dst_ptrs, self.n)

    def fused(self, a: torch.Tensor, sync: bool = True) -> torch.Tensor:
        """One kernel: this rank's column block, written into every rank's output.  With sync (default) the call
        returns when the [m, n] matrix is complete on every rank; with sync=False it only enqueues this rank's
        kernel, and complete() has to follow before anybody reads."""
        if self._shared is None or a.shape[0] != self._shared.rows:
            raise RuntimeError("enable_fused_scatter(m) first, with m = a.shape[0]")
        if self.weight_image is None:
            raise RuntimeError("load_weight_shard() first")
        self._scatter(a)
        if sync:
            self.complete()
        return self._shared.tensor

    def complete(self):
        """Makes the scattered result readable everywhere.  A rank may pass the barrier only when its OWN stores into
        the peers are done, so it first waits for its kernel -- whatever backend the group uses and whatever stream
        the kernel ran on; a barrier alone orders nothing that is still in flight on a device."""
        self._wait_local()
        if self.world > 1:
            dist.barrier(group=self.group)

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
