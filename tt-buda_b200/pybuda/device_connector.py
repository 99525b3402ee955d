"""Direct device connectors (reference: pybuda/pybuda/device_connector.py:131-375): the objects through which a
host process pushes a set of tensors into a device's input queues and reads / pops its output queues.  The
pusher converts each tensor to a type the queue's converter accepts, describes the runtime tensor transform and the tile
padding to the pack kernel as a source view (the data itself is not rewritten on the host) and pushes the whole set in
one backend call — on the caller's thread (sequential) or on a pusher thread fed through a
bounded command queue, as in the reference.  Inter-process transports (multiprocessing queues, torch queues) of
the reference are not part of this path."""
import queue
import threading
from typing import List, Optional, Tuple, Union

import torch

from . import TILE_DIM
from ._C import DataFormat
from ._C.backend_api import DramIODesc, PytorchTensorDesc, SourceView, SourceViewMode
from .backend import BackendAPI
from .tensor import (RuntimeTensorTransform, RuntimeTensorTransformType, Tensor, TilePadding, embedding_index_layout,
                     is_equivalent_data_format, pytorch_tensor_to_tensor_desc)


class DirectPusherDeviceConnector:
    """Connector in which one side directly pushes (tilizes) into the other's queues."""

    def __init__(self, shutdown_event: Optional[threading.Event], sequential: bool, microbatch=1):
        self.shutdown_event = shutdown_event
        self.direct_push_queues = None
        self.sequential = sequential
        self.tile_broadcast_dims = None
        self.runtime_tensor_transforms: List[RuntimeTensorTransform] = None
        self.constant_tensors = None
        self.tile_dims = None
        self.microbatch = microbatch
        self.pusher_thread = None
        self.pusher_thread_queue = None
        self.push_error = None

    _QUIT = "quit"

    def pusher_thread_main(self, cmdqueue: queue.Queue):
        """Body of the pusher thread: sets of tensors arrive through the command queue and are pushed in order.  The
        thread wakes ten times a second to see whether the process is shutting down."""
        stop = self.shutdown_event
        while stop is None or not stop.is_set():
            try:
                work = cmdqueue.get(timeout=0.1)
            except queue.Empty:
                continue
            try:
                if isinstance(work, str) and work == self._QUIT:
                    return
                self._internal_push(work)
            except Exception as exc:  # noqa: BLE001  handed to the caller by wait_for_pushes()
                self.push_error = exc
            finally:
                cmdqueue.task_done()

    def shutdown(self):
        thread, self.pusher_thread = self.pusher_thread, None
        if thread is not None:
            self.pusher_thread_queue.put(self._QUIT)
            thread.join(timeout=10)

    def initialize(self):
        if self.sequential or self.pusher_thread is not None:
            return
        # a short command queue: pushes must not run far ahead of the device, their tensors are kept alive meanwhile
        self.pusher_thread_queue = queue.Queue(maxsize=3)
        self.pusher_thread = threading.Thread(target=self.pusher_thread_main, args=(self.pusher_thread_queue,), daemon=True)
        self.pusher_thread.start()

    def wait_for_pushes(self):
        """Blocks until the pusher thread has drained its command queue; re-raises a push that failed there."""
        if self.pusher_thread_queue is not None:
            self.pusher_thread_queue.join()
        if self.push_error is not None:
            err, self.push_error = self.push_error, None
            raise err

    # Which torch dtypes a queue's converter takes as they are, and what everything else is cast to first.
    _FLOAT_FAMILIES = (
        ((DataFormat.Float16, DataFormat.Bfp8, DataFormat.Bfp4, DataFormat.Bfp2), (torch.float16,), DataFormat.Float16),
        ((DataFormat.Float16_b, DataFormat.Bfp8_b, DataFormat.Bfp4_b, DataFormat.Bfp2_b), (torch.float32, torch.bfloat16),
         DataFormat.Float16_b),
    )

    def _convert_tensor_for_tilize(self, tensor: Tensor, q: DramIODesc) -> Tensor:
        """The tensor in a torch dtype the queue's converter accepts: the 5-bit-exponent family takes float16, the
        8-bit-exponent family float32 or bfloat16, integers are cast to the queue's own type; anything the table does
        not know is left for the converter to judge."""
        have = tensor.pt_data_format
        if is_equivalent_data_format(have, q.data_format):
            return tensor
        if not tensor.value().is_floating_point():
            return tensor.to_format(q.data_format)
        for family, accepted, fallback in self._FLOAT_FAMILIES:
            if q.data_format in family:
                return tensor if have in accepted else tensor.to_format(fallback)
        return tensor

    def _tile_dims(self, slot: int) -> Tuple[int, int]:
        return tuple(self.tile_dims[slot]) if self.tile_dims is not None else (TILE_DIM, TILE_DIM)

    def _stage(self, slot: int, item: Union[Tensor, torch.Tensor]):
        """One pushed tensor -> (torch value to keep alive, descriptor, source view or None).  Padding, tile broadcast
        and the embedding-index layout are not applied to the data here: they are handed to the pack kernel as a
        source view, which reads the tensor accordingly while it writes the queue's tiles."""
        q = self.direct_push_queues[slot]
        transform = self.runtime_tensor_transforms[slot]
        kind = transform.type
        if kind == RuntimeTensorTransformType.ConstantInput:
            assert self.constant_tensors[slot] is not None, "a constant input needs its tensor"
            item, kind = self.constant_tensors[slot], RuntimeTensorTransformType.NoTransform
        if isinstance(item, Tensor):
            item = self._convert_tensor_for_tilize(item, q)
        value = item.value() if isinstance(item, Tensor) else item
        df = item.data_format if isinstance(item, Tensor) and int(item.data_format) >= 0xF0 else None

        if kind == RuntimeTensorTransformType.EmbeddingIndex:
            count = transform.original_shape.dims[-1]
            idx = value.reshape(-1, value.shape[-1]).to(torch.int32).contiguous()
            q_rt = q.bufq_grid_dim_r * q.mblock_m * q.ublock_rt
            view = SourceView()
            view.mode = SourceViewMode.EmbeddingIndex
            view.count = count
            view.group, _ = embedding_index_layout(count, idx.shape[-1], q_rt)
            return idx, pytorch_tensor_to_tensor_desc(idx.view(idx.shape[0], 1, 1, idx.shape[1]), df=DataFormat.RawUInt32), view
        if kind == RuntimeTensorTransformType.Prestride:
            return value, pytorch_tensor_to_tensor_desc(value, df=df), None          # the queue's stride descriptor does the rest
        if kind == RuntimeTensorTransformType.ReinterpretShape:
            dims = list(transform.reinterpreted_shape.dims)
            if isinstance(item, Tensor) and dims[0] == 1:
                dims[0] = self.microbatch
            value = value.contiguous().view(dims)
        elif kind != RuntimeTensorTransformType.NoTransform:
            raise AssertionError(f"Unsupported runtime transform type: {kind}")

        tile_r, tile_c = self._tile_dims(slot)
        plan = TilePadding(value, self.tile_broadcast_dims[slot], True, self.microbatch, tile_r, tile_c)
        if plan.aligned:
            return plan.view, pytorch_tensor_to_tensor_desc(plan.view, df=df), None
        if plan.view.dim() != 4 or tile_r != TILE_DIM or tile_c != TILE_DIM or plan.view.stride(-1) != 1:
            padded = plan.materialise()                                               # tiny tiles and odd layouts: pad on the host
            return padded, pytorch_tensor_to_tensor_desc(padded, df=df), None
        view = SourceView()
        view.mode = SourceViewMode.Padded
        view.broadcast_rows, view.broadcast_cols = plan.rep_r, plan.rep_c
        src = plan.view.contiguous()
        return src, pytorch_tensor_to_tensor_desc(src, df=df), view

    def _internal_push(self, tensors: List[Union[Tensor, torch.Tensor]]):
        queues = self.direct_push_queues
        assert queues, "set_dram_io_push_queues() has not been called"
        assert self.tile_broadcast_dims is not None and self.runtime_tensor_transforms, "push queues were set without their transforms"
        assert len(tensors) == len(queues) == len(self.runtime_tensor_transforms), (
            f"{len(tensors)} tensors pushed to {len(queues)} queues")
        staged = [self._stage(slot, item) for slot, item in enumerate(tensors)]
        BackendAPI.push_staged(queues, [(desc, view) for _, desc, view in staged], single_input=False)
        self.save_tensors = [value for value, _, _ in staged]

    def push(self, tensors: List[Tensor]):
        if self.sequential:
            self._internal_push(tensors)
            return
        assert self.pusher_thread is not None, "initialize() starts the pusher thread"
        self.pusher_thread_queue.put(tensors)

    def set_dram_io_push_queues(self, direct_push_queues: List[DramIODesc], tile_broadcast_dims: List[List[int]],
                                runtime_tensor_transforms: Optional[List[RuntimeTensorTransform]],
                                constant_tensors: Optional[List[Tensor]] = None, tile_dims: Optional[List[List[int]]] = None):
        self.direct_push_queues = direct_push_queues
        self.tile_broadcast_dims = tile_broadcast_dims
        self.runtime_tensor_transforms = (runtime_tensor_transforms if runtime_tensor_transforms is not None
                                          else [RuntimeTensorTransform() for _ in range(len(direct_push_queues))])
        self.constant_tensors = constant_tensors if constant_tensors is not None else [None for _ in range(len(direct_push_queues))]
        self.tile_dims = tile_dims


class DirectPopperDeviceConnector:
    """Connector in which one side produces data directly into queues, and the other pops from them."""

    def __init__(self, shutdown_event: Optional[threading.Event]):
        self.shutdown_event = shutdown_event
        self.direct_pop_queues = None
        self.original_shapes = None
        self.requires_grad = None
        self.runtime_tensor_transforms = None

    def _queues(self) -> List[DramIODesc]:
        assert self.direct_pop_queues is not None, "set_dram_io_pop_queues() has not been called"
        return self.direct_pop_queues

    def read(self) -> List[Tensor]:
        queues = self._queues()
        if not queues:
            return []
        assert self.original_shapes is not None, "pop queues were set without the tensors' original shapes"
        return BackendAPI.read_queues(queues, self.original_shapes, self.runtime_tensor_transforms, requires_grad=self.requires_grad,
                                      single_output=False, shutdown_event=self.shutdown_event, clone=False)

    def pop(self):
        queues = self._queues()
        if queues:
            BackendAPI.pop_queues(queues, single_output=False)

    def set_dram_io_pop_queues(self, direct_pop_queues: List[DramIODesc], original_shapes: List[Tuple[int, ...]],
                               requires_grad: List[bool], runtime_tensor_transforms: Optional[List[RuntimeTensorTransform]]):
        self.direct_pop_queues = direct_pop_queues
        self.original_shapes = original_shapes
        self.requires_grad = requires_grad
        self.runtime_tensor_transforms = runtime_tensor_transforms
