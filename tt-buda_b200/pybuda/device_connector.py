"""Direct device connectors (reference: pybuda/pybuda/device_connector.py:131-375): the objects through which a
host process pushes a set of tensors into a device's input queues and reads / pops its output queues.  The
pusher converts each tensor to a type the queue's converter accepts, applies the runtime tensor transform, pads to
tiles and calls BackendAPI.push_to_queues — on the caller's thread (sequential) or on a pusher thread fed through a
bounded command queue, as in the reference.  Inter-process transports (multiprocessing queues, torch queues) of
the reference are not part of this path."""
import queue
import threading
from typing import List, Optional, Tuple, Union

import torch

from . import TILE_DIM
from ._C import DataFormat
from ._C.backend_api import DramIODesc, PytorchTensorDesc
from .backend import BackendAPI
from .tensor import (RuntimeTensorTransform, RuntimeTensorTransformType, Tensor, _embedding_index, is_equivalent_data_format,
                     pad_pytorch_tensor_to_buda, pytorch_tensor_to_tensor_desc)


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

    def pusher_thread_main(self, cmdqueue: queue.Queue):
        while True:
            while True:
                try:
                    cmd = cmdqueue.get(timeout=0.1)
                    break
                except queue.Empty:
                    if self.shutdown_event is not None and self.shutdown_event.is_set():
                        return
                    continue
            if cmd == "quit":
                return
            try:
                self._internal_push(cmd)
            except Exception as exc:  # noqa: BLE001  surfaced to the caller by wait_for_pushes()
                self.push_error = exc
            finally:
                cmdqueue.task_done()

    def shutdown(self):
        if self.pusher_thread:
            self.pusher_thread_queue.put("quit")
            self.pusher_thread.join(timeout=10)
            self.pusher_thread = None

    def initialize(self):
        if not self.sequential and not self.pusher_thread:
            # don't allow pushes to go too far ahead, or we'll run out of memory
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

    def _convert_tensor_for_tilize(self, tensor: Tensor, q: DramIODesc) -> Tensor:
        """Convert formats to the closest format the queue's converter takes."""
        if is_equivalent_data_format(tensor.pt_data_format, q.data_format):
            return tensor
        pt_format = tensor.value().dtype
        if not tensor.value().is_floating_point():
            return tensor.to_format(q.data_format)
        if q.data_format in [DataFormat.Float16, DataFormat.Bfp8, DataFormat.Bfp4, DataFormat.Bfp2]:
            if pt_format != torch.float16:          # tensor has to be float16
                return tensor.to_format(DataFormat.Float16)
            return tensor
        if q.data_format in [DataFormat.Float16_b, DataFormat.Bfp8_b, DataFormat.Bfp4_b, DataFormat.Bfp2_b]:
            if pt_format not in [torch.float32, torch.bfloat16]:   # tensor can be bfloat or fp32
                return tensor.to_format(DataFormat.Float16_b)
            return tensor
        return tensor

    def _internal_push(self, tensors: List[Union[Tensor, torch.Tensor]]):
        assert self.direct_push_queues, "Direct push queues have not been set"
        assert self.tile_broadcast_dims is not None
        assert len(tensors) == len(self.direct_push_queues), (
            f"Incorrect number of tensors provided on input: {len(tensors)} vs {len(self.direct_push_queues)}")
        assert self.runtime_tensor_transforms, "Runtime tensor transforms have not been set"
        assert len(tensors) == len(self.runtime_tensor_transforms)
        tensors = list(tensors)
        tensor_dtypes = [None] * len(tensors)

        for i, t in enumerate(tensors):
            if isinstance(t, Tensor):
                tensors[i] = self._convert_tensor_for_tilize(t, self.direct_push_queues[i])

        for i, t in enumerate(tensors):
            transform = self.runtime_tensor_transforms[i]
            if transform.type == RuntimeTensorTransformType.EmbeddingIndex:
                if isinstance(t, Tensor):
                    t = t.value()
                t = _embedding_index(t, transform.original_shape.dims, self.direct_push_queues[i])
                tensors[i] = t
                tensor_dtypes[i] = DataFormat.RawUInt32
                continue
            elif transform.type == RuntimeTensorTransformType.ConstantInput:
                assert self.constant_tensors[i] is not None
                tensors[i] = self.constant_tensors[i]
                t = tensors[i]

            if isinstance(tensors[i], torch.Tensor):
                if transform.type == RuntimeTensorTransformType.ReinterpretShape:
                    t = t.contiguous().view(list(transform.reinterpreted_shape.dims))
                elif transform.type == RuntimeTensorTransformType.Prestride:
                    continue
                tile_r = self.tile_dims[i][0] if self.tile_dims is not None else TILE_DIM
                tile_c = self.tile_dims[i][1] if self.tile_dims is not None else TILE_DIM
                tensors[i] = pad_pytorch_tensor_to_buda(t, self.tile_broadcast_dims[i], squeeze=True, microbatch=self.microbatch,
                                                        tile_r=tile_r, tile_c=tile_c)
            else:
                if transform.type == RuntimeTensorTransformType.ReinterpretShape:
                    tensors[i] = t.to_buda_shape(self.tile_broadcast_dims[i], reinterpret_shape=list(transform.reinterpreted_shape.dims),
                                                 clone=False, squeeze=True, microbatch=self.microbatch)
                elif transform.type == RuntimeTensorTransformType.Prestride:
                    pass
                elif transform.type == RuntimeTensorTransformType.NoTransform:
                    tensors[i] = t.to_buda_shape(self.tile_broadcast_dims[i], reinterpret_shape=None, clone=False, squeeze=True,
                                                 microbatch=self.microbatch)

        def to_tensor_desc(t: Union[Tensor, torch.Tensor], df: Optional[DataFormat]) -> PytorchTensorDesc:
            if isinstance(t, Tensor):
                return t.to_tensor_desc()
            return pytorch_tensor_to_tensor_desc(t, df=df)

        BackendAPI.push_to_queues(self.direct_push_queues, [to_tensor_desc(t, df) for t, df in zip(tensors, tensor_dtypes)],
                                  single_input=False)
        self.save_tensors = tensors

    def push(self, tensors: List[Tensor]):
        if not self.sequential:
            assert self.pusher_thread is not None, "initialize() starts the pusher thread"
            self.pusher_thread_queue.put(tensors)
        else:
            self._internal_push(tensors)

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

    def read(self) -> List[Tensor]:
        assert self.direct_pop_queues is not None, "Direct pop queues have not been set"
        if len(self.direct_pop_queues) == 0:
            return []
        assert self.original_shapes is not None
        return BackendAPI.read_queues(self.direct_pop_queues, self.original_shapes, self.runtime_tensor_transforms,
                                      requires_grad=self.requires_grad, single_output=False, shutdown_event=self.shutdown_event,
                                      clone=False)

    def pop(self):
        assert self.direct_pop_queues is not None, "Direct pop queues have not been set"
        if len(self.direct_pop_queues) == 0:
            return
        BackendAPI.pop_queues(self.direct_pop_queues, single_output=False)

    def set_dram_io_pop_queues(self, direct_pop_queues: List[DramIODesc], original_shapes: List[Tuple[int, ...]],
                               requires_grad: List[bool], runtime_tensor_transforms: Optional[List[RuntimeTensorTransform]]):
        self.direct_pop_queues = direct_pop_queues
        self.original_shapes = original_shapes
        self.requires_grad = requires_grad
        self.runtime_tensor_transforms = runtime_tensor_transforms
