"""Queue side of the reference's BackendAPI (pybuda/pybuda/backend.py:341-493): the class methods that push
tensors into device queues, read them back and pop them.  Same names, arguments, retry and assertion behaviour.
The compile / run side of that class (netlists, programs, device bring-up) is not part of this path."""
from threading import Event
from typing import Dict, List, Optional, Tuple, Union

import torch

from ._C.backend_api import (BackendStatusCode, DramIODesc, PytorchTensorDesc, TilizedTensorDesc, free_tensor, get_output,
                             pop_output, push_input, push_input_batch, push_input_view)
from .tensor import (RuntimeTensorTransform, RuntimeTensorTransformType, Tensor, pytorch_tensor_to_tensor_desc)


class BackendAPI:
    @classmethod
    def push_input(cls, queue_desc: DramIODesc, tensor_desc: Union[PytorchTensorDesc, TilizedTensorDesc], single_input: bool = True,
                   timeout_secs: int = 1, ram_address: int = 0):
        if isinstance(tensor_desc, TilizedTensorDesc):
            assert push_input(queue_desc, tensor_desc, timeout_secs, ram_address) == BackendStatusCode.Success, \
                "Error while pushing tilized inputs"
        else:
            assert push_input(queue_desc, tensor_desc, single_input, timeout_secs, ram_address) == BackendStatusCode.Success, \
                "Error while pushing inputs"

    @classmethod
    def push_to_queues(cls, ordered_input_queues: List[DramIODesc], tensors: List[PytorchTensorDesc], single_input: bool):
        assert len(tensors) == len(ordered_input_queues), (
            f"Incorrect number of tensors provided on input: tensors:{len(tensors)} vs ordered_input_queues:{len(ordered_input_queues)}")
        for i, inq in enumerate(ordered_input_queues):
            BackendAPI.push_input(inq, tensors[i], single_input, 1, -1)

    @classmethod
    def push_staged(cls, queues: List[DramIODesc], staged: List[Tuple[PytorchTensorDesc, object]], single_input: bool,
                    ram_addresses: Optional[List[int]] = None):
        """(descriptor, source view or None) pairs to their queues.  Descriptors without a view travel together in one
        push_input_batch call (one conversion launch per format combination instead of one per tensor); a descriptor
        with a view, or one for a prestriding queue, is pushed by itself."""
        assert len(staged) == len(queues), f"{len(staged)} tensors staged for {len(queues)} queues"
        ram = list(ram_addresses) if ram_addresses is not None else [-1] * len(queues)
        together = []
        for i, (q, (desc, view)) in enumerate(zip(queues, staged)):
            if view is not None:
                rc = push_input_view(q, desc, view, single_input, 1, ram[i])
                assert rc == BackendStatusCode.Success, "Error while pushing inputs"
            elif isinstance(desc, TilizedTensorDesc) or q.s_descriptor.stride > 1:
                BackendAPI.push_input(q, desc, single_input, 1, ram[i])
            else:
                together.append(i)
        if together:
            rc = push_input_batch([queues[i] for i in together], [staged[i][0] for i in together], single_input, 1,
                                  [ram[i] for i in together])
            assert rc == BackendStatusCode.Success, "Error while pushing inputs"

    @classmethod
    def read_queues(cls, queues: List[DramIODesc], original_shapes: List[Tuple[int, ...]],
                    runtime_tensor_transforms: Optional[List[RuntimeTensorTransform]], requires_grad: List[bool],
                    single_output: bool, rd_ptr: int = -1, shutdown_event: Optional[Event] = None, clone: bool = False,
                    has_microbatch_dim: bool = True) -> List[Tensor]:
        """get_output on every queue (a read that times out is retried up to 10 times, as in the reference), then the
        tile padding is cut off.  clone=False returns views of backend-owned memory that stay valid until pop_queues."""
        count = len(queues)
        assert len(original_shapes) == count and len(requires_grad) == count, "one original shape and one requires_grad flag per queue"
        transforms = runtime_tensor_transforms if runtime_tensor_transforms is not None else [None] * count

        def fetch(q: DramIODesc) -> PytorchTensorDesc:
            desc, status = PytorchTensorDesc(), BackendStatusCode.TimeoutError
            for _attempt in range(10):                      # one-second reads, so a shutdown request is noticed between them
                status = get_output(q, desc, single_output, 1, rd_ptr)
                if status != BackendStatusCode.TimeoutError or (shutdown_event is not None and shutdown_event.is_set()):
                    break
            if status == BackendStatusCode.TimeoutError:
                if shutdown_event is not None:
                    shutdown_event.set()                    # whoever else waits on this device should give up too
                raise RuntimeError("Timeout while reading " + q.name)
            assert status == BackendStatusCode.Success, "Error while reading output"
            return desc

        def dims_of(shape_field) -> Optional[list]:
            return list(shape_field.dims) if shape_field is not None and shape_field.dims else None

        descs = [fetch(q) for q in queues]
        results = []
        for desc, shape, tr, grad in zip(descs, original_shapes, transforms, requires_grad):
            t = Tensor.create_from_tensor_descriptor(desc).narrow_to_original_shape(
                tuple(shape), dims_of(tr.reinterpreted_shape) if tr is not None else None, has_microbatch_dim=has_microbatch_dim,
                unpadded_shape=dims_of(tr.unpadded_shape) if tr is not None else None)
            if grad:
                t = t.detach()
                t.set_requires_grad(True)
            if clone:
                t = t.clone()
                free_tensor(desc)
            results.append(t)
        return results

    @classmethod
    def pop_queues(cls, queues: List[DramIODesc], single_output: bool):
        for outq in queues:
            assert pop_output(outq, single_output, 1) == BackendStatusCode.Success, "Error while popping output"

    @classmethod
    def push_constants_and_parameters(cls, queues: Dict[str, DramIODesc], values: Dict[str, torch.Tensor]):
        """Every constant and parameter of a model to its RandomAccess queue at address 0.  The reference walks the
        compiled graph's names and pushes them one by one (backend.py:458-493); here the caller names the queues and the
        whole set goes down in ONE backend call: tensors of different shapes share a conversion launch."""
        names = list(queues)
        descs = []
        for name in names:
            q = queues[name]
            df = q.data_format if int(q.data_format) >= 0xF0 else None       # raw formats keep their integer bits
            descs.append((pytorch_tensor_to_tensor_desc(values[name].contiguous(), df), None))
        BackendAPI.push_staged([queues[n] for n in names], descs, True, ram_addresses=[0] * len(names))

    @classmethod
    def update_device_paramaters(cls, queues: Dict[str, DramIODesc], values: Dict[str, torch.Tensor]):
        """New values for parameters that already live on the device (name as the reference spells it,
        backend.py:495-517): the same batched push, into the same addresses."""
        BackendAPI.push_constants_and_parameters({n: queues[n] for n in values}, values)
