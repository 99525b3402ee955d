"""The reference's OWN caller code driving this repository's pybuda._C.

Runs where a checkout of the reference is present (the path in REFERENCE_ROOT, else a directory `reference` beside this
repository) and is skipped elsewhere.  The reference's Python package cannot be imported (tensorflow, jax, its unbuilt C++ module), so the
functions under test are taken out of its source files by name -- pybuda/pybuda/tensor.py:
pytorch_tensor_to_tensor_desc, tensor_desc_to_pytorch_tensor, pad_pytorch_tensor_to_buda, narrow_buda_tensor_to_pytorch,
is_equivalent_data_format, the dtype maps; pybuda/pybuda/device_connector.py: DirectPusherDeviceConnector;
pybuda/pybuda/backend.py: BackendAPI.push_input / push_to_queues -- and executed against this build's DataFormat,
PytorchTensorDesc, DramIODesc and push_input.  No GPU is needed: what is checked is that every call the reference
makes is accepted (names, argument order and types, buffer protocol, pickling) and that results that do not involve the
device equal this repository's own mirrors; the conversion itself is covered by the GPU tests."""
import ast
import os
import pickle
import threading
import types
import typing

import numpy as np
import pytest
import torch

REF = os.environ.get("REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
pytestmark = pytest.mark.skipif(not os.path.isfile(os.path.join(REF, "pybuda/pybuda/tensor.py")),
                                reason="needs a checkout of the reference")


def _take(path, names, namespace, class_methods=None):
    """Executes the named top-level functions (and, for class_methods = {class: [methods]}, those methods as a new
    class of that name) of a reference source file inside `namespace`."""
    with open(os.path.join(REF, path)) as f:
        tree = ast.parse(f.read())
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    assert {n.name for n in body} == set(names), path
    for cls, methods in (class_methods or {}).items():
        node = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == cls)
        node.bases, node.keywords, node.decorator_list = [], [], []
        node.body = [m for m in node.body if isinstance(m, ast.FunctionDef) and m.name in methods]
        assert {m.name for m in node.body} == set(methods), (path, cls)
        body.append(node)
    exec(compile(ast.Module(body=body, type_ignores=[]), path, "exec"), namespace)


@pytest.fixture(scope="module")
def ref():
    import pybuda._C as C
    from pybuda import tensor as ours

    B = C.backend_api
    logger = types.SimpleNamespace(debug=lambda *a, **k: None, info=lambda *a, **k: None, warning=lambda *a, **k: None,
                                   trace=lambda *a, **k: None)
    ns = {"torch": torch, "np": np, "TILE_DIM": 32, "DataFormat": C.DataFormat, "PytorchTensorDesc": B.PytorchTensorDesc,
          "TilizedTensorDesc": B.TilizedTensorDesc, "DramIODesc": B.DramIODesc, "BackendStatusCode": B.BackendStatusCode,
          "Tuple": typing.Tuple, "List": typing.List, "Optional": typing.Optional, "Union": typing.Union, "Dict": typing.Dict,
          "logger": logger, "align_up": lambda v, a: (v + a - 1) // a * a, "align_up_tile": lambda v: (v + 31) // 32 * 32,
          "reduce": __import__("functools").reduce, "mul": __import__("operator").mul, "os": os, "queue": __import__("queue"),
          "threading": threading, "Tensor": ours.Tensor, "RuntimeTensorTransformType": ours.RuntimeTensorTransformType,
          "RuntimeTensorTransform": ours.RuntimeTensorTransform}
    _take("pybuda/pybuda/tensor.py",
          ["pytorch_dtype_to_buda_dataformat", "buda_dataformat_to_pytorch_dtype", "is_equivalent_data_format",
           "pytorch_tensor_to_tensor_desc", "tensor_desc_to_pytorch_tensor", "is_buda_shape", "pad_pytorch_tensor_to_buda",
           "narrow_buda_tensor_to_pytorch"], ns)
    ns["push_input"] = B.push_input
    _take("pybuda/pybuda/backend.py", [], ns, {"BackendAPI": ["push_input", "push_to_queues"]})
    _take("pybuda/pybuda/device_connector.py", [], ns,
          {"DirectPusherDeviceConnector": ["_convert_tensor_for_tilize", "_embedding_index", "_internal_push"]})
    ns["DirectPusherDeviceConnector"].push_to_side_queue = lambda self, tensors: None     # DeviceConnector base-class hook
    ns["BackendAPI"]._capture_tensor = classmethod(lambda cls, desc, q: None)             # the archive-capture hook of the run loop
    return types.SimpleNamespace(**ns), ours, B, C.DataFormat


def test_reference_descriptor_builders_accept_this_builds_types(ref):
    R, ours, B, DF = ref
    for dt in (torch.float32, torch.bfloat16, torch.float16, torch.int8, torch.int32):
        assert R.pytorch_dtype_to_buda_dataformat(dt) == ours.pytorch_dtype_to_buda_dataformat(dt)
    for df in (DF.Float32, DF.Float16, DF.Float16_b, DF.Bfp8_b, DF.Bfp4_b, DF.Bfp2_b, DF.Bfp8, DF.Int8, DF.RawUInt32):
        assert R.buda_dataformat_to_pytorch_dtype(df) == ours.buda_dataformat_to_pytorch_dtype(df)
        for dt in (torch.float32, torch.bfloat16, torch.float16, torch.int8):
            assert R.is_equivalent_data_format(dt, df) == ours.is_equivalent_data_format(dt, df)
    g = torch.Generator().manual_seed(1)
    for shape, df in (((2, 3, 64, 96), None), ((64, 32), None), ((1, 1, 1, 2, 32, 32), None), ((4, 32, 64), DF.Float16_b)):
        t = torch.randn(shape, generator=g)
        theirs, mine = R.pytorch_tensor_to_tensor_desc(t, df), ours.pytorch_tensor_to_tensor_desc(t, df)
        assert isinstance(theirs, B.PytorchTensorDesc)
        for f in ("itemsize", "format", "dim"):
            assert getattr(theirs, f) == getattr(mine, f), f
        assert list(theirs.shape) == list(mine.shape) and list(theirs.strides) == list(mine.strides)
        # the reference reads results back through the descriptor's buffer protocol
        back = R.tensor_desc_to_pytorch_tensor(R.pytorch_tensor_to_tensor_desc(t.float().contiguous()))
        assert torch.equal(back.reshape(t.shape), t.float())
        assert pickle.loads(pickle.dumps(theirs)).shape == theirs.shape
    with pytest.raises(RuntimeError):
        R.pytorch_tensor_to_tensor_desc(torch.zeros(2, 1, 32, 32, 32))       # a leading dim that is not 1 cannot be dropped


def test_reference_pad_and_narrow_agree_with_the_mirrors(ref):
    R, ours, B, DF = ref
    g = torch.Generator().manual_seed(2)
    cases = [((1, 3, 50, 70), [], 1), ((2, 1, 1, 40), [2], 2), ((1, 2, 33, 1), [3], 1), ((4, 17), [], 1), ((7,), [], 1),
             ((2, 5, 31), [], 2), ((1, 1, 64, 64), [], 1)]
    for shape, bcast, mb in cases:
        x = torch.randn(shape, generator=g)
        theirs = R.pad_pytorch_tensor_to_buda(x, bcast, squeeze=True, microbatch=mb)
        mine = ours.pad_pytorch_tensor_to_buda(x, bcast, squeeze=True, microbatch=mb)
        assert theirs.shape == mine.shape and torch.equal(theirs, mine), (shape, bcast)
        if not bcast:
            assert torch.equal(R.narrow_buda_tensor_to_pytorch(theirs, list(shape)), ours.narrow_buda_tensor_to_pytorch(mine, list(shape)))
            assert torch.equal(ours.narrow_buda_tensor_to_pytorch(mine, list(shape)), x)


def test_reference_pusher_reaches_this_builds_push_input(ref):
    """The reference's DirectPusherDeviceConnector._internal_push, unchanged, calling this build's BackendAPI entry:
    every argument is accepted; without a GPU the push itself answers RuntimeError and the reference's own assertion
    fires, with this library's reason on record."""
    R, ours, B, DF = ref
    pusher = R.DirectPusherDeviceConnector()          # its constructor belongs to the transport classes around it: fields set by hand
    queues = [B.DramIODesc.for_tensor("ref_act", [1, 1, 64, 96], DF.Bfp8_b), B.DramIODesc.for_tensor("ref_idx", [1, 1, 32, 32], DF.RawUInt32)]
    pusher.direct_push_queues = queues
    pusher.tile_broadcast_dims = [[], []]
    pusher.runtime_tensor_transforms = [ours.RuntimeTensorTransform(),
                                        ours.RuntimeTensorTransform(ours.RuntimeTensorTransformType.EmbeddingIndex, original_shape=(40,))]
    pusher.constant_tensors, pusher.tile_dims, pusher.microbatch = [None, None], None, 1
    # the reference reads transform.original_shape as a sequence and transform.reinterpreted_shape.as_list()
    assert pusher.runtime_tensor_transforms[1].original_shape[-1] == 40
    # format conversion rules, their code against this build's Tensor wrapper
    half = ours.Tensor.create_from_torch(torch.randn(1, 33, 64).half())
    assert pusher._convert_tensor_for_tilize(half, queues[0]).pt_data_format == torch.bfloat16
    assert pusher._convert_tensor_for_tilize(ours.Tensor.create_from_torch(torch.randn(1, 33, 64)), queues[0]).pt_data_format == torch.float32
    # their embedding layout equals the mirror's (and, on the device, the pack kernel's embedding view)
    idx = torch.arange(40, dtype=torch.int32)
    assert torch.equal(pusher._embedding_index(idx.clone(), (40,), queues[1]), ours._embedding_index(idx, (40,), queues[1]))
    if torch.cuda.is_available():
        pusher._internal_push([ours.Tensor.create_from_torch(torch.randn(1, 50, 70)), idx.clone()])
        assert B.queue_occupancy(queues[0]) == 1 and B.queue_occupancy(queues[1]) == 1
        B.release_all_queues()
    else:
        with pytest.raises(AssertionError, match="Error while pushing inputs"):
            pusher._internal_push([ours.Tensor.create_from_torch(torch.randn(1, 50, 70)), idx.clone()])
        assert "CUDA" in B.last_error()
