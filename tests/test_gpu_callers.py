"""GPU tests of the caller side of the path, written the way the reference's host code drives it
(pybuda/pybuda/device_connector.py: DirectPusherDeviceConnector / DirectPopperDeviceConnector; pybuda/pybuda/backend.py:
BackendAPI.push_to_queues / read_queues / pop_queues / push_constants_and_parameters)."""
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    import pybuda._C as C
    from pybuda import backend, device_connector, parameter, tensor as T
    yield C.backend_api, C.DataFormat, T, backend, device_connector, parameter
    C.backend_api.release_all_queues()


def _quantised(oracle, x4, fmt):
    return oracle.unpack_untilize(oracle.tilize_pack(x4, fmt), fmt, x4.shape)


@pytest.mark.parametrize("sequential", [True, False])
def test_connector_push_read_pop(mods, oracle, sequential):
    B, DF, T, backend, dc, _ = mods
    mb = 2
    g = torch.Generator().manual_seed(3)
    act = torch.randn(mb, 50, 70, generator=g)                       # padded to [2, 1, 64, 96] on the way in
    half = torch.randn(mb, 33, 64, generator=g).half()               # float16 into a Float16_b queue: converted to bfloat16
    rowv = torch.randn(mb, 1, 96, generator=g)                       # a row vector tile-broadcast along r
    idx = torch.arange(40, dtype=torch.int32).repeat(mb, 1)          # embedding indices
    tag = "seq" if sequential else "thr"
    queues = [B.DramIODesc.for_tensor(f"act_{tag}", [mb, 1, 64, 96], DF.Bfp8_b, grid=(1, 3)),
              B.DramIODesc.for_tensor(f"half_{tag}", [mb, 1, 64, 64], DF.Float16_b),
              B.DramIODesc.for_tensor(f"rowv_{tag}", [mb, 1, 32, 96], DF.Bfp4_b),
              B.DramIODesc.for_tensor(f"idx_{tag}", [mb, 1, 32, 32], DF.RawUInt32)]
    transforms = [T.RuntimeTensorTransform(), T.RuntimeTensorTransform(), T.RuntimeTensorTransform(),
                  T.RuntimeTensorTransform(T.RuntimeTensorTransformType.EmbeddingIndex, original_shape=(40,))]
    shutdown = threading.Event()
    pusher = dc.DirectPusherDeviceConnector(shutdown, sequential=sequential, microbatch=mb)
    pusher.set_dram_io_push_queues(queues, [[], [], [-2], []], transforms)
    pusher.initialize()
    popper = dc.DirectPopperDeviceConnector(shutdown)
    popper.set_dram_io_pop_queues(queues[:3], [tuple(act.shape), tuple(half.shape), (mb, 32, 96)], [False, False, False], None)
    try:
        for _ in range(2):                                           # two rounds through the rings
            pusher.push([T.Tensor.create_from_torch(act), T.Tensor.create_from_torch(half), T.Tensor.create_from_torch(rowv),
                         idx.clone()])
            pusher.wait_for_pushes()
            got = popper.read()
            # activations: Bfp8_b of the zero-padded tensor, narrowed back
            padded = np.zeros((mb, 1, 64, 96), np.float32)
            padded[:, 0, :50, :70] = act.numpy()
            want = _quantised(oracle, padded, oracle.Bfp8_b)[:, 0, :50, :70]
            # a Bfp queue reads back as bfloat16 by default (tensor.py:730-740): exact for 7-bit magnitudes
            assert got[0].value().shape == act.shape
            assert np.array_equal(got[0].value().float().numpy().view(np.uint32), want.view(np.uint32))
            # float16 input was converted to bfloat16 for the Float16_b queue
            assert torch.equal(got[1].value().float(), half.bfloat16().float())
            # the row vector was replicated down the tile before packing
            rep = np.repeat(rowv.numpy()[:, None, :, :], 32, axis=2).reshape(mb, 1, 32, 96)
            want_row = _quantised(oracle, rep, oracle.Bfp4_b)
            assert np.array_equal(got[2].value().float().numpy().reshape(mb, 1, 32, 96).view(np.uint32), want_row.view(np.uint32))
            popper.pop()
            # the index queue: raw 32-bit values in the embedding layout, padding = all ones
            out = B.PytorchTensorDesc()
            assert B.get_output(queues[3], out, False, 1, -1) == B.BackendStatusCode.Success, B.last_error()
            raw = T.tensor_desc_to_pytorch_tensor(out).clone()
            B.pop_output(queues[3], False, 1)
            B.free_tensor(out)
            assert raw.shape == (mb, 1, 32, 32) and raw[0, 0, 0, :32].tolist() == list(range(32))
            assert raw[0, 0, 1, :8].tolist() == list(range(32, 40)) and raw[0, 0, 1, 8].item() == -1
    finally:
        pusher.shutdown()


def test_threaded_pusher_reports_a_failed_push(mods):
    B, DF, T, backend, dc, _ = mods
    q = B.DramIODesc.for_tensor("too_small", [1, 1, 32, 32], DF.Bfp8_b, num_slots=1)
    pusher = dc.DirectPusherDeviceConnector(threading.Event(), sequential=False)
    pusher.set_dram_io_push_queues([q], [[]], None)
    pusher.initialize()
    try:
        pusher.push([T.Tensor.create_from_torch(torch.randn(1, 32, 32))])
        pusher.wait_for_pushes()
        pusher.push([T.Tensor.create_from_torch(torch.randn(1, 32, 32))])   # the ring is full: the push times out
        with pytest.raises(AssertionError, match="Error while pushing inputs"):
            pusher.wait_for_pushes()
    finally:
        pusher.shutdown()


def test_read_queues_retries_then_raises_on_an_empty_queue(mods):
    B, DF, T, backend, dc, _ = mods
    q = B.DramIODesc.for_tensor("never_filled_but_created", [1, 1, 32, 32], DF.Float32)
    assert B.push_input(q, T.pytorch_tensor_to_tensor_desc(torch.zeros(1, 1, 32, 32)), False, 1, -1) == B.BackendStatusCode.Success
    backend.BackendAPI.pop_queues([q], single_output=False)                    # now empty
    ev = threading.Event()
    ev.set()                                                                   # a set shutdown event ends the retry loop at once
    with pytest.raises(RuntimeError, match="Timeout while reading"):
        backend.BackendAPI.read_queues([q], [(1, 32, 32)], None, [False], single_output=False, shutdown_event=ev)


def test_parameters_pushed_to_random_access_queues(mods, oracle):
    B, DF, T, backend, dc, parameter = mods
    g = torch.Generator().manual_seed(8)
    p = parameter.Parameter(torch.randn(128, 256, generator=g) * 0.02, name="ffn.w")
    p.set_data_format(DF.Bfp8_b)
    assert p.value().dtype == torch.bfloat16 and p.pt_data_format == torch.bfloat16
    table = torch.arange(64 * 32, dtype=torch.int32).reshape(64, 32)
    queues = {"ffn.w": B.DramIODesc.for_tensor("ffn.w", [1, 1, 128, 256], DF.Bfp8_b, io_type=B.IOType.RandomAccess, num_slots=1),
              "lut": B.DramIODesc.for_tensor("lut", [1, 1, 64, 32], DF.RawUInt32, io_type=B.IOType.RandomAccess, num_slots=1)}
    backend.BackendAPI.push_constants_and_parameters(queues, {"ffn.w": p.value(), "lut": table})
    backend.BackendAPI.push_constants_and_parameters(queues, {"ffn.w": p.value(), "lut": table})   # RAM queues are overwritten in place
    out = B.PytorchTensorDesc()
    out.format = DF.Float32
    assert B.get_output(queues["ffn.w"], out, True, 1, 0) == B.BackendStatusCode.Success, B.last_error()
    w = T.tensor_desc_to_pytorch_tensor(out).clone()
    B.free_tensor(out)
    want = _quantised(oracle, p.value().float().numpy().reshape(1, 1, 128, 256), oracle.Bfp8_b)
    assert np.array_equal(w.numpy().reshape(1, 1, 128, 256).view(np.uint32), want.view(np.uint32))
    out = B.PytorchTensorDesc()
    assert B.get_output(queues["lut"], out, True, 1, 0) == B.BackendStatusCode.Success, B.last_error()
    assert torch.equal(T.tensor_desc_to_pytorch_tensor(out).reshape(64, 32), table)
    B.free_tensor(out)


def test_parameter_set_goes_down_in_one_launch_per_format(mods, oracle):
    """push_constants_and_parameters / update_device_paramaters: a model's whole parameter set -- different shapes,
    queue geometries and formats -- in one backend call; tensors that share a (source, queue) format pair share a
    conversion launch.  Device-resident and host values alike."""
    B, DF, T, backend, dc, parameter = mods
    from pybuda import _cabi
    g = torch.Generator().manual_seed(12)
    shapes = {"q": (1024, 1024), "k": (1024, 1024), "ffn1": (1024, 4096), "ffn2": (4096, 1024), "ln": (32, 1024), "emb": (64, 32)}
    for where in ("host", "device"):
        values, queues = {}, {}
        for i, (name, shp) in enumerate(shapes.items()):
            v = torch.randn(shp, generator=g) * 0.02
            if name == "emb":
                v = torch.randint(0, 1000, shp, generator=g, dtype=torch.int32)
            values[name] = v.cuda() if where == "device" else v
            fmt = DF.RawUInt32 if name == "emb" else (DF.Bfp4_b if name == "ln" else DF.Bfp8_b)
            grid = (2, 2) if name == "ffn1" else (1, 1)
            queues[name] = B.DramIODesc.for_tensor(f"{where}_{name}", [1, 1, *shp], fmt, grid=grid, io_type=B.IOType.RandomAccess, num_slots=1)
        n0 = _cabi.launch_count()
        backend.BackendAPI.push_constants_and_parameters(queues, values)
        launches = _cabi.launch_count() - n0
        if where == "device":
            assert launches == 3, launches          # fp32 -> Bfp8_b (4 tensors), fp32 -> Bfp4_b, int32 -> RawUInt32
        for name, shp in shapes.items():
            out = B.PytorchTensorDesc()
            if name != "emb":
                out.format = DF.Float32
            assert B.get_output(queues[name], out, True, 1, 0) == B.BackendStatusCode.Success, B.last_error()
            got = T.tensor_desc_to_pytorch_tensor(out).clone().reshape(shp)
            B.free_tensor(out)
            if name == "emb":
                assert torch.equal(got, values[name].cpu())
            else:
                fmt = oracle.Bfp4_b if name == "ln" else oracle.Bfp8_b
                want = _quantised(oracle, values[name].cpu().numpy().reshape(1, 1, *shp), fmt).reshape(shp)
                assert np.array_equal(got.numpy().view(np.uint32), want.view(np.uint32)), (where, name)
        # new values for two of them, into the same addresses
        upd = {"q": values["q"] * 2, "ln": values["ln"] + 1}
        backend.BackendAPI.update_device_paramaters(queues, upd)
        out = B.PytorchTensorDesc()
        out.format = DF.Float32
        assert B.get_output(queues["q"], out, True, 1, 0) == B.BackendStatusCode.Success
        want = _quantised(oracle, upd["q"].cpu().numpy().reshape(1, 1, 1024, 1024), oracle.Bfp8_b).reshape(1024, 1024)
        assert np.array_equal(T.tensor_desc_to_pytorch_tensor(out).numpy().reshape(1024, 1024).view(np.uint32), want.view(np.uint32))
        B.free_tensor(out)
    # the same queue twice in one call is refused
    q = queues["q"]
    d = T.pytorch_tensor_to_tensor_desc(torch.zeros(1, 1, 1024, 1024))
    assert B.push_input_batch([q, q], [d, d], True, 1, [0, 0]) == B.BackendStatusCode.RuntimeError
    assert "twice" in B.last_error()


def test_connector_pushes_reinterpreted_and_prestrided_inputs(mods, oracle):
    """ReinterpretShape (the tensor's elements read in another shape, then padded by the kernel) and Prestride (the queue
    carries a stride descriptor; the kernel gathers the phases) through the connector."""
    B, DF, T, backend, dc, _ = mods
    g = torch.Generator().manual_seed(13)
    flat = torch.randn(1, 2 * 45 * 50, generator=g)                       # reinterpreted as [1, 2, 45, 50] -> queue [1, 2, 64, 64]
    act = torch.randn(1, 3, 10, 12, generator=g)                          # stride 2 -> [1, 1, 12, 30] -> queue [1, 1, 32, 32]
    q0 = B.DramIODesc.for_tensor("reint", [1, 2, 64, 64], DF.Float32)
    q1 = B.DramIODesc.for_tensor("prestr", [1, 1, 32, 32], DF.Float32)
    tr0 = T.RuntimeTensorTransform(T.RuntimeTensorTransformType.ReinterpretShape, original_shape=tuple(flat.shape), reinterpreted_shape=(1, 2, 45, 50))
    tr1 = T.RuntimeTensorTransform(T.RuntimeTensorTransformType.Prestride, stride_height=2, stride_width=2)
    _, q1 = T.eval_runtime_transform(tr1, act, q1, [])                    # attaches the stride descriptor to the queue
    pusher = dc.DirectPusherDeviceConnector(threading.Event(), sequential=True)
    pusher.set_dram_io_push_queues([q0, q1], [[], []], [tr0, tr1])
    for dev in ("cpu", "cuda"):
        pusher.push([flat.to(dev), act.to(dev)])
        out = B.PytorchTensorDesc()
        assert B.get_output(q0, out, True, 1, -1) == B.BackendStatusCode.Success, B.last_error()
        got = T.tensor_desc_to_pytorch_tensor(out).clone()
        B.free_tensor(out)
        B.pop_output(q0, True, 1)
        want = oracle.pad_to_tiles(flat.numpy().reshape(1, 2, 45, 50))
        assert np.array_equal(got.numpy(), want), dev
        out = B.PytorchTensorDesc()
        assert B.get_output(q1, out, True, 1, -1) == B.BackendStatusCode.Success, B.last_error()
        got = T.tensor_desc_to_pytorch_tensor(out).clone()
        B.free_tensor(out)
        B.pop_output(q1, True, 1)
        assert np.array_equal(got.numpy(), oracle.pad_to_tiles(oracle.prestride_act(act.numpy(), 2))), dev
