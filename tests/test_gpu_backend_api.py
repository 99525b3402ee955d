"""GPU tests of the drop-in boundary: the reference's backend_api entry points (tilize_tensor,
push_input, get_output, pop_output, free_tensor, binarize / debinarize) called the way
pybuda/pybuda/backend.py and tti/archive.py call them, with results checked against the oracle."""
import threading

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def api():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    import pybuda._C as C
    from pybuda import tensor as T

    yield C, C.backend_api, C.DataFormat, T
    C.backend_api.release_all_queues()


def _ok(B, status):
    assert status == B.BackendStatusCode.Success, B.last_error()


def test_tilize_tensor_matches_oracle_and_tbin_round_trip(api, oracle, tmp_path):
    C, B, DF, T = api
    x = torch.randn(1, 1, 1024, 1024, generator=torch.Generator().manual_seed(0))
    q = B.DramIODesc.for_tensor("cfg1", [1, 1, 1024, 1024], DF.Bfp8_b)
    td = B.tilize_tensor(q, T.pytorch_tensor_to_tensor_desc(x))
    assert (td.num_buffers, td.buf_size_bytes, td.format) == (1, 1114112, DF.Bfp8_b)
    img = np.frombuffer(td, dtype=np.uint8)
    ref = oracle.tilize_pack(x.numpy(), oracle.Bfp8_b)
    assert np.array_equal(img, ref)
    # the .tbin path of the device image archive: dump, reload, push without re-tilizing, read back
    path = str(tmp_path / "w.tbin")
    _ok(B, B.binarize_tensor(td, path))
    assert open(path, "rb").read() == ref.tobytes()
    td2 = B.TilizedTensorDesc()
    td2.num_buffers, td2.buf_size_bytes, td2.format = td.num_buffers, td.buf_size_bytes, td.format
    _ok(B, B.debinarize_tensor(td2, path))
    _ok(B, B.push_input(q, td2, 1, -1))
    out = B.PytorchTensorDesc()
    out.format = DF.Float32
    _ok(B, B.get_output(q, out, True, 1, -1))
    y = T.tensor_desc_to_pytorch_tensor(out).clone()
    _ok(B, B.pop_output(q, True, 1))
    _ok(B, B.free_tensor(out))
    _ok(B, B.free_tensor(td))
    _ok(B, B.free_tensor(td2))
    assert np.array_equal(y.numpy().view(np.uint32), oracle.unpack_untilize(ref, oracle.Bfp8_b, x.shape).view(np.uint32))
    # a CUDA tensor goes through the same entry point
    td3 = B.tilize_tensor(q, T.pytorch_tensor_to_tensor_desc(x.cuda()))
    assert np.array_equal(np.frombuffer(td3, dtype=np.uint8), ref)
    B.free_tensor(td3)
    # multi-buffer image: one buffer per grid core
    q4 = B.DramIODesc.for_tensor("cfg1_grid", [1, 1, 1024, 1024], DF.Bfp4_b, grid=(2, 2), ublock=(2, 2))
    td4 = B.tilize_tensor(q4, T.pytorch_tensor_to_tensor_desc(x))
    assert (td4.num_buffers, td4.buf_size_bytes) == (4, 256 * 576)
    go = oracle.Geom.for_shape([1, 1, 1024, 1024], (2, 2), (2, 2), 0)
    assert np.array_equal(np.frombuffer(td4, dtype=np.uint8), oracle.tilize_pack(x.numpy(), oracle.Bfp4_b, go))
    B.free_tensor(td4)


@pytest.mark.parametrize("df_name,dtype", [("Bfp8_b", torch.float32), ("Bfp8_b", torch.bfloat16), ("Bfp4_b", torch.float32),
                                           ("Bfp2_b", torch.bfloat16), ("Float16_b", torch.bfloat16), ("Float32", torch.float32)])
def test_push_get_pop_round_trip(api, oracle, df_name, dtype):
    C, B, DF, T = api
    df = getattr(DF, df_name)
    shape = [4, 2, 96, 160]                       # a microbatch of 4 entries, t = 2
    x = torch.randn(shape, generator=torch.Generator().manual_seed(5)).to(dtype)
    q = B.DramIODesc.for_tensor(f"rt_{df_name}_{dtype}", shape, df, grid=(1, 1), ublock=(3, 1), ublock_order="c")
    assert q.num_slots == 8
    _ok(B, B.push_input(q, T.pytorch_tensor_to_tensor_desc(x), False, 1, -1))
    assert B.queue_occupancy(q) == 4 and B.queue_device_address(q) != 0
    out = B.PytorchTensorDesc()
    if dtype == torch.float32:
        out.format = DF.Float32
    _ok(B, B.get_output(q, out, False, 1, -1))
    assert list(out.shape) == shape and out.dim == 4
    y = T.Tensor.create_from_tensor_descriptor(out).value(clone=True)
    _ok(B, B.free_tensor(out))
    _ok(B, B.pop_output(q, False, 1))
    assert B.queue_occupancy(q) == 0
    if df_name.startswith("Bfp"):
        xn = x.view(torch.int16).numpy().view(np.uint16) if dtype == torch.bfloat16 else x.numpy()
        go = oracle.Geom.for_shape(shape, (1, 1), (3, 1), 1)
        img = oracle.tilize_pack(xn, getattr(oracle, df_name), go,
                                 src_df=oracle.Float16_b if dtype == torch.bfloat16 else oracle.Float32)
        if dtype == torch.float32:
            want = oracle.unpack_untilize(img, getattr(oracle, df_name), shape, geom=go)
            assert np.array_equal(y.numpy().view(np.uint32), want.view(np.uint32))
        else:
            want = oracle.unpack_untilize(img, getattr(oracle, df_name), shape, dst_dtype=np.uint16, geom=go,
                                          dst_df=oracle.Float16_b)
            assert np.array_equal(y.view(torch.int16).numpy().view(np.uint16), want)
    else:
        assert torch.equal(y, x)                  # plain formats come back unchanged


def test_queue_is_a_ring_with_timeouts(api):
    C, B, DF, T = api
    shape = [1, 1, 32, 64]
    q = B.DramIODesc.for_tensor("ring", shape, DF.Float32, num_slots=3)
    out = B.PytorchTensorDesc()
    assert B.get_output(q, out, True, 0, -1) == B.BackendStatusCode.RuntimeError       # never written
    xs = [torch.full(shape, float(i)) for i in range(5)]
    for i in range(3):
        _ok(B, B.push_input(q, T.pytorch_tensor_to_tensor_desc(xs[i]), True, 1, -1))
    assert B.push_input(q, T.pytorch_tensor_to_tensor_desc(xs[3]), True, 0, -1) == B.BackendStatusCode.TimeoutError
    assert "stayed full" in B.last_error()
    got = []
    for i in range(5):                              # wraps around the 3 slots
        _ok(B, B.get_output(q, out, True, 1, -1))
        got.append(float(T.tensor_desc_to_pytorch_tensor(out)[0, 0, 0, 0]))
        B.free_tensor(out)
        _ok(B, B.pop_output(q, True, 1))
        if i + 3 < 5:
            _ok(B, B.push_input(q, T.pytorch_tensor_to_tensor_desc(xs[i + 3]), True, 1, -1))
    assert got == [0.0, 1.0, 2.0, 3.0, 4.0]
    assert B.get_output(q, out, True, 0, -1) == B.BackendStatusCode.TimeoutError       # empty again
    assert B.pop_output(q, True, 0) == B.BackendStatusCode.TimeoutError
    # a reader blocked on an empty queue is released by a push from another thread
    res = {}

    def reader():
        o = B.PytorchTensorDesc()
        res["status"] = B.get_output(q, o, True, 10, -1)
        res["v"] = float(T.tensor_desc_to_pytorch_tensor(o)[0, 0, 0, 0]) if res["status"] == B.BackendStatusCode.Success else None

    th = threading.Thread(target=reader)
    th.start()
    _ok(B, B.push_input(q, T.pytorch_tensor_to_tensor_desc(torch.full(shape, 42.0)), True, 1, -1))
    th.join(20)
    assert res["status"] == B.BackendStatusCode.Success and res["v"] == 42.0
    # mismatched tensors are refused with a status, not an exception
    assert B.push_input(q, T.pytorch_tensor_to_tensor_desc(torch.zeros(1, 1, 64, 64)), True, 1, -1) == B.BackendStatusCode.RuntimeError
    assert "does not match queue" in B.last_error()
    _ok(B, B.release_queue(q))
    assert B.queue_device_address(q) == 0


def test_parameter_ram_queue_and_concurrent_pushers(api, oracle):
    C, B, DF, T = api
    # parameters go to random-access queues at an explicit slot (push_constants_and_parameters)
    w = torch.randn(1, 1, 128, 256, generator=torch.Generator().manual_seed(9)) * 0.02
    pq = B.DramIODesc.for_tensor("param", [1, 1, 128, 256], DF.Bfp8_b, num_slots=1, io_type=B.IOType.RandomAccess)
    _ok(B, B.push_input(pq, T.pytorch_tensor_to_tensor_desc(w), True, 1, 0))
    out = B.PytorchTensorDesc()
    out.format = DF.Float32
    _ok(B, B.get_output(pq, out, True, 1, 0))
    y = T.tensor_desc_to_pytorch_tensor(out).clone()
    B.free_tensor(out)
    ref = oracle.unpack_untilize(oracle.tilize_pack(w.numpy(), oracle.Bfp8_b), oracle.Bfp8_b, w.shape)
    assert np.array_equal(y.numpy().view(np.uint32), ref.view(np.uint32))
    assert B.push_input(pq, T.pytorch_tensor_to_tensor_desc(w), True, 1, 5) == B.BackendStatusCode.RuntimeError
    # several pusher threads, one queue each (the reference runs one pusher thread per connector)
    shape = [2, 1, 64, 128]
    qs = [B.DramIODesc.for_tensor(f"thr{i}", shape, DF.Bfp4_b) for i in range(4)]
    xs = [torch.randn(shape, generator=torch.Generator().manual_seed(20 + i)) for i in range(4)]
    errs = []

    def pusher(i):
        for _ in range(3):
            if B.push_input(qs[i], T.pytorch_tensor_to_tensor_desc(xs[i]), False, 5, -1) != B.BackendStatusCode.Success:
                errs.append(B.last_error())
            o = B.PytorchTensorDesc()
            o.format = DF.Float32
            if B.get_output(qs[i], o, False, 5, -1) != B.BackendStatusCode.Success:
                errs.append(B.last_error())
                continue
            got = T.tensor_desc_to_pytorch_tensor(o).clone()
            B.free_tensor(o)
            B.pop_output(qs[i], False, 5)
            want = oracle.unpack_untilize(oracle.tilize_pack(xs[i].numpy(), oracle.Bfp4_b), oracle.Bfp4_b, shape)
            if not np.array_equal(got.numpy().view(np.uint32), want.view(np.uint32)):
                errs.append(f"thread {i}: data mismatch")

    ths = [threading.Thread(target=pusher, args=(i,)) for i in range(4)]
    [t.start() for t in ths]
    [t.join(60) for t in ths]
    assert not errs, errs


def test_binarize_pytorch_desc(api, tmp_path):
    C, B, DF, T = api
    x = torch.randn(2, 1, 32, 64)
    path = str(tmp_path / "x.bin")
    _ok(B, B.binarize_tensor(T.pytorch_tensor_to_tensor_desc(x), path))
    d = B.PytorchTensorDesc()
    d.itemsize, d.format, d.shape, d.dim = 4, DF.Float32, [2, 1, 32, 64], 4
    _ok(B, B.debinarize_tensor(d, path))
    assert torch.equal(T.tensor_desc_to_pytorch_tensor(d), x)
    B.free_tensor(d)
    d.shape = [2, 1, 32, 32]
    assert B.debinarize_tensor(d, path) == B.BackendStatusCode.RuntimeError


def _golden_stack(x, h, v, row_major):
    """hstack / vstack of the t slices as the reference's golden TMs define them
    (pybuda/pybuda/op/eval/buda/tm.py:114-137), in the order the output host TM applies them."""
    def hstack(t, f):
        w, z, r, c = t.shape
        return t.reshape(w, z // f, f, r, c).permute(0, 1, 3, 2, 4).reshape(w, z // f, r, c * f)

    def vstack(t, f):
        w, z, r, c = t.shape
        return t.reshape(w, z // f, r * f, c)

    return vstack(hstack(x, h), v) if row_major else hstack(vstack(x, v), h)


@pytest.mark.parametrize("h,v,row_major,t", [(4, 1, True, 4), (1, 3, True, 6), (2, 2, True, 4), (2, 3, False, 12), (3, 2, True, 12)])
def test_output_host_transforms(api, oracle, h, v, row_major, t):
    C, B, DF, T = api
    shape = [2, t, 64, 96]
    x = torch.randn(shape, generator=torch.Generator().manual_seed(33))
    for df_name in ("Float32", "Bfp8_b"):
        q = B.DramIODesc.for_tensor(f"tm_{df_name}_{h}{v}{int(row_major)}{t}", shape, getattr(DF, df_name), ublock=(2, 1))
        _ok(B, B.push_input(q, T.pytorch_tensor_to_tensor_desc(x), False, 1, -1))
        q.hstack_factor, q.vstack_factor, q.stack_row_major = h, v, row_major
        out = B.PytorchTensorDesc()
        out.format = DF.Float32
        _ok(B, B.get_output(q, out, False, 1, -1))
        y = T.tensor_desc_to_pytorch_tensor(out).clone()
        B.free_tensor(out)
        _ok(B, B.pop_output(q, False, 1))
        assert list(y.shape) == [2, t // (h * v), 64 * v, 96 * h]
        if df_name == "Float32":
            want = x
        else:
            go = oracle.Geom.for_shape(shape, (1, 1), (2, 1), 0)
            want = torch.from_numpy(oracle.unpack_untilize(oracle.tilize_pack(x.numpy(), oracle.Bfp8_b, go), oracle.Bfp8_b, shape, geom=go))
        assert torch.equal(y, _golden_stack(want, h, v, row_major)), df_name


def test_prestriding_queue_stores_the_prestrided_activation(api, oracle):
    """push_input on a queue with a StrideDescriptor: the original [w, z, H, W] activation goes in, the queue holds
    its prestrided form (golden op/eval/pybuda/tm.py:316-335), zero-padded to tiles."""
    C, B, DF, T = api
    g = torch.Generator().manual_seed(41)
    x = torch.randn(2, 3, 30, 45, generator=g)                 # odd sizes: padding to the stride is exercised
    for stride, fmt, tdtype in ((2, DF.Float32, torch.float32), (4, DF.Float16_b, torch.bfloat16), (2, DF.Bfp8_b, torch.float32)):
        xs = x.to(tdtype)
        gold = oracle.prestride_act(xs.float().numpy(), stride)            # [2, 1, 3*s*s, ceil(30/s)*ceil(45/s)]
        rows, cols = T.align_up_tile(gold.shape[2]), T.align_up_tile(gold.shape[3])
        q = B.DramIODesc.for_tensor(f"conv_act_{stride}_{int(fmt)}", [2, 1, rows, cols], fmt)
        tr = T.RuntimeTensorTransform(T.RuntimeTensorTransformType.Prestride, stride_height=stride, stride_width=stride)
        xs2, q = T.do_runtime_transform(tr, xs, q, [])
        for src in (xs2, xs2.cuda()):                                       # host and device sources
            _ok(B, B.push_input(q, T.pytorch_tensor_to_tensor_desc(src), False, 1, -1))
            out = B.PytorchTensorDesc()
            out.format = DF.Float32 if fmt != DF.Float16_b else DF.Float16_b
            _ok(B, B.get_output(q, out, False, 1, -1))
            y = T.tensor_desc_to_pytorch_tensor(out).clone().float()
            _ok(B, B.pop_output(q, False, 1))
            _ok(B, B.free_tensor(out))
            want = np.zeros((2, 1, rows, cols), np.float32)
            want[:, :, :gold.shape[2], :gold.shape[3]] = gold
            if fmt == DF.Bfp8_b:
                want = oracle.unpack_untilize(oracle.tilize_pack(want, oracle.Bfp8_b), oracle.Bfp8_b, want.shape)
            assert np.array_equal(y.numpy().view(np.uint32), want.view(np.uint32))
    # a descriptor that does not fit its queue is refused
    small = B.DramIODesc.for_tensor("conv_act_small", [2, 1, 32, 32], DF.Float32)
    _, small = T._prestride_shape(x, 2, 2, small)
    assert B.push_input(small, T.pytorch_tensor_to_tensor_desc(x), False, 1, -1) == B.BackendStatusCode.RuntimeError
    assert "does not fit" in B.last_error()


@pytest.mark.parametrize("th", [1, 16])
def test_tiny_tile_queue_round_trip(api, oracle, th):
    C, B, DF, T = api
    x = torch.randn(2, 1, th, 96, generator=torch.Generator().manual_seed(th))
    q = B.DramIODesc.for_tensor(f"bias_th{th}", [2, 1, th, 96], DF.Bfp8_b, tile_height=th)
    assert q.tile_height == th
    _ok(B, B.push_input(q, T.pytorch_tensor_to_tensor_desc(x), False, 1, -1))
    out = B.PytorchTensorDesc()
    out.format = DF.Float32
    _ok(B, B.get_output(q, out, False, 1, -1))
    y = T.tensor_desc_to_pytorch_tensor(out).clone()
    _ok(B, B.pop_output(q, False, 1))
    _ok(B, B.free_tensor(out))
    og = oracle.Geom.for_shape(x.shape, tile_height=th)
    img = oracle.tilize_pack(x.numpy(), oracle.Bfp8_b, og)
    assert img.size == 2 * 3 * 1088                                         # full-size records
    want = oracle.unpack_untilize(img, oracle.Bfp8_b, x.shape, geom=og)
    assert y.shape == x.shape and np.array_equal(y.numpy().view(np.uint32), want.view(np.uint32))

