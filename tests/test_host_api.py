"""CPU tests of the host layer: the pybind module pybuda._C (DataFormat, descriptors, sizes, tile
order) and the Python tensor / data-format API, checked against the reference's documented
behaviour.  No GPU compute is called here."""
import ctypes
import os
import pickle
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def C():
    import pybuda._C as C

    return C


@pytest.fixture(scope="module")
def T():
    from pybuda import tensor

    return tensor


def test_cabi_exports_every_declared_symbol():
    from pybuda import _cabi

    total = 0
    for h in ("buda_cuda.h", "buda_cuda_testing.h"):
        header = open(os.path.join(ROOT, "include", h)).read()
        declared = set(re.findall(r"\b(buda_[a-z0-9_]+)\s*\(", header))
        declared -= {"buda_status", "buda_queue_geom", "buda_tensor_job", "buda_bfp_policy"}
        total += len(declared)
        for name in sorted(declared):
            assert hasattr(_cabi.lib, name), f"{name} is declared in include/{h} but not exported"
    assert total >= 50
    # the measurement probe is not part of this library
    assert not hasattr(_cabi.lib, "buda_stream_probe")
    assert b"sm_100a" in _cabi.lib.buda_version()


def test_cabi_sizes_match_oracle(oracle):
    from pybuda import _cabi

    for df in (0, 1, 2, 3, 11, 5, 6, 7, 15, 10, 12, 14, 8, 0xF0, 0xF1, 0xF2, 0xFF, 99):
        for hdr in (0, 1):
            assert _cabi.lib.buda_tile_bytes(df, hdr) == oracle.tile_bytes(df, hdr)
        assert _cabi.lib.buda_data_format_byte_size(df, 4096) == oracle.lib().ref_data_format_byte_size(df, 4096)
    g = _cabi.QueueGeom.for_shape([1, 1, 1024, 1024])
    assert _cabi.tilized_bytes(g, [1, 1, 1024, 1024], 6) == 1114112
    for df, n in ((6, 17825792), (7, 9437184), (15, 5242880)):
        assert _cabi.tilized_bytes(_cabi.QueueGeom.for_shape([1, 1, 4096, 4096]), [1, 1, 4096, 4096], df) == n
    # queues are sized with the 32-byte per-tile header, as the reference compiler sizes them
    assert _cabi.lib.buda_io_size_bytes(6, 0, 1, 1, 2, 4, 1, 2, 32, 32) == 16 * 1120
    assert _cabi.lib.buda_io_size_bytes(0, 1, 1, 1, 2, 4, 1, 2, 32, 32) == 16 * 4096
    assert _cabi.lib.buda_io_size_bytes(6, 0, 1, 1, 2, 4, 1, 2, 4, 32) == 16 * 1120      # tiny tiles keep full-size records


def test_cabi_tile_map_matches_oracle(oracle):
    from pybuda import _cabi

    for grid, ublock, order in (((1, 1), (1, 1), 0), ((2, 3), (2, 1), 0), ((1, 2), (3, 2), 1)):
        shape = [1, 3, 32 * 12, 32 * 12]
        gq = _cabi.QueueGeom.for_shape(shape, grid, ublock, order)
        go = oracle.Geom.for_shape(shape, grid, ublock, order)
        for t in range(3):
            for r in range(12):
                for c in range(12):
                    cr, cc, addr = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint64()
                    assert _cabi.lib.buda_tile_map(ctypes.byref(gq), t, r, c, ctypes.byref(cr), ctypes.byref(cc),
                                                   ctypes.byref(addr)) == 0
                    assert (cr.value, cc.value, addr.value) == oracle.tile_map(go, t, r, c)
    cr, cc, addr = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint64()
    assert _cabi.lib.buda_tile_map(ctypes.byref(gq), 3, 0, 0, ctypes.byref(cr), ctypes.byref(cc), ctypes.byref(addr)) == 1
    assert "outside the queue" in _cabi.last_error()


def test_no_gpu_calls_fail_with_status_not_exception():
    # without a device every compute entry point reports RuntimeError and says why
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from pybuda import _cabi

    g = _cabi.QueueGeom.for_shape([1, 1, 32, 32])
    rc = _cabi.lib.buda_tilize_pack(1, 0, _cabi.u32x4([1, 1, 32, 32]), _cabi.u64x4([4096, 4096, 128, 4]), ctypes.byref(g), 6,
                                    0, 1, 1088, None)
    assert rc == _cabi.RUNTIME_ERROR
    assert "no CPU path" in _cabi.last_error()


def test_dataformat_enum_values_json_pickle(C):
    DF = C.DataFormat
    want = dict(Float32=0, Float16=1, Bfp8=2, Bfp4=3, Bfp2=11, Float16_b=5, Bfp8_b=6, Bfp4_b=7, Bfp2_b=15, Lf8=10, UInt16=12,
                Int8=14, Int32=8, RawUInt8=0xF0, RawUInt16=0xF1, RawUInt32=0xF2, Invalid=0xFF)
    for name, v in want.items():
        assert int(getattr(DF, name)) == v
        assert getattr(DF, name).to_json() == name
        assert DF.from_json(name) == getattr(DF, name)
        assert pickle.loads(pickle.dumps(getattr(DF, name))) == getattr(DF, name)
    with pytest.raises(KeyError):
        DF.from_json("Bfp16")
    assert C.backend_api.get_format_from_string("bfp8_b") == DF.Bfp8_b
    assert C.backend_api.get_format_from_string("nonsense") == DF.Invalid
    assert C.data_format_byte_size(DF.Bfp8_b, 1024) == 1088 and C.data_format_byte_size(DF.Bfp2, 1024) == 320
    assert C.tile_size_bytes(DF.Bfp4_b) == 608 and C.tile_size_bytes(DF.Bfp4_b, False) == 576
    assert C.to_a_data_format(DF.Bfp8_b) == DF.Bfp8 and C.to_b_data_format(DF.Float16) == DF.Float16_b
    assert C.preserve_lower_precision_cast(DF.Bfp8, DF.Float16_b) == DF.Bfp8_b
    assert C.preserve_lower_precision_cast(DF.Float32, DF.Bfp4_b) == DF.Bfp4_b
    assert int(C.MathFidelity.HiFi3) == 3 and C.MathFidelity.from_json("LoFi") == C.MathFidelity.LoFi


def test_descriptors(C):
    B, DF = C.backend_api, C.DataFormat
    t = torch.arange(2 * 64 * 96, dtype=torch.float32).reshape(2, 1, 64, 96)
    import sys

    rc0 = sys.getrefcount(t)
    d = B.PytorchTensorDesc(t, 4, DF.Float32, 4, [2, 1, 64, 96], [64 * 96 * 4, 64 * 96 * 4, 96 * 4, 4])
    assert d.ptr == t.data_ptr() and d.itemsize == 4 and d.format == DF.Float32 and d.dim == 4
    assert list(d.shape) == [2, 1, 64, 96] and list(d.strides) == [24576, 24576, 384, 4]
    assert sys.getrefcount(t) == rc0 + 1  # the descriptor keeps the tensor alive
    back = torch.frombuffer(d, dtype=torch.float32).reshape(2, 1, 64, 96)
    assert torch.equal(back, t)
    d2 = pickle.loads(pickle.dumps(d))
    assert d2.ptr == d.ptr and list(d2.shape) == list(d.shape) and d2.format == d.format
    del back, d
    assert sys.getrefcount(t) == rc0
    tz = B.TilizedTensorDesc()
    tz.num_buffers, tz.buf_size_bytes, tz.format = 4, 8704, DF.Bfp8_b
    tz2 = pickle.loads(pickle.dumps(tz))
    assert (tz2.num_buffers, tz2.buf_size_bytes, tz2.format, tz2.ptr) == (4, 8704, DF.Bfp8_b, 0)

    q = B.DramIODesc.for_tensor("acts", [4, 2, 128, 256], DF.Bfp8_b, grid=(2, 1), ublock=(1, 4), ublock_order="c")
    assert (q.name, q.data_format, q.t, q.input_count) == ("acts", DF.Bfp8_b, 2, 4)
    assert (q.bufq_grid_dim_r, q.bufq_grid_dim_c, q.mblock_m, q.mblock_n, q.ublock_rt, q.ublock_ct) == (2, 1, 2, 2, 1, 4)
    assert q.entry_size == 2 * 2 * 2 * 4 * 1088 and q.num_slots == 8 and q.ublock_order == "c"
    q2 = pickle.loads(pickle.dumps(q))
    assert (q2.name, q2.entry_size, q2.ublock_order, q2.mblock_n) == ("acts", q.entry_size, "c", 2)
    with pytest.raises(RuntimeError):
        B.DramIODesc.for_tensor("bad", [1, 1, 100, 64], DF.Bfp8_b)
    with pytest.raises(RuntimeError):
        B.DramIODesc.for_tensor("bad", [1, 1, 96, 64], DF.Bfp8_b, grid=(2, 1))
    s = B.StrideDescriptor()
    s.xy_offsets, s.stride = [(0, 1), (1, 0)], 2
    s2 = pickle.loads(pickle.dumps(s))
    assert s2.xy_offsets == [(0, 1), (1, 0)] and s2.stride == 2
    assert B.get_next_aligned_address(33) == 64 and B.get_next_aligned_address(64) == 64
    assert B.get_io_size_in_bytes(DF.Float16_b, False, 2, 2, 1, 1, 1, 3) == 3 * 4 * 2080
    assert int(B.BackendStatusCode.Success) == 0 and int(B.BackendStatusCode.TimeoutError) == 2


def test_tile_layout_binding_round_trip(C, oracle):
    bal = C.balancer
    for grid, mb, ub, order in (((2, 3), (2, 1), (1, 2), bal.UBlockOrder.R), ((1, 2), (3, 2), (2, 2), bal.UBlockOrder.C)):
        L = bal.TileLayout(grid, 2, mb[0], mb[1], ub, order)
        go = oracle.Geom(grid[0], grid[1], mb[0], mb[1], ub[0], ub[1], 2, 0 if order == bal.UBlockOrder.R else 1)
        for t in range(L.t):
            for r in range(L.rt):
                for c in range(L.ct):
                    lin = L.map(t, r, c)
                    assert lin == oracle.tile_map(go, t, r, c)
                    assert L.unmap(*lin) == (t, r, c)
    with pytest.raises(IndexError):
        L.map(0, 999, 0)


def test_dtype_format_maps(C, T):
    DF = C.DataFormat
    assert T.pytorch_dtype_to_buda_dataformat(torch.bfloat16) == DF.Float16_b
    assert T.pytorch_dtype_to_buda_dataformat(torch.float32, fp32_fallback=DF.Float16_b) == DF.Float16_b
    assert T.pytorch_dtype_to_buda_dataformat(torch.bool) == DF.Bfp2_b
    assert T.pytorch_dtype_to_buda_dataformat(DF.Bfp4) == DF.Bfp4
    with pytest.raises(RuntimeError):
        T.pytorch_dtype_to_buda_dataformat(torch.float64)
    for df in (DF.Bfp8_b, DF.Bfp4_b, DF.Bfp2_b, DF.Float16_b):
        assert T.buda_dataformat_to_pytorch_dtype(df) == torch.bfloat16
    for df in (DF.Bfp8, DF.Bfp4, DF.Bfp2, DF.Float16):
        assert T.buda_dataformat_to_pytorch_dtype(df) == torch.float16
    assert T.buda_dataformat_to_pytorch_dtype(DF.RawUInt32) == torch.int
    with pytest.raises(RuntimeError):
        T.buda_dataformat_to_pytorch_dtype(DF.Lf8)
    assert T.is_equivalent_data_format(torch.bfloat16, DF.Float16_b)
    assert not T.is_equivalent_data_format(torch.bfloat16, DF.Bfp8_b)


def test_tensor_desc_building(C, T):
    DF = C.DataFormat
    d = T.pytorch_tensor_to_tensor_desc(torch.zeros(64, 96))
    assert list(d.shape) == [1, 1, 64, 96] and d.dim == 3 and d.format == DF.Float32
    assert list(d.strides) == [384, 384, 384, 4]          # missing dims repeat the outermost stride
    d = T.pytorch_tensor_to_tensor_desc(torch.zeros(1, 1, 2, 3, 32, 64, dtype=torch.bfloat16))
    assert list(d.shape) == [2, 3, 32, 64] and d.itemsize == 2 and d.format == DF.Float16_b
    with pytest.raises(RuntimeError):
        T.pytorch_tensor_to_tensor_desc(torch.zeros(2, 1, 2, 3, 32, 64))
    d = T.pytorch_tensor_to_tensor_desc(torch.zeros(32, 32, dtype=torch.int64))
    assert d.format == DF.RawUInt32 and d.itemsize == 4
    d = T.pytorch_tensor_to_tensor_desc(torch.zeros(32, 32), df=DF.Bfp8_b)    # cast to the dtype Bfp8_b travels as
    assert d.format == DF.Bfp8_b and d.itemsize == 2
    nc = torch.zeros(64, 64).t()[:, ::2]
    d = T.pytorch_tensor_to_tensor_desc(nc)
    assert list(d.strides)[-2:] == [128, 4]                                    # made contiguous first
    with pytest.raises(RuntimeError):
        T.pytorch_tensor_to_tensor_desc(torch.zeros(4, dtype=torch.float64))
    x = torch.randn(1, 1, 32, 64)
    y = T.tensor_desc_to_pytorch_tensor(T.pytorch_tensor_to_tensor_desc(x))
    assert torch.equal(x, y) and y.data_ptr() == x.data_ptr()
    z = T.buffer_to_pytorch_tensor(x.data_ptr(), (32, 64), DF.Float32)
    assert list(z.shape) == [1, 1, 32, 64] and torch.equal(z[0, 0], x[0, 0])


def test_pad_and_narrow(T):
    x = torch.randn(3, 50, 70)
    p = T.pad_pytorch_tensor_to_buda(x, [])
    assert list(p.shape) == [1, 3, 64, 96]
    assert torch.equal(p[0, :, :50, :70], x) and p[..., 50:, :].abs().sum() == 0 and p[..., 70:].abs().sum() == 0
    assert torch.equal(T.narrow_buda_tensor_to_pytorch(p, (3, 50, 70)), x)
    b = torch.randn(1, 1, 1, 70)
    pb = T.pad_pytorch_tensor_to_buda(b, [-2])
    assert list(pb.shape) == [1, 1, 32, 96] and torch.equal(pb[0, 0, 17, :70], b[0, 0, 0])   # row replicated
    col = torch.randn(1, 1, 40, 1)
    pc = T.pad_pytorch_tensor_to_buda(col, [3])
    assert list(pc.shape) == [1, 1, 64, 32] and torch.equal(pc[0, 0, :40, 31], col[0, 0, :, 0])
    a = torch.randn(1, 1, 64, 64)
    assert T.pad_pytorch_tensor_to_buda(a, []) is a                              # already a buda shape
    m = T.pad_pytorch_tensor_to_buda(torch.randn(1, 33), [], microbatch=4)
    assert list(m.shape) == [4, 1, 32, 64]
    i8 = T.pad_pytorch_tensor_to_buda(torch.ones(5, 5, dtype=torch.int8), [])
    assert i8.dtype == torch.int8 and list(i8.shape) == [1, 1, 32, 32] and int(i8.sum()) == 25
    v = torch.randn(10)
    pv = T.pad_pytorch_tensor_to_buda(v, [])
    assert torch.equal(T.narrow_buda_tensor_to_pytorch(pv, (10,)), v)
    s = T.pad_pytorch_tensor_to_buda(torch.tensor(3.5), [])
    assert float(T.narrow_buda_tensor_to_pytorch(s, ())) == 3.5
    assert T.is_buda_shape(torch.zeros(1, 1, 32, 64)) and not T.is_buda_shape(torch.zeros(32, 64))
    assert T.is_buda_shape(torch.zeros(32, 64), min_dim=2)
    assert list(T.change_rank(torch.zeros(1, 1, 4, 5), 2).shape) == [4, 5]


def test_tensor_wrappers(C, T):
    DF = C.DataFormat
    t = T.Tensor.create_from_torch(torch.randn(2, 40, 40))
    assert t.data_format == DF.Float32 and t.pt_data_format == torch.float32 and t.has_value()
    assert t.shape.r == 40 and t.shape.rt == 2 and t.shape.z == 2 and t.shape.w == 1 and len(t.shape) == 3
    b = t.to_format(DF.Bfp8_b)
    assert b.data_format == DF.Bfp8_b and b.value().dtype == torch.bfloat16       # tagged + cast, never packed here
    p = t.to_buda_shape([])
    assert list(p.value().shape) == [1, 2, 64, 64]
    d = p.to_tensor_desc()
    back = T.Tensor.create_from_tensor_descriptor(d)
    assert back.data_format == DF.Float32 and back.shape == (1, 2, 64, 64)
    n = back.narrow_to_original_shape((2, 40, 40))
    assert torch.equal(n.value(), t.value())
    with pytest.raises(RuntimeError):
        back.to_buda_shape()
    assert T.to_pt_tensors([t, torch.zeros(1)])[0] is t.value()


# ------------------------------------------------------------------------------------------------
# runtime tensor transforms (reference: pybuda/pybuda/tensor.py:1382-1447)
# ------------------------------------------------------------------------------------------------
def test_runtime_transform_record_round_trips_through_json():
    import json
    from pybuda import tensor as T
    tr = T.RuntimeTensorTransform(T.RuntimeTensorTransformType.Prestride, original_shape=(1, 3, 224, 224), stride_height=2,
                                  stride_width=2, kernel_height=7, kernel_width=7)
    back = T.RuntimeTensorTransform.from_json(json.loads(json.dumps(tr.to_json())))
    assert back.to_json() == tr.to_json() and back.type is T.RuntimeTensorTransformType.Prestride


def test_embedding_index_layout():
    import pybuda._C as C
    from pybuda import tensor as T
    q = C.backend_api.DramIODesc.for_tensor("emb", [1, 1, 32, 64], C.DataFormat.RawUInt32)
    idx = torch.arange(1100, dtype=torch.int32)
    tr = T.RuntimeTensorTransform(T.RuntimeTensorTransformType.EmbeddingIndex, original_shape=(1100,))
    t, q2 = T.do_runtime_transform(tr, idx.clone(), q, [])
    assert t.shape == (1, 1, 32, 64) and q2 is q
    # 1100 indices pad to 1120 = 35 rows of 32 with all-ones, rows pad to 64 with zeros; tile row j of 32 indices
    # ends up as row j % 32 of the column block j // 32
    flat = torch.full((1120,), -1, dtype=torch.int32)
    flat[:1100] = idx
    rows = torch.zeros(64, 32, dtype=torch.int32)
    rows[:35] = flat.view(35, 32)
    want = rows.view(2, 32, 32).transpose(0, 1).reshape(32, 64)
    assert torch.equal(t[0, 0], want)


def test_prestride_transform_sets_the_stride_descriptor(oracle):
    import pybuda._C as C
    from pybuda import tensor as T
    q = C.backend_api.DramIODesc.for_tensor("conv_act", [1, 1, 32, 32], C.DataFormat.Float16_b)
    x = torch.randn(1, 3, 8, 8)
    y, q2 = T.eval_runtime_transform('{"type": "Prestride", "stride_height": 2, "stride_width": 2}', x, q, [])
    assert y is x and q2.s_descriptor.stride == 2
    assert q2.s_descriptor.xy_offsets == [(0, 0), (1, 0), (0, 1), (1, 1)]
    # the oracle's restatement of the golden prestride against the golden's own torch formulation (tm.py:316-335)
    a = torch.arange(2 * 3 * 5 * 7, dtype=torch.float32).reshape(2, 3, 5, 7)
    act = torch.nn.functional.pad(a, (0, 1, 0, 1))
    gold = torch.cat([act[:, :, yy::2, xx::2] for yy in range(2) for xx in range(2)], dim=-3)
    gold = gold.view(2, 1, 12, 12)
    assert np.array_equal(oracle.prestride_act(a.numpy(), 2), gold.numpy())
    with pytest.raises(AssertionError):
        T._prestride_shape(x, 2, 3, q)


def test_reinterpret_shape_pads_to_the_queue_tiles():
    import pybuda._C as C
    from pybuda import tensor as T
    q = C.backend_api.DramIODesc.for_tensor("r", [1, 1, 32, 64], C.DataFormat.Float32)
    x = torch.arange(2 * 3 * 10, dtype=torch.float32).reshape(2, 30)
    tr = T.RuntimeTensorTransform(T.RuntimeTensorTransformType.ReinterpretShape, reinterpreted_shape=(1, 1, 1, 60))
    y, _ = T.do_runtime_transform(tr, x, q, [])
    assert y.shape == (1, 1, 32, 64) and torch.equal(y[0, 0, 0, :60], x.reshape(-1)) and y[0, 0, 1:].abs().sum() == 0



def test_cpp_twins_of_the_torch_device_descriptor_helpers():
    """to_pytorch_tensor_desc / pad_to_buda_shape of the reference's torch device plugin
    (pybuda/csrc/tt_torch_device/tt_device.cpp:109-189), restated on (pointer, sizes, strides)."""
    import pybuda._C as C
    B, DF = C.backend_api, C.DataFormat
    t = torch.zeros(3, 50, 70)
    d = B.to_pytorch_tensor_desc(t.data_ptr(), 4, DF.Float32, list(t.shape), list(t.stride()))
    # sizes right-aligned, r / c rounded UP to the tile, byte strides, the missing w stride copied from z
    assert (list(d.shape), list(d.strides), d.dim, d.itemsize, d.format) == ([1, 3, 64, 96], [14000, 14000, 280, 4], 4, 4, DF.Float32)
    v = torch.zeros(17, dtype=torch.bfloat16)
    d = B.to_pytorch_tensor_desc(v.data_ptr(), 2, DF.Float16_b, [17], [1])
    assert (list(d.shape), list(d.strides)) == ([1, 1, 32, 32], [64, 64, 64, 2])          # 1-D: one tile row per implied row
    assert list(B.buda_padded_shape([3, 50, 70])) == [1, 3, 64, 96]
    assert list(B.buda_padded_shape([5])) == [1, 1, 32, 32]
    with pytest.raises(ValueError):
        B.to_pytorch_tensor_desc(t.data_ptr(), 4, DF.Float32, [1, 2, 3, 4, 5], [1, 1, 1, 1, 1])
    with pytest.raises(ValueError):
        B.buda_padded_shape([1, 2, 3, 4, 5])
