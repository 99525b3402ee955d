"""GPU tests of the Lf8 conversions (one 1-5-2 float per element, docs/public/dataformats.rst:24 of the reference):
binary32 / bfloat16 / binary16 -> Lf8 tile records and back, checked against the CPU oracle and against the
committed vectors of the exact-arithmetic spec.  Parity unpinned: the reference documents the field widths only."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    from pybuda import cuda_ops

    return cuda_ops


def _np_of(x):
    if x.dtype == torch.bfloat16:
        return x.view(torch.int16).numpy().view(np.uint16)
    return x.numpy()


def _src_df(oracle, x):
    return {torch.float32: oracle.Float32, torch.bfloat16: oracle.Float16_b, torch.float16: oracle.Float16}[x.dtype]


def _values(shape, seed, dtype):
    """Spread over the whole Lf8 range and beyond both ends, with ties, zeros, Inf and NaN."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g) * torch.exp(torch.empty(shape).uniform_(-13.0, 12.0, generator=g))
    flat = x.view(-1)
    special = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan"), 57344.0, 61440.0, 61439.0, 65504.0, 1e9, -1e9,
                            2.0 ** -14, 2.0 ** -15, 2.0 ** -16, 2.0 ** -17, 1.5 * 2.0 ** -16, 2.5 * 2.0 ** -16, 3.5 * 2.0 ** -16,
                            1.125, 1.375, 1.625, 1.875, -1.125, -1.375, 1e-30, 1e-45])
    flat[: special.numel()] = special
    flat[1000: 1000 + special.numel()] = -special
    return x.to(dtype)


def test_committed_vectors_on_the_gpu(ops, oracle):
    kat = np.load(os.path.join(HERE, "golden", "lf8_kat.npz"))
    bits, codes = kat["bits"], kat["codes"]
    n = bits.size
    cols = 64
    rows = -(-n // cols)
    rows += (-rows) % 32
    padded = np.zeros(rows * cols, dtype=np.uint32)
    padded[:n] = bits
    x = torch.from_numpy(padded.view(np.float32).reshape(1, 1, rows, cols).copy())
    img = ops.tilize_pack(x.cuda(), ops.DF.Lf8)
    # a relayout (uint8 row-major side) brings the codes back into the order of the inputs
    got = ops.unpack_untilize(img, ops.DF.Lf8, (1, 1, rows, cols), dtype=torch.uint8).cpu().numpy().reshape(-1)[:n]
    nan = np.isnan(bits.view(np.float32))
    assert np.array_equal(got[~nan], codes[~nan])
    assert np.all((got[nan] & 0x7F) == 0x7F)
    # decode of every code, into each float type
    allc = torch.arange(256, dtype=torch.uint8).repeat(4 * 32).reshape(1, 1, 32, 1024)
    cimg = ops.tilize_pack(allc.cuda(), ops.DF.Lf8)
    f = ops.unpack_untilize(cimg, ops.DF.Lf8, (1, 1, 32, 1024), dtype=torch.float32).cpu().numpy().view(np.uint32)
    assert np.array_equal(f[0, 0, 0, :256], kat["decode"])
    h = ops.unpack_untilize(cimg, ops.DF.Lf8, (1, 1, 32, 1024), dtype=torch.float16).cpu().view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(h[0, 0, 5, :256], np.arange(256, dtype=np.uint16) << 8)
    b = ops.unpack_untilize(cimg, ops.DF.Lf8, (1, 1, 32, 1024), dtype=torch.bfloat16).cpu().view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(b[0, 0, 31, :256], (kat["decode"] >> 16).astype(np.uint16))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hdr", [False, True])
def test_pack_and_unpack_match_the_oracle(ops, oracle, dtype, hdr):
    shape = (2, 2, 96, 160)
    x = _values(shape, 7, dtype)
    gq = ops.QueueGeom.for_shape(shape, (1, 1), (3, 1), 1)
    go = oracle.Geom.for_shape(shape, (1, 1), (3, 1), 1)
    want = oracle.tilize_pack(_np_of(x), oracle.Lf8, go, hdr, src_df=_src_df(oracle, x))
    img = ops.tilize_pack(x.cuda(), ops.DF.Lf8, gq, hdr)
    assert np.array_equal(img.cpu().numpy(), want)
    # arbitrary bytes decode the same way (NaN codes included)
    raw = torch.randint(0, 256, (want.size,), dtype=torch.uint8, generator=torch.Generator().manual_seed(8))
    np_dt = {torch.float32: np.float32, torch.bfloat16: np.uint16, torch.float16: np.float16}[dtype]
    ref = oracle.unpack_untilize(raw.numpy(), oracle.Lf8, shape, np_dt, geom=go, with_header=hdr, dst_df=_src_df(oracle, x))
    got = ops.unpack_untilize(raw.cuda(), ops.DF.Lf8, shape, dtype, gq, hdr).cpu()
    assert np.array_equal(got.view(torch.uint8).numpy(), np.ascontiguousarray(ref).view(np.uint8).reshape(got.view(torch.uint8).shape))


def test_against_an_independent_e5m2_cast(ops):
    if not hasattr(torch, "float8_e5m2"):
        pytest.skip("this torch has no float8_e5m2")
    shape = (1, 1, 256, 512)
    x = _values(shape, 11, torch.float32)
    img = ops.tilize_pack(x.cuda(), ops.DF.Lf8)
    codes = ops.unpack_untilize(img, ops.DF.Lf8, shape, dtype=torch.uint8).cpu()
    want = x.to(torch.float8_e5m2).view(torch.uint8)
    nan = torch.isnan(x)
    assert torch.equal(codes[~nan], want[~nan])


def test_unaligned_views_tiny_tiles_and_face_order(ops, oracle):
    from pybuda._cabi import QueueGeom
    base = _values((1, 1, 64, 132), 21, torch.float32).cuda()
    v = base[..., 1:129]
    assert v.data_ptr() % 16 != 0
    want = oracle.tilize_pack(v.cpu().contiguous().numpy(), oracle.Lf8)
    assert np.array_equal(ops.tilize_pack(v, ops.DF.Lf8).cpu().numpy(), want)
    out = torch.full((1, 1, 64, 132), 7.0, device="cuda")
    ops.unpack_untilize(torch.from_numpy(want).cuda(), ops.DF.Lf8, (1, 1, 64, 128), out=out[..., 1:129])
    assert torch.all(out[..., 0] == 7.0) and torch.all(out[..., 129:] == 7.0)
    ref = oracle.unpack_untilize(want, oracle.Lf8, (1, 1, 64, 128))
    assert np.array_equal(out[..., 1:129].cpu().contiguous().numpy().view(np.uint32), ref.view(np.uint32))
    # 8 x 32 tiles
    shape = (2, 1, 32, 96)
    x = _values(shape, 22, torch.bfloat16)
    geom = QueueGeom.for_shape(shape, tile_height=8)
    ogeom = oracle.Geom.for_shape(shape, (1, 1), (1, 1), 0, 8)
    want = oracle.tilize_pack(_np_of(x), oracle.Lf8, ogeom, src_df=oracle.Float16_b)
    assert np.array_equal(ops.tilize_pack(x.cuda(), ops.DF.Lf8, geom).cpu().numpy(), want)
    # another face order moves the blocks of the record, nothing else
    from pybuda import _cabi
    try:
        ops.set_bfp_policy(_cabi.BfpPolicy(face_order=(0, 2, 1, 3)))
        oracle.set_bfp_policy(oracle.BfpPolicy(face_order=(0, 2, 1, 3)))
        y = _values((1, 1, 64, 64), 23, torch.float32)
        want = oracle.tilize_pack(y.numpy(), oracle.Lf8)
        img = ops.tilize_pack(y.cuda(), ops.DF.Lf8)
        assert np.array_equal(img.cpu().numpy(), want)
        back = ops.unpack_untilize(img, ops.DF.Lf8, (1, 1, 64, 64)).cpu().numpy()
        assert np.array_equal(back.view(np.uint32), oracle.unpack_untilize(want, oracle.Lf8, (1, 1, 64, 64)).view(np.uint32))
    finally:
        ops.set_bfp_policy(None)
        oracle.set_bfp_policy(None)
    # the staged kernels do not convert to Lf8: asking for them by name is refused
    with pytest.raises(ops._cabi.BudaError, match="staged path"):
        ops.tilize_pack(_values((1, 1, 32, 64), 24, torch.float32).cuda(), ops.DF.Lf8, path=0)


def test_lf8_queue_through_the_backend_api(oracle):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device; there is no CPU fallback to test")
    import pybuda._C as C
    from pybuda import tensor as T
    B, DF = C.backend_api, C.DataFormat
    try:
        x = _values((1, 2, 64, 96), 31, torch.float32)
        q = B.DramIODesc.for_tensor("lf8_q", [1, 2, 64, 96], DF.Lf8)
        assert B.push_input(q, T.pytorch_tensor_to_tensor_desc(x), True, 1, -1) == B.BackendStatusCode.Success, B.last_error()
        out = B.PytorchTensorDesc()
        out.format = DF.Float32
        assert B.get_output(q, out, True, 1, -1) == B.BackendStatusCode.Success, B.last_error()
        y = T.tensor_desc_to_pytorch_tensor(out).clone()
        B.pop_output(q, True, 1)
        B.free_tensor(out)
        want = oracle.unpack_untilize(oracle.tilize_pack(x.numpy(), oracle.Lf8), oracle.Lf8, x.shape)
        nan = np.isnan(want)
        assert np.array_equal(y.numpy().view(np.uint32)[~nan], want.view(np.uint32)[~nan])
        assert np.all(np.isnan(y.numpy()[nan]))
    finally:
        B.release_all_queues()
