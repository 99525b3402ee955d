"""GPU tests with ONE tensor above 4 GiB: every byte offset the kernels form must be 64-bit (the reference pushes
parameters of 1-8 GB, pybuda/test/test_large_parameters.py).  The whole tensor cannot go through the CPU oracle in test
time, so the checks are: the two kernel paths and the job-table flavour agree on the whole image; the tile rows past
the 4 GiB mark equal the oracle's image of that slice, byte for byte; the round trip of a plain relayout gives the
tensor back exactly."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

R_ROWS, C_COLS = 36864, 32768          # 4.83e9 bytes of float32: rows past 32768 start beyond 2^32


@pytest.fixture(scope="module")
def big():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    free, _ = torch.cuda.mem_get_info()
    if free < 24 * 2 ** 30:
        pytest.skip("needs 24 GiB of free device memory")
    from pybuda import cuda_ops

    g = torch.Generator(device="cuda").manual_seed(2024)
    x = torch.randn(1, 1, R_ROWS, C_COLS, device="cuda", generator=g)
    x[0, 0, R_ROWS - 40, 100:116] = torch.tensor([3.0e5, -2.5e-7, 0.0, 1.0] * 4, device="cuda")   # an outlier block near the end
    assert x.numel() * 4 > 2 ** 32
    yield cuda_ops, x
    del x
    torch.cuda.empty_cache()


def _tail(x, rows):
    return x[:, :, R_ROWS - rows:, :].contiguous().cpu().numpy()


def test_block_float_pack_of_a_tensor_above_4_gib(big, oracle):
    ops, x = big
    img = ops.tilize_pack(x, ops.DF.Bfp8_b)                       # staged kernel
    img_direct = ops.tilize_pack(x, ops.DF.Bfp8_b, path=1)        # direct kernel
    assert torch.equal(img, img_direct)
    del img_direct
    img_jobs = ops.tilize_pack_jobs([x], ops.DF.Bfp8_b)[0]        # job-table flavour
    assert torch.equal(img, img_jobs)
    del img_jobs
    # the last two tile rows (source offsets above 2^32) against the oracle's image of that slice: with a 1 x 1 grid the
    # records of a tile row are contiguous and tile rows follow one another
    rows = 64
    want = oracle.tilize_pack(_tail(x, rows), oracle.Bfp8_b)
    tail_bytes = (rows // 32) * (C_COLS // 32) * 1088
    assert want.size == tail_bytes
    assert np.array_equal(img[-tail_bytes:].cpu().numpy(), want)
    head = oracle.tilize_pack(x[:, :, :32, :].contiguous().cpu().numpy(), oracle.Bfp8_b)
    assert np.array_equal(img[: head.size].cpu().numpy(), head)
    # and back: the tail rows of the unpacked tensor equal the oracle's decode of that slice
    y = ops.unpack_untilize(img, ops.DF.Bfp8_b, x.shape)
    ref = oracle.unpack_untilize(want, oracle.Bfp8_b, (1, 1, rows, C_COLS))
    assert np.array_equal(_tail(y, rows).view(np.uint32), ref.view(np.uint32))
    y2 = ops.unpack_untilize(img, ops.DF.Bfp8_b, x.shape, path=1)
    assert torch.equal(y.view(torch.int32), y2.view(torch.int32))
    rc, st = ops._cabi.device_status()
    assert rc == 0 and st == 0


def test_plain_relayout_with_both_sides_above_4_gib(big, oracle):
    ops, x = big
    img = ops.tilize_pack(x, ops.DF.Float32)
    assert img.numel() == x.numel() * 4 and img.numel() > 2 ** 32
    rows = 32
    want = oracle.tilize_pack(_tail(x, rows), oracle.Float32)
    assert np.array_equal(img[-want.size:].cpu().numpy(), want)   # image offsets above 2^32
    y = ops.unpack_untilize(img, ops.DF.Float32, x.shape)
    assert torch.equal(y.view(torch.int32), x.view(torch.int32))
    del y
    img_direct = ops.tilize_pack(x, ops.DF.Float32, path=1)
    assert torch.equal(img, img_direct)
    rc, st = ops._cabi.device_status()
    assert rc == 0 and st == 0


def test_host_buffer_pipeline_with_a_tensor_above_4_gib(big, oracle):
    """The sliced host pipeline (buda_tilize_pack_host / buda_unpack_untilize_host) forms host-side offsets above 2^32 too."""
    import ctypes

    ops, x = big
    cabi = ops._cabi
    shape = list(x.shape)
    xh = x.cpu()                                   # pageable host memory: the entry point stages it itself
    gq = ops.QueueGeom.for_shape(shape)
    n = cabi.tilized_bytes(gq, shape, int(ops.DF.Bfp8_b))
    img = torch.empty(n, dtype=torch.uint8)
    st = cabi.u64x4(cabi.dense_strides(shape, 4))
    cabi.check(cabi.lib.buda_tilize_pack_host(xh.data_ptr(), int(ops.DF.Float32), cabi.u32x4(shape), st, ctypes.byref(gq),
                                              int(ops.DF.Bfp8_b), 0, img.data_ptr(), n, None))
    want = ops.tilize_pack(x, ops.DF.Bfp8_b).cpu()
    assert torch.equal(img, want)
    del want
    y = torch.empty(shape, dtype=torch.float32)
    cabi.check(cabi.lib.buda_unpack_untilize_host(img.data_ptr(), int(ops.DF.Bfp8_b), 0, ctypes.byref(gq), y.data_ptr(),
                                                  int(ops.DF.Float32), cabi.u32x4(shape), st, None))
    rows = 64
    tail_bytes = (rows // 32) * (C_COLS // 32) * 1088
    ref = oracle.unpack_untilize(img[-tail_bytes:].numpy(), oracle.Bfp8_b, (1, 1, rows, C_COLS))
    assert np.array_equal(y[:, :, R_ROWS - rows:, :].contiguous().numpy().view(np.uint32), ref.view(np.uint32))
    rc, st_ = cabi.device_status()
    assert rc == 0 and st_ == 0


@pytest.mark.parametrize("shape", [(1, 1, 32, 262144), (1, 1, 131072, 32), (256, 4, 32, 32), (3, 5, 96, 4128)])
@pytest.mark.parametrize("df_name", ["Bfp8_b", "Bfp2_b", "Float16_b"])
def test_extreme_aspect_ratios_against_the_oracle(oracle, shape, df_name):
    """One tile row of 8192 tiles, 4096 tile rows of one tile, a thousand single-tile slices, a ragged width: whole images
    against the oracle on both kernel paths, and back."""
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    from pybuda import cuda_ops as ops

    g = torch.Generator().manual_seed(sum(shape))
    x = torch.randn(shape, generator=g) * torch.exp(torch.empty(shape).uniform_(-3.0, 3.0, generator=g))
    if df_name == "Float16_b":
        x = x.bfloat16()
        xn = x.view(torch.int16).numpy().view(np.uint16)
        want = oracle.tilize_pack(xn, oracle.Float16_b, src_df=oracle.Float16_b)
    else:
        want = oracle.tilize_pack(x.numpy(), getattr(oracle, df_name))
    df = getattr(ops.DF, df_name)
    for path in (0, 1):
        img = ops.tilize_pack(x.cuda(), df, path=path)
        assert np.array_equal(img.cpu().numpy(), want), path
        y = ops.unpack_untilize(img, df, shape, dtype=x.dtype, path=path).cpu()
        if df_name == "Float16_b":
            assert torch.equal(y.view(torch.int16), x.view(torch.int16)), path
        else:
            ref = oracle.unpack_untilize(want, getattr(oracle, df_name), shape)
            assert np.array_equal(y.numpy().view(np.uint32), ref.view(np.uint32)), path
