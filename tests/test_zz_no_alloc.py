"""GPU test of the tilize + pack entry point that allocates nothing.

Some users of the library cannot call cudaMalloc at the moment they need a conversion: a pusher
thread sharing a process with a framework whose caching allocator already owns the device heap, or a
loop that must not pay the device-wide synchronisation an allocation implies.  For them
buda_tilize_pack_host_noalloc stages through a fixed 8 MiB array inside the library.  This test
calls it through the C ABI twice in a row (second call with another shape and format, so bytes left
in the shared array by the first call would show) and compares every output byte with the ordinary
host-buffer entry point and with the CPU oracle; it also checks that an oversize request is refused with a
clear message."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(cabi, x, dst_df, with_header, geom):
    shape = list(x.shape)
    n = cabi.tilized_bytes(geom, shape, dst_df, with_header)
    st = cabi.u64x4(cabi.dense_strides(shape, x.element_size()))
    src_df = 0 if x.dtype == torch.float32 else 5
    ref = torch.zeros(n, dtype=torch.uint8)
    got = torch.full((n,), 0xAB, dtype=torch.uint8)
    cabi.check(cabi.lib.buda_tilize_pack_host(x.data_ptr(), src_df, cabi.u32x4(shape), st, ctypes.byref(geom), dst_df,
                                              int(with_header), ref.data_ptr(), n, None))
    cabi.check(cabi.lib.buda_tilize_pack_host_noalloc(x.data_ptr(), src_df, cabi.u32x4(shape), st, ctypes.byref(geom), dst_df,
                                                      int(with_header), got.data_ptr(), n, None))
    return got, ref


def _oracle_image(oracle, x, df, with_header, grid=(1, 1), ublock=(1, 1), order=0):
    import numpy as np
    geom = oracle.Geom.for_shape(list(x.shape), grid, ublock, order)
    if x.dtype == torch.bfloat16:
        return oracle.tilize_pack(x.view(torch.int16).numpy().view(np.uint16), df, geom, with_header, src_df=oracle.Float16_b)
    return oracle.tilize_pack(x.numpy(), df, geom, with_header)


def test_no_alloc_entry_point_matches_host_entry_point_on_two_calls(oracle):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device; there is no CPU fallback to test")
    import numpy as np
    from pybuda import _cabi as cabi

    g = torch.Generator().manual_seed(123)
    # call 1: the single-tensor config, fp32 [1,1,1024,1024] -> Bfp8_b (4 MiB + 1.06 MiB of the 8 MiB)
    x1 = torch.randn(1, 1, 1024, 1024, generator=g)
    got1, ref1 = _both(cabi, x1, 6, False, cabi.QueueGeom.for_shape(list(x1.shape)))
    assert torch.equal(got1, ref1)
    assert np.array_equal(got1.numpy(), _oracle_image(oracle, x1, oracle.Bfp8_b, False))
    # call 2, straight after: smaller tensor, other format, tile headers, another queue geometry
    x2 = (torch.randn(2, 3, 128, 160, generator=g) * 100).bfloat16()
    got2, ref2 = _both(cabi, x2, 7, True, cabi.QueueGeom.for_shape(list(x2.shape), (2, 1), (1, 5), 1))
    assert torch.equal(got2, ref2)
    assert np.array_equal(got2.numpy(), _oracle_image(oracle, x2, oracle.Bfp4_b, True, (2, 1), (1, 5), 1))
    # and the first input once more gives the first answer
    got3, _ = _both(cabi, x1, 6, False, cabi.QueueGeom.for_shape(list(x1.shape)))
    assert torch.equal(got3, ref1)
    rc, st = cabi.device_status()
    assert rc == 0 and st == 0


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device; there is no CPU fallback to test")
    from pybuda import _cabi as cabi

    x = torch.zeros(1, 1, 2048, 1024)  # 8 MiB of fp32 alone fills the array: no room for the image
    shape = list(x.shape)
    geom = cabi.QueueGeom.for_shape(shape)
    n = cabi.tilized_bytes(geom, shape, 6, False)
    out = torch.zeros(n, dtype=torch.uint8)
    rc = cabi.lib.buda_tilize_pack_host_noalloc(x.data_ptr(), 0, cabi.u32x4(shape), cabi.u64x4(cabi.dense_strides(shape, 4)),
                                                ctypes.byref(geom), 6, 0, out.data_ptr(), n, None)
    assert rc == cabi.RUNTIME_ERROR
    msg = cabi.last_error()
    assert "static scratch" in msg and "8388608" in msg
