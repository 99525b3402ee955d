"""GPU tests of the block-float layout policies and of the job-table entry points (tensors of different shapes in one
launch; a selection of tile rows per tensor).  Everything is compared byte for byte with the CPU oracle under the
same policy, and the policy known-answer vectors (exact-arithmetic spec) are checked on both kernel paths."""
import ctypes
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


def _policies():
    kp = np.load(os.path.join(HERE, "golden", "bfp_kat_policies.npz"))
    return kp, [tuple(int(v) for v in row) for row in kp["policies"]]


def _set_both(ops, oracle, row):
    from pybuda import _cabi
    if row is None:
        ops.set_bfp_policy(None)
        oracle.set_bfp_policy(None)
        return
    ops.set_bfp_policy(_cabi.BfpPolicy(row[0], row[1], row[2:6], row[6], row[7]))
    oracle.set_bfp_policy(oracle.BfpPolicy(row[0], row[1], row[2:6], row[6], row[7]))


def _kat_tiles():
    k = np.load(os.path.join(HERE, "golden", "bfp_kat.npz"))
    x = np.zeros((1, 1, 32, 128), np.uint32)
    for b in range(256):
        t, blk = divmod(b, 64)
        face, fr = divmod(blk, 16)
        x[0, 0, (face >> 1) * 16 + fr, t * 32 + (face & 1) * 16: t * 32 + (face & 1) * 16 + 16] = k["x"][b]
    return x


def _special(shape, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    flat = x.view(-1)
    flat[torch.rand(flat.numel(), generator=g) < 0.01] *= 1e3
    flat[torch.rand(flat.numel(), generator=g) < 0.005] = 0.0
    rows = flat.view(-1, 16)
    k = rows.shape[0]
    rows[k // 7] = 0.0
    rows[k // 6] = torch.randn(16, generator=g) * 2.0 ** -124
    rows[k // 5] = torch.randn(16, generator=g) * 1e-41
    rows[k // 4] = torch.randn(16, generator=g) * 2.0 ** 126
    rows[k // 3] = torch.tensor([float("inf"), float("-inf"), float("nan"), 1e38, -1e30, 1.0, 0.0, -0.0] * 2)
    rows[k // 2] = torch.tensor([1.0, 1.9999, -1.9999, 1.984375, 1.9921875, 1.99609375, 1.0078125, 1.00390625] * 2)
    rows[k // 2 + 1] = torch.tensor([3.4e38, 3.39e38, -3.4e38, 1e38] * 4)     # rounds up at the top exponent
    return x


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("df_name,m", [("Bfp8_b", 7), ("Bfp4_b", 3), ("Bfp2_b", 1)])
def test_policy_known_answers_on_the_gpu(ops, oracle, df_name, m, path):
    kp, rows = _policies()
    xt = torch.from_numpy(_kat_tiles().view(np.float32)).cuda()
    df = getattr(ops.DF, df_name)
    try:
        for pi, row in enumerate(rows):
            _set_both(ops, oracle, row)
            img = ops.tilize_pack(xt, df, path=path).cpu().numpy()
            want = kp[f"records{m}"][pi].reshape(-1)
            assert np.array_equal(img, want), (pi, row, int(np.argmax(img != want)))
            back = ops.unpack_untilize(torch.from_numpy(want).cuda(), df, (1, 1, 32, 128), path=path).cpu().numpy()
            ref = oracle.unpack_untilize(want, getattr(oracle, df_name), (1, 1, 32, 128))
            assert np.array_equal(back.view(np.uint32), ref.view(np.uint32)), (pi, row, "decode")
    finally:
        _set_both(ops, oracle, None)
    assert tuple(ops.get_bfp_policy().face_order) == (0, 1, 2, 3)


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("src", ["f32", "bf16"])
def test_policies_against_the_oracle_on_special_values(ops, oracle, path, src):
    _, rows = _policies()
    shape = (2, 2, 64, 160)          # ragged last band of tiles for the staged kernel (5 tile columns)
    x = _special(shape, 31)
    try:
        for row in rows:
            _set_both(ops, oracle, row)
            for df_name in ("Bfp8_b", "Bfp4_b", "Bfp2_b"):
                df = getattr(ops.DF, df_name)
                if src == "f32":
                    img = ops.tilize_pack(x.cuda(), df, path=path)
                    ref = oracle.tilize_pack(x.numpy(), getattr(oracle, df_name))
                else:
                    xb = x.bfloat16()
                    img = ops.tilize_pack(xb.cuda(), df, path=path)
                    ref = oracle.tilize_pack(xb.view(torch.int16).numpy().view(np.uint16), getattr(oracle, df_name), src_df=oracle.Float16_b)
                assert np.array_equal(img.cpu().numpy(), ref), (row, df_name, "pack")
                y = ops.unpack_untilize(img, df, shape, path=path)
                yref = oracle.unpack_untilize(ref, getattr(oracle, df_name), shape)
                assert np.array_equal(y.cpu().numpy().view(np.uint32), yref.view(np.uint32)), (row, df_name, "unpack")
    finally:
        _set_both(ops, oracle, None)


def test_policies_cover_plain_formats_a_formats_headers_and_geometry(ops, oracle):
    """Face order applies to every format; the "a" formats raise their 5-bit exponent only below 31."""
    _, rows = _policies()
    shape = (1, 2, 128, 128)
    g = torch.Generator().manual_seed(9)
    xi = torch.randint(-2 ** 31, 2 ** 31 - 1, shape, generator=g, dtype=torch.int32)
    xh = (torch.randn(shape, generator=g) * 8).half()
    xh.view(-1)[::37] = float("inf")
    xh.view(-1)[5::41] = 65504.0
    gq, go = ops.QueueGeom.for_shape(shape, (2, 1), (1, 2), 1), oracle.Geom.for_shape(shape, (2, 1), (1, 2), 1)
    try:
        for row in rows[4:]:
            _set_both(ops, oracle, row)
            for path in (0, 1):
                img = ops.tilize_pack(xi.cuda(), ops.DF.Int32, gq, with_header=True, path=path)
                ref = oracle.tilize_pack(xi.numpy(), oracle.Int32, go, with_header=True)
                assert np.array_equal(img.cpu().numpy(), ref), (row, path, "int32 relayout")
                back = ops.unpack_untilize(img, ops.DF.Int32, shape, dtype=torch.int32, geom=gq, with_header=True, path=path)
                assert torch.equal(back.cpu(), xi)
                for df_name in ("Bfp8", "Bfp4", "Bfp2"):
                    img = ops.tilize_pack(xh.cuda(), getattr(ops.DF, df_name), gq, path=path)
                    ref = oracle.tilize_pack(xh.numpy(), getattr(oracle, df_name), go)
                    assert np.array_equal(img.cpu().numpy(), ref), (row, path, df_name)
                    y = ops.unpack_untilize(img, getattr(ops.DF, df_name), shape, dtype=torch.float16, geom=gq, path=path)
                    yref = oracle.unpack_untilize(ref, getattr(oracle, df_name), shape, dst_dtype=np.float16, geom=go)
                    assert np.array_equal(y.cpu().numpy().view(np.uint16), yref.view(np.uint16)), (row, path, df_name, "unpack")
    finally:
        _set_both(ops, oracle, None)


def test_matmul_refuses_a_layout_it_cannot_read(ops):
    from pybuda import _cabi
    a = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    w = ops.tilize_pack(torch.zeros(1, 1, 64, 256, device="cuda"), ops.DF.Bfp8_b)
    try:
        ops.set_bfp_policy(_cabi.BfpPolicy(rounding=1, overflow=1))       # rounding / overflow do not change how bytes are read
        ops.bfp8b_matmul(a, w, 256)
        ops.set_bfp_policy(_cabi.BfpPolicy(datum_order=1))
        with pytest.raises(_cabi.BudaError):
            ops.bfp8b_matmul(a, w, 256)
        with pytest.raises(_cabi.BudaError):
            ops.set_bfp_policy(_cabi.BfpPolicy(face_order=(0, 1, 1, 3)))
    finally:
        ops.set_bfp_policy(None)


# ------------------------------------------------------------------------------------------------
# job tables: tensors of different shapes in one launch; a selection of tile rows per tensor
# ------------------------------------------------------------------------------------------------
def _mixed_set(seed):
    g = torch.Generator().manual_seed(seed)
    shapes = [(1, 1, 64, 64), (1, 1, 32, 4096), (2, 3, 96, 160), (1, 1, 1024, 1024), (1, 2, 256, 32), (1, 1, 4096, 1024)]
    return [torch.randn(s, generator=g) * 0.02 for s in shapes]


@pytest.mark.parametrize("df_name", ["Bfp8_b", "Bfp4_b", "Bfp2_b"])
def test_job_table_packs_and_unpacks_a_mixed_set_in_one_launch(ops, oracle, df_name):
    from pybuda import _cabi
    xs = _mixed_set(3)
    df = getattr(ops.DF, df_name)
    n0 = _cabi.launch_count()
    imgs = ops.tilize_pack_jobs([x.cuda() for x in xs], df)
    assert _cabi.launch_count() - n0 == 1
    for x, img in zip(xs, imgs):
        assert np.array_equal(img.cpu().numpy(), oracle.tilize_pack(x.numpy(), getattr(oracle, df_name))), tuple(x.shape)
    outs = [torch.empty(x.shape, device="cuda") for x in xs]
    n0 = _cabi.launch_count()
    ops.unpack_untilize_jobs(imgs, df, outs)
    assert _cabi.launch_count() - n0 == 1
    for x, img, y in zip(xs, imgs, outs):
        ref = oracle.unpack_untilize(img.cpu().numpy(), getattr(oracle, df_name), tuple(x.shape))
        assert np.array_equal(y.cpu().numpy().view(np.uint32), ref.view(np.uint32)), tuple(x.shape)


def test_job_table_geometries_headers_bf16_and_plain(ops, oracle):
    g = torch.Generator().manual_seed(4)
    specs = [((1, 2, 128, 256), (2, 2), (1, 2), 1), ((2, 1, 64, 64), (1, 1), (2, 1), 0), ((1, 1, 96, 96), (3, 1), (1, 3), 0),
             ((1, 4, 32, 32), (1, 1), (1, 1), 0)]
    xs = [torch.randn(s[0], generator=g) for s in specs]
    gq = [ops.QueueGeom.for_shape(s[0], s[1], s[2], s[3]) for s in specs]
    go = [oracle.Geom.for_shape(s[0], s[1], s[2], s[3]) for s in specs]
    imgs = ops.tilize_pack_jobs([x.bfloat16().cuda() for x in xs], ops.DF.Bfp8_b, geoms=gq, with_header=True)
    for x, img, o in zip(xs, imgs, go):
        ref = oracle.tilize_pack(x.bfloat16().view(torch.int16).numpy().view(np.uint16), oracle.Bfp8_b, o, with_header=True,
                                 src_df=oracle.Float16_b)
        assert np.array_equal(img.cpu().numpy(), ref), tuple(x.shape)
    outs = [torch.empty(x.shape, dtype=torch.bfloat16, device="cuda") for x in xs]
    ops.unpack_untilize_jobs(imgs, ops.DF.Bfp8_b, outs, geoms=gq, with_header=True)
    for x, img, y, o in zip(xs, imgs, outs, go):
        ref = oracle.unpack_untilize(img.cpu().numpy(), oracle.Bfp8_b, tuple(x.shape), dst_dtype=np.uint16, geom=o, with_header=True,
                                     dst_df=oracle.Float16_b)
        assert np.array_equal(y.view(torch.int16).cpu().numpy().view(np.uint16), ref), tuple(x.shape)
    xi = [torch.randint(-128, 128, s[0], generator=g, dtype=torch.int8) for s in specs]
    imgs = ops.tilize_pack_jobs([x.cuda() for x in xi], ops.DF.Int8, geoms=gq)
    for x, img, o in zip(xi, imgs, go):
        assert np.array_equal(img.cpu().numpy(), oracle.tilize_pack(x.numpy(), oracle.Int8, o)), tuple(x.shape)


def test_job_table_spills_into_several_launches_and_takes_unaligned_tensors(ops, oracle):
    from pybuda import _cabi
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(1, 1, 32, 32 * (1 + i % 3), generator=g) for i in range(200)]      # more than one table holds
    base = torch.randn(33 * 64 + 1, generator=g).cuda()
    odd = base[1:].view(1, 1, 33, 64)[:, :, :32, :]                                        # rows start 4 bytes off a 16-byte boundary
    n0 = _cabi.launch_count()
    imgs = ops.tilize_pack_jobs([x.cuda() for x in xs] + [odd], ops.DF.Bfp4_b)
    assert _cabi.launch_count() - n0 == 3          # 192 + 8 table entries, and the direct kernel for the unaligned tensor
    for x, img in zip(xs + [odd.cpu()], imgs):
        assert np.array_equal(img.cpu().numpy(), oracle.tilize_pack(x.contiguous().numpy(), oracle.Bfp4_b))


@pytest.mark.parametrize("world", [2, 3, 8])
def test_tile_row_bands_of_one_tensor_land_in_one_image(ops, oracle, world):
    """Band b -> rank b mod world: every rank converts its tile rows straight into the shared image; after all ranks
    the image equals the whole-tensor conversion.  Also through a grid / ublock geometry, where a band's records are
    not contiguous."""
    g = torch.Generator().manual_seed(6)
    for shape, grid, ub, order in (((1, 1, 1024, 1024), (1, 1), (1, 1), 0), ((2, 2, 256, 192), (2, 3), (2, 1), 1)):
        x = torch.randn(shape, generator=g)
        x.view(-1)[::101] *= 1e3
        xc = x.cuda()
        gq, go = ops.QueueGeom.for_shape(shape, grid, ub, order), oracle.Geom.for_shape(shape, grid, ub, order)
        ref = oracle.tilize_pack(x.numpy(), oracle.Bfp8_b, go)
        img = torch.full((ref.size,), 0xAB, dtype=torch.uint8, device="cuda")
        rt = shape[2] // 32
        for rank in range(world):
            count = len(range(rank, rt, world))
            if count:
                ops.tilize_pack_jobs([xc], ops.DF.Bfp8_b, geoms=[gq], outs=[img], bands=[(rank, world, count)])
            if rank == 0 and world > 1 and grid == (1, 1):
                # only rank 0's bands are written so far: band b is the contiguous slice [b*Ct*1088, (b+1)*Ct*1088)
                got = img.cpu().numpy().reshape(rt, -1)
                assert np.array_equal(got[0], ref.reshape(rt, -1)[0]) and (got[1] == 0xAB).all()
        assert np.array_equal(img.cpu().numpy(), ref), (shape, world)
        # and back: every rank untilizes its bands into one row-major tensor
        y = torch.full(shape, float("nan"), device="cuda")
        for rank in range(world):
            count = len(range(rank, rt, world))
            if count:
                ops.unpack_untilize_jobs([img], ops.DF.Bfp8_b, [y], geoms=[gq], bands=[(rank, world, count)])
        yref = oracle.unpack_untilize(ref, oracle.Bfp8_b, shape, geom=go)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), yref.view(np.uint32))


def test_job_table_rejects_bad_jobs(ops):
    from pybuda import _cabi
    x = torch.zeros(1, 1, 64, 64, device="cuda")
    with pytest.raises(_cabi.BudaError):
        ops.tilize_pack_jobs([x], ops.DF.Bfp8_b, bands=[(1, 1, 2)])             # tile rows 1, 2 of a 2-row tensor
    with pytest.raises(_cabi.BudaError):
        ops.tilize_pack_jobs([x], ops.DF.Bfp8_b, outs=[torch.empty(100, dtype=torch.uint8, device="cuda")])
    with pytest.raises(_cabi.BudaError):
        ops.tilize_pack_jobs([x], ops.DF.Bfp8_b, bands=[(0, 0, 1)])


def test_host_jobs_pipeline_mixed_shapes(ops, oracle):
    """buda_tilize_pack_host_jobs / buda_unpack_untilize_host_jobs: host tensors of different shapes through one
    pipeline run, images on the host or left on the device."""
    from pybuda import _cabi
    xs = [x.contiguous() for x in _mixed_set(8)]
    imgs = [np.zeros(oracle.tilize_pack(x.numpy(), oracle.Bfp8_b).size, np.uint8) for x in xs]
    jobs = (_cabi.TensorJob * len(xs))()
    for j, x, im in zip(jobs, xs, imgs):
        shape = _cabi.shape4(x.shape)
        j.tensor, j.image, j.image_bytes = x.data_ptr(), im.ctypes.data, im.size
        j.shape, j.strides_bytes = _cabi.u32x4(shape), _cabi.u64x4(_cabi.dense_strides(shape, 4))
        j.geom = _cabi.QueueGeom.for_shape(shape)
    _cabi.check(_cabi.lib.buda_tilize_pack_host_jobs(len(xs), jobs, 0, 6, 0, 0, None))
    for x, im in zip(xs, imgs):
        assert np.array_equal(im, oracle.tilize_pack(x.numpy(), oracle.Bfp8_b)), tuple(x.shape)
    # images on the device: the same call leaves them in device buffers
    dimgs = [torch.empty(im.size, dtype=torch.uint8, device="cuda") for im in imgs]
    for j, d in zip(jobs, dimgs):
        j.image = d.data_ptr()
    _cabi.check(_cabi.lib.buda_tilize_pack_host_jobs(len(xs), jobs, 0, 6, 0, 1, None))
    for d, im in zip(dimgs, imgs):
        assert np.array_equal(d.cpu().numpy(), im)
    backs = [torch.empty_like(x) for x in xs]
    for j, b in zip(jobs, backs):
        j.tensor = b.data_ptr()
    _cabi.check(_cabi.lib.buda_unpack_untilize_host_jobs(len(xs), jobs, 6, 0, 0, 1, None))
    for x, b, im in zip(xs, backs, imgs):
        ref = oracle.unpack_untilize(im, oracle.Bfp8_b, tuple(x.shape))
        assert np.array_equal(b.numpy().view(np.uint32), ref.view(np.uint32))
