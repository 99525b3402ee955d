"""GPU tests of the source views: a tensor pushed through one of the reference's runtime tensor transforms is
converted by ONE kernel whose index arithmetic does the transform.  Checked byte for byte against the CPU oracle
(transform restated in numpy and pinned by vectors the reference's own functions produced, then the oracle's tilize),
and against those reference vectors directly."""
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


def _golden():
    return np.load(os.path.join(HERE, "golden", "transform_golden.npz"))


def test_embedding_index_view_matches_the_reference_vectors(ops, oracle):
    from pybuda import _cabi
    g = _golden()
    k = 0
    while f"emb{k}_in" in g.files:
        n, w, q_rt, q_ct = (int(v) for v in g[f"emb{k}_meta"])
        idx = torch.from_numpy(g[f"emb{k}_in"].reshape(w, n)).cuda()
        view = _cabi.SourceView(mode=2, emb_count=n, emb_group=((n + 31) // 32 * 32) // q_rt)
        qshape = (w, 1, q_rt * 32, q_ct * 32)
        img = ops.tilize_pack_view(idx, ops.DF.RawUInt32, qshape, view, strides_bytes=[n * 4, 0, 0, 4])
        want = oracle.tilize_pack(np.ascontiguousarray(g[f"emb{k}_out"]).view(np.uint32), oracle.RawUInt32)
        assert np.array_equal(img.cpu().numpy(), want), k
        k += 1
    assert k == 5


def test_embedding_index_view_beyond_one_tile_column(ops, oracle):
    """More than 1024 indices per queue tile row (several tile columns), several entries, 16-bit indices."""
    from pybuda import _cabi
    g = torch.Generator().manual_seed(2)
    for n, w, q_rt, dt, df in ((5000, 2, 1, torch.int32, "RawUInt32"), (8100, 1, 2, torch.int32, "Int32"), (3000, 3, 1, torch.int16, "RawUInt16")):
        idx = torch.randint(0, 30000, (w, n), generator=g, dtype=dt)
        ref = oracle.embedding_index(idx.numpy(), n, q_rt)
        view = _cabi.SourceView(mode=2, emb_count=n, emb_group=((n + 31) // 32 * 32) // q_rt)
        img = ops.tilize_pack_view(idx.cuda(), getattr(ops.DF, df), ref.shape, view, strides_bytes=[n * idx.element_size(), 0, 0, idx.element_size()])
        npdt = np.uint16 if dt == torch.int16 else (np.uint32 if df == "RawUInt32" else np.int32)
        want = oracle.tilize_pack(ref.view(npdt), getattr(oracle, df), src_df=getattr(oracle, df) if dt == torch.int16 else None)
        assert np.array_equal(img.cpu().numpy(), want), (n, w, q_rt)


def test_prestride_view_matches_the_reference_vectors_and_packs(ops, oracle):
    from pybuda import _cabi
    g = _golden()
    k = 0
    while f"pre{k}_in" in g.files:
        act, s, want_t = g[f"pre{k}_in"], int(g[f"pre{k}_stride"][0]), g[f"pre{k}_out"]
        w, z, h, wd = act.shape
        xy = [(x, y) for y in range(s) for x in range(s)]
        view = _cabi.SourceView(mode=3, ps_stride=s, ps_z=z, ps_h=h, ps_w=wd, ps_n_offsets=len(xy))
        for i, (x, y) in enumerate(xy):
            view.ps_xy[2 * i], view.ps_xy[2 * i + 1] = x, y
        padded = oracle.pad_to_tiles(want_t)
        for df_name, src in (("Float32", torch.from_numpy(act)), ("Bfp8_b", torch.from_numpy(act)), ("Bfp8_b", torch.from_numpy(act).bfloat16())):
            img = ops.tilize_pack_view(src.cuda(), getattr(ops.DF, df_name), padded.shape, view)
            if src.dtype == torch.bfloat16:
                pb = torch.from_numpy(padded).bfloat16().view(torch.int16).numpy().view(np.uint16)
                want = oracle.tilize_pack(pb, getattr(oracle, df_name), src_df=oracle.Float16_b)
            else:
                want = oracle.tilize_pack(padded, getattr(oracle, df_name))
            assert np.array_equal(img.cpu().numpy(), want), (k, df_name, str(src.dtype))
        k += 1
    assert k == 4


def test_padded_view_pads_and_broadcasts_like_the_reference(ops, oracle):
    from pybuda import _cabi
    g = _golden()
    k = 0
    while f"pad{k}_in" in g.files:
        x, bc, want_t = g[f"pad{k}_in"], list(g[f"pad{k}_bcast"]), g[f"pad{k}_out"]
        x4 = x.reshape((1,) * (4 - x.ndim) + x.shape)
        want4 = want_t.reshape((1,) * (4 - want_t.ndim) + want_t.shape)
        view = _cabi.SourceView(mode=1, valid_r=x4.shape[2], valid_c=x4.shape[3], bcast_r=int(2 in bc), bcast_c=int(3 in bc))
        for df_name in ("Float32", "Bfp4_b"):
            img = ops.tilize_pack_view(torch.from_numpy(x4).cuda(), getattr(ops.DF, df_name), want4.shape, view)
            assert np.array_equal(img.cpu().numpy(), oracle.tilize_pack(want4, getattr(oracle, df_name))), (k, df_name)
        k += 1
    assert k == 5
    # a reinterpreted, non-contiguous source under a layout policy, into a grid geometry with tile headers
    gq, go = ops.QueueGeom.for_shape((2, 2, 64, 96), (2, 1), (1, 3), 1), oracle.Geom.for_shape((2, 2, 64, 96), (2, 1), (1, 3), 1)
    base = torch.randn(2, 2, 50, 100, generator=torch.Generator().manual_seed(3))
    xs = base[:, :, :, :70]                                            # row stride 100 elements, 70 valid columns
    view = _cabi.SourceView(mode=1, valid_r=50, valid_c=70)
    try:
        ops.set_bfp_policy(_cabi.BfpPolicy(rounding=1, face_order=(0, 2, 1, 3)))
        oracle.set_bfp_policy(oracle.BfpPolicy(rounding=1, face_order=(0, 2, 1, 3)))
        img = ops.tilize_pack_view(base.cuda()[:, :, :, :70], ops.DF.Bfp8_b, (2, 2, 64, 96), view, geom=gq, with_header=True)
        want = oracle.tilize_pack(oracle.pad_to_tiles(xs.contiguous().numpy()), oracle.Bfp8_b, go, with_header=True)
        assert np.array_equal(img.cpu().numpy(), want)
    finally:
        ops.set_bfp_policy(None)
        oracle.set_bfp_policy(None)


def test_views_reject_what_does_not_fit(ops):
    from pybuda import _cabi
    x = torch.zeros(1, 1, 40, 40, device="cuda")
    with pytest.raises(_cabi.BudaError):
        ops.tilize_pack_view(x, ops.DF.Float32, (1, 1, 32, 64), _cabi.SourceView(mode=1, valid_r=40, valid_c=40))
    with pytest.raises(_cabi.BudaError):
        ops.tilize_pack_view(x, ops.DF.Float32, (1, 1, 64, 64), _cabi.SourceView(mode=1, valid_r=40, valid_c=40, bcast_r=1))
    with pytest.raises(_cabi.BudaError):
        ops.tilize_pack_view(x, ops.DF.Float32, (1, 1, 64, 64), _cabi.SourceView(mode=7))
    idx = torch.zeros(100, dtype=torch.int32, device="cuda")
    with pytest.raises(_cabi.BudaError):
        ops.tilize_pack_view(idx, ops.DF.Bfp8_b, (1, 1, 32, 32), _cabi.SourceView(mode=2, emb_count=100, emb_group=128),
                             strides_bytes=[400, 0, 0, 4])     # indices do not go through a block-float pack
    with pytest.raises(_cabi.BudaError):
        ops.tilize_pack_view(x, ops.DF.Float32, (1, 1, 64, 64), _cabi.SourceView(mode=3, ps_stride=2, ps_z=1, ps_h=40, ps_w=40, ps_n_offsets=0))
