"""The tensor side of the device-image archive (reference: pybuda/pybuda/tti/archive.py, tti/utils.py):
JSON descriptors, .pkl / .bin / .tbin files, lazy loading, checksum sidecar.  Writing row-major .bin
files and the JSON needs no GPU; producing and reloading .tbin files does (they are packed on the GPU
and land in pinned host memory)."""
import json
import os

import numpy as np
import pytest
import torch


@pytest.fixture(scope="module")
def mods():
    import pybuda.tti as tti
    from pybuda._C import DataFormat, backend_api
    from pybuda.config import TTIDumpFormat
    return tti, TTIDumpFormat, DataFormat, backend_api


def test_dump_format_enum(mods):
    _, F, _, _ = mods
    assert [f.extension() for f in (F.DEFAULT, F.BACKEND, F.BACKEND_TILIZED)] == ["pkl", "bin", "tbin"]
    assert F.from_json("backend_tilized") is F.BACKEND_TILIZED and F.to_json(F.BACKEND) == "BACKEND"


def test_checksum_helpers(mods, tmp_path):
    tti = mods[0]
    p = tmp_path / "blob"
    p.write_bytes(b"abc" * 100000)
    import hashlib
    c = tti.compute_file_checksum(str(p))
    assert c == hashlib.sha256(b"abc" * 100000).hexdigest()
    assert tti.read_checksum_from_file(str(p) + ".checksum") is None
    tti.write_checksum_to_file(c, str(p) + ".checksum")
    assert tti.read_checksum_from_file(str(p) + ".checksum") == c


def test_bin_archive_layout_and_json(mods, tmp_path):
    tti, F, DF, _ = mods
    w = torch.randn(64, 96, generator=torch.Generator().manual_seed(0))
    tensors = {"layer/w": w, "nested": {"idx": torch.arange(12, dtype=torch.int32).reshape(3, 4), torch.float32: 7},
               "cpueval_outputs": [torch.ones(3)]}
    path = tti.save_tensor_archive(str(tmp_path), tensors, F.BACKEND)
    body = json.load(open(path))
    assert body["tti_dump_format"] == "BACKEND"
    e = body["tensors"]["layer/w"]
    assert e == {"bin": "tensors/torch.Tensor.layer_w.bin", "itemsize": 4, "shape": [1, 1, 64, 96],
                 "strides": [96 * 4, 96 * 4, 96 * 4, 4], "dim": 3, "format": "Float32"}   # 2-D: dim 3, leading stride repeated
    raw = open(tmp_path / e["bin"], "rb").read()
    assert raw == w.numpy().tobytes()                       # the .bin is the row-major bytes, nothing else
    assert body["tensors"]["nested"]["idx"]["format"] == "Int32" and body["tensors"]["nested"]["torch.float32"] == 7
    assert body["tensors"]["cpueval_outputs"].endswith(".pkl")   # golden outputs always stay pickled
    # checksum sidecar guards the descriptor
    assert tti.read_checksum_from_file(path + ".checksum") == tti.compute_file_checksum(path)
    with open(path, "a") as f:
        f.write(" ")
    with pytest.raises(RuntimeError, match="checksum"):
        tti.load_tensor_archive(str(tmp_path))
    back = tti.load_tensor_archive(str(tmp_path), verify_checksum=False)
    assert callable(back["layer/w"]) and callable(back["nested"]["idx"])      # lazy: nothing read yet
    assert back["nested"][torch.float32] == 7                                  # dtype keys restored
    assert torch.equal(back["cpueval_outputs"][0], torch.ones(3))


def test_pickle_archive_round_trip(mods, tmp_path):
    tti, F, _, _ = mods
    w = torch.randn(5, 7)
    tti.save_tensor_archive(str(tmp_path), {"w": w}, F.DEFAULT)
    back = tti.load_tensor_archive(str(tmp_path))
    assert torch.equal(back["w"], w)


def test_tbin_needs_a_queue_descriptor(mods, tmp_path):
    tti, F, _, _ = mods
    with pytest.raises(KeyError, match="queue descriptor"):
        tti.save_tensor_archive(str(tmp_path), {"w": torch.zeros(32, 32)}, F.BACKEND_TILIZED, {})


@pytest.mark.gpu
def test_tbin_archive_packs_once_and_pushes_without_conversion(mods, oracle, tmp_path):
    tti, F, DF, B = mods
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device; there is no CPU fallback to test")
    from pybuda import tensor as T
    g = torch.Generator().manual_seed(5)
    tensors = {"ffn.w1": torch.randn(1024, 4096, generator=g) * 0.02, "attn.q": torch.randn(1024, 1024, generator=g) * 0.02,
               "bias": torch.randn(1, 1024, generator=g)}
    qd = {"ffn.w1": B.DramIODesc.for_tensor("ffn.w1", [1, 1, 1024, 4096], DF.Bfp8_b, grid=(2, 4), ublock=(2, 2)),
          "attn.q": B.DramIODesc.for_tensor("attn.q", [1, 1, 1024, 1024], DF.Bfp4_b),
          "bias": B.DramIODesc.for_tensor("bias", [1, 1, 32, 1024], DF.Float16_b)}
    padded = dict(tensors)
    # a plain-format queue takes the tensor in its own element type (the reference converts before tilizing:
    # pybuda/pybuda/device_connector.py:177-201), and tile-aligned
    padded["bias"] = T.pad_pytorch_tensor_to_buda(tensors["bias"], []).bfloat16()
    tti.save_tensor_archive(str(tmp_path), padded, F.BACKEND_TILIZED, qd)
    body = json.load(open(tmp_path / "device_image.json"))["tensors"]
    assert body["ffn.w1"]["format"] == "Bfp8_b" and body["ffn.w1"]["num_buffers"] == 8
    assert body["ffn.w1"]["buf_size_bytes"] == (1024 * 4096 // 1024 // 8) * 1088
    # file bytes = the oracle's queue image
    go = oracle.Geom.for_shape([1, 1, 1024, 4096], (2, 4), (2, 2), 0)
    want = oracle.tilize_pack(tensors["ffn.w1"].reshape(1, 1, 1024, 4096).numpy(), oracle.Bfp8_b, go)
    assert open(tmp_path / body["ffn.w1"]["bin"], "rb").read() == want.tobytes()
    # reload lazily, push the pre-tilized bytes, read back through the normal output path
    back = tti.load_tensor_archive(str(tmp_path))
    for name, fmt in (("ffn.w1", oracle.Bfp8_b), ("attn.q", oracle.Bfp4_b)):
        td = back[name]()
        assert isinstance(td, B.TilizedTensorDesc)
        assert B.push_input(qd[name], td, 1, -1) == B.BackendStatusCode.Success, B.last_error()
        out = B.PytorchTensorDesc()
        out.format = DF.Float32
        assert B.get_output(qd[name], out, True, 1, -1) == B.BackendStatusCode.Success, B.last_error()
        y = T.tensor_desc_to_pytorch_tensor(out).clone()
        B.pop_output(qd[name], True, 1)
        B.free_tensor(out)
        B.free_tensor(td)
        x = tensors[name]
        shape = (1, 1) + tuple(x.shape)
        geom = go if name == "ffn.w1" else None
        img = oracle.tilize_pack(x.reshape(shape).numpy(), fmt, geom) if geom else oracle.tilize_pack(x.reshape(shape).numpy(), fmt)
        ref = oracle.unpack_untilize(img, fmt, shape, geom=geom)
        assert np.array_equal(y.numpy().reshape(shape).view(np.uint32), ref.view(np.uint32))
    B.release_all_queues()
