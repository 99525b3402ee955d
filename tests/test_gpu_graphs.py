"""GPU test: the conversion, quantise and matmul launches recorded into a CUDA graph and replayed.  A launch-bound loop
(many small conversions per step) is where a graph pays; what has to hold is that a replay computes on the buffers'
current contents and that the device work counters a captured launch was given stay its own."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_captured_launches_replay_on_new_data(oracle):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    from pybuda import cuda_ops as ops

    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(17)
    shape = (1, 1, 256, 512)
    xs = [torch.randn(shape, generator=g).to(dev) for _ in range(3)]
    mixed = [torch.randn(1, 1, 64, 96, generator=g).to(dev), torch.randn(2, 1, 128, 32, generator=g).to(dev)]
    imgs = ops.tilize_pack_batch(xs, ops.DF.Bfp8_b)                       # eager first: one-time set-up happens outside the capture
    ys = ops.unpack_untilize_batch(imgs, ops.DF.Bfp8_b, shape)
    tj = ops.TensorJobs(mixed, ops.DF.Bfp4_b)
    tj.pack()
    xq = torch.randn(64, 1024, generator=g).to(dev) * 4
    sc = torch.tensor([0.05], device=dev)
    q_out = ops.quantize(xq, sc, 3)
    M, K, N = 512, 128, 256
    a = torch.randn(M, K, generator=g).bfloat16().to(dev)
    w = (torch.randn(1, 1, K, N, generator=g) * 0.05).to(dev)
    wimg = ops.tilize_pack(w, ops.DF.Bfp8_b)
    c = ops.bfp8b_matmul(a, wimg, N)
    torch.cuda.synchronize()

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.tilize_pack_batch(xs, ops.DF.Bfp8_b, outs=imgs)
        ops.unpack_untilize_batch(imgs, ops.DF.Bfp8_b, shape, outs=ys)
        tj.pack()
        q_cap = ops.quantize(xq, sc, 3)
        ops.tilize_pack(w, ops.DF.Bfp8_b, out=wimg)
        ops.bfp8b_matmul(a, wimg, N, out=c)

    for it in range(3):
        for x in xs + mixed:
            x.copy_(torch.randn(x.shape, generator=g) * (it + 1))
        xq.copy_(torch.randn(64, 1024, generator=g) * 4)
        w.copy_(torch.randn(1, 1, K, N, generator=g) * 0.05)
        graph.replay()
        torch.cuda.synchronize()
        for x, im, y in zip(xs, imgs, ys):
            want = oracle.tilize_pack(x.cpu().numpy(), oracle.Bfp8_b)
            assert np.array_equal(im.cpu().numpy(), want), it
            assert np.array_equal(y.cpu().numpy().view(np.uint32), oracle.unpack_untilize(want, oracle.Bfp8_b, shape).view(np.uint32)), it
        for x, im in zip(mixed, tj.images):
            assert np.array_equal(im.cpu().numpy(), oracle.tilize_pack(x.cpu().numpy(), oracle.Bfp4_b)), it
        assert np.array_equal(q_cap.cpu().numpy(), oracle.quantize(xq.cpu().numpy(), sc.cpu().numpy(), 3)), it
        assert torch.equal(c, ops.bfp8b_matmul(a, ops.tilize_pack(w, ops.DF.Bfp8_b), N)), it
    rc, st = ops._cabi.device_status()
    assert rc == 0 and st == 0
