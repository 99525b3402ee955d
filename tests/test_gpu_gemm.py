"""GPU tests of the Bfp8_b-weight matmul (tcgen05 kernel) against binary32 matmul of the
oracle-decoded operands.

Tolerance (stated by the target: rel-err 1e-3 against an fp32 matmul of the decoded operands):
  * norm-wise   ||C - bf16(ref)||_F / ||ref||_F <= 1e-3, the reference rounded to the kernel's
    bfloat16 output type first (rounding to bfloat16 alone costs ~1.5e-3 norm-wise);
  * element-wise |C - ref| <= 2^-8 |ref| + 1e-3 max|ref|  (half an ulp of bfloat16 plus a floor).
One-hot activations make the product a copy of decoded weight rows, which must then be exact."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device; there is no CPU fallback to test")
    from pybuda import cuda_ops

    torch.backends.cuda.matmul.allow_tf32 = False
    return cuda_ops


def _weights(oracle, ops, K, N, seed, scale=0.02):
    w = torch.randn(1, 1, K, N, generator=torch.Generator().manual_seed(seed)) * scale
    img = ops.tilize_pack(w.cuda(), ops.DF.Bfp8_b)
    ref_img = oracle.tilize_pack(w.numpy(), oracle.Bfp8_b)
    assert np.array_equal(img.cpu().numpy(), ref_img)
    wd = torch.from_numpy(oracle.unpack_untilize(ref_img, oracle.Bfp8_b, (1, 1, K, N)))[0, 0]
    return img, wd


def _check(c, ref):
    c = c.float()
    refb = ref.bfloat16().float()
    rel = ((c - refb).norm() / ref.norm()).item()
    assert rel <= 1e-3, f"norm-wise relative error {rel}"
    bound = ref.abs() * 2.0 ** -8 + 1e-3 * ref.abs().max()
    bad = (c - ref).abs() > bound
    assert not bad.any(), f"{int(bad.sum())} elements outside the element-wise bound; first {bad.nonzero()[:5].tolist()}"


def test_one_hot_rows_copy_decoded_weights_exactly(ops, oracle):
    K, N, M = 128, 512, 256
    img, wd = _weights(oracle, ops, K, N, seed=7, scale=1.0)
    a = torch.zeros(M, K)
    ks = torch.arange(M) % K
    a[torch.arange(M), ks] = 1.0
    c = ops.bfp8b_matmul(a.bfloat16().cuda(), img, N).cpu().float()
    want = wd[ks]            # decoded values have 7 significant bits: exact in bfloat16
    if not torch.equal(c, want):
        bad = (c != want).nonzero()
        pytest.fail(f"{bad.shape[0]} of {c.numel()} elements differ; first {bad[:8].tolist()}; "
                    f"got {c[tuple(bad[0])].item()} want {want[tuple(bad[0])].item()}")


@pytest.fixture(params=["single", "pair", "pair_register_epilogue"])
def kernel(request, ops):
    """Both tensor-core kernels (one CTA per tile; a CTA pair per tile, with either epilogue) run every shape."""
    prev = ops.select_gemm_kernel(request.param)
    yield request.param
    ops.select_gemm_kernel(prev)


@pytest.mark.parametrize("M,K,N", [(256, 64, 256), (256, 256, 256), (512, 512, 768), (128, 192, 256), (300, 128, 512),
                                   (1024, 1024, 1024), (1500, 320, 1280)])
def test_matmul_small_shapes(ops, oracle, kernel, M, K, N):
    img, wd = _weights(oracle, ops, K, N, seed=M + K + N)
    a = torch.randn(M, K, generator=torch.Generator().manual_seed(1)).bfloat16()
    c = ops.bfp8b_matmul(a.cuda(), img, N).cpu()
    _check(c, a.float() @ wd)
    if M * K * N <= 256 * 256 * 256:
        # and against the oracle's own k-ordered binary32 accumulation
        ref2 = torch.from_numpy(oracle.bfp8b_matmul(a.view(torch.int16).numpy().view(np.uint16), img.cpu().numpy(), K, N))
        _check(c, ref2)


def test_pair_and_single_kernels_agree_bit_for_bit(ops, oracle):
    M, K, N = 2048, 1024, 1536
    img, _ = _weights(oracle, ops, K, N, seed=11)
    a = torch.randn(M, K, generator=torch.Generator().manual_seed(12)).bfloat16().cuda()
    prev = ops.select_gemm_kernel("single")
    try:
        c1 = ops.bfp8b_matmul(a, img, N)
        ops.select_gemm_kernel("pair")
        c2 = ops.bfp8b_matmul(a, img, N)
        ops.select_gemm_kernel("pair_register_epilogue")
        c3 = ops.bfp8b_matmul(a, img, N)
        # rows past M are clipped by the bulk tensor store, and a wider output keeps its other columns
        wide = torch.full((M - 37 + 5, N + 64), 7.0, dtype=torch.bfloat16, device="cuda")
        ops.select_gemm_kernel("pair")
        ops.bfp8b_matmul(a[: M - 37], img, N, out=wide[: M - 37, :N])
    finally:
        ops.select_gemm_kernel(prev)
    assert torch.equal(c1, c2)    # same k order, same binary32 accumulation
    assert torch.equal(c2, c3)
    assert torch.equal(wide[: M - 37, :N], c2[: M - 37])
    assert torch.all(wide[M - 37:] == 7.0) and torch.all(wide[:, N:] == 7.0)
    rc, st = ops._cabi.device_status()
    assert rc == 0 and st == 0


def test_scatter_writes_every_destination(ops, oracle, kernel):
    M, K, N = 768, 256, 512
    img, wd = _weights(oracle, ops, K, N, seed=21)
    a = torch.randn(M, K, generator=torch.Generator().manual_seed(22)).bfloat16().cuda()
    # three full-width outputs [M, 2N]; this "rank" owns columns N..2N of each
    outs = [torch.zeros(M, 2 * N, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    ops.bfp8b_matmul_scatter(a, img, N, [o.data_ptr() + N * 2 for o in outs], 2 * N)
    torch.cuda.synchronize()
    _check(outs[0][:, N:].cpu(), a.cpu().float() @ wd)
    for o in outs:
        assert torch.all(o[:, :N] == 0)
        assert torch.equal(o, outs[0])
    with pytest.raises(ops._cabi.BudaError):
        ops.bfp8b_matmul_scatter(a, img, N, [outs[0].data_ptr()] * 9, 2 * N)


def _ipc_child(handle, m, k, n, seed, q):
    """Another process of the box: maps the parent's matrix and lets the matmul epilogue store into it."""
    import os, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [root, os.path.join(root, "tt-buda_b200")]
    try:
        from pybuda import cuda_ops
        g = torch.Generator().manual_seed(seed)
        a = torch.randn(m, k, generator=g).bfloat16().cuda()
        w = torch.randn(1, 1, k, n, generator=g) * 0.02
        img = cuda_ops.tilize_pack(w.cuda(), cuda_ops.DF.Bfp8_b)
        mine = cuda_ops.SharedDeviceMatrix(m, n)
        peer = mine.open_peer(handle)
        cuda_ops.bfp8b_matmul_scatter(a, img, n, [mine.ptr, peer], n)
        torch.cuda.synchronize()
        local = mine.tensor.cpu().view(torch.int16).numpy().tobytes()   # plain bytes: nothing shared with this process
        mine.close()
        q.put(("ok", local))
    except Exception as e:  # noqa: BLE001
        q.put(("error", repr(e)))


def test_scatter_into_another_process_memory(ops, oracle):
    """The inter-process mapping the column-parallel matmul relies on, exercised on one GPU: a child process
    computes the product and its epilogue stores it into THIS process's matrix as well as its own."""
    import torch.multiprocessing as mp
    m, k, n, seed = 512, 128, 256, 31
    shared = ops.SharedDeviceMatrix(m, n)
    shared.tensor.zero_()
    torch.cuda.synchronize()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    child = ctx.Process(target=_ipc_child, args=(shared.handle(), m, k, n, seed, q))
    child.start()
    status, payload = q.get(timeout=300)
    child.join(timeout=60)
    assert status == "ok", payload
    torch.cuda.synchronize()
    got = shared.tensor.cpu()
    shared.close()
    assert got.view(torch.int16).numpy().tobytes() == payload
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = torch.randn(1, 1, k, n, generator=g) * 0.02
    wd = torch.from_numpy(oracle.unpack_untilize(oracle.tilize_pack(w.numpy(), oracle.Bfp8_b), oracle.Bfp8_b, (1, 1, k, n)))[0, 0]
    _check(got, a.float() @ wd)


def test_strided_operands_and_reuse(ops, oracle, kernel):
    M, K, N = 256, 128, 256
    img, wd = _weights(oracle, ops, K, N, seed=3)
    big = torch.randn(M, K + 64, generator=torch.Generator().manual_seed(2)).bfloat16().cuda()
    a = big[:, :K]                                    # row stride K + 64
    out = torch.zeros(M, N + 128, dtype=torch.bfloat16, device="cuda")
    for _ in range(3):                                # the persistent kernel is relaunched safely
        ops.bfp8b_matmul(a, img, N, out=out[:, :N])
    _check(out[:, :N].cpu(), a.cpu().float() @ wd)
    assert torch.all(out[:, N:] == 0)
    rc, st = ops._cabi.device_status()
    assert rc == 0 and st == 0


def test_bad_shapes_are_refused(ops):
    a = torch.zeros(128, 96, dtype=torch.bfloat16, device="cuda")
    img = torch.zeros(3 * 8 * 1088, dtype=torch.uint8, device="cuda")
    with pytest.raises(ops._cabi.BudaError) as e:
        ops.bfp8b_matmul(a, img, 256)
    assert "K % 64" in str(e.value)


def test_config4_full_size(ops, oracle, kernel):
    # activations bf16 [8192,4096] ~ N(0,1); weights fp32 [4096,16384] ~ N(0,0.02) packed to Bfp8_b
    M, K, N = 8192, 4096, 16384
    a = torch.randn(M, K, generator=torch.Generator().manual_seed(6)).bfloat16().cuda()
    w = torch.randn(1, 1, K, N, generator=torch.Generator().manual_seed(7)) * 0.02
    img = ops.tilize_pack(w.cuda(), ops.DF.Bfp8_b)
    assert img.numel() == 71303168
    c = ops.bfp8b_matmul(a, img, N)
    # decoded weights: the kernel's own unpack was proven bit-exact against the oracle above
    wd = ops.unpack_untilize(img, ops.DF.Bfp8_b, (1, 1, K, N))[0, 0]
    ref = a.float() @ wd                               # binary32 matmul (TF32 off)
    cf = c.float()
    rel = ((cf - ref.bfloat16().float()).norm() / ref.norm()).item()
    assert rel <= 1e-3, rel
    bound = ref.abs() * 2.0 ** -8 + 1e-3 * ref.abs().max()
    assert not ((cf - ref).abs() > bound).any()
    # a sample of rows against the CPU oracle's decode + matmul, end to end
    rows = torch.tensor([0, 1, 127, 128, 255, 256, 4095, 8191])
    wd_cpu = torch.from_numpy(oracle.unpack_untilize(oracle.tilize_pack(w.numpy(), oracle.Bfp8_b), oracle.Bfp8_b, (1, 1, K, N)))[0, 0]
    ref_rows = a[rows.cuda()].cpu().float() @ wd_cpu
    _check(c[rows.cuda()].cpu(), ref_rows)


# ------------------------------------------------------------------------------------------------
# int8 matmul with the requantisation / dequantisation epilogue (bit-exact: integer accumulation, then the
# golden evaluation's float operations one by one)
# ------------------------------------------------------------------------------------------------
def _i8_operands(ops, oracle, M, K, N, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-128, 128, (K, N), generator=g, dtype=torch.int8)
    img = ops.tilize_pack(w.reshape(1, 1, K, N).cuda(), ops.DF.Int8)
    ref_img = oracle.tilize_pack(w.reshape(1, 1, K, N).numpy(), oracle.Int8)
    assert np.array_equal(img.cpu().numpy(), ref_img)
    return a, w, img


@pytest.mark.parametrize("M,K,N", [(512, 128, 256), (128, 256, 256), (700, 384, 512), (1024, 1024, 1024)])
def test_i8_matmul_accumulators_exact(ops, oracle, M, K, N):
    a, w, img = _i8_operands(ops, oracle, M, K, N, seed=M + K + N)
    c = ops.i8_matmul(a.cuda(), img, N).cpu()
    want = a.int() @ w.int()
    assert torch.equal(c, want)
    if M * K * N <= 512 * 384 * 512:
        assert np.array_equal(c.numpy(), oracle.i8_matmul(a.numpy(), img.cpu().numpy(), K, N))
    rc, st = ops._cabi.device_status()
    assert rc == 0 and st == 0


@pytest.mark.parametrize("per_column", [False, True])
def test_i8_matmul_requant_and_dequant_epilogues(ops, oracle, per_column, kernel):
    if kernel == "single":
        pytest.skip("the int8 matmul has the pair kernel only")
    M, K, N = 640, 256, 512
    a, w, img = _i8_operands(ops, oracle, M, K, N, seed=77)
    g = torch.Generator().manual_seed(78)
    scale = (torch.rand(N if per_column else 1, generator=g) * (1e-3 - 1e-5) + 1e-5)
    acc = a.int() @ w.int()
    # the golden chain: matmul (int32) then requantization / dequantization of its result
    zp = 3.0
    want_q = torch.clamp(torch.round(acc.float() * scale + zp), -128, 127).to(torch.int8)
    got_q = ops.i8_matmul(a.cuda(), img, N, scale=scale, zero_point=zp, out="int8").cpu()
    assert torch.equal(got_q, want_q)
    assert got_q.min() == -128 and got_q.max() == 127 and (got_q.abs() < 100).any()     # saturation and interior both exercised
    want_f = (acc.float() - zp) * scale
    got_f = ops.i8_matmul(a.cuda(), img, N, scale=scale, zero_point=zp, out="float32").cpu()
    assert torch.equal(got_f, want_f)
    assert np.array_equal(got_q.numpy(), oracle.i8_matmul(a.numpy(), img.cpu().numpy(), K, N, scale.numpy(), zp, 1))
    assert np.array_equal(got_f.numpy(), oracle.i8_matmul(a.numpy(), img.cpu().numpy(), K, N, scale.numpy(), zp, 2))


def test_i8_matmul_full_size_against_float_matmul(ops):
    # 8192 x 4096 x 16384: partial sums stay far below 2^24, so a binary32 matmul of the same integers is exact
    M, K, N = 8192, 4096, 16384
    g = torch.Generator().manual_seed(5)
    a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8).cuda()
    w = torch.randint(-128, 128, (K, N), generator=g, dtype=torch.int8).cuda()
    img = ops.tilize_pack(w.reshape(1, 1, K, N), ops.DF.Int8)
    c = ops.i8_matmul(a, img, N)
    rows = torch.arange(0, M, 61, device="cuda")
    want = (a[rows].float() @ w.float()).int()
    assert torch.equal(c[rows], want)
    scale = torch.rand(N, generator=g).cuda() * 2e-5
    q = ops.i8_matmul(a, img, N, scale=scale, zero_point=-2.0, out="int8")
    want_q = torch.clamp(torch.round(want.float() * scale - 2.0), -128, 127).to(torch.int8)
    assert torch.equal(q[rows], want_q)


def test_i8_matmul_refuses_bad_arguments(ops):
    a = torch.zeros(128, 96, dtype=torch.int8, device="cuda")
    img = torch.zeros(3 * 8 * 1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(ops._cabi.BudaError, match="K % 128"):
        ops.i8_matmul(a, img, 256)
    a = torch.zeros(128, 128, dtype=torch.int8, device="cuda")
    img = torch.zeros(4 * 8 * 1024, dtype=torch.uint8, device="cuda")
    with pytest.raises(ops._cabi.BudaError, match="scale"):
        ops.i8_matmul(a, img, 256, scale=torch.ones(7), out="int8")


def test_weight_blocks_at_the_ends_of_the_exponent_range(ops, oracle, kernel):
    """Blocks whose shared exponent is below 7 hold values under 2^-126 and enter the product as zero; every other finite
    block -- down to exponent 7 and up to 253 -- enters exactly.  One-hot activations make the product a copy of weight rows."""
    K, N, M = 64, 256, 256
    w = torch.zeros(1, 1, K, N)
    g = torch.Generator().manual_seed(5)
    base = torch.randint(1, 128, (K, N), generator=g).float() * torch.where(torch.rand(K, N, generator=g) < 0.5, -1.0, 1.0)
    # rows of K use different magnitudes: 2^-135 (exponent field 3 after the block maximum), 2^-125, 1, 2^100, 2^119
    scales = {0: 2.0 ** -140, 1: 2.0 ** -128, 2: 2.0 ** -126, 3: 1.0, 4: 2.0 ** 100, 5: 2.0 ** 119}
    for k in range(K):
        w[0, 0, k] = base[k] * scales[k % 6]
    img = ops.tilize_pack(w.cuda(), ops.DF.Bfp8_b)
    ref_img = oracle.tilize_pack(w.numpy(), oracle.Bfp8_b)
    assert np.array_equal(img.cpu().numpy(), ref_img)
    wd = torch.from_numpy(oracle.unpack_untilize(ref_img, oracle.Bfp8_b, (1, 1, K, N)))[0, 0]
    exps = torch.from_numpy(ref_img.reshape(-1, 1088)[:, :64].astype(np.int32))          # [tile, block]
    a = torch.zeros(M, K)
    ks = torch.arange(M) % K
    a[torch.arange(M), ks] = 1.0
    c = ops.bfp8b_matmul(a.bfloat16().cuda(), img, N).cpu().float()
    # expected: decoded weights, with the blocks of exponent < 7 taken as zero
    want = wd.clone()
    for kt in range(K // 32):
        for nt in range(N // 32):
            e = exps[kt * (N // 32) + nt]
            for blk in range(64):
                if int(e[blk]) < 7:
                    face, fr = divmod(blk, 16)
                    r0, c0 = kt * 32 + (face >> 1) * 16 + fr, nt * 32 + (face & 1) * 16
                    want[r0, c0:c0 + 16] = 0.0
    assert (exps < 7).any() and (exps >= 7).any()
    assert torch.equal(c, want[ks].bfloat16().float())
    rc, st = ops._cabi.device_status()
    assert rc == 0 and st == 0
