"""Device-resident entry points: the data-format kernels applied to CUDA torch tensors.

torch is used for device memory and streams only; every byte of arithmetic happens in
libbuda_cuda.so (hand-written sm_100a kernels) reached through its C ABI.  Functions raise if
the tensor is not on a CUDA device: there is no CPU path here.
"""
import ctypes
import enum

import torch

from . import _cabi
from ._cabi import QueueGeom, check


class DF(enum.IntEnum):
    """Integer values of the reference's DataFormat (pybuda/csrc/lower_to_buda/common.hpp:92-111)."""

    Float32 = 0
    Float16 = 1
    Bfp8 = 2
    Bfp4 = 3
    Bfp2 = 11
    Float16_b = 5
    Bfp8_b = 6
    Bfp4_b = 7
    Bfp2_b = 15
    Lf8 = 10
    UInt16 = 12
    Int8 = 14
    Int32 = 8
    RawUInt8 = 0xF0
    RawUInt16 = 0xF1
    RawUInt32 = 0xF2
    Invalid = 0xFF


_TORCH_TO_DF = {
    torch.float32: DF.Float32, torch.bfloat16: DF.Float16_b, torch.float16: DF.Float16,
    torch.int8: DF.Int8, torch.int32: DF.Int32, torch.uint8: DF.RawUInt8, torch.int16: DF.RawUInt16,
}
_DF_TO_TORCH = {
    DF.Float32: torch.float32, DF.Float16_b: torch.bfloat16, DF.Float16: torch.float16, DF.Int8: torch.int8,
    DF.Int32: torch.int32, DF.RawUInt8: torch.uint8, DF.RawUInt16: torch.int16, DF.RawUInt32: torch.int32,
    DF.UInt16: torch.int16, DF.Lf8: torch.uint8,
}


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("pybuda.cuda_ops works on CUDA tensors only (no CPU fallback)")


def _desc(t):
    """[w,z,r,c] shape and byte strides of a tensor of up to 4 dims (leading 1s dropped above 4),
    as pytorch_tensor_to_tensor_desc builds them (pybuda/pybuda/tensor.py:695-713)."""
    shape = list(t.shape)
    strides = list(t.stride())
    while len(shape) > 4:
        if shape[0] != 1:
            raise RuntimeError("Dropping a dimension that's not 1 to reduce shape to 4D: " + str(tuple(t.shape)))
        shape, strides = shape[1:], strides[1:]
    while len(shape) < 4:
        shape = [1] + shape
        strides = [strides[0] if strides else 1] + strides
    es = t.element_size()
    return shape, [s * es for s in strides]


def tilize_pack_batch(tensors, dst_df, geom=None, with_header=False, outs=None, path=None):
    """Tilize (and block-float pack) n same-shaped CUDA tensors into n queue images in one launch.
    Returns the list of uint8 image tensors."""
    _need_cuda(*tensors)
    t0 = tensors[0]
    shape, strides = _desc(t0)
    for t in tensors[1:]:
        if _desc(t) != (shape, strides):
            raise RuntimeError("tilize_pack_batch needs tensors of one shape and stride pattern")
    src_df = _TORCH_TO_DF[t0.dtype]
    if geom is None:
        geom = QueueGeom.for_shape(shape)
    nbytes = _cabi.tilized_bytes(geom, shape, int(dst_df), with_header)
    if outs is None:
        outs = [torch.empty(nbytes, dtype=torch.uint8, device=t0.device) for _ in tensors]
    srcs = _cabi.ptr_array([t.data_ptr() for t in tensors])
    dsts = _cabi.ptr_array([o.data_ptr() for o in outs])
    with torch.cuda.device(t0.device):
        if path is None:
            rc = _cabi.lib.buda_tilize_pack_batch(len(tensors), srcs, int(src_df), _cabi.u32x4(shape), _cabi.u64x4(strides),
                                                  ctypes.byref(geom), int(dst_df), int(with_header), dsts, nbytes, _stream())
        else:
            rc = _cabi.lib.buda_tilize_pack_batch_path(len(tensors), srcs, int(src_df), _cabi.u32x4(shape),
                                                       _cabi.u64x4(strides), ctypes.byref(geom), int(dst_df),
                                                       int(with_header), dsts, nbytes, _stream(), int(path))
    check(rc)
    return outs


def tilize_pack(t, dst_df, geom=None, with_header=False, out=None, path=None):
    return tilize_pack_batch([t], dst_df, geom, with_header, None if out is None else [out], path)[0]


def unpack_untilize_batch(images, src_df, shape, dtype=torch.float32, geom=None, with_header=False, outs=None, path=None):
    """Inverse of tilize_pack_batch: n queue images -> n row-major tensors of `shape` and `dtype`."""
    _need_cuda(*images)
    if outs is None:
        outs = [torch.empty(tuple(shape), dtype=dtype, device=images[0].device) for _ in images]
    shape4, strides = _desc(outs[0])
    dst_df = _TORCH_TO_DF[outs[0].dtype]
    if geom is None:
        geom = QueueGeom.for_shape(shape4)
    need = _cabi.tilized_bytes(geom, shape4, int(src_df), with_header)
    for im in images:
        if im.numel() * im.element_size() < need:
            raise RuntimeError(f"queue image holds {im.numel() * im.element_size()} bytes, needs {need}")
    srcs = _cabi.ptr_array([im.data_ptr() for im in images])
    dsts = _cabi.ptr_array([o.data_ptr() for o in outs])
    with torch.cuda.device(images[0].device):
        if path is None:
            rc = _cabi.lib.buda_unpack_untilize_batch(len(images), srcs, int(src_df), int(with_header), ctypes.byref(geom),
                                                      dsts, int(dst_df), _cabi.u32x4(shape4), _cabi.u64x4(strides), _stream())
        else:
            rc = _cabi.lib.buda_unpack_untilize_batch_path(len(images), srcs, int(src_df), int(with_header),
                                                           ctypes.byref(geom), dsts, int(dst_df), _cabi.u32x4(shape4),
                                                           _cabi.u64x4(strides), _stream(), int(path))
    check(rc)
    return outs


def unpack_untilize(image, src_df, shape, dtype=torch.float32, geom=None, with_header=False, out=None, path=None):
    return unpack_untilize_batch([image], src_df, shape, dtype, geom, with_header, None if out is None else [out], path)[0]


def _scale_args(x, scale, axis):
    scale = scale.reshape(-1)
    if scale.numel() == 1:
        return scale, 1, 1
    ax = axis if axis >= 0 else x.dim() + axis
    if x.shape[ax] != scale.numel():
        raise RuntimeError(f"scale has {scale.numel()} entries, axis {axis} of the input has {x.shape[ax]}")
    inner = 1
    for d in x.shape[ax + 1:]:
        inner *= d
    return scale, scale.numel(), inner


def quantize(x, scale, zero_point, axis=-1, buda=False, lo=-128.0, hi=127.0):
    """Quantize (divide by scale) or BudaQuantize (multiply by scale): float32 -> int8."""
    _need_cuda(x, scale)
    x = x.contiguous().float()
    s, sl, inner = _scale_args(x, scale.float().contiguous(), axis)
    out = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    with torch.cuda.device(x.device):
        check(_cabi.lib.buda_quantize(x.data_ptr(), x.numel(), s.data_ptr(), sl, inner, float(zero_point), int(buda),
                                      float(lo), float(hi), out.data_ptr(), _stream()))
    return out


def dequantize(x, scale, zero_point, axis=-1):
    _need_cuda(x, scale)
    x = x.contiguous()
    assert x.dtype == torch.int8
    s, sl, inner = _scale_args(x, scale.float().contiguous(), axis)
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(_cabi.lib.buda_dequantize(x.data_ptr(), x.numel(), s.data_ptr(), sl, inner, float(zero_point),
                                        out.data_ptr(), _stream()))
    return out


def requantize(x, inp_scale, out_scale, out_zp, axis=-1, lo=-128.0, hi=127.0):
    """Requantize: int32 -> int8 with scale inp_scale / out_scale."""
    _need_cuda(x, inp_scale, out_scale)
    x = x.contiguous()
    assert x.dtype == torch.int32
    a, sl, inner = _scale_args(x, inp_scale.float().contiguous(), axis)
    b = out_scale.float().reshape(-1).expand(a.shape).contiguous()
    out = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    with torch.cuda.device(x.device):
        check(_cabi.lib.buda_requantize(x.data_ptr(), x.numel(), a.data_ptr(), b.data_ptr(), sl, inner, float(out_zp), 0,
                                        float(lo), float(hi), out.data_ptr(), _stream()))
    return out


def buda_requantize(x, scale, zp, axis=-1, lo=-128.0, hi=127.0):
    """BudaRequantize: int32 -> int8 with the given (already combined) scale."""
    _need_cuda(x, scale)
    x = x.contiguous()
    assert x.dtype == torch.int32
    a, sl, inner = _scale_args(x, scale.float().contiguous(), axis)
    out = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    with torch.cuda.device(x.device):
        check(_cabi.lib.buda_requantize(x.data_ptr(), x.numel(), a.data_ptr(), None, sl, inner, float(zp), 1, float(lo),
                                        float(hi), out.data_ptr(), _stream()))
    return out


def bfp8b_matmul(a, w_image, n, out=None):
    """C = A @ W with A bfloat16 [M,K] and W the Bfp8_b queue image of a [K,N] tensor (default
    geometry, no header).  Returns bfloat16 [M,N]."""
    _need_cuda(a, w_image)
    assert a.dtype == torch.bfloat16 and a.dim() == 2 and a.stride(1) == 1
    m, k = a.shape
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    with torch.cuda.device(a.device):
        check(_cabi.lib.buda_bfp8b_gemm(a.data_ptr(), m, k, a.stride(0), w_image.data_ptr(), n, out.data_ptr(),
                                        out.stride(0), _stream()))
    return out


def i8_matmul(a, w_image, n, scale=None, zero_point=0.0, out="int32"):
    """int8 [M,K] @ W, W the tilized image of an Int8 queue holding a [K,N] tensor (tilize_pack(w_int8, DF.Int8)).
    out = "int32": the accumulators; "int8": requantised, clamp(round(acc * scale + zero_point), -128, 127);
    "float32": dequantised, (acc - zero_point) * scale.  scale: 1 value or N values (per output column)."""
    _need_cuda(a, w_image)
    assert a.dtype == torch.int8 and a.dim() == 2 and a.stride(1) == 1
    m, k = a.shape
    mode = {"int32": 0, "int8": 1, "float32": 2}[out]
    c = torch.empty((m, n), dtype=[torch.int32, torch.int8, torch.float32][mode], device=a.device)
    sc = None
    if mode:
        sc = scale.to(device=a.device, dtype=torch.float32).reshape(-1).contiguous()
    with torch.cuda.device(a.device):
        check(_cabi.lib.buda_i8_gemm(a.data_ptr(), m, k, a.stride(0), w_image.data_ptr(), n, sc.data_ptr() if mode else None,
                                     sc.numel() if mode else 0, float(zero_point), mode, c.data_ptr(), c.stride(0), _stream()))
    return c


def select_gemm_kernel(which):
    """'auto' (default), 'single', 'pair' or 'pair_register_epilogue': which tensor-core kernel the matmul launches.
    Returns the previous choice."""
    names = ["auto", "single", "pair", "pair_register_epilogue"]
    return names[_cabi.lib.buda_gemm_select_kernel(names.index(which))]


def bfp8b_matmul_scatter(a, w_image, n, dst_ptrs, ldc):
    """The same product stored to every device address in `dst_ptrs` (this device's first; the others
    usually peers' copies of the output mapped with SharedDeviceMatrix), row stride `ldc` elements."""
    _need_cuda(a, w_image)
    assert a.dtype == torch.bfloat16 and a.dim() == 2 and a.stride(1) == 1
    m, k = a.shape
    with torch.cuda.device(a.device):
        check(_cabi.lib.buda_bfp8b_gemm_scatter(a.data_ptr(), m, k, a.stride(0), w_image.data_ptr(), n,
                                                _cabi.ptr_array(dst_ptrs), len(dst_ptrs), ldc, _stream()))


def bfp8b_matmul_multicast(a, w_image, n, local_ptr, multicast_ptr, ldc):
    """The same product stored to this device's copy (local_ptr) and, through one multimem store per 16 bytes, to
    every device bound to the multicast address (multicast_ptr); both already point at this device's column block."""
    _need_cuda(a, w_image)
    assert a.dtype == torch.bfloat16 and a.dim() == 2 and a.stride(1) == 1
    m, k = a.shape
    with torch.cuda.device(a.device):
        check(_cabi.lib.buda_bfp8b_gemm_multicast(a.data_ptr(), m, k, a.stride(0), w_image.data_ptr(), n, local_ptr, multicast_ptr,
                                                  ldc, _stream()))


class _RawCudaBuffer:
    """Lets torch view memory it did not allocate (buda_malloc / a mapped peer allocation)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


class SharedDeviceMatrix:
    """A [rows, cols] bfloat16 matrix in plain device memory that the other processes of the box can map:
    `handle()` is the 64-byte token to send them, `open_peer(handle)` maps one of theirs here."""

    def __init__(self, rows, cols, device=None):
        import ctypes

        self.rows, self.cols = int(rows), int(cols)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.nbytes = self.rows * self.cols * 2
        ptr = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            check(_cabi.lib.buda_malloc(ctypes.byref(ptr), self.nbytes))
        self.ptr = ptr.value
        self._peers = []
        self.tensor = torch.as_tensor(_RawCudaBuffer(self.ptr, self.nbytes), device=self.device).view(torch.bfloat16).view(
            self.rows, self.cols)

    def handle(self) -> bytes:
        import ctypes

        buf = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            check(_cabi.lib.buda_ipc_export(self.ptr, buf))
        return buf.raw

    def open_peer(self, handle: bytes) -> int:
        import ctypes

        ptr = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            check(_cabi.lib.buda_ipc_open(ctypes.create_string_buffer(handle, 64), ctypes.byref(ptr)))
        self._peers.append(ptr.value)
        return ptr.value

    def close(self):
        with torch.cuda.device(self.device):
            for p in self._peers:
                _cabi.lib.buda_ipc_close(p)
            self._peers = []
            if self.ptr:
                self.tensor = None
                _cabi.lib.buda_free(self.ptr)
                self.ptr = None


def set_bfp_policy(policy=None):
    """Process-wide block-float layout policy (a _cabi.BfpPolicy; None restores the default)."""
    check(_cabi.lib.buda_set_bfp_policy(ctypes.byref(policy) if policy is not None else None))


def get_bfp_policy():
    p = _cabi.BfpPolicy()
    check(_cabi.lib.buda_get_bfp_policy(ctypes.byref(p)))
    return p


def _job_table(tensors, images, q_df, geoms, with_header, bands):
    jobs = (_cabi.TensorJob * len(tensors))()
    for i, (t, im) in enumerate(zip(tensors, images)):
        shape, strides = _desc(t)
        g = geoms[i] if geoms is not None and geoms[i] is not None else QueueGeom.for_shape(shape)
        j = jobs[i]
        j.tensor, j.image = t.data_ptr(), im.data_ptr()
        j.image_bytes = im.numel() * im.element_size()
        j.shape = _cabi.u32x4(shape)
        j.strides_bytes = _cabi.u64x4(strides)
        j.geom = g
        if bands is not None and bands[i] is not None:
            j.band_first, j.band_step, j.band_count = bands[i]
    return jobs


class TensorJobs:
    """A prepared job table: n CUDA tensors of one dtype but any shapes, their queue images, geometries and
    (optionally) selections of tile rows.  Building the table costs a few microseconds of Python per tensor, so a
    caller that converts the same set repeatedly (a parameter set every step) prepares it once; pack() and unpack()
    are then one C call each."""

    def __init__(self, tensors, q_df, images=None, geoms=None, with_header=False, bands=None):
        _need_cuda(*tensors)
        self.tensors = list(tensors)
        self.q_df, self.with_header = int(q_df), bool(with_header)
        self.rm_df = int(_TORCH_TO_DF[tensors[0].dtype])
        if images is None:
            images = []
            for i, t in enumerate(tensors):
                shape, _ = _desc(t)
                g = geoms[i] if geoms is not None and geoms[i] is not None else QueueGeom.for_shape(shape)
                images.append(torch.empty(_cabi.tilized_bytes(g, shape, self.q_df, with_header), dtype=torch.uint8, device=t.device))
        _need_cuda(*images)
        self.images = list(images)
        self._jobs = _job_table(self.tensors, self.images, q_df, geoms, with_header, bands)
        self._n = len(self.tensors)

    def pack(self):
        """tensors -> images"""
        with torch.cuda.device(self.tensors[0].device):
            check(_cabi.lib.buda_tilize_pack_jobs(self._n, self._jobs, self.rm_df, self.q_df, int(self.with_header), _stream()))
        return self.images

    def unpack(self):
        """images -> tensors"""
        with torch.cuda.device(self.tensors[0].device):
            check(_cabi.lib.buda_unpack_untilize_jobs(self._n, self._jobs, self.q_df, int(self.with_header), self.rm_df, _stream()))
        return self.tensors


def tilize_pack_jobs(tensors, dst_df, geoms=None, with_header=False, outs=None, bands=None):
    """Tilize (and block-float pack) CUDA tensors of DIFFERENT shapes (one dtype) in as few launches as possible.
    geoms: per-tensor QueueGeom or None; bands: per-tensor (first, step, count) selection of tile rows or None.
    Returns the list of uint8 image tensors."""
    return TensorJobs(tensors, dst_df, outs, geoms, with_header, bands).pack()


def unpack_untilize_jobs(images, src_df, outs, geoms=None, with_header=False, bands=None):
    """Inverse of tilize_pack_jobs: images[i] -> outs[i] (CUDA tensors of one dtype, any shapes)."""
    return TensorJobs(outs, src_df, images, geoms, with_header, bands).unpack()


def tilize_pack_view(src, dst_df, queue_shape, view, geom=None, with_header=False, out=None, strides_bytes=None):
    """Tilize a CUDA tensor that is read through a source view (_cabi.SourceView: tile padding / broadcast, an
    embedding-index vector, a prestrided convolution activation) straight into the queue image of `queue_shape`
    ([w, t, R, C], whole tiles): one kernel, no intermediate tensor."""
    _need_cuda(src)
    qshape = _cabi.shape4(queue_shape)
    if geom is None:
        geom = QueueGeom.for_shape(qshape)
    nbytes = _cabi.tilized_bytes(geom, qshape, int(dst_df), with_header)
    if out is None:
        out = torch.empty(nbytes, dtype=torch.uint8, device=src.device)
    if strides_bytes is None:
        _, strides_bytes = _desc(src)
    with torch.cuda.device(src.device):
        check(_cabi.lib.buda_queue_write_view(src.data_ptr(), int(_TORCH_TO_DF[src.dtype]), _cabi.u32x4(qshape), _cabi.u64x4(strides_bytes),
                                              ctypes.byref(view), ctypes.byref(geom), int(dst_df), int(with_header), out.data_ptr(),
                                              out.numel(), 0, 0, _stream()))
    return out
