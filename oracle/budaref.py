"""ctypes front-end of the CPU oracle (oracle/budaref.c).  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this module: only tests, the smoke check and the
benchmark's CPU-baseline leg do.  Parity status of each part is stated in the header of
budaref.c (tile order, quantise ops and sizes are pinned; face order and Bfp bytes are
"parity unpinned" because the reference's converter source is not in its checkout).

All tensors cross this boundary as C-contiguous numpy arrays.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libbudaref.so")

# DataFormat values, pybuda/csrc/lower_to_buda/common.hpp:92-111
Float32, Float16, Bfp8, Bfp4, Bfp2, Float16_b = 0, 1, 2, 3, 11, 5
Bfp8_b, Bfp4_b, Bfp2_b, Lf8, UInt16, Int8, Int32 = 6, 7, 15, 10, 12, 14, 8
RawUInt8, RawUInt16, RawUInt32, Invalid = 0xF0, 0xF1, 0xF2, 0xFF


class Geom(ctypes.Structure):
    """Queue geometry; field order matches ref_geom in budaref.c."""

    _fields_ = [
        ("grid_r", ctypes.c_uint32), ("grid_c", ctypes.c_uint32),
        ("mblock_m", ctypes.c_uint32), ("mblock_n", ctypes.c_uint32),
        ("ublock_rt", ctypes.c_uint32), ("ublock_ct", ctypes.c_uint32),
        ("t", ctypes.c_uint32), ("ublock_order", ctypes.c_uint32), ("tile_height", ctypes.c_uint32),
    ]

    @classmethod
    def for_shape(cls, shape, grid=(1, 1), ublock=(1, 1), ublock_order=0, tile_height=32):
        """Geometry covering a [w,z,R,C] tensor: R = grid_r*mblock_m*ublock_rt*tile_height and
        C = grid_c*mblock_n*ublock_ct*32 (pybuda/pybuda/tensor.py:1382-1404)."""
        _, z, r, c = shape
        rt, ct = r // tile_height, c // 32
        assert r % tile_height == 0 and rt % (grid[0] * ublock[0]) == 0 and ct % (grid[1] * ublock[1]) == 0
        return cls(grid[0], grid[1], rt // (grid[0] * ublock[0]), ct // (grid[1] * ublock[1]),
                   ublock[0], ublock[1], z, ublock_order, tile_height)


class BfpPolicy(ctypes.Structure):
    """ref_bfp_policy; the default constructor is the default layout."""

    _fields_ = [
        ("rounding", ctypes.c_uint32), ("overflow", ctypes.c_uint32), ("face_order", ctypes.c_uint8 * 4),
        ("exponent_order", ctypes.c_uint32), ("datum_order", ctypes.c_uint32),
    ]

    def __init__(self, rounding=0, overflow=0, face_order=(0, 1, 2, 3), exponent_order=0, datum_order=0):
        super().__init__(rounding, overflow, (ctypes.c_uint8 * 4)(*face_order), exponent_order, datum_order)


def set_bfp_policy(policy=None):
    """Process-wide layout policy of the oracle (None: the default)."""
    rc = lib().ref_set_bfp_policy(ctypes.byref(policy) if policy is not None else None)
    if rc:
        raise ValueError("invalid block-float policy")


def build(force=False):
    """Compile libbudaref.so with the committed Makefile (building the checker is not using it)."""
    if force or not os.path.exists(_LIB_PATH) or (
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "budaref.c"))):
        env = {k: v for k, v in os.environ.items() if k not in ("CC", "CFLAGS")}
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True, env=env,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        vp, i32, i64, u32p = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.POINTER(ctypes.c_uint32)
        gp = ctypes.POINTER(Geom)
        L.ref_threads.restype = i32
        L.ref_set_threads.restype = i32
        L.ref_set_threads.argtypes = [i32]
        L.ref_set_bfp_policy.restype = i32
        L.ref_set_bfp_policy.argtypes = [ctypes.POINTER(BfpPolicy)]
        L.ref_tile_bytes.restype = ctypes.c_long
        L.ref_tile_bytes.argtypes = [i32, i32]
        L.ref_data_format_byte_size.restype = ctypes.c_long
        L.ref_data_format_byte_size.argtypes = [i32, ctypes.c_long]
        L.ref_tile_map.restype = None
        L.ref_tile_map.argtypes = [gp, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, u32p, u32p,
                                   ctypes.POINTER(ctypes.c_uint64)]
        L.ref_tile_unmap.restype = None
        L.ref_tile_unmap.argtypes = [gp, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint64, u32p, u32p, u32p]
        L.ref_tilized_bytes.restype = i64
        L.ref_tilized_bytes.argtypes = [gp, u32p, i32, i32]
        L.ref_tilize_pack.restype = i32
        L.ref_tilize_pack.argtypes = [vp, i32, u32p, u32p, gp, i32, i32, vp]
        L.ref_unpack_untilize.restype = i32
        L.ref_unpack_untilize.argtypes = [vp, i32, i32, gp, vp, i32, u32p, u32p]
        L.ref_lf8_encode.restype = ctypes.c_uint8
        L.ref_lf8_encode.argtypes = [ctypes.c_double]
        L.ref_lf8_decode.restype = ctypes.c_double
        L.ref_lf8_decode.argtypes = [ctypes.c_uint8]
        L.ref_bfp_pack_block.restype = None
        L.ref_bfp_pack_block.argtypes = [vp, i32, vp, vp]
        L.ref_bfp_unpack_block.restype = None
        L.ref_bfp_unpack_block.argtypes = [ctypes.c_uint8, vp, i32, vp]
        L.ref_bfp_a_pack_block.restype = None
        L.ref_bfp_a_pack_block.argtypes = [vp, i32, vp, vp]
        L.ref_bfp_a_unpack_block.restype = None
        L.ref_bfp_a_unpack_block.argtypes = [ctypes.c_uint8, vp, i32, vp]
        L.ref_quantize.restype = None
        L.ref_quantize.argtypes = [vp, i64, vp, i64, i64, ctypes.c_float, i32, ctypes.c_float, ctypes.c_float, vp]
        L.ref_dequantize.restype = None
        L.ref_dequantize.argtypes = [vp, i64, vp, i64, i64, ctypes.c_float, vp]
        L.ref_requantize.restype = None
        L.ref_requantize.argtypes = [vp, i64, vp, vp, i64, i64, ctypes.c_float, i32, ctypes.c_float,
                                     ctypes.c_float, vp]
        L.ref_bfp8b_matmul.restype = i32
        L.ref_bfp8b_matmul.argtypes = [vp, ctypes.c_long, ctypes.c_long, vp, gp, ctypes.c_long, vp]
        L.ref_i8_matmul.restype = i32
        L.ref_i8_matmul.argtypes = [vp, ctypes.c_long, ctypes.c_long, vp, gp, ctypes.c_long, vp, ctypes.c_long, ctypes.c_float,
                                    i32, vp]
        _lib = L
    return _lib


def threads():
    return lib().ref_threads()


def set_threads(n):
    """Limit the OpenMP team of the following calls; returns the previous limit."""
    return lib().ref_set_threads(int(n))


_NP_DF = {np.dtype(np.float32): Float32, np.dtype(np.int8): Int8, np.dtype(np.int32): Int32,
          np.dtype(np.float16): Float16, np.dtype(np.uint8): RawUInt8, np.dtype(np.uint32): RawUInt32}


def _u32x4(v):
    return (ctypes.c_uint32 * 4)(*[int(x) for x in v])


def _shape4(a):
    s = list(a.shape)
    while len(s) < 4:
        s = [1] + s
    assert len(s) == 4
    return s


def _strides4(shape, es):
    st = [es] * 4
    for i in (2, 1, 0):
        st[i] = st[i + 1] * shape[i + 1]
    return st


def tile_bytes(df, with_header=False):
    return lib().ref_tile_bytes(df, int(with_header))


def tile_map(geom, t, r, c):
    cr, cc, addr = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint64()
    lib().ref_tile_map(ctypes.byref(geom), t, r, c, ctypes.byref(cr), ctypes.byref(cc), ctypes.byref(addr))
    return cr.value, cc.value, addr.value


def tile_unmap(geom, core_r, core_c, addr):
    t, r, c = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint32()
    lib().ref_tile_unmap(ctypes.byref(geom), core_r, core_c, addr, ctypes.byref(t), ctypes.byref(r), ctypes.byref(c))
    return t.value, r.value, c.value


def tilize_pack(x, dst_df, geom=None, with_header=False, src_df=None):
    """x: C-contiguous numpy array of up to 4 dims (bfloat16 is passed as uint16 with
    src_df=Float16_b).  Returns the queue image as a uint8 array."""
    x = np.ascontiguousarray(x)
    shape = _shape4(x)
    if src_df is None:
        src_df = _NP_DF[x.dtype]
    if geom is None:
        geom = Geom.for_shape(shape)
    n = lib().ref_tilized_bytes(ctypes.byref(geom), _u32x4(shape), dst_df, int(with_header))
    assert n >= 0, "shape does not fit the queue geometry"
    out = np.zeros(n, dtype=np.uint8)
    rc = lib().ref_tilize_pack(x.ctypes.data, src_df, _u32x4(shape), _u32x4(_strides4(shape, x.itemsize)),
                               ctypes.byref(geom), dst_df, int(with_header), out.ctypes.data)
    assert rc == 0, "ref_tilize_pack rejected its arguments"
    return out


def unpack_untilize(img, src_df, shape, dst_dtype=np.float32, geom=None, with_header=False, dst_df=None):
    """Inverse of tilize_pack.  dst_dtype np.uint16 with dst_df=Float16_b yields bfloat16 bits."""
    img = np.ascontiguousarray(img, dtype=np.uint8)
    shape4 = _shape4(np.empty(shape, dtype=np.uint8))
    if geom is None:
        geom = Geom.for_shape(shape4)
    if dst_df is None:
        dst_df = _NP_DF[np.dtype(dst_dtype)]
    out = np.zeros(shape4, dtype=dst_dtype)
    rc = lib().ref_unpack_untilize(img.ctypes.data, src_df, int(with_header), ctypes.byref(geom), out.ctypes.data,
                                   dst_df, _u32x4(shape4), _u32x4(_strides4(shape4, out.itemsize)))
    assert rc == 0, "ref_unpack_untilize rejected its arguments"
    return out.reshape(shape)


def lf8_encode(v):
    """One value -> its Lf8 code (1-5-2 float, round to nearest even)."""
    return int(lib().ref_lf8_encode(float(v)))


def lf8_decode(code):
    return float(lib().ref_lf8_decode(int(code)))


def bfp_pack_block(bits16, mant_bits):
    bits16 = np.ascontiguousarray(bits16, dtype=np.uint32)
    assert bits16.size == 16
    exp = np.zeros(1, dtype=np.uint8)
    out = np.zeros(16 * (mant_bits + 1) // 8, dtype=np.uint8)
    lib().ref_bfp_pack_block(bits16.ctypes.data, mant_bits, exp.ctypes.data, out.ctypes.data)
    return int(exp[0]), out


def bfp_unpack_block(exp, data, mant_bits):
    data = np.ascontiguousarray(data, dtype=np.uint8)
    out = np.zeros(16, dtype=np.float32)
    lib().ref_bfp_unpack_block(int(exp), data.ctypes.data, mant_bits, out.ctypes.data)
    return out


def bfp_a_pack_block(half_bits16, mant_bits):
    """One block of an "a" format (5-bit shared exponent) from 16 binary16 bit patterns."""
    h = np.ascontiguousarray(half_bits16, dtype=np.uint16)
    assert h.size == 16
    exp = np.zeros(1, dtype=np.uint8)
    out = np.zeros(16 * (mant_bits + 1) // 8, dtype=np.uint8)
    lib().ref_bfp_a_pack_block(h.ctypes.data, mant_bits, exp.ctypes.data, out.ctypes.data)
    return int(exp[0]), out


def bfp_a_unpack_block(exp, data, mant_bits):
    data = np.ascontiguousarray(data, dtype=np.uint8)
    out = np.zeros(16, dtype=np.float32)
    lib().ref_bfp_a_unpack_block(int(exp), data.ctypes.data, mant_bits, out.ctypes.data)
    return out


def _scale_args(x, scale, axis):
    scale = np.ascontiguousarray(scale, dtype=np.float32).reshape(-1)
    if scale.size == 1:
        return scale, 1, 1
    ax = axis if axis >= 0 else x.ndim + axis
    assert x.shape[ax] == scale.size
    inner = int(np.prod(x.shape[ax + 1:], dtype=np.int64))
    return scale, scale.size, inner


def quantize(x, scale, zero_point, axis=-1, buda=False, lo=-128.0, hi=127.0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    s, sl, inner = _scale_args(x, scale, axis)
    out = np.empty(x.shape, dtype=np.int8)
    lib().ref_quantize(x.ctypes.data, x.size, s.ctypes.data, sl, inner, float(zero_point), int(buda), lo, hi,
                       out.ctypes.data)
    return out


def dequantize(x, scale, zero_point, axis=-1):
    x = np.ascontiguousarray(x, dtype=np.int8)
    s, sl, inner = _scale_args(x, scale, axis)
    out = np.empty(x.shape, dtype=np.float32)
    lib().ref_dequantize(x.ctypes.data, x.size, s.ctypes.data, sl, inner, float(zero_point), out.ctypes.data)
    return out


def requantize(x, inp_scale, out_scale, out_zp, axis=-1, lo=-128.0, hi=127.0):
    x = np.ascontiguousarray(x, dtype=np.int32)
    a, sl, inner = _scale_args(x, inp_scale, axis)
    b = np.ascontiguousarray(np.broadcast_to(np.asarray(out_scale, dtype=np.float32).reshape(-1), a.shape))
    out = np.empty(x.shape, dtype=np.int8)
    lib().ref_requantize(x.ctypes.data, x.size, a.ctypes.data, b.ctypes.data, sl, inner, float(out_zp), 0, lo, hi,
                         out.ctypes.data)
    return out


def buda_requantize(x, scale, zp, axis=-1, lo=-128.0, hi=127.0):
    x = np.ascontiguousarray(x, dtype=np.int32)
    a, sl, inner = _scale_args(x, scale, axis)
    out = np.empty(x.shape, dtype=np.int8)
    lib().ref_requantize(x.ctypes.data, x.size, a.ctypes.data, a.ctypes.data, sl, inner, float(zp), 1, lo, hi,
                         out.ctypes.data)
    return out


def bfp8b_matmul(a_bf16_bits, w_img, K, N, geom=None):
    a = np.ascontiguousarray(a_bf16_bits, dtype=np.uint16)
    M = a.shape[0]
    assert a.shape[1] == K
    if geom is None:
        geom = Geom.for_shape([1, 1, K, N])
    w = np.ascontiguousarray(w_img, dtype=np.uint8)
    out = np.zeros((M, N), dtype=np.float32)
    rc = lib().ref_bfp8b_matmul(a.ctypes.data, M, K, w.ctypes.data, ctypes.byref(geom), N, out.ctypes.data)
    assert rc == 0
    return out


def i8_matmul(a_i8, w_img, K, N, scale=None, zp=0.0, mode=0, geom=None):
    """int8 [M,K] @ Int8 queue image of [K,N]: mode 0 int32 accumulators, 1 requantised int8, 2 dequantised float32."""
    a = np.ascontiguousarray(a_i8, dtype=np.int8)
    M = a.shape[0]
    assert a.shape[1] == K
    if geom is None:
        geom = Geom.for_shape([1, 1, K, N])
    w = np.ascontiguousarray(w_img, dtype=np.uint8)
    out = np.zeros((M, N), dtype=[np.int32, np.int8, np.float32][mode])
    sc = None if scale is None else np.ascontiguousarray(scale, dtype=np.float32).reshape(-1)
    rc = lib().ref_i8_matmul(a.ctypes.data, M, K, w.ctypes.data, ctypes.byref(geom), N,
                             None if sc is None else sc.ctypes.data, 0 if sc is None else sc.size, ctypes.c_float(zp), mode,
                             out.ctypes.data)
    assert rc == 0
    return out


def prestride_act(act, stride):
    """Golden prestride of a [w, z, H, W] activation (pybuda/pybuda/op/eval/pybuda/tm.py:316-335): pad H and W with
    zeros to multiples of the stride, take the stride x stride phase images act[:, :, y::s, x::s] (y outer, x inner),
    stack them along z, flatten each image into one row -> [w, 1, z*s*s, (H/s)*(W/s)]."""
    act = np.asarray(act)
    w, z, h, wd = act.shape
    hp, wp = -(-h // stride) * stride, -(-wd // stride) * stride
    padded = np.zeros((w, z, hp, wp), dtype=act.dtype)
    padded[:, :, :h, :wd] = act
    phases = [padded[:, :, y::stride, x::stride] for y in range(stride) for x in range(stride)]
    out = np.concatenate(phases, axis=-3)
    return out.reshape(w, 1, out.shape[1], out.shape[2] * out.shape[3])



# ------------------------------------------------------------------------------------------------
# Runtime tensor transforms of the push path, restated in numpy (checker for the kernels' source views).
# Pinned by tests/golden/transform_golden.npz, which the reference's own functions produced.
# ------------------------------------------------------------------------------------------------
def _align32(v):
    return (v + 31) // 32 * 32


def embedding_index(indices, count, q_rt):
    """Row indices laid out for an embedding op (pybuda/pybuda/tensor.py:1382-1405): padded to whole tiles with
    all-ones from position `count` on, cut into q_rt groups (one per queue tile row), every 32 consecutive indices a
    row, rows zero-padded to a multiple of 32, and each 32x32 block of rows transposed into place so that a tile holds
    1024 consecutive indices.  Returns [w, 1, q_rt * 32, columns]."""
    idx = np.atleast_2d(np.asarray(indices))
    w, n = idx.shape
    n_pad = _align32(n)
    flat = np.zeros((w, n_pad), dtype=idx.dtype)
    flat[:, :n] = idx
    flat[:, count:] = ~np.zeros((), dtype=idx.dtype)
    assert n_pad % (q_rt * 32) == 0, "the padded index count must split evenly over the queue's tile rows"
    rows = n_pad // q_rt // 32
    p_rows = _align32(rows)
    t = np.zeros((w, q_rt, p_rows, 32), dtype=idx.dtype)
    t[:, :, :rows, :] = flat.reshape(w, q_rt, rows, 32)
    t = t.reshape(w, q_rt, p_rows // 32, 32, 32).transpose(0, 1, 3, 2, 4)
    return np.ascontiguousarray(t).reshape(w, 1, q_rt * 32, p_rows)


def prestride_act(act, stride, xy_offsets=None):
    """Convolution activation cut into its stride phases (golden pybuda/pybuda/op/eval/pybuda/tm.py:316-335; the
    offsets are the queue's StrideDescriptor, pybuda/pybuda/tensor.py:1415-1422): [w, z, H, W], zero-padded to
    multiples of the stride -> [w, 1, n_offsets * z, ceil(H/s) * ceil(W/s)]."""
    act = np.asarray(act)
    w, z, h, wd = act.shape
    if xy_offsets is None:
        xy_offsets = [(x, y) for y in range(stride) for x in range(stride)]
    hp, wp = -(-h // stride) * stride, -(-wd // stride) * stride
    padded = np.zeros((w, z, hp, wp), dtype=act.dtype)
    padded[:, :, :h, :wd] = act
    phases = [padded[:, :, y::stride, x::stride] for (x, y) in xy_offsets]
    out = np.concatenate(phases, axis=1)
    return np.ascontiguousarray(out).reshape(w, 1, out.shape[1], out.shape[2] * out.shape[3])


def pad_to_tiles(x, replicate_rows=False, replicate_cols=False):
    """Rows and columns of a 4-D tensor rounded up to whole 32x32 tiles: zeros, or the single row / column repeated
    for a tile-broadcast dim (pad_pytorch_tensor_to_buda, pybuda/pybuda/tensor.py:805-877)."""
    x = np.asarray(x)
    w, z, r, c = x.shape
    out = np.zeros((w, z, _align32(r), _align32(c)), dtype=x.dtype)
    out[:, :, :r, :c] = x
    if replicate_cols:
        assert c == 1
        out[:, :, :r, :] = x
    if replicate_rows:
        assert r == 1
        out[:, :, :, :] = out[:, :, :1, :]
    return out
