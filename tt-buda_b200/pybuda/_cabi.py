"""ctypes view of libbuda_cuda.so (include/buda_cuda.h, include/buda_cuda_testing.h) for callers that already hold device
pointers, e.g. CUDA torch tensors.  There is no fallback: if the library is missing this module
raises at import, and every compute call needs a CUDA device.
"""
import ctypes
import os

_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libbuda_cuda.so")
if not os.path.exists(_LIB_PATH):
    raise ImportError(
        f"{_LIB_PATH} is missing: build it with `python tt-buda_b200/build.py` (there is no CPU fallback)")

lib = ctypes.CDLL(_LIB_PATH)

SUCCESS, RUNTIME_ERROR, TIMEOUT_ERROR = 0, 1, 2


class QueueGeom(ctypes.Structure):
    """buda_queue_geom"""

    _fields_ = [
        ("grid_r", ctypes.c_uint32), ("grid_c", ctypes.c_uint32),
        ("mblock_m", ctypes.c_uint32), ("mblock_n", ctypes.c_uint32),
        ("ublock_rt", ctypes.c_uint32), ("ublock_ct", ctypes.c_uint32),
        ("t", ctypes.c_uint32), ("ublock_order", ctypes.c_uint32), ("tile_height", ctypes.c_uint32),
    ]

    @classmethod
    def for_shape(cls, shape, grid=(1, 1), ublock=(1, 1), ublock_order=0, tile_height=32):
        _, z, r, c = shape
        if r % tile_height or c % 32:
            raise ValueError(f"[{r},{c}] is not a whole number of {tile_height}x32 tiles")
        rt, ct = r // tile_height, c // 32
        if rt % (grid[0] * ublock[0]) or ct % (grid[1] * ublock[1]):
            raise ValueError("grid x ublock does not divide the tensor's tile counts")
        return cls(grid[0], grid[1], rt // (grid[0] * ublock[0]), ct // (grid[1] * ublock[1]),
                   ublock[0], ublock[1], z, ublock_order, tile_height)


class TensorJob(ctypes.Structure):
    """buda_tensor_job"""

    _fields_ = [
        ("tensor", ctypes.c_void_p), ("image", ctypes.c_void_p), ("image_bytes", ctypes.c_uint64),
        ("shape", ctypes.c_uint32 * 4), ("strides_bytes", ctypes.c_uint64 * 4), ("geom", QueueGeom),
        ("band_first", ctypes.c_uint32), ("band_step", ctypes.c_uint32), ("band_count", ctypes.c_uint32),
        ("slots", ctypes.c_uint32), ("first_slot", ctypes.c_uint32),
    ]


class BfpPolicy(ctypes.Structure):
    """buda_bfp_policy; the default constructor gives the library's default layout"""

    _fields_ = [
        ("rounding", ctypes.c_uint32), ("overflow", ctypes.c_uint32), ("face_order", ctypes.c_uint8 * 4),
        ("exponent_order", ctypes.c_uint32), ("datum_order", ctypes.c_uint32),
    ]

    def __init__(self, rounding=0, overflow=0, face_order=(0, 1, 2, 3), exponent_order=0, datum_order=0):
        super().__init__(rounding, overflow, (ctypes.c_uint8 * 4)(*face_order), exponent_order, datum_order)


class SourceView(ctypes.Structure):
    """buda_source_view"""

    _fields_ = [
        ("mode", ctypes.c_uint32), ("valid_r", ctypes.c_uint32), ("valid_c", ctypes.c_uint32),
        ("bcast_r", ctypes.c_uint32), ("bcast_c", ctypes.c_uint32),
        ("emb_count", ctypes.c_uint64), ("emb_group", ctypes.c_uint64),
        ("ps_stride", ctypes.c_uint32), ("ps_z", ctypes.c_uint32), ("ps_h", ctypes.c_uint32), ("ps_w", ctypes.c_uint32),
        ("ps_n_offsets", ctypes.c_uint32), ("ps_xy", ctypes.c_int32 * 128),
    ]


_vp, _i, _i64, _u64, _u32, _f = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_uint64, ctypes.c_uint32,
                                 ctypes.c_float)
_jp, _pp = ctypes.POINTER(TensorJob), ctypes.POINTER(BfpPolicy)
_u32p, _u64p, _gp, _vpp = (ctypes.POINTER(ctypes.c_uint32), ctypes.POINTER(ctypes.c_uint64),
                           ctypes.POINTER(QueueGeom), ctypes.POINTER(ctypes.c_void_p))

_SIGS = {
    "buda_tile_bytes": (_i64, [_i, _i]),
    "buda_data_format_byte_size": (_i64, [_i, _i64]),
    "buda_io_size_bytes": (_i64, [_i, _i, _u32, _u32, _u32, _u32, _u32, _u32, _u32, _u32]),
    "buda_tilized_bytes": (_i64, [_gp, _u32p, _i, _i]),
    "buda_tile_map": (_i, [_gp, _u32, _u32, _u32, _u32p, _u32p, _u64p]),
    "buda_tilize_pack": (_i, [_vp, _i, _u32p, _u64p, _gp, _i, _i, _vp, _u64, _vp]),
    "buda_tilize_pack_batch": (_i, [_i, _vpp, _i, _u32p, _u64p, _gp, _i, _i, _vpp, _u64, _vp]),
    "buda_tilize_pack_batch_path": (_i, [_i, _vpp, _i, _u32p, _u64p, _gp, _i, _i, _vpp, _u64, _vp, _i]),
    "buda_tilize_pack_host": (_i, [_vp, _i, _u32p, _u64p, _gp, _i, _i, _vp, _u64, _vp]),
    "buda_tilize_pack_host_batch": (_i, [_i, _vpp, _i, _u32p, _u64p, _gp, _i, _i, _vpp, _u64, _vp]),
    "buda_tilize_pack_host_noalloc": (_i, [_vp, _i, _u32p, _u64p, _gp, _i, _i, _vp, _u64, _vp]),
    "buda_tilize_pack_jobs": (_i, [_i, _jp, _i, _i, _i, _vp]),
    "buda_tilize_pack_host_jobs": (_i, [_i, _jp, _i, _i, _i, _i, _vp]),
    "buda_unpack_untilize_jobs": (_i, [_i, _jp, _i, _i, _i, _vp]),
    "buda_unpack_untilize_host_jobs": (_i, [_i, _jp, _i, _i, _i, _i, _vp]),
    "buda_set_bfp_policy": (_i, [_pp]),
    "buda_get_bfp_policy": (_i, [_pp]),
    "buda_unpack_untilize": (_i, [_vp, _i, _i, _gp, _vp, _i, _u32p, _u64p, _vp]),
    "buda_unpack_untilize_batch": (_i, [_i, _vpp, _i, _i, _gp, _vpp, _i, _u32p, _u64p, _vp]),
    "buda_unpack_untilize_batch_path": (_i, [_i, _vpp, _i, _i, _gp, _vpp, _i, _u32p, _u64p, _vp, _i]),
    "buda_unpack_untilize_host": (_i, [_vp, _i, _i, _gp, _vp, _i, _u32p, _u64p, _vp]),
    "buda_queue_bytes": (_i64, [_gp, _i, _i, _u32]),
    "buda_queue_write": (_i, [_vp, _i, _i, _u32p, _u64p, _gp, _i, _i, _vp, _u32, _u32, _vp]),
    "buda_queue_write_view": (_i, [_vp, _i, _u32p, _u64p, ctypes.POINTER(SourceView), _gp, _i, _i, _vp, _u64, _u32, _u32, _vp]),
    "buda_queue_read": (_i, [_vp, _i, _i, _gp, _u32, _u32, _vp, _i, _i, _u32p, _u64p, _vp]),
    "buda_queue_read_stacked": (_i, [_vp, _i, _i, _gp, _u32, _u32, _u32, _u32, _u32, _i, _vp, _i, _vp]),
    "buda_malloc": (_i, [_vpp, _u64]),
    "buda_free": (_i, [_vp]),
    "buda_host_alloc": (_i, [_vpp, _u64]),
    "buda_host_free": (_i, [_vp]),
    "buda_memcpy": (_i, [_vp, _vp, _u64, _i, _vp]),
    "buda_stream_synchronize": (_i, [_vp]),
    "buda_pointer_is_device": (_i, [_vp, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]),
    "buda_get_device": (_i, [ctypes.POINTER(ctypes.c_int)]),
    "buda_set_device": (_i, [_i]),
    "buda_device_count": (_i, [ctypes.POINTER(ctypes.c_int)]),
    "buda_quantize": (_i, [_vp, _i64, _vp, _i64, _i64, _f, _i, _f, _f, _vp, _vp]),
    "buda_dequantize": (_i, [_vp, _i64, _vp, _i64, _i64, _f, _vp, _vp]),
    "buda_requantize": (_i, [_vp, _i64, _vp, _vp, _i64, _i64, _f, _i, _f, _f, _vp, _vp]),
    "buda_bfp8b_gemm": (_i, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _vp]),
    "buda_bfp8b_gemm_scatter": (_i, [_vp, _i64, _i64, _i64, _vp, _i64, ctypes.POINTER(ctypes.c_void_p), _i, _i64, _vp]),
    "buda_bfp8b_gemm_multicast": (_i, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _vp, _i64, _vp]),
    "buda_prestride": (_i, [_vp, _i, _u32p, _u64p, _i, ctypes.POINTER(ctypes.c_int), _i, _vp, _u32, _u32, _vp]),
    "buda_i8_gemm": (_i, [_vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _f, _i, _vp, _i64, _vp]),
    "buda_gemm_select_kernel": (_i, [_i]),
    "buda_selftest_bounded_wait": (_i, [_u32, _vp]),
    "buda_ipc_export": (_i, [_vp, ctypes.c_char_p]),
    "buda_ipc_open": (_i, [ctypes.c_char_p, _vpp]),
    "buda_ipc_close": (_i, [_vp]),
    "buda_last_error": (ctypes.c_size_t, [ctypes.c_char_p, ctypes.c_size_t]),
    "buda_device_status": (_i, [ctypes.POINTER(ctypes.c_int)]),
    "buda_launch_count": (_u64, []),
    "buda_version": (ctypes.c_char_p, []),
}
for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTED = tuple(_SIGS)


class BudaError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"status {code}: {msg}")
        self.code = code


def last_error():
    buf = ctypes.create_string_buffer(512)
    lib.buda_last_error(buf, 512)
    return buf.value.decode()


def check(rc):
    if rc != SUCCESS:
        raise BudaError(rc, last_error())


def u32x4(v):
    return (ctypes.c_uint32 * 4)(*[int(x) for x in v])


def u64x4(v):
    return (ctypes.c_uint64 * 4)(*[int(x) for x in v])


def ptr_array(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def shape4(shape):
    s = [int(x) for x in shape]
    while len(s) > 4:
        if s[0] != 1:
            raise ValueError("cannot drop a leading dimension that is not 1")
        s = s[1:]
    return [1] * (4 - len(s)) + s


def dense_strides(shape, es):
    st = [es] * 4
    for i in (2, 1, 0):
        st[i] = st[i + 1] * shape[i + 1]
    return st


def tilized_bytes(geom, shape, df, with_header=False):
    n = lib.buda_tilized_bytes(ctypes.byref(geom), u32x4(shape), df, int(with_header))
    if n < 0:
        raise BudaError(RUNTIME_ERROR, last_error())
    return n


def device_status():
    st = ctypes.c_int(0)
    rc = lib.buda_device_status(ctypes.byref(st))
    return rc, st.value


def launch_count():
    return lib.buda_launch_count()
