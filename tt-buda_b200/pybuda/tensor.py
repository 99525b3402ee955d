"""Tensor wrappers and the torch <-> backend descriptor conversions of the data-format path.

Same names, arguments and results as the reference's pybuda/pybuda/tensor.py for the part of it
that feeds the converters: dtype <-> DataFormat maps (563-651), descriptor building (653-745),
padding to 4-D tile-aligned shapes (799-877) and narrowing back (879-954), and the Tensor
wrappers around a torch value or a descriptor (151-546).  TensorFlow / JAX / sparse / traced
tensors of the reference are not part of this path.
"""
from functools import reduce
from operator import mul
from typing import List, Optional, Tuple

import torch

from . import TILE_DIM
from ._C import DataFormat
from ._C.backend_api import DramIODesc, PytorchTensorDesc, StrideDescriptor, TilizedTensorDesc

SomeTensor = torch.Tensor


def align_up_tile(v: int) -> int:
    return (v + TILE_DIM - 1) // TILE_DIM * TILE_DIM


class TensorShape:
    """Shape of up to four named dims (w, z, r, c counted from the back)."""

    def __init__(self, *dims):
        self.dims = tuple(int(d) for d in dims)

    def _from_back(self, i):
        return self.dims[-i] if len(self.dims) >= i else 1

    @property
    def c(self):
        return self._from_back(1)

    @property
    def r(self):
        return self._from_back(2)

    @property
    def z(self):
        return self._from_back(3)

    @property
    def w(self):
        return self._from_back(4)

    @property
    def rt(self):
        return (self.r + TILE_DIM - 1) // TILE_DIM

    @property
    def ct(self):
        return (self.c + TILE_DIM - 1) // TILE_DIM

    def rc_divisible_by_tile_dim(self) -> bool:
        return self.r % TILE_DIM == 0 and self.c % TILE_DIM == 0

    def get_pytorch_shape(self) -> Tuple[int, ...]:
        return self.dims

    @classmethod
    def from_pytorch_tuple(cls, w, z, r, c):
        return cls(w, z, r, c)

    def numel(self):
        return reduce(mul, self.dims, 1)

    def __len__(self):
        return len(self.dims)

    def __getitem__(self, i):
        return self.dims[i]

    def __repr__(self):
        return str(self.dims)

    def __eq__(self, other):
        return tuple(other) == self.dims if not isinstance(other, TensorShape) else other.dims == self.dims


# ------------------------------------------------------------------------------------------------
# torch dtype <-> DataFormat
# ------------------------------------------------------------------------------------------------
_DTYPE_TO_DF = {
    torch.float16: DataFormat.Float16,
    torch.bfloat16: DataFormat.Float16_b,
    torch.float32: DataFormat.Float32,
    torch.int8: DataFormat.Int8,
    torch.bool: DataFormat.Bfp2_b,
    torch.int32: DataFormat.Int32,
    torch.int64: DataFormat.Int8,  # the reference narrows int64 parameters to int8 (with a warning)
}

_DF_TO_DTYPE = {
    DataFormat.Float32: torch.float32,
    DataFormat.Float16: torch.float16,
    DataFormat.Float16_b: torch.bfloat16,
    DataFormat.Bfp8_b: torch.bfloat16, DataFormat.Bfp4_b: torch.bfloat16, DataFormat.Bfp2_b: torch.bfloat16,
    DataFormat.Bfp8: torch.float16, DataFormat.Bfp4: torch.float16, DataFormat.Bfp2: torch.float16,
    DataFormat.Int8: torch.int8,
    DataFormat.RawUInt32: torch.int,
    DataFormat.UInt16: torch.int,
    DataFormat.Int32: torch.int32,
}

_EXACT_PAIRS = {
    DataFormat.Float32: torch.float32, DataFormat.Float16: torch.float16, DataFormat.Float16_b: torch.bfloat16,
    DataFormat.Int8: torch.int8,
}


def pytorch_dtype_to_buda_dataformat(dtype, fp32_fallback: Optional[DataFormat] = None) -> DataFormat:
    if isinstance(dtype, DataFormat):
        return dtype
    assert isinstance(dtype, torch.dtype)
    if dtype == torch.float32 and fp32_fallback is not None:
        return fp32_fallback
    try:
        return _DTYPE_TO_DF[dtype]
    except KeyError:
        raise RuntimeError("Unsupported torch dtype " + str(dtype))


def buda_dataformat_to_pytorch_dtype(data_format: DataFormat) -> torch.dtype:
    assert isinstance(data_format, DataFormat)
    try:
        return _DF_TO_DTYPE[data_format]
    except KeyError:
        raise RuntimeError("Unsupported DataFormat for conversion to torch dtype: " + str(data_format))


def is_equivalent_data_format(pt_df: torch.dtype, tt_df: DataFormat) -> bool:
    """True when the torch dtype and the device format hold exactly the same values."""
    return _EXACT_PAIRS.get(tt_df) == pt_df


# ------------------------------------------------------------------------------------------------
# descriptors
# ------------------------------------------------------------------------------------------------
_TILIZE_NDIM = 4

_INFERRED_FORMAT = {
    torch.float32: DataFormat.Float32, torch.bfloat16: DataFormat.Float16_b, torch.float16: DataFormat.Float16,
    torch.int32: DataFormat.Int32, torch.int8: DataFormat.Int8,
}


def _to_4d(values: list, what: str, fill) -> list:
    values = list(values)
    while len(values) > _TILIZE_NDIM:
        if what == "shape" and values[0] != 1:
            raise RuntimeError("Dropping a dimension that's not 1 to reduce shape to 4D: " + str(values))
        values = values[1:]
    while len(values) < _TILIZE_NDIM:
        values = [fill(values)] + values
    return values


def pytorch_tensor_to_tensor_desc(t: torch.Tensor, df: DataFormat = None, element_size=None) -> "PytorchTensorDesc":
    """Describe a torch tensor (host or CUDA) to the converters: 4-D [w,z,r,c] shape and BYTE strides.
    With `df` given the tensor is first cast to the torch dtype that format travels as."""
    if isinstance(t, (PytorchTensorDesc, TilizedTensorDesc)):
        return t
    if not t.is_contiguous():
        t = t.contiguous()
    if df is None:
        if t.dtype == torch.int64:
            t = t.to(torch.int32)  # the reference pushes int64 as raw 32-bit words
            fmt = DataFormat.RawUInt32
        elif t.dtype in _INFERRED_FORMAT:
            fmt = _INFERRED_FORMAT[t.dtype]
        else:
            raise RuntimeError("Unsupported torch tensor type for tilization: " + str(t.dtype))
    else:
        fmt = df
        want = buda_dataformat_to_pytorch_dtype(fmt)
        if t.dtype != want:
            t = t.type(want)

    dim = 3 if t.dim() == 2 else t.dim()
    shape = _to_4d(t.shape, "shape", lambda v: 1)
    strides = _to_4d(t.stride(), "strides", lambda v: v[0])
    if element_size is None:
        element_size = t.element_size()
    return PytorchTensorDesc(t, element_size, fmt, dim, shape, [s * element_size for s in strides])


_READBACK_DTYPE = {
    DataFormat.Float32: torch.float32, DataFormat.Float16_b: torch.bfloat16, DataFormat.Float16: torch.float16,
    DataFormat.RawUInt32: torch.int,
}


def tensor_desc_to_pytorch_tensor(desc: "PytorchTensorDesc") -> torch.Tensor:
    """Zero-copy torch view of a (host) descriptor's memory."""
    try:
        dtype = _READBACK_DTYPE[desc.format]
    except KeyError:
        raise RuntimeError(f"Unsupported tensor type({desc.format}) for untilization")
    return torch.frombuffer(desc, dtype=dtype).reshape(list(desc.shape))


def buffer_to_pytorch_tensor(buf_ptr: int, shape: Tuple, format: DataFormat) -> torch.Tensor:
    """Torch view of a dense row-major host buffer at address buf_ptr."""
    sizes = {DataFormat.Float32: 4, DataFormat.Float16_b: 2, DataFormat.Float16: 2}
    if format not in sizes:
        raise RuntimeError("Unsupported format")
    dim = len(shape)
    shape = list(shape)
    while len(shape) > _TILIZE_NDIM:
        if shape[0] != 1:
            raise RuntimeError("Trimming a dimension that's not 1")
        shape = shape[1:]
    shape = [1] * (_TILIZE_NDIM - len(shape)) + shape
    es = sizes[format]
    strides = [es] * _TILIZE_NDIM
    for i in range(_TILIZE_NDIM - 2, -1, -1):
        strides[i] = strides[i + 1] * shape[i + 1]
    return tensor_desc_to_pytorch_tensor(PytorchTensorDesc(int(buf_ptr), es, format, dim, shape, strides))


# ------------------------------------------------------------------------------------------------
# padding to tile-aligned 4-D shapes and back
# ------------------------------------------------------------------------------------------------
def is_buda_shape(tensor: torch.Tensor, min_dim=-1) -> bool:
    nd = len(tensor.shape)
    if nd > 4 or (nd < min_dim if min_dim > 0 else nd != 4):
        return False
    return tensor.shape[-1] % TILE_DIM == 0 and tensor.shape[-2] % TILE_DIM == 0


class TilePadding:
    """What stands between a torch tensor and the 4-D tile-aligned shape a queue takes: the tensor viewed in 4-D (with
    the microbatch dimension broadcast if it was missing), how many rows / columns of padding the last two dims need,
    and whether that padding repeats the single row / column (a tile-broadcast dim) instead of being zero.  The host
    path materialises it (pad_pytorch_tensor_to_buda); a push to a device queue hands it to the pack kernel instead,
    which pads while it reads."""

    __slots__ = ("view", "pad_r", "pad_c", "rep_r", "rep_c")

    def __init__(self, tensor: torch.Tensor, tile_broadcast_dims, squeeze: bool, microbatch: int, tile_r: int, tile_c: int):
        if tensor.dim() == 0:
            tensor = tensor.reshape(1)                      # a scalar pads like a one-element vector
        rank = 2 if (squeeze and tensor.dim() > 2 and tensor.shape[0] != microbatch) else 4
        if is_buda_shape(tensor, rank):
            self.view, self.pad_r, self.pad_c, self.rep_r, self.rep_c = tensor, 0, 0, False, False
            return
        v = tensor
        while v.dim() < rank:
            v = v.unsqueeze(1 if v.shape[0] == microbatch else 0)
        while v.dim() > 5:
            assert v.shape[0] == 1, "only leading dimensions of size 1 can be dropped"
            v = v.squeeze(0)
        if v.shape[0] < microbatch:
            v = v.broadcast_to([microbatch, *v.shape[1:]])
        self.view = v
        dims = set(d % 4 for d in tile_broadcast_dims) if tile_broadcast_dims else set()
        self.rep_r, self.rep_c = 2 in dims, 3 in dims
        if self.rep_r:
            assert v.shape[-2] == 1, "a tile-broadcast dimension must have size 1"
        if self.rep_c:
            assert v.shape[-1] == 1, "a tile-broadcast dimension must have size 1"
        self.pad_r, self.pad_c = (-v.shape[-2]) % tile_r, (-v.shape[-1]) % tile_c

    @property
    def aligned(self) -> bool:
        return self.pad_r == 0 and self.pad_c == 0

    def padded_shape(self):
        return (*self.view.shape[:-2], self.view.shape[-2] + self.pad_r, self.view.shape[-1] + self.pad_c)

    def materialise(self) -> torch.Tensor:
        v = self.view
        if self.aligned:
            return v.detach().contiguous()
        out = torch.zeros(self.padded_shape(), dtype=v.dtype, device=v.device)
        rows, cols = v.shape[-2], v.shape[-1]
        # columns first, then rows: a repeated row carries the (zero or repeated) column padding with it
        out[..., :rows, :cols] = v.detach()
        if self.rep_c:
            out[..., :rows, :] = v.detach()
        if self.rep_r:
            out[..., :, :] = out[..., :1, :].clone()
        return out


def pad_pytorch_tensor_to_buda(tensor: torch.Tensor, tile_broadcast_dims: List[int], squeeze: bool = False, microbatch=1,
                               tile_r=TILE_DIM, tile_c=TILE_DIM) -> torch.Tensor:
    """Pad a torch tensor to 4-D with rows / columns rounded up to the tile.  Dims listed in
    tile_broadcast_dims (size 1) are replicated across the tile instead of zero padded."""
    plan = TilePadding(tensor, tile_broadcast_dims, squeeze, microbatch, tile_r, tile_c)
    if plan.view is tensor and plan.aligned:
        return tensor
    out = plan.materialise()
    if out.is_floating_point():
        out.requires_grad = tensor.requires_grad
    return out


def narrow_buda_tensor_to_pytorch(tensor: torch.Tensor, shape: List[int], has_microbatch_dim: bool = False) -> torch.Tensor:
    """Undo pad_pytorch_tensor_to_buda: cut the tile padding off and reshape to `shape`."""
    shape = tuple(shape)
    if len(shape) == 0:  # a scalar that was padded to one tile
        return tensor.narrow(-1, 0, 1).narrow(-2, 0, 1).squeeze()
    out = tensor
    if len(shape) == 1:  # a vector that was padded to tiles
        if out.dim() == 1:
            out = out.narrow(0, 0, shape[0])
        elif out.dim() > 2 and out.shape[0] == shape[0]:
            out = out.narrow(-1, 0, 1).narrow(-2, 0, 1)
        else:
            out = out.narrow(-1, 0, shape[0]).narrow(-2, 0, 1)
    elif reduce(mul, shape, 1) != reduce(mul, out.shape, 1):
        # z may have been swapped with r by a transform attached upstream: narrow in that frame
        swap = out.dim() == 4 and len(shape) == 4 and out.shape[-3] != shape[-3]
        if swap:
            out = out.transpose(-3, -2)
        inner = shape[1:] if has_microbatch_dim else shape
        out = out.narrow(-2, 0, 1 if len(inner) == 1 else inner[-2])
        out = out.narrow(-1, 0, inner[-1])
        if swap:
            out = out.transpose(-3, -2)
    return out.reshape(shape)


def change_rank(tensor: torch.Tensor, rank: int):
    while tensor.dim() > rank:
        assert tensor.shape[0] == 1
        tensor = tensor.select(0, 0)
    while tensor.dim() < rank:
        tensor = tensor.unsqueeze(0)
    return tensor


# ------------------------------------------------------------------------------------------------
# Tensor wrappers
# ------------------------------------------------------------------------------------------------
class Tensor:
    """A tensor on its way to or from a device queue: a torch value plus the device data format."""

    def __init__(self):
        self.src_layer = None

    def set_src_layer(self, layer: str):
        self.src_layer = layer
        return self

    def to_pytorch(self) -> torch.Tensor:
        return self.value()

    def has_value(self) -> bool:
        raise RuntimeError("Children should override")

    def value(self) -> torch.Tensor:
        raise RuntimeError("Children should override")

    def is_constant(self) -> bool:
        return False

    def __repr__(self):
        if self.has_value():
            return f"Buda Tensor: {self.value()}, {self.data_format}"
        return f"Buda Empty Tensor: {self.shape}"

    @classmethod
    def create_from_torch(cls, torch_tensor: torch.Tensor, dev_data_format: Optional[DataFormat] = None,
                          constant: bool = False) -> "TensorFromPytorch":
        return TensorFromPytorch(torch_tensor, dev_data_format, constant)

    @classmethod
    def create_from_tensor_descriptor(cls, descriptor: "PytorchTensorDesc") -> "TensorFromDescriptor":
        return TensorFromDescriptor(descriptor)


class TensorFromPytorch(Tensor):
    """A torch value tagged with the device data format it is meant for."""

    def __init__(self, torch_tensor: torch.Tensor, dev_data_format: Optional[DataFormat], constant: bool):
        super().__init__()
        self._value, self._constant = torch_tensor, bool(constant)
        self._data_format = pytorch_dtype_to_buda_dataformat(torch_tensor.dtype) if dev_data_format is None else dev_data_format

    # --- what it holds
    def has_value(self) -> bool:
        return True

    def value(self) -> torch.Tensor:
        return self._value

    def is_constant(self) -> bool:
        return self._constant

    shape = property(lambda self: TensorShape(*self._value.shape))
    pt_data_format = property(lambda self: self._value.dtype)
    data_format = property(lambda self: self._data_format)
    requires_grad = property(lambda self: self._value.requires_grad)

    def set_requires_grad(self, requires_grad: bool):
        self._value.requires_grad = requires_grad

    # --- copies
    def _like(self, value: torch.Tensor, data_format: Optional[DataFormat] = None) -> "Tensor":
        return Tensor.create_from_torch(value, dev_data_format=data_format)

    def clone(self) -> Tensor:
        return self._like(self._value.clone())

    def detach(self) -> Tensor:
        return self._like(self._value.detach())

    def to_format(self, data_format: DataFormat) -> "Tensor":
        """The same values in the torch dtype that `data_format` travels as (bfloat16 for the Bfp*_b formats), tagged
        with it.  Nothing is packed here: tile bytes only come into being when the tensor is pushed."""
        return self._like(self._value.to(buda_dataformat_to_pytorch_dtype(data_format)), data_format)

    # --- on the way to a queue
    def to_tensor_desc(self) -> "PytorchTensorDesc":
        return pytorch_tensor_to_tensor_desc(self._value)

    def to_buda_shape(self, tile_broadcast_dims: List[int], reinterpret_shape: Optional[List[int]] = None, clone: bool = False,
                      squeeze: bool = False, microbatch=1, tile_r=TILE_DIM, tile_c=TILE_DIM) -> "Tensor":
        """This tensor in the 4-D tile-aligned shape the queues take (itself when it already has it)."""
        if reinterpret_shape is None and not clone and is_buda_shape(self._value):
            return self
        value = self._value.clone() if clone else self._value
        if reinterpret_shape is not None:
            dims = list(reinterpret_shape)
            dims[0] = microbatch if dims[0] == 1 else dims[0]
            value = value.view(dims)
        return self._like(pad_pytorch_tensor_to_buda(value, tile_broadcast_dims, squeeze, microbatch, tile_r, tile_c))


class TensorFromDescriptor(Tensor):
    """Tensor wrapper around a descriptor returned by the backend (e.g. by get_output)."""

    def __init__(self, descriptor: "PytorchTensorDesc"):
        super().__init__()
        self.descriptor = descriptor
        self.requires_grad = False

    def clone(self) -> "TensorFromPytorch":
        return Tensor.create_from_torch(self.value(clone=True))

    def has_value(self) -> bool:
        return True

    def value(self, clone=False) -> torch.Tensor:
        t = tensor_desc_to_pytorch_tensor(self.descriptor)
        return t.clone() if clone else t

    def to_buda_shape(self) -> "Tensor":
        raise RuntimeError("Tensor descriptor should not be converted to buda shape")

    def to_tensor_desc(self) -> "PytorchTensorDesc":
        return self.descriptor

    def narrow_to_original_shape(self, original_shape: Tuple[int, ...], reinterpret_shape: Optional[Tuple[int, ...]] = None,
                                 has_microbatch_dim: bool = False, unpadded_shape: Optional[Tuple[int, ...]] = None) -> "Tensor":
        """Cut the tile padding off a read-back tensor and give it its original shape."""
        assert type(original_shape) == tuple, "original_shape must be a tuple"
        tensor = self.value()
        reinterpret = reinterpret_shape if reinterpret_shape else None
        if reinterpret is None and self.shape.get_pytorch_shape() == original_shape:
            return Tensor.create_from_torch(tensor)
        target = original_shape if reinterpret is None else tuple(reinterpret)
        if len(target) > 1:
            new_shape = (*target[:-2], target[-2], target[-1])
        else:
            new_shape = (target[-1],)
        narrowed = narrow_buda_tensor_to_pytorch(tensor, new_shape, has_microbatch_dim=has_microbatch_dim)
        return Tensor.create_from_torch(narrowed.reshape(original_shape))

    @property
    def pt_data_format(self) -> torch.dtype:
        return buda_dataformat_to_pytorch_dtype(self.descriptor.format)

    @property
    def data_format(self) -> DataFormat:
        return self.descriptor.format

    def to_format(self, data_format: DataFormat) -> "Tensor":
        t = self.value().type(buda_dataformat_to_pytorch_dtype(data_format))
        t.requires_grad = self.requires_grad
        return Tensor.create_from_torch(t, dev_data_format=data_format)

    @property
    def shape(self):
        return TensorShape(*self.descriptor.shape)


def to_pt_tensors(tensors, convert_format: bool = False) -> Tuple[torch.Tensor, ...]:
    """torch tensors out of a mix of torch tensors and Tensor wrappers."""
    if not isinstance(tensors, (list, tuple)):
        tensors = (tensors,)
    out = []
    for t in tensors:
        if isinstance(t, torch.Tensor):
            out.append(t)
        elif isinstance(t, Tensor):
            v = t.value()
            out.append(v.type(buda_dataformat_to_pytorch_dtype(t.data_format)) if convert_format else v)
        else:
            raise RuntimeError(f"Unsupported tensor type {type(t)}")
    return tuple(out)


def to_buda_tensors(tensors) -> Tuple[Tensor, ...]:
    return tuple(t if isinstance(t, Tensor) else Tensor.create_from_torch(t) for t in tensors)


# ------------------------------------------------------------------------------------------------
# Runtime tensor transforms: what the host does to an input right before it is pushed
# (reference: pybuda/pybuda/tensor.py:1382-1447; the transform record is bound from C++ at
# pybuda/csrc/graph_lib/python_bindings.cpp:317-371 — the graph library is not part of this path, so the
# record is a plain Python class with the same field names and JSON form).
# ------------------------------------------------------------------------------------------------
import json
from enum import Enum


def align_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


class RuntimeTensorTransformType(Enum):
    NoTransform = 0
    ReinterpretShape = 1
    Prestride = 2
    EmbeddingIndex = 3
    ConstantInput = 4
    Unpad = 5
    Concatenate = 6


class RuntimeTensorTransform:
    def __init__(self, type=RuntimeTensorTransformType.NoTransform, original_shape=(), reinterpreted_shape=(), unpadded_shape=(),
                 stride_height=1, stride_width=1, kernel_height=1, kernel_width=1):
        self.type = type
        self.original_shape = TensorShape(*original_shape)
        self.reinterpreted_shape = TensorShape(*reinterpreted_shape)
        self.unpadded_shape = TensorShape(*unpadded_shape)
        self.stride_height, self.stride_width = stride_height, stride_width
        self.kernel_height, self.kernel_width = kernel_height, kernel_width

    def to_json(self):
        return {"type": self.type.name, "original_shape": list(self.original_shape.dims),
                "reinterpreted_shape": list(self.reinterpreted_shape.dims), "unpadded_shape": list(self.unpadded_shape.dims),
                "stride_height": self.stride_height, "stride_width": self.stride_width,
                "kernel_height": self.kernel_height, "kernel_width": self.kernel_width}

    @classmethod
    def from_json(cls, j):
        return cls(RuntimeTensorTransformType[j["type"]], j.get("original_shape", ()), j.get("reinterpreted_shape", ()),
                   j.get("unpadded_shape", ()), j.get("stride_height", 1), j.get("stride_width", 1), j.get("kernel_height", 1),
                   j.get("kernel_width", 1))

    def __repr__(self):
        return f"RuntimeTensorTransform({self.to_json()})"


def embedding_index_layout(count: int, length: int, queue_tile_rows: int):
    """Geometry of an embedding-index push: `length` indices per entry (of which the first `count` are real), dealt
    evenly over the queue's tile rows.  Returns (indices per tile row, tile columns): every 32x32 tile holds 1024
    consecutive indices, so a tile row needs ceil(group / 1024) tile columns."""
    padded = align_up(length, TILE_DIM)
    assert padded % (queue_tile_rows * TILE_DIM) == 0, "the padded index vector must split evenly over the queue's tile rows"
    group = padded // queue_tile_rows
    return group, align_up(group // TILE_DIM, TILE_DIM) // TILE_DIM


def _embedding_index(tensor: torch.Tensor, original_shape: Tuple[int, ...], queue: DramIODesc):
    """Host form of the embedding-index transform (what the pack kernel's embedding view produces on the device):
    out[w, 0, g*32 + i, j*32 + k] = index[w, g*group + (j*32 + i)*32 + k]; all ones from position original_shape[-1]
    on, zero where (j*32 + i)*32 reaches past the group."""
    assert queue.data_format in (DataFormat.RawUInt8, DataFormat.RawUInt16, DataFormat.RawUInt32), "indices travel in a raw integer queue"
    assert tensor.dim() <= 2 and all(d == 1 for d in tuple(original_shape)[:-1][-2:]), "embedding indices form a vector"
    idx = tensor.reshape(-1, tensor.shape[-1])
    w, length = idx.shape
    q_rt = queue.bufq_grid_dim_r * queue.mblock_m * queue.ublock_rt
    group, ct = embedding_index_layout(original_shape[-1], length, q_rt)
    r = torch.arange(q_rt * TILE_DIM).unsqueeze(1)
    c = torch.arange(ct * TILE_DIM).unsqueeze(0)
    a = (c // TILE_DIM) * TILE_DIM + r % TILE_DIM
    flat = (r // TILE_DIM) * group + a * TILE_DIM + c % TILE_DIM
    ones = torch.tensor(-1, dtype=idx.dtype)
    src = torch.cat([idx, torch.zeros(w, 1, dtype=idx.dtype)], dim=1)                 # one spare slot to gather from
    out = src[:, flat.clamp(max=length - 1)]
    out = torch.where(flat >= original_shape[-1], ones, out)
    out = torch.where(a * TILE_DIM >= group, torch.zeros((), dtype=idx.dtype), out)
    out = out.reshape(w, 1, q_rt * TILE_DIM, ct * TILE_DIM)
    assert out.shape[1] == queue.t and out.shape[3] == queue.bufq_grid_dim_c * queue.mblock_n * queue.ublock_ct * TILE_DIM, \
        "the index layout does not match the queue's geometry"
    return out


def _reinterpret_shape(tensor: torch.Tensor, shape: List[int], queue: DramIODesc, tile_bcast_dims: List[int]):
    """The tensor's elements read in the shape the compiled graph expects, padded to the queue's tiles."""
    reshaped = tensor.contiguous().view(shape)
    return pad_pytorch_tensor_to_buda(reshaped, tile_bcast_dims, squeeze=True, microbatch=queue.input_count,
                                      tile_r=queue.tile_height, tile_c=queue.tile_width), queue


def _prestride_shape(tensor: torch.Tensor, stride_height: int, stride_width: int, queue: DramIODesc):
    """Nothing happens to the tensor here: the queue gets a stride descriptor (all stride x stride phase offsets, row
    by row) and push_input stores the activation in its prestrided form."""
    assert stride_height == stride_width, "prestriding works with square strides only"
    desc = StrideDescriptor()
    desc.stride = stride_height
    desc.xy_offsets = [(k % stride_width, k // stride_width) for k in range(stride_height * stride_width)]
    queue.s_descriptor = desc
    return tensor, queue


def do_runtime_transform(transform, tensor, q, tile_bcast_dims):
    kind = transform.type
    if kind == RuntimeTensorTransformType.NoTransform:
        return tensor, q
    if kind == RuntimeTensorTransformType.EmbeddingIndex:
        return _embedding_index(tensor, transform.original_shape.dims, q), q
    if kind == RuntimeTensorTransformType.ReinterpretShape:
        return _reinterpret_shape(tensor, list(transform.reinterpreted_shape.dims), q, tile_bcast_dims)
    if kind == RuntimeTensorTransformType.Prestride:
        return _prestride_shape(tensor, transform.stride_height, transform.stride_width, q)
    raise AssertionError(f"Unsupported runtime transform type: {kind}")


def eval_runtime_transform(transform, inp, q, tile_bcast_dims):
    if isinstance(transform, str):
        transform = RuntimeTensorTransform.from_json(json.loads(transform))
    return do_runtime_transform(transform, inp, q, tile_bcast_dims)
