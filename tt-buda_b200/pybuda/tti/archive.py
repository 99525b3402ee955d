"""Tensors of a device image on disk (reference: pybuda/pybuda/tti/archive.py:52-66 load_tensor_from_disk,
:69-148 TTDeviceImageJsonEncoder, :186-260 TTDeviceImageJsonDecoder).

Each tensor becomes one file under tensors/ and one JSON entry:
    .pkl   pickled torch tensor                                   (TTIDumpFormat.DEFAULT)
    .bin   raw row-major bytes + {itemsize, shape, strides, dim, format}   (BACKEND)
    .tbin  the queue's tilized bytes, packed on the GPU by tilize_tensor,
           + {format, num_buffers, buf_size_bytes}                 (BACKEND_TILIZED)
A .tbin loads back as a TilizedTensorDesc that push_input copies into the device queue as is, so
weights are converted once, not on every start.  Loading is lazy: the JSON entry turns into a callable
that reads the file when called.  The reference asks the compiled netlist for a tensor's queue
descriptor; there is no netlist here, so the caller passes a {name: DramIODesc} table.
"""
import functools
import json
import os
import pickle
from collections.abc import Iterable
from typing import Callable, Dict, Optional

import torch

from pybuda._C import DataFormat
from pybuda._C.backend_api import (BackendStatusCode, DramIODesc, PytorchTensorDesc, TilizedTensorDesc, binarize_tensor,
                                   debinarize_tensor, free_tensor, tilize_tensor)
from pybuda.config import TTIDumpFormat
from pybuda.tensor import pytorch_tensor_to_tensor_desc

from .utils import compute_file_checksum, read_checksum_from_file, write_checksum_to_file

DESCRIPTOR_FILE = "device_image.json"


def _ok(status, what):
    if status != BackendStatusCode.Success:
        raise RuntimeError(f"{what} failed with {status}")


def load_tensor_from_disk(filepath, value):
    """JSON entry + file -> TilizedTensorDesc (.tbin) or PytorchTensorDesc (.bin); backend-owned memory,
    released with free_tensor."""
    if filepath.endswith(TTIDumpFormat.BACKEND_TILIZED.extension()):
        desc = TilizedTensorDesc()
        desc.format = DataFormat.from_json(value["format"])
        desc.num_buffers = value["num_buffers"]
        desc.buf_size_bytes = value["buf_size_bytes"]
    else:
        desc = PytorchTensorDesc()
        desc.itemsize = value["itemsize"]
        desc.format = DataFormat.from_json(value["format"])
        desc.shape = value["shape"]
        desc.strides = value["strides"]
        if "dim" in value:
            desc.dim = value["dim"]
    _ok(debinarize_tensor(desc, filepath), f"debinarize_tensor({filepath})")
    return desc


class TTDeviceImageJsonEncoder(json.JSONEncoder):
    @staticmethod
    def encode_descriptor(filename: str, tensor_desc: PytorchTensorDesc, tilized_tensor_desc: Optional[TilizedTensorDesc] = None):
        encoding = {
            "bin": filename,
            "itemsize": tensor_desc.itemsize,
            "shape": list(tensor_desc.shape),
            "strides": list(tensor_desc.strides),
            "dim": tensor_desc.dim,
            "format": tensor_desc.format,
        }
        if tilized_tensor_desc:
            encoding.update({
                "format": tilized_tensor_desc.format,
                "num_buffers": tilized_tensor_desc.num_buffers,
                "buf_size_bytes": tilized_tensor_desc.buf_size_bytes,
            })
        return encoding

    @staticmethod
    def rehash_as_pickled_object(d, key, object_value, filename_encoding, base_directory):
        with open(os.path.join(base_directory, filename_encoding), "wb") as pkl_file:
            pickle.dump(object_value, pkl_file, pickle.HIGHEST_PROTOCOL)
        d[key] = filename_encoding

    @staticmethod
    def rehash_tensor_as_pickled_object(d, key, object_value, base_directory):
        filename_encoding = os.path.join("tensors", f"torch.Tensor.{key}.pkl".replace("/", "_"))
        TTDeviceImageJsonEncoder.rehash_as_pickled_object(d, key, object_value, filename_encoding, base_directory)

    @staticmethod
    def rehash_tensor_as_bin_object(d, key, object_value, base_directory, tti_dump_format: TTIDumpFormat,
                                    queue_descriptors: Optional[Dict[str, DramIODesc]] = None):
        filename_encoding = os.path.join("tensors", f"torch.Tensor.{key}.{tti_dump_format.extension()}".replace("/", "_"))
        assert isinstance(object_value, torch.Tensor), "rehash_tensor_as_bin_object expects a torch.Tensor"
        tensor = object_value.contiguous()
        tensor_desc = pytorch_tensor_to_tensor_desc(tensor)
        tilized = None
        if tti_dump_format == TTIDumpFormat.BACKEND_TILIZED:
            if not queue_descriptors or key not in queue_descriptors:
                raise KeyError(f"no queue descriptor for tensor '{key}': a .tbin needs the queue it will be pushed to")
            tilized = tilize_tensor(queue_descriptors[key], tensor_desc)     # packed on the GPU
        path = os.path.join(base_directory, filename_encoding)
        try:
            _ok(binarize_tensor(tilized if tilized else tensor_desc, path), f"binarize_tensor({path})")
            d[key] = TTDeviceImageJsonEncoder.encode_descriptor(filename_encoding, tensor_desc, tilized)
        finally:
            if tilized:
                free_tensor(tilized)

    @staticmethod
    def preprocess_keys(d, base_directory: str, tti_dump_format: Optional[TTIDumpFormat] = None,
                        queue_descriptors: Optional[Dict[str, DramIODesc]] = None):
        """Tensors (and iterables holding tensors) move out to files; dtype keys become strings."""
        for key, value in list(d.items()):
            if not isinstance(key, str) and isinstance(key, torch.dtype):
                d[str(key)] = value
                del d[key]
            elif isinstance(value, torch.Tensor) or (not isinstance(value, (str, dict)) and isinstance(value, Iterable)
                                                     and any(isinstance(v, torch.Tensor) for v in value)):
                use_backend_format = tti_dump_format in (TTIDumpFormat.BACKEND, TTIDumpFormat.BACKEND_TILIZED)
                if use_backend_format and key != "cpueval_outputs" and isinstance(value, torch.Tensor):
                    TTDeviceImageJsonEncoder.rehash_tensor_as_bin_object(d, key, value, base_directory, tti_dump_format,
                                                                         queue_descriptors)
                else:
                    TTDeviceImageJsonEncoder.rehash_tensor_as_pickled_object(d, key, value, base_directory)
            elif isinstance(value, dict):
                d[key] = TTDeviceImageJsonEncoder.preprocess_keys(value, base_directory, tti_dump_format, queue_descriptors)
        return d

    def default(self, obj):
        if hasattr(obj, "to_json"):
            return obj.to_json()
        try:
            return json.JSONEncoder.default(self, obj)
        except TypeError as e:
            raise RuntimeError(f"JSON Serialization failed: {e}. {obj.__class__.__name__}.to_json(..) method needs to be "
                               f"implemented. Object={obj}.")


class TTDeviceImageJsonDecoder(json.JSONDecoder):
    DICT_KEY_DECODING = {"torch.": torch}

    @staticmethod
    def rehash_as_tensor(value, directory) -> Callable:
        """Lazy: the returned callable reads the file when (and every time) it is called."""
        return functools.partial(load_tensor_from_disk, os.path.join(directory, value["bin"]), value)

    @staticmethod
    def postprocess_keys(d, directory):
        for key, value in list(d.items()):
            if isinstance(value, dict):
                if "bin" in value:
                    d[key] = value = TTDeviceImageJsonDecoder.rehash_as_tensor(value, directory)
                else:
                    value = TTDeviceImageJsonDecoder.postprocess_keys(value, directory)
            if isinstance(value, str) and value.endswith(".pkl"):
                with open(os.path.join(directory, value), "rb") as pkl_file:
                    d[key] = value = pickle.load(pkl_file)
            for encoded_string, decoded_type in TTDeviceImageJsonDecoder.DICT_KEY_DECODING.items():
                if isinstance(key, str) and key.startswith(encoded_string):
                    d[getattr(decoded_type, key[len(encoded_string):])] = value
                    del d[key]
        return d


def save_tensor_archive(directory: str, tensors: dict, tti_dump_format: TTIDumpFormat = TTIDumpFormat.BACKEND_TILIZED,
                        queue_descriptors: Optional[Dict[str, DramIODesc]] = None) -> str:
    """Write `tensors` (a possibly nested dict) under `directory`: tensors/<files>, device_image.json and its
    .checksum sidecar.  Returns the descriptor path."""
    os.makedirs(os.path.join(directory, "tensors"), exist_ok=True)
    body = TTDeviceImageJsonEncoder.preprocess_keys(dict(tensors), directory, tti_dump_format, queue_descriptors)
    path = os.path.join(directory, DESCRIPTOR_FILE)
    with open(path, "w") as f:
        json.dump({"tti_dump_format": TTIDumpFormat.to_json(tti_dump_format), "tensors": body}, f, cls=TTDeviceImageJsonEncoder, indent=1)
    write_checksum_to_file(compute_file_checksum(path), path + ".checksum")
    return path


def load_tensor_archive(directory: str, verify_checksum: bool = True) -> dict:
    """The inverse: {name: callable -> descriptor} for .bin/.tbin entries, tensors for .pkl entries."""
    path = os.path.join(directory, DESCRIPTOR_FILE)
    if verify_checksum:
        want = read_checksum_from_file(path + ".checksum")
        if want is not None and want != compute_file_checksum(path):
            raise RuntimeError(f"{path}: checksum mismatch, the archive was modified or truncated")
    with open(path, "r") as f:
        body = json.load(f, cls=TTDeviceImageJsonDecoder)
    return TTDeviceImageJsonDecoder.postprocess_keys(body["tensors"], directory)
