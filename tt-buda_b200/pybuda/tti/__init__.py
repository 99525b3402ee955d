"""Tensor side of the device-image archive: tensors written as .pkl / .bin / .tbin files beside a JSON
descriptor, loaded lazily (reference: pybuda/pybuda/tti/archive.py)."""
from .archive import (TTDeviceImageJsonDecoder, TTDeviceImageJsonEncoder, load_tensor_from_disk, load_tensor_archive,
                      save_tensor_archive)
from .utils import compute_file_checksum, read_checksum_from_file, write_checksum_to_file
