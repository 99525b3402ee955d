"""A module parameter as the data-format path sees it (reference: pybuda/pybuda/parameter.py:20-240): a named torch
value with a device data format; set_data_format casts the value to the torch dtype that feeds that format
(Bfp*_b and Float16_b travel as bfloat16, Bfp* "a" and Float16 as float16: tensor.py:602-632)."""
from typing import Optional

import torch

from ._C import DataFormat
from .tensor import buda_dataformat_to_pytorch_dtype, pytorch_dtype_to_buda_dataformat


class Parameter:
    def __init__(self, *args, requires_grad: bool = True, name: Optional[str] = None, dev_data_format: Optional[DataFormat] = None):
        self._name = name
        self.requires_grad = requires_grad
        self._value = None
        self._data_format = dev_data_format
        if len(args) == 1 and isinstance(args[0], torch.Tensor):
            self._value = args[0]
            if self._data_format is None:
                self._data_format = pytorch_dtype_to_buda_dataformat(self._value.dtype)

    def get_name(self) -> str:
        return self._name

    def value(self) -> torch.Tensor:
        return self._value

    def set_value(self, value: torch.Tensor):
        self._value = value.type(self.pt_data_format) if self._data_format is not None else value

    @property
    def data_format(self) -> DataFormat:
        assert self._data_format is not None, "No data type set for parameter yet"
        return self._data_format

    @property
    def pt_data_format(self) -> torch.dtype:
        assert self._data_format is not None, "No data type set for parameter yet"
        return buda_dataformat_to_pytorch_dtype(self._data_format)

    def set_data_format(self, df: DataFormat):
        self._data_format = df
        if self._value is not None:
            self._value = self._value.type(buda_dataformat_to_pytorch_dtype(df))

    @classmethod
    def create_from_torch(cls, torch_tensor: torch.Tensor) -> "Parameter":
        return cls(torch_tensor, requires_grad=torch_tensor.requires_grad)
