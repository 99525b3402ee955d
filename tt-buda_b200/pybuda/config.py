"""The one piece of the reference's configuration module this path needs: the on-disk tensor formats
of a device image (reference: pybuda/pybuda/config.py:121-144)."""
from enum import Enum


class TTIDumpFormat(Enum):
    """How tensors of a device image are written: pickled torch tensors, raw row-major bytes (.bin),
    or the queue's own tilized bytes (.tbin) that can be pushed without conversion."""
    DEFAULT = "DEFAULT"
    BACKEND = "BACKEND"
    BACKEND_TILIZED = "BACKEND_TILIZED"

    def extension(self) -> str:
        return {TTIDumpFormat.DEFAULT: "pkl", TTIDumpFormat.BACKEND: "bin", TTIDumpFormat.BACKEND_TILIZED: "tbin"}[self]

    @classmethod
    def to_json(cls, value):
        return value.name

    @classmethod
    def from_json(cls, value):
        return cls[value.upper()]
