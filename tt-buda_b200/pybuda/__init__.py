"""pybuda: the tensor / data-format conversion surface of TT-Buda, backed by hand-written
sm_100a CUDA kernels (libbuda_cuda.so) behind the reference's backend_api entry points.

Only the data-format path is here: tilize / untilize, Bfp8_b / Bfp4_b / Bfp2_b pack and unpack,
the golden int8 quantise ops and the Bfp8_b-weight matmul.  There is no CPU fallback.
"""
TILE_DIM = 32

# The names of the reference's top-level package that belong to this path (pybuda/pybuda/__init__.py:56-60), resolved
# on first use so that `import pybuda` itself stays free of the compiled modules.
_LAZY = {
    "Parameter": ("parameter", "Parameter"),
    "Tensor": ("tensor", "Tensor"),
    "SomeTensor": ("tensor", "SomeTensor"),
    "TensorShape": ("tensor", "TensorShape"),
    "DataFormat": ("_C", "DataFormat"),
    "MathFidelity": ("_C", "MathFidelity"),
}


def __getattr__(name):
    if name in _LAZY:
        import importlib

        mod, attr = _LAZY[name]
        value = getattr(importlib.import_module(f"{__name__}.{mod}"), attr)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
