"""thunderkittens_b200 — B200 (sm_100a) kernels for the quantized-inference path of ThunderKittens.

The product is the C-ABI shared library `libtkb200.so` (include/tkb200.h), built in-tree from
`csrc/`.  `ops` mirrors the reference's pybind entry points on top of it for torch callers.
Importing this package does not load the library; the first call does, and raises if it is absent.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib", "ops"]


def __getattr__(name):
    if name == "ops":
        import importlib
        return importlib.import_module(".ops", __name__)
    raise AttributeError(name)
