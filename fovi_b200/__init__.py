"""fovi_b200: the foveated hot path of nblauch/fovi (sensor grid-sample + KNNConv) as
hand-written CUDA kernels for NVIDIA B200 (sm_100a) behind a C ABI.

Importing the package loads ``libfovi_b200.so``; it raises if the library has not been built.
"""
from . import _lib  # noqa: F401  (fails loudly when the native library is missing)
from . import ops  # noqa: F401

__version__ = "0.1"
