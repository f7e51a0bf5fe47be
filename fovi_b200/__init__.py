"""fovi_b200: the foveated hot path of nblauch/fovi (sensor grid-sample + KNNConv) as
hand-written CUDA kernels for NVIDIA B200 (sm_100a) behind a C ABI.

``fovi_b200.build`` compiles the native library; every other submodule loads
``libfovi_b200.so`` on import and raises if it is missing or stale — there is no CPU or PyTorch
fallback.  Submodules are imported lazily so that the build recipe can run before the library
exists.
"""
import importlib

__version__ = "0.1"
_LAZY = ("ops", "sensing", "knn", "alexnet", "tables", "policies", "pipeline", "coords", "dist", "build", "_lib")


def __getattr__(name):
    if name in _LAZY:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
