"""deepx_b200 — B200 (sm_100a) executor for the deepxIR op hot path.

Layers, bottom up:
  * ``libdeepx_b200.so``   hand-written CUDA kernels behind a C ABI (include/dx_kernels.h)
  * ``tensorfunc``         the reference's tensorfunc interface (same names, argument
                           meaning, error behaviour) over that ABI, on CUDA tensors
  * ``executor``           the deepxIR text boundary: parser, op registry, tensor store
  * ``sharded``            axis-0 sharding across the GPUs of one node

Submodules load on first use (``deepx_b200.build`` must be importable before the native
library exists).  ``_native`` raises, with the build command, when the library is missing:
there is no CPU fallback.
"""
import importlib

_SUBMODULES = ("_native", "tensorfunc", "executor", "sharded", "build")


def __getattr__(name):
    if name in _SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
