"""deepx_b200 — B200 (sm_100a) executor for the deepxIR op hot path.

Layers, bottom up:
  * ``libdeepx_b200.so``   hand-written CUDA kernels behind a C ABI (include/dx_kernels.h)
  * ``tensorfunc``         the reference's tensorfunc interface (same names, argument
                           meaning, error behaviour) over that ABI, on CUDA tensors
  * ``executor``           the deepxIR text boundary: parser, op registry, tensor store
  * ``sharded``            axis-0 sharding across the GPUs of one node
"""
from . import _native  # noqa: F401  (fails loudly when the CUDA library is missing)

__all__ = ["_native"]
