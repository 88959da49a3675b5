"""ctypes front of oracle/_ref/libdeepx_ref_cuda.so — TEST INFRASTRUCTURE, NOT PRODUCT.

The library holds the reference's own CUDA kernels (executor/op-cuda/src/deepx/tensorfunc/*.cu,
compiled where they lie by oracle/Makefile) behind the small C harness of ref_cuda_harness.cu.
It exists only where the reference tree was present at build time; ``load()`` returns None
otherwise.  Used by the GPU parity tests to pin the CPU oracle to code the reference holds, and
by bench.py's baseline legs to time the reference's kernels as they are today.  All calls are
synchronous and run on the default stream, as the reference's launch wrappers do.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "_ref" / "libdeepx_ref_cuda.so"
_lib = None


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        return None
    lib = C.CDLL(str(LIB_PATH))
    vp, i64p, i32p = C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int32)
    lib.refcu_last_error.restype = C.c_char_p
    lib.refcu_binary.argtypes = [C.c_int, C.c_int, vp, vp, vp, C.c_int]
    lib.refcu_scalar.argtypes = [C.c_int, C.c_int, vp, C.c_double, C.c_int64, vp, C.c_int]
    lib.refcu_unary.argtypes = [C.c_int, C.c_int, vp, vp, C.c_int]
    lib.refcu_compare.argtypes = [C.c_int, C.c_int, vp, vp, C.c_float, vp, C.c_int]
    lib.refcu_compare_scalar.argtypes = [C.c_int, C.c_int, vp, C.c_double, C.c_int64, C.c_float, vp, C.c_int]
    lib.refcu_switch.argtypes = [C.c_int, C.POINTER(vp), C.c_int, C.c_int, vp, vp, C.c_int]
    lib.refcu_cast.argtypes = [C.c_int, vp, C.c_int, vp, C.c_int]
    lib.refcu_sum.argtypes = [C.c_int, vp, i64p, C.c_int, i32p, C.c_int, C.c_int, vp]
    lib.refcu_transpose.argtypes = [C.c_int, vp, i64p, C.c_int, i32p, vp]
    lib.refcu_broadcast_to.argtypes = [C.c_int, vp, i64p, C.c_int, i64p, C.c_int, vp]
    lib.refcu_indexselect.argtypes = [C.c_int, vp, i64p, C.c_int, C.c_int, vp, i64p, C.c_int, C.c_int, vp]
    lib.refcu_matmul.argtypes = [C.c_int, vp, vp, vp, i64p, i64p, C.c_int]
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError("reference op-cuda: " + _lib.refcu_last_error().decode())


def i64(v):
    v = [int(x) for x in v]
    return (C.c_int64 * max(len(v), 1))(*v)


def i32(v):
    v = [int(x) for x in v]
    return (C.c_int32 * max(len(v), 1))(*v)
