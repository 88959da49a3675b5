"""numpy front end of the CPU oracle (``oracle/liboracle.so``) — TEST INFRASTRUCTURE, NOT PRODUCT.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` may
import this module, as the checker or as the timed CPU baseline.  Function names and
argument order follow the reference's tensorfunc interface so a parity test reads
``tensorfunc.add(A, B, C)`` against ``oracle.add(a, b)``.

16-bit floats travel as numpy arrays of ``ml_dtypes.bfloat16`` / ``numpy.float16``.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path
from typing import Sequence

import ml_dtypes
import numpy as np

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "liboracle.so"
REF_LIB_PATH = _HERE / "_ref" / "libdeepx_ref.so"

F64, F32, F16, BF16, I64, I32, I16, I8, BOOL = range(9)
ADD, SUB, MUL, DIV, MAX, MIN, POW = range(7)
ADDS, SUBS, RSUBS, MULS, DIVS, RDIVS, MAXS, MINS, POWS, RPOWS = range(10)
SQRT, LOG, EXP, SIN, COS, TAN, INVERT = range(7)
EQ, NE, LT, GT = range(4)
SUM, PROD, RMAX, RMIN = range(4)

bfloat16 = ml_dtypes.bfloat16

_NP2DX = {
    np.dtype(np.float64): F64, np.dtype(np.float32): F32, np.dtype(np.float16): F16, np.dtype(bfloat16): BF16,
    np.dtype(np.int64): I64, np.dtype(np.int32): I32, np.dtype(np.int16): I16, np.dtype(np.int8): I8,
    np.dtype(np.bool_): BOOL,
}
DX2NP = {v: k for k, v in _NP2DX.items()}


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference harness when the reference tree is present)."""
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < (_HERE / "oracle.cpp").stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "liboracle.so"], check=True, capture_output=True)
    subprocess.run(["make", "-C", str(_HERE), "ref"], check=False, capture_output=True)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        _lib = C.CDLL(str(LIB_PATH))
    return _lib


def code(a: np.ndarray) -> int:
    return _NP2DX[a.dtype]


def _p(a: np.ndarray) -> C.c_void_p:
    return C.c_void_p(a.ctypes.data)


def _i64(v) -> C.Array:
    vals = [int(x) for x in v]
    return (C.c_int64 * (len(vals) or 1))(*vals)


def _i32(v) -> C.Array:
    vals = [int(x) for x in v]
    return (C.c_int32 * (len(vals) or 1))(*vals)


def _ck(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"oracle {what} failed with status {rc}")


def _c(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a)


def _fs_is(dtype, value) -> tuple[float, int]:
    if np.dtype(dtype).kind == "f" or np.dtype(dtype) == np.dtype(bfloat16):
        return float(value), 0
    return 0.0, int(value)


# ---- elementwise -----------------------------------------------------------------------------
def binary(op: int, a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a, b = _c(a), _c(b)
    assert a.shape == b.shape and a.dtype == b.dtype
    out = np.empty_like(a)
    _ck(lib().orc_ew_binary(op, code(a), _p(a), _p(b), _p(out), C.c_int64(a.size)), "ew_binary")
    return out


def add(a, b): return binary(ADD, a, b)
def sub(a, b): return binary(SUB, a, b)
def mul(a, b): return binary(MUL, a, b)
def div(a, b): return binary(DIV, a, b)
def max(a, b): return binary(MAX, a, b)  # noqa: A001
def min(a, b): return binary(MIN, a, b)  # noqa: A001
def pow(a, b): return binary(POW, a, b)  # noqa: A001


def scalar(op: int, a: np.ndarray, value) -> np.ndarray:
    a = _c(a)
    out = np.empty_like(a)
    fs, is_ = _fs_is(a.dtype, value)
    _ck(lib().orc_ew_scalar(op, code(a), _p(a), C.c_double(fs), C.c_int64(is_), _p(out), C.c_int64(a.size)), "ew_scalar")
    return out


def addscalar(a, v): return scalar(ADDS, a, v)
def subscalar(a, v): return scalar(SUBS, a, v)
def rsubscalar(v, a): return scalar(RSUBS, a, v)
def mulscalar(a, v): return scalar(MULS, a, v)
def divscalar(a, v): return scalar(DIVS, a, v)
def rdivscalar(v, a): return scalar(RDIVS, a, v)
def maxscalar(a, v): return scalar(MAXS, a, v)
def minscalar(a, v): return scalar(MINS, a, v)
def powscalar(a, v): return scalar(POWS, a, v)
def rpowscalar(v, a): return scalar(RPOWS, a, v)


def unary(op: int, a: np.ndarray) -> np.ndarray:
    a = _c(a)
    out = np.empty_like(a)
    _ck(lib().orc_ew_unary(op, code(a), _p(a), _p(out), C.c_int64(a.size)), "ew_unary")
    return out


def sqrt(a): return unary(SQRT, a)
def log(a): return unary(LOG, a)
def exp(a): return unary(EXP, a)
def sin(a): return unary(SIN, a)
def cos(a): return unary(COS, a)
def tan(a): return unary(TAN, a)
def invert(a): return unary(INVERT, a)


def compare(op: int, a: np.ndarray, b: np.ndarray, epsilon: float = 0.0) -> np.ndarray:
    a, b = _c(a), _c(b)
    assert a.shape == b.shape and a.dtype == b.dtype
    out = np.empty(a.shape, dtype=np.bool_)
    _ck(lib().orc_ew_compare(op, code(a), _p(a), _p(b), C.c_float(epsilon), _p(out), C.c_int64(a.size)), "ew_compare")
    return out


def compare_scalar(op: int, a: np.ndarray, value, epsilon: float = 0.0) -> np.ndarray:
    a = _c(a)
    out = np.empty(a.shape, dtype=np.bool_)
    fs, is_ = _fs_is(a.dtype, value)
    _ck(lib().orc_ew_compare_scalar(op, code(a), _p(a), C.c_double(fs), C.c_int64(is_), C.c_float(epsilon), _p(out),
                                    C.c_int64(a.size)), "ew_compare_scalar")
    return out


def equal(a, b, eps=0.0): return compare(EQ, a, b, eps)
def notequal(a, b, eps=0.0): return compare(NE, a, b, eps)
def less(a, b): return compare(LT, a, b)
def greater(a, b): return compare(GT, a, b)
def equalscalar(a, v, eps=0.0): return compare_scalar(EQ, a, v, eps)
def notequalscalar(a, v, eps=0.0): return compare_scalar(NE, a, v, eps)
def lessscalar(a, v): return compare_scalar(LT, a, v)
def greaterscalar(a, v): return compare_scalar(GT, a, v)


def Switch(tensors: Sequence[np.ndarray], cases: np.ndarray) -> np.ndarray:
    ts = [_c(t) for t in tensors]
    cases = _c(cases)
    out = np.empty_like(ts[0])
    ptrs = (C.c_void_p * len(ts))(*[t.ctypes.data for t in ts])
    _ck(lib().orc_switch(code(ts[0]), ptrs, len(ts), code(cases), _p(cases), _p(out), C.c_int64(out.size)), "switch")
    return out


def todtype(a: np.ndarray, dst_dtype) -> np.ndarray:
    a = _c(a)
    out = np.empty(a.shape, dtype=dst_dtype)
    _ck(lib().orc_cast(code(a), _p(a), code(out), _p(out), C.c_int64(a.size)), "cast")
    return out


# ---- reduce -------------------------------------------------------------------------------------
def checked_dims(shape, dims) -> list[int]:
    n = len(shape)
    if len(dims) == 0:
        return list(range(n))
    out = []
    for d in dims:
        d = int(d)
        if d < 0:
            d += n
        if d >= n or d < 0:
            raise ValueError("Dimension out of range")
        out.append(d)
    return sorted(set(out))


def reduced_shape(shape, dims, keepdims) -> list[int]:
    red = set(dims)
    out = []
    for i, s in enumerate(shape):
        if i not in red:
            out.append(int(s))
        elif keepdims:
            out.append(1)
    return out or [1]


def reduce(op: int, a: np.ndarray, dims, keepdims: bool = False) -> np.ndarray:
    a = _c(a)
    cd = checked_dims(a.shape, dims)
    out = np.empty(reduced_shape(a.shape, cd, keepdims), dtype=a.dtype)
    _ck(lib().orc_reduce(op, code(a), _p(a), _i64(a.shape), a.ndim, _i32(cd), len(cd), _p(out)), "reduce")
    return out


def sum(a, dims, keepdims=False): return reduce(SUM, a, dims, keepdims)  # noqa: A001
def prod(a, dims, keepdims=False): return reduce(PROD, a, dims, keepdims)
def reducemax(a, dims, keepdims=False): return reduce(RMAX, a, dims, keepdims)
def reducemin(a, dims, keepdims=False): return reduce(RMIN, a, dims, keepdims)


def reduce_all_parallel(op: int, a: np.ndarray) -> np.ndarray:
    """Whole-array reduce split over all host threads (for the timed CPU baseline)."""
    a = _c(a)
    out = np.empty((1,), dtype=a.dtype)
    _ck(lib().orc_reduce_all_parallel(op, code(a), _p(a), C.c_int64(a.size), _p(out)), "reduce_all_parallel")
    return out


# ---- changeshape -----------------------------------------------------------------------------------
def transpose(a: np.ndarray, dim_order) -> np.ndarray:
    a = _c(a)
    out = np.empty([a.shape[d] for d in dim_order], dtype=a.dtype)
    _ck(lib().orc_transpose(code(a), _p(a), _i64(a.shape), a.ndim, _i32(dim_order), _p(out)), "transpose")
    return out


def concat(tensors: Sequence[np.ndarray], axis: int) -> np.ndarray:
    ts = [_c(t) for t in tensors]
    oshape = list(ts[0].shape)
    oshape[axis] = int(np.sum([t.shape[axis] for t in ts]))
    out = np.empty(oshape, dtype=ts[0].dtype)
    ptrs = (C.c_void_p * len(ts))(*[t.ctypes.data for t in ts])
    _ck(lib().orc_concat(code(out), ptrs, _i64(t.shape[axis] for t in ts), len(ts), _i64(oshape), len(oshape), axis,
                         _p(out)), "concat")
    return out


def broadcastTo(a: np.ndarray, new_shape) -> np.ndarray:
    a = _c(a)
    out = np.empty(list(new_shape), dtype=a.dtype)
    _ck(lib().orc_broadcast_to(code(a), _p(a), _i64(a.shape), a.ndim, _i64(new_shape), len(new_shape), _p(out)),
        "broadcastTo")
    return out


def indexselect(a: np.ndarray, index: np.ndarray, axis: int) -> np.ndarray:
    a, index = _c(a), _c(index)
    g = axis + a.ndim if axis < 0 else axis
    oshape = list(a.shape[:g]) + list(index.shape) + list(a.shape[g + 1:])
    out = np.empty(oshape, dtype=a.dtype)
    _ck(lib().orc_indexselect(code(a), _p(a), _i64(a.shape), a.ndim, code(index), _p(index), _i64(index.shape), index.ndim,
                              g, _p(out)), "indexselect")
    return out


def repeat(a: np.ndarray, repeats) -> np.ndarray:
    a = _c(a)
    out = np.empty([s * int(r) for s, r in zip(a.shape, repeats)], dtype=a.dtype)
    _ck(lib().orc_repeat(code(a), _p(a), _i64(a.shape), a.ndim, _i64(repeats), _p(out)), "repeat")
    return out


def matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a, b = _c(a), _c(b)
    M, K, Nn = a.shape[-2], a.shape[-1], b.shape[-1]
    batch = a.size // (M * K)
    out = np.empty(list(a.shape[:-1]) + [Nn], dtype=a.dtype)
    _ck(lib().orc_matmul(code(a), _p(a), _p(b), _p(out), C.c_int64(batch), C.c_int64(M), C.c_int64(Nn), C.c_int64(K)),
        "matmul")
    return out


def num_threads() -> int:
    return int(lib().orc_num_threads())


# ---- the reference's own code (oracle/_ref), where it could be built ------------------------------------
_ref = None


def ref_lib():
    """``oracle/_ref/libdeepx_ref.so`` or None when it has not been built (no reference tree)."""
    global _ref
    if _ref is None and REF_LIB_PATH.exists():
        _ref = C.CDLL(str(REF_LIB_PATH))
        _ref.ref_factory_new.restype = C.c_void_p
        _ref.ref_factory_free.argtypes = [C.c_void_p]
        _ref.ref_factory_add.argtypes = [C.c_void_p, C.c_char_p]
        _ref.ref_factory_get.argtypes = [C.c_void_p, C.c_char_p]
        _ref.ref_dtype_value.restype = C.c_uint
    return _ref
