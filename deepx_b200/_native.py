"""ctypes binding of ``libdeepx_b200.so`` (the C ABI declared in ``include/dx_kernels.h``).

The library is the product: there is no Python or CPU fallback.  If it has not been
built, importing this module raises with the build command.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libdeepx_b200.so"

# dtype codes (dx_dtype)
F64, F32, F16, BF16, I64, I32, I16, I8, BOOL = range(9)
DTYPE_NAMES = {F64: "float64", F32: "float32", F16: "float16", BF16: "bfloat16", I64: "int64", I32: "int32",
               I16: "int16", I8: "int8", BOOL: "bool"}
DTYPE_CODES = {v: k for k, v in DTYPE_NAMES.items()}
DTYPE_SIZE = {F64: 8, F32: 4, F16: 2, BF16: 2, I64: 8, I32: 4, I16: 2, I8: 1, BOOL: 1}

# op codes
ADD, SUB, MUL, DIV, MAX, MIN, POW = range(7)
ADDS, SUBS, RSUBS, MULS, DIVS, RDIVS, MAXS, MINS, POWS, RPOWS = range(10)
SQRT, LOG, EXP, SIN, COS, TAN, INVERT = range(7)
EQ, NE, LT, GT = range(4)
SUM, PROD, RMAX, RMIN = range(4)

OK, E_DTYPE, E_SHAPE, E_ARG, E_CUDA, E_WORKSPACE, E_ALIAS, E_UNSUPPORTED = 0, -1, -2, -3, -4, -5, -6, -7
MAX_DIMS = 12
SWITCH_MAX = 16

_vp, _i, _i64, _d, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_double, C.c_float, C.c_size_t
_pi64, _pi32, _pvp = C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.POINTER(C.c_void_p)

# name → (restype, argtypes); every symbol include/dx_kernels.h declares
SIGNATURES = {
    "dx_last_error": (C.c_char_p, []),
    "dx_dtype_size": (_i, [_i]),
    "dx_sm_count": (_i, []),
    "dx_launch_count": (C.c_ulonglong, []),
    "dx_ew_binary": (_i, [_i, _i, _vp, _vp, _vp, _i64, _vp]),
    "dx_ew_scalar": (_i, [_i, _i, _vp, _d, _i64, _vp, _i64, _vp]),
    "dx_ew_unary": (_i, [_i, _i, _vp, _vp, _i64, _vp]),
    "dx_ew_compare": (_i, [_i, _i, _vp, _vp, _f, _vp, _i64, _vp]),
    "dx_ew_compare_scalar": (_i, [_i, _i, _vp, _d, _i64, _f, _vp, _i64, _vp]),
    "dx_switch": (_i, [_i, _pvp, _i, _i, _vp, _vp, _i64, _vp]),
    "dx_cast": (_i, [_i, _vp, _i, _vp, _i64, _vp]),
    "dx_fill": (_i, [_i, _vp, _d, _i64, _i64, _vp]),
    "dx_arange": (_i, [_i, _vp, _d, _d, _i64, _vp]),
    "dx_uniform": (_i, [_i, _vp, _d, _d, C.c_uint64, _i64, _vp]),
    "dx_normal": (_i, [_i, _vp, _d, _d, C.c_uint64, _i64, _vp]),
    "dx_dropout": (_i, [_i, _vp, _d, C.c_uint64, _i64, _vp]),
    "dx_reduce_workspace_bytes": (_sz, [_i, _i, _pi64, _i, _pi32, _i]),
    "dx_reduce": (_i, [_i, _i, _vp, _pi64, _i, _pi32, _i, _vp, _vp, _sz, _vp]),
    "dx_reduce_noalloc": (_i, [_i, _i, _vp, _pi64, _i, _pi32, _i, _vp, _vp]),
    "dx_comm_max_bytes": (_sz, []),
    "dx_comm_create": (_vp, [_i, _i, _i]),
    "dx_comm_handle": (_i, [_vp, C.c_char_p]),
    "dx_comm_connect": (_i, [_vp, C.c_char_p]),
    "dx_comm_set_timeout_ms": (_i, [_vp, _i]),
    "dx_comm_allreduce": (_i, [_vp, _i, _i, _vp, _i64, _vp]),
    "dx_comm_status": (_i, [_vp, _vp]),
    "dx_comm_wait_stats": (_i, [_vp, C.POINTER(C.c_double), C.POINTER(C.c_longlong), _i, _vp]),
    "dx_comm_destroy": (None, [_vp]),
    "dx_reduce_allreduce": (_i, [_vp, _i, _i, _vp, _pi64, _i, _pi32, _i, _vp, _vp, _sz, _vp]),
    "dx_comm_emulate": (_vp, [_i, _i]),
    "dx_comm_emulated_allreduce": (_i, [_vp, _i, _i, _pvp, _i, _i64, _vp]),
    "dx_comm_rank": (_i, [_vp]),
    "dx_comm_world": (_i, [_vp]),
    "dx_comm_allreduce_begin": (_i, [_vp, _i, _i, _vp, _i64, _vp]),
    "dx_comm_allreduce_finish": (_i, [_vp, _vp]),
    "dx_comm_pending": (_i, [_vp, _pvp]),
    "dx_shard_rows": (None, [_i64, _i, _i, _pi64, _pi64]),
    "dx_comm_allgather_rows": (_i, [_vp, _vp, _i64, _i64, _vp]),
    "dx_reduce_allreduce_begin": (_i, [_vp, _i, _i, _vp, _pi64, _i, _pi32, _i, _vp, _vp, _sz, _vp]),
    "dx_comm_emulated_publish": (_i, [_vp, _i, _i, _pvp, _i, _i64, _vp]),
    "dx_comm_emulated_combine": (_i, [_vp, _i, _i, _pvp, _i, _i64, _vp]),
    "dx_comm_emulated_allgather_rows": (_i, [_vp, _pvp, _i64, _i64, _vp]),
    "dx_rmsnorm": (_i, [_i, _vp, _vp, _vp, _i64, _i64, _d, _d, _vp]),
    "dx_softmax": (_i, [_i, _vp, _vp, _i64, _i64, _vp]),
    "dx_transpose": (_i, [_i, _vp, _pi64, _i, _pi32, _vp, _vp]),
    "dx_concat": (_i, [_i, _pvp, _pi64, _i, _pi64, _i, _i, _vp, _vp]),
    "dx_broadcast_to": (_i, [_i, _vp, _pi64, _i, _pi64, _i, _vp, _vp]),
    "dx_indexselect": (_i, [_i, _vp, _pi64, _i, _i, _vp, _pi64, _i, _i, _vp, _vp, _vp]),
    "dx_repeat": (_i, [_i, _vp, _pi64, _i, _pi64, _vp, _vp]),
    "dx_matmul": (_i, [_i, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "dx_matmul_workspace_bytes": (_sz, [_i, _i64, _i64, _i64, _i64]),
    "dx_matmul_ws": (_i, [_i, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp, _sz, _vp]),
    "dx_matmul_status": (_i, [_vp]),
    "dx_pool_create": (_vp, [_i, _sz]),
    "dx_pool_destroy": (None, [_vp]),
    "dx_pool_alloc": (_vp, [_vp, _sz]),
    "dx_pool_free": (_i, [_vp, _vp]),
    "dx_pool_stats": (None, [_vp, C.POINTER(C.c_size_t)]),
    "dx_pool_trim": (None, [_vp]),
}


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA kernel library has not been built. "
            "Run `python -m deepx_b200.build` (needs nvcc; no GPU required to build). "
            "There is no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class DxError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[dx {code}] {message}")
        self.code = code
        self.message = message


def check(code: int) -> None:
    if code != OK:
        raise DxError(code, lib.dx_last_error().decode("utf-8", "replace"))


def i64_array(values) -> C.Array:
    vals = [int(v) for v in values]
    return (C.c_int64 * max(len(vals), 1))(*vals)


def i32_array(values) -> C.Array:
    vals = [int(v) for v in values]
    return (C.c_int32 * max(len(vals), 1))(*vals)


def ptr_array(values) -> C.Array:
    vals = [C.c_void_p(int(v)) for v in values]
    return (C.c_void_p * max(len(vals), 1))(*vals)
