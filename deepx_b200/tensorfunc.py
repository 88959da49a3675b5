"""The reference's ``tensorfunc`` interface on B200 kernels.

Same function names, argument order (inputs first, output tensor last) and error
behaviour as ``executor/deepxcore/src/deepx/tensorfunc/{elementwise,reduce,changeshape,
matmul,init}.hpp`` of the reference; every function is a thin call into the C ABI of
``libdeepx_b200.so``.  Tensors are contiguous ``torch.Tensor`` objects on a CUDA device —
torch only provides device memory and the current stream here.  Nothing in this module
computes on the host and nothing falls back to torch ops.

Shape errors raise ``ValueError`` (the reference throws ``std::invalid_argument`` /
``TensorShapeError``); dtype errors raise ``TypeError``; kernel-library failures raise
``_native.DxError``.
"""
from __future__ import annotations

import builtins
from typing import Sequence

import torch

from . import _native as N

_TORCH2DX = {
    torch.float64: N.F64, torch.float32: N.F32, torch.float16: N.F16, torch.bfloat16: N.BF16,
    torch.int64: N.I64, torch.int32: N.I32, torch.int16: N.I16, torch.int8: N.I8, torch.bool: N.BOOL,
}
DX2TORCH = {v: k for k, v in _TORCH2DX.items()}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _TORCH2DX[t.dtype]
    except KeyError:
        raise TypeError(f"Unsupported dtype: {t.dtype}") from None


def _dev(*ts: torch.Tensor) -> None:
    d = None
    for t in ts:
        if not t.is_cuda:
            raise ValueError("tensor is not on a CUDA device (this executor has no CPU path)")
        if not t.is_contiguous():
            raise ValueError("tensor is not contiguous")
        if d is None:
            d = t.device
        elif t.device != d:
            raise ValueError("tensors are on different devices")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _same_shape(*ts: torch.Tensor) -> None:
    s = ts[0].shape
    for t in ts[1:]:
        if t.shape != s:
            raise ValueError("shape mismatch")


def _same_dtype(*ts: torch.Tensor) -> None:
    d = ts[0].dtype
    for t in ts[1:]:
        if t.dtype != d:
            raise TypeError("Type mismatch: " + " != ".join(N.DTYPE_NAMES[dtype_code(x)] for x in ts))


def _scalar(dtype: torch.dtype, value) -> tuple[float, int]:
    """(fscalar, iscalar) for the C ABI; the caller decides how the text became a number."""
    if dtype.is_floating_point:
        return float(value), 0
    return 0.0, int(value)


# ---- elementwise: tensor ∘ tensor ----------------------------------------------------------
def _binary(op: int, A: torch.Tensor, B: torch.Tensor, Cc: torch.Tensor) -> None:
    _dev(A, B, Cc)
    _same_shape(A, B, Cc)
    _same_dtype(A, B, Cc)
    with torch.cuda.device(A.device):
        N.check(N.lib.dx_ew_binary(op, dtype_code(A), A.data_ptr(), B.data_ptr(), Cc.data_ptr(), A.numel(), _stream(A)))


def add(A, B, Cc): _binary(N.ADD, A, B, Cc)
def sub(A, B, Cc): _binary(N.SUB, A, B, Cc)
def mul(A, B, Cc): _binary(N.MUL, A, B, Cc)
def div(A, B, Cc): _binary(N.DIV, A, B, Cc)
def max(A, B, Cc): _binary(N.MAX, A, B, Cc)  # noqa: A001 (reference name)
def min(A, B, Cc): _binary(N.MIN, A, B, Cc)  # noqa: A001
def pow(A, B, Cc): _binary(N.POW, A, B, Cc)  # noqa: A001


# ---- elementwise: tensor ∘ scalar ------------------------------------------------------------
def _scalar_op(op: int, A: torch.Tensor, value, Cc: torch.Tensor) -> None:
    _dev(A, Cc)
    _same_shape(A, Cc)
    _same_dtype(A, Cc)
    fs, is_ = _scalar(A.dtype, value)
    with torch.cuda.device(A.device):
        N.check(N.lib.dx_ew_scalar(op, dtype_code(A), A.data_ptr(), fs, is_, Cc.data_ptr(), A.numel(), _stream(A)))


def addscalar(A, value, Cc): _scalar_op(N.ADDS, A, value, Cc)
def subscalar(A, value, Cc): _scalar_op(N.SUBS, A, value, Cc)
def rsubscalar(value, A, Cc): _scalar_op(N.RSUBS, A, value, Cc)
def mulscalar(A, value, Cc): _scalar_op(N.MULS, A, value, Cc)
def divscalar(A, value, Cc): _scalar_op(N.DIVS, A, value, Cc)
def rdivscalar(value, A, Cc): _scalar_op(N.RDIVS, A, value, Cc)
def maxscalar(A, value, Cc): _scalar_op(N.MAXS, A, value, Cc)
def minscalar(A, value, Cc): _scalar_op(N.MINS, A, value, Cc)
def powscalar(A, value, Cc): _scalar_op(N.POWS, A, value, Cc)
def rpowscalar(value, A, Cc): _scalar_op(N.RPOWS, A, value, Cc)


# ---- elementwise: unary ------------------------------------------------------------------------
def _unary(op: int, A: torch.Tensor, Cc: torch.Tensor) -> None:
    _dev(A, Cc)
    _same_shape(A, Cc)
    _same_dtype(A, Cc)
    with torch.cuda.device(A.device):
        N.check(N.lib.dx_ew_unary(op, dtype_code(A), A.data_ptr(), Cc.data_ptr(), A.numel(), _stream(A)))


def sqrt(A, Cc): _unary(N.SQRT, A, Cc)
def log(A, Cc): _unary(N.LOG, A, Cc)
def exp(A, Cc): _unary(N.EXP, A, Cc)
def sin(A, Cc): _unary(N.SIN, A, Cc)
def cos(A, Cc): _unary(N.COS, A, Cc)
def tan(A, Cc): _unary(N.TAN, A, Cc)
def invert(A, Cc): _unary(N.INVERT, A, Cc)


# ---- compare → bool mask --------------------------------------------------------------------------
def _compare(op: int, A: torch.Tensor, B: torch.Tensor, epsilon: float, mask: torch.Tensor) -> None:
    _dev(A, B, mask)
    _same_shape(A, B, mask)
    _same_dtype(A, B)
    if mask.dtype != torch.bool:
        raise TypeError("mask must be bool")
    with torch.cuda.device(A.device):
        N.check(N.lib.dx_ew_compare(op, dtype_code(A), A.data_ptr(), B.data_ptr(), float(epsilon), mask.data_ptr(),
                                    A.numel(), _stream(A)))


def _compare_scalar(op: int, A: torch.Tensor, value, epsilon: float, mask: torch.Tensor) -> None:
    _dev(A, mask)
    _same_shape(A, mask)
    if mask.dtype != torch.bool:
        raise TypeError("mask must be bool")
    fs, is_ = _scalar(A.dtype, value)
    with torch.cuda.device(A.device):
        N.check(N.lib.dx_ew_compare_scalar(op, dtype_code(A), A.data_ptr(), fs, is_, float(epsilon), mask.data_ptr(),
                                           A.numel(), _stream(A)))


def equal(A, B, epsilon, mask): _compare(N.EQ, A, B, epsilon, mask)
def notequal(A, B, epsilon, mask): _compare(N.NE, A, B, epsilon, mask)
def less(A, B, mask): _compare(N.LT, A, B, 0.0, mask)
def greater(A, B, mask): _compare(N.GT, A, B, 0.0, mask)
def equalscalar(A, value, epsilon, mask): _compare_scalar(N.EQ, A, value, epsilon, mask)
def notequalscalar(A, value, epsilon, mask): _compare_scalar(N.NE, A, value, epsilon, mask)
def lessscalar(A, value, mask): _compare_scalar(N.LT, A, value, 0.0, mask)
def greaterscalar(A, value, mask): _compare_scalar(N.GT, A, value, 0.0, mask)


def Switch(tensors: Sequence[torch.Tensor], cases: torch.Tensor, Cc: torch.Tensor) -> None:
    """C[i] = tensors[cases[i]][i]; bool cases need exactly two tensors (false → tensors[0])."""
    _dev(cases, Cc, *tensors)
    if cases.shape != Cc.shape:
        raise ValueError("shape mismatch")
    _same_dtype(Cc, *tensors)
    for t in tensors:
        if t.shape != Cc.shape:
            raise ValueError("shape mismatch")
    if cases.dtype == torch.bool and len(tensors) != 2:
        raise ValueError("For bool cases, tensors size must be 2")
    ptrs = N.ptr_array(t.data_ptr() for t in tensors)
    with torch.cuda.device(Cc.device):
        N.check(N.lib.dx_switch(dtype_code(Cc), ptrs, len(tensors), dtype_code(cases), cases.data_ptr(), Cc.data_ptr(),
                                Cc.numel(), _stream(Cc)))


def todtype(A: torch.Tensor, Cc: torch.Tensor) -> None:
    _dev(A, Cc)
    if A.numel() != Cc.numel():
        raise ValueError(f"Shape mismatch: {A.numel()} != {Cc.numel()}")
    with torch.cuda.device(A.device):
        N.check(N.lib.dx_cast(dtype_code(A), A.data_ptr(), dtype_code(Cc), Cc.data_ptr(), A.numel(), _stream(A)))


def constant(Cc: torch.Tensor, value) -> None:
    _dev(Cc)
    if Cc.dtype == torch.bool:
        fs, is_ = 0.0, int(bool(value))
    else:
        fs, is_ = _scalar(Cc.dtype, value)
    with torch.cuda.device(Cc.device):
        N.check(N.lib.dx_fill(dtype_code(Cc), Cc.data_ptr(), fs, is_, Cc.numel(), _stream(Cc)))


# ---- reduce --------------------------------------------------------------------------------------------
def checked_dims(shape: Sequence[int], dims: Sequence[int]) -> list[int]:
    """checkedDims (executor/deepxcore/src/deepx/shape_reduce.cpp:11-45): empty = all axes,
    negatives wrap, sorted, unique; out of range raises."""
    n = len(shape)
    if len(dims) == 0:
        return list(range(n))
    out = []
    for d in dims:
        d = int(d)
        if d < 0:
            d += n
        if d >= n or d < 0:
            raise ValueError("Tensor shape error for operation: Dimension out of range in sum")
        out.append(d)
    return sorted(set(out))


def reduced_shape(shape: Sequence[int], dims: Sequence[int], keepdims: bool) -> list[int]:
    """reducedShape (shape_reduce.cpp:47-75); `dims` already checked."""
    red = set(dims)
    out = []
    for i, s in enumerate(shape):
        if i not in red:
            out.append(int(s))
        elif keepdims:
            out.append(1)
    return out or [1]


_workspace: dict[tuple, torch.Tensor] = {}


def _get_workspace(device: torch.device, nbytes: int, floor: int = 1 << 20, what: str = "reduce") -> torch.Tensor:
    """Scratch memory of (device, current stream, purpose): launches on different streams may overlap, so they must not share it."""
    key = (device, torch.cuda.current_stream(device).cuda_stream, what)
    ws = _workspace.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(builtins.max(int(nbytes), floor), dtype=torch.uint8, device=device)
        _workspace[key] = ws
    return ws


def _reduce(op: int, A: torch.Tensor, dims: Sequence[int], keepdims: bool, B: torch.Tensor, comm_handle=None, defer: bool = False) -> None:
    """`comm_handle` (a dx_comm): the local reduction is followed by the combine over its ranks, fused
    into the reduction's finish kernel where that is a single CTA.  `defer`: stop after this rank's result
    has been published to the peers; dx_comm_allreduce_finish completes the exchange later on the stream."""
    _dev(A, B)
    _same_dtype(A, B)
    cd = checked_dims(A.shape, dims)
    want = reduced_shape(A.shape, cd, keepdims)
    n_want = 1
    for s in want:
        n_want *= s
    if B.numel() != n_want:
        raise ValueError("shape mismatch")
    shape = N.i64_array(A.shape)
    cdims = N.i32_array(cd)
    code = dtype_code(A)
    with torch.cuda.device(A.device):
        need = N.lib.dx_reduce_workspace_bytes(op, code, shape, A.dim(), cdims, len(cd))
        ws = _get_workspace(A.device, need) if need else None
        if comm_handle is not None:
            fn = N.lib.dx_reduce_allreduce_begin if defer else N.lib.dx_reduce_allreduce
            N.check(fn(comm_handle, op, code, A.data_ptr(), shape, A.dim(), cdims, len(cd), B.data_ptr(),
                     ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, _stream(A)))
            return
        N.check(N.lib.dx_reduce(op, code, A.data_ptr(), shape, A.dim(), cdims, len(cd), B.data_ptr(),
                                ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                _stream(A)))


def sum(A, dims, keepdims, B): _reduce(N.SUM, A, dims, keepdims, B)  # noqa: A001
def prod(A, dims, keepdims, B): _reduce(N.PROD, A, dims, keepdims, B)
def reducemax(A, dims, keepdims, B): _reduce(N.RMAX, A, dims, keepdims, B)
def reducemin(A, dims, keepdims, B): _reduce(N.RMIN, A, dims, keepdims, B)


# ---- fused row chains (no single reference function: the front end's RMSNorm / softmax op chains) --------
def rmsnorm(X: torch.Tensor, weight, divisor: float, eps: float, Out: torch.Tensor) -> None:
    """Out = weight * (X * 1/sqrt(sum(X^2, last axis)/divisor + eps)); `weight` [cols] or None."""
    _dev(X, Out) if weight is None else _dev(X, Out, weight)
    _same_dtype(X, Out) if weight is None else _same_dtype(X, Out, weight)
    if X.shape != Out.shape or X.dim() < 1:
        raise ValueError("shape mismatch")
    cols = X.shape[-1]
    if weight is not None and weight.numel() != cols:
        raise ValueError("weight does not match the last axis")
    rows = X.numel() // cols if cols else 0
    with torch.cuda.device(X.device):
        N.check(N.lib.dx_rmsnorm(dtype_code(X), X.data_ptr(), None if weight is None else weight.data_ptr(), Out.data_ptr(),
                                 rows, cols, float(divisor), float(eps), _stream(X)))


def softmax(X: torch.Tensor, Out: torch.Tensor) -> None:
    """Out = softmax(X) over the last axis, as the chain reducemax, sub, exp, sum, div computes it."""
    _dev(X, Out)
    _same_dtype(X, Out)
    if X.shape != Out.shape or X.dim() < 1:
        raise ValueError("shape mismatch")
    cols = X.shape[-1]
    rows = X.numel() // cols if cols else 0
    with torch.cuda.device(X.device):
        N.check(N.lib.dx_softmax(dtype_code(X), X.data_ptr(), Out.data_ptr(), rows, cols, _stream(X)))


# ---- changeshape -----------------------------------------------------------------------------------------
def transpose(A: torch.Tensor, dim_order: Sequence[int], Cc: torch.Tensor) -> None:
    _dev(A, Cc)
    _same_dtype(A, Cc)
    if len(dim_order) != A.dim():
        raise ValueError("dimOrder size does not match the number of dimensions in the TensorCPU.")
    if Cc.numel() != A.numel():
        raise RuntimeError("transpose error!shape")
    with torch.cuda.device(A.device):
        N.check(N.lib.dx_transpose(dtype_code(A), A.data_ptr(), N.i64_array(A.shape), A.dim(), N.i32_array(dim_order),
                                   Cc.data_ptr(), _stream(A)))


def concat(tensors: Sequence[torch.Tensor], axis: int, Cc: torch.Tensor) -> None:
    _dev(Cc, *tensors)
    _same_dtype(Cc, *tensors)
    nd = Cc.dim()
    total = 0
    for t in tensors:
        if t.dim() != nd:
            raise ValueError("Tensor shape error for operation: All input tensors must have the same dimension size for concat")
        for j in range(nd):
            if j != axis and t.shape[j] != Cc.shape[j]:
                raise ValueError("Tensor shape error for operation: All input tensors must have the same dimension size for concat")
        total += t.shape[axis]
    if total != Cc.shape[axis]:
        raise ValueError("Tensor shape error for operation: Output tensor shape size must match the sum of input tensor shape sizes for concat")
    with torch.cuda.device(Cc.device):
        N.check(N.lib.dx_concat(dtype_code(Cc), N.ptr_array(t.data_ptr() for t in tensors),
                                N.i64_array(t.shape[axis] for t in tensors), len(tensors), N.i64_array(Cc.shape), nd,
                                axis, Cc.data_ptr(), _stream(Cc)))


def broadcastTo(A: torch.Tensor, new_shape: Sequence[int], B: torch.Tensor) -> None:
    _dev(A, B)
    _same_dtype(A, B)
    if list(B.shape) != [int(s) for s in new_shape]:
        raise ValueError("Tensor shape error for operation: Broadcast shape mismatch")
    with torch.cuda.device(A.device):
        try:
            N.check(N.lib.dx_broadcast_to(dtype_code(A), A.data_ptr(), N.i64_array(A.shape), A.dim(),
                                          N.i64_array(new_shape), len(new_shape), B.data_ptr(), _stream(A)))
        except N.DxError as e:
            if e.code == N.E_SHAPE:
                raise ValueError("Tensor shape error for operation: Broadcast shape mismatch") from None
            raise


def indexselect_shape(input_shape: Sequence[int], index_shape: Sequence[int], axis: int) -> list[int]:
    """indexselectShape (shape_changeshape.cpp:122-141)."""
    return [int(s) for s in input_shape[:axis]] + [int(s) for s in index_shape] + [int(s) for s in input_shape[axis + 1:]]


def indexselect(A: torch.Tensor, index: torch.Tensor, axis: int, B: torch.Tensor, oob_flag: torch.Tensor | None = None) -> None:
    _dev(A, index, B)
    _same_dtype(A, B)
    if index.dtype not in (torch.int32, torch.int64):
        raise TypeError("index_type only support int64 or int32")
    g = axis + A.dim() if axis < 0 else axis
    if g < 0 or g >= A.dim():
        raise ValueError("Axis is out of bounds")
    if list(B.shape) != indexselect_shape(A.shape, index.shape, g):
        raise ValueError("Tensor shape error for operation: Indexselect shape mismatch")
    with torch.cuda.device(A.device):
        N.check(N.lib.dx_indexselect(dtype_code(A), A.data_ptr(), N.i64_array(A.shape), A.dim(), dtype_code(index),
                                     index.data_ptr(), N.i64_array(index.shape), index.dim(), g, B.data_ptr(),
                                     oob_flag.data_ptr() if oob_flag is not None else None, _stream(A)))


def repeat(A: torch.Tensor, repeats: Sequence[int], B: torch.Tensor) -> None:
    _dev(A, B)
    _same_dtype(A, B)
    if len(repeats) != A.dim():
        raise ValueError("Shape and repeats must have the same number of dimensions")
    if list(B.shape) != [int(s) * int(r) for s, r in zip(A.shape, repeats)]:
        raise ValueError("Tensor shape error for operation: Repeat shape mismatch")
    with torch.cuda.device(A.device):
        N.check(N.lib.dx_repeat(dtype_code(A), A.data_ptr(), N.i64_array(A.shape), A.dim(), N.i64_array(repeats),
                                B.data_ptr(), _stream(A)))


# ---- matmul -------------------------------------------------------------------------------------------------
def check_matmul_shape(a: Sequence[int], b: Sequence[int]) -> bool:
    """check_matmul_shape (executor/deepxcore/src/deepx/tensorfunc/matmul.hpp:9-27)."""
    if len(a) < 2 or len(b) < 2 or a[-1] != b[-2] or len(a) != len(b):
        return False
    return all(a[i] == b[i] for i in range(len(a) - 2))


def matmul(A: torch.Tensor, B: torch.Tensor, Cc: torch.Tensor) -> None:
    _dev(A, B, Cc)
    _same_dtype(A, B, Cc)
    if not check_matmul_shape(list(A.shape), list(B.shape)):
        raise ValueError("A.shape could matmul with B.shape")
    M, K, Nn = A.shape[-2], A.shape[-1], B.shape[-1]
    batch = A.numel() // (M * K) if M * K else 0
    if list(Cc.shape) != list(A.shape[:-1]) + [Nn]:
        raise ValueError("shape mismatch")
    with torch.cuda.device(A.device):
        code = dtype_code(A)
        need = N.lib.dx_matmul_workspace_bytes(code, batch, M, Nn, K)  # > 0 for a few rows of tiles: K split through scratch memory
        if need:
            ws = _get_workspace(A.device, need, 32 << 20, "matmul")
            N.check(N.lib.dx_matmul_ws(code, A.data_ptr(), B.data_ptr(), Cc.data_ptr(), batch, M, Nn, K, ws.data_ptr(), ws.numel(), _stream(A)))
        else:
            N.check(N.lib.dx_matmul(code, A.data_ptr(), B.data_ptr(), Cc.data_ptr(), batch, M, Nn, K, _stream(A)))
