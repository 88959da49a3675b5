"""CPU tests: the C-ABI libraries load without a GPU and export exactly what the headers declare."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared(header: str) -> set[str]:
    text = (ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(dx_[a-z0-9_]+)\s*\(", text))


def test_kernel_library_exports_every_declared_symbol():
    from deepx_b200 import _native as N
    names = declared("dx_kernels.h")
    assert len(names) >= 30
    lib = C.CDLL(str(N.LIB_PATH))
    for n in sorted(names):
        assert hasattr(lib, n), f"{n} is declared in dx_kernels.h but not exported"
    assert names == set(N.SIGNATURES), "ctypes table and header disagree: " + str(names ^ set(N.SIGNATURES))


def test_executor_library_exports_every_declared_symbol():
    from deepx_b200 import executor as E
    names = declared("dx_executor.h")
    lib = E.lib()
    for n in sorted(names):
        assert hasattr(lib, n), f"{n} is declared in dx_executor.h but not exported"
    assert names == set(E.SIGNATURES)


def test_heapmem_symbols_are_exported():
    from deepx_b200 import heapmem as H
    names = declared("dx_heapmem.h")
    lib = H.lib()
    for n in sorted(names):
        assert hasattr(lib, n), f"{n} is declared in dx_heapmem.h but not exported"
    assert names == set(H.SIGNATURES)


def test_fused_calls_validate_on_the_host():
    from deepx_b200 import _native as N
    assert N.lib.dx_rmsnorm(N.I32, 8, None, 8, 4, 4, 4.0, 1e-6, None) == N.E_DTYPE
    assert N.lib.dx_softmax(N.F32, 8, 8, 4, 0, None) == N.E_SHAPE
    assert N.lib.dx_softmax(N.F32, 8, 8, 0, 16, None) == N.OK            # no rows: nothing to do
    assert N.lib.dx_rmsnorm(N.F32, None, None, None, 4, 4, 4.0, 1e-6, None) == N.E_ARG


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected on the host before anything touches a device."""
    from deepx_b200 import _native as N
    assert N.lib.dx_dtype_size(N.BF16) == 2 and N.lib.dx_dtype_size(99) == 0
    assert N.lib.dx_ew_binary(99, N.F32, 8, 8, 8, 4, None) == N.E_ARG
    assert b"unknown op" in N.lib.dx_last_error()
    assert N.lib.dx_ew_binary(N.POW, N.I32, 8, 8, 8, 4, None) == N.E_DTYPE
    assert N.lib.dx_ew_binary(N.ADD, N.F32, 8, 8, 8, 0, None) == N.OK          # empty tensor: nothing to do
    shape, dims = N.i64_array([4, 5]), N.i32_array([2])
    assert N.lib.dx_reduce(N.SUM, N.F32, 8, shape, 2, dims, 1, 8, None, 0, None) == N.E_SHAPE
    assert N.lib.dx_transpose(N.F32, 8, shape, 2, N.i32_array([0, 0]), 16, None) == N.E_SHAPE
    assert N.lib.dx_concat(N.F32, N.ptr_array([8]), N.i64_array([3]), 1, N.i64_array([2, 5]), 2, 1, 16, None) == N.E_SHAPE
    assert N.lib.dx_broadcast_to(N.F32, 8, N.i64_array([3, 2]), 2, N.i64_array([4, 3, 3]), 3, 16, None) == N.E_SHAPE
    assert N.lib.dx_matmul(N.I32, 8, 8, 8, 1, 2, 2, 2, None) == N.E_DTYPE
    with pytest.raises(N.DxError):
        N.check(N.E_SHAPE)


def test_tensorfunc_refuses_cpu_tensors():
    import torch
    from deepx_b200 import tensorfunc as TF
    a = torch.zeros(4)
    with pytest.raises(ValueError, match="no CPU path"):
        TF.add(a, a, a)
