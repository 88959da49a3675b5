"""The CPU oracle and this library's kernels against the REFERENCE'S OWN CUDA kernels.

oracle/_ref/libdeepx_ref_cuda.so is the reference's executor/op-cuda/src/deepx/tensorfunc/*.cu,
compiled unchanged for sm_100 (oracle/Makefile) behind a small C harness.  Each case runs the
reference's launch_* wrapper, the oracle (oracle.cpp, the restatement of op-ompsimd every other
parity test trusts) and this library's C ABI on the same seeded input:

  * integers, IEEE float + - * / sqrt max min (float32/float64), compares, switch, casts, every
    changeshape op: all three must agree bit for bit;
  * float16 / bfloat16 arithmetic: the reference's CUDA code uses the native half instructions, the
    CPU executor has no 16-bit floats at all; the oracle (compute in float32, round once) may differ
    from a native half add or divide by one unit in the last place, which is the tolerance here;
  * exp / log / pow: relative 1e-5 (float32), 1e-12 (float64) — CUDA's and the C library's routines
    are different implementations of the same function;
  * float sum: 1e-5 of sum|x| (the reference adds with atomics in arbitrary order); int32 sum bit-exact.

Not run (read, not executed): the reference's sum over every axis without keepdims (reads an uninitialised output
index), its concat (device-side allocation per thread), reducemax /
reducemin / prod (unsynchronised read-modify-write), sum on int64/int16/int8, sin/cos/tan.

equal/notequal with a tolerance: the reference's CUDA kernels test |a-b| < eps, its CPU executor
|a-b| <= eps (op-ompsimd elementwise_miaobyte.hpp:778-785).  The oracle and this library follow the
CPU executor; the cases here use data with no difference exactly equal to eps.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import ALL_NUMERIC, FLOATS, INTS, NP_DTYPES, assert_bit_exact, bits, make, seed_of, to_gpu, to_np

pytestmark = pytest.mark.gpu

SIZES = [1, 7, 4099, (1 << 20) + 3]
CODES = {"float64": 0, "float32": 1, "float16": 2, "bfloat16": 3, "int64": 4, "int32": 5, "int16": 6, "int8": 7, "bool": 8}


@pytest.fixture(scope="module")
def R():
    from oracle import ref_cuda
    lib = ref_cuda.load()
    if lib is None:
        pytest.skip("oracle/_ref/libdeepx_ref_cuda.so was not built (the reference tree was absent at build time)")
    return ref_cuda


@pytest.fixture(scope="module")
def mods():
    from deepx_b200 import tensorfunc as TF
    from oracle import oracle as O
    return TF, O


def _ulp_close(got, want, dtype, what, ulps=1):
    """16-bit floats: equal up to `ulps` units in the last place (sign-magnitude order of the bit patterns)."""
    g, w = bits(got).astype(np.int64), bits(want).astype(np.int64)
    g = np.where(g & 0x8000, 0x8000 - g, g)
    w = np.where(w & 0x8000, 0x8000 - w, w)
    bad = np.abs(g - w) > ulps
    assert not bad.any(), f"{what}: {int(bad.sum())} of {g.size} elements differ by more than {ulps} ulp"


def _rel_close(got, want, dtype, what):
    tol = {"float64": 1e-12, "float32": 1e-5}[dtype]
    g, w = got.astype(np.float64), want.astype(np.float64)
    ok = np.isclose(g, w, rtol=tol, atol=0) | (g == w)
    assert ok.all(), f"{what}: max rel err {np.max(np.abs(g - w) / np.maximum(np.abs(w), 1e-300))}"


def _same(got, want, dtype, what):
    if dtype in ("float16", "bfloat16"):
        _ulp_close(got, want, dtype, what)
    else:
        assert_bit_exact(got, want, what)


@pytest.mark.parametrize("dtype", ALL_NUMERIC)
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "max", "min"])
def test_binary(R, mods, op, dtype):
    TF, O = mods
    lib = R.load()
    code = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5}[op]
    rng = np.random.default_rng(seed_of("refcu", op, dtype))
    for n in SIZES:
        a = make(rng, dtype, (n,))
        b = make(rng, dtype, (n,), nonzero=(op == "div"))
        A, B = to_gpu(a), to_gpu(b)
        ref, ours = torch.empty_like(A), torch.empty_like(A)
        R.check(lib.refcu_binary(code, CODES[dtype], A.data_ptr(), B.data_ptr(), ref.data_ptr(), n))
        getattr(TF, op)(A, B, ours)
        want = getattr(O, op)(a, b)
        _same(to_np(ref), want, dtype, f"reference {op}<{dtype}> n={n} vs oracle")
        _same(to_np(ours), to_np(ref), dtype, f"ours {op}<{dtype}> n={n} vs reference")


@pytest.mark.parametrize("dtype", ALL_NUMERIC)
@pytest.mark.parametrize("op", ["addscalar", "subscalar", "rsubscalar", "mulscalar", "divscalar", "rdivscalar", "maxscalar", "minscalar"])
def test_scalar(R, mods, op, dtype):
    TF, O = mods
    lib = R.load()
    code = ["addscalar", "subscalar", "rsubscalar", "mulscalar", "divscalar", "rdivscalar", "maxscalar", "minscalar"].index(op)
    rng = np.random.default_rng(seed_of("refcu", op, dtype))
    value = 3 if dtype in INTS else 2.5
    for n in SIZES:
        a = make(rng, dtype, (n,), nonzero=(op == "rdivscalar"))
        A = to_gpu(a)
        ref, ours = torch.empty_like(A), torch.empty_like(A)
        R.check(lib.refcu_scalar(code, CODES[dtype], A.data_ptr(), float(value), int(value), ref.data_ptr(), n))
        if op.startswith("r"):
            getattr(TF, op)(value, A, ours)
            want = getattr(O, op)(value, a)
        else:
            getattr(TF, op)(A, value, ours)
            want = getattr(O, op)(a, value)
        _same(to_np(ref), want, dtype, f"reference {op}<{dtype}> n={n} vs oracle")
        _same(to_np(ours), to_np(ref), dtype, f"ours {op}<{dtype}> n={n} vs reference")


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("op", ["sqrt", "exp", "log"])
def test_unary_math(R, mods, op, dtype):
    TF, O = mods
    lib = R.load()
    code = {"sqrt": 0, "log": 1, "exp": 2}[op]
    rng = np.random.default_rng(seed_of("refcu", op, dtype))
    for n in SIZES:
        a = make(rng, dtype, (n,), 0.05, 8.0) if op != "exp" else make(rng, dtype, (n,), -8.0, 8.0)
        A = to_gpu(a)
        ref, ours = torch.empty_like(A), torch.empty_like(A)
        R.check(lib.refcu_unary(code, CODES[dtype], A.data_ptr(), ref.data_ptr(), n))
        getattr(TF, op)(A, ours)
        want = getattr(O, op)(a)
        what = f"{op}<{dtype}> n={n}"
        if dtype in ("float16", "bfloat16"):
            # hexp / hlog / hsqrt against float32-and-round: one unit in the last place (two for the native log/exp)
            _ulp_close(to_np(ref), want, dtype, "reference " + what, ulps=1 if op == "sqrt" else 2)
            _ulp_close(to_np(ours), want, dtype, "ours " + what, ulps=1)
        elif op == "sqrt":
            assert_bit_exact(to_np(ref), want, "reference " + what + " vs oracle")
            assert_bit_exact(to_np(ours), to_np(ref), "ours " + what + " vs reference")
        else:
            _rel_close(to_np(ref), want, dtype, "reference " + what + " vs oracle")
            _rel_close(to_np(ours), to_np(ref), dtype, "ours " + what + " vs reference")


@pytest.mark.parametrize("dtype", ["float64", "float32"])
def test_pow_family(R, mods, dtype):
    TF, O = mods
    lib = R.load()
    rng = np.random.default_rng(seed_of("refcu", "pow", dtype))
    n = 100003
    a = make(rng, dtype, (n,), 0.1, 4.0)
    b = make(rng, dtype, (n,), -3.0, 3.0)
    A, B = to_gpu(a), to_gpu(b)
    ref, ours = torch.empty_like(A), torch.empty_like(A)
    R.check(lib.refcu_binary(6, CODES[dtype], A.data_ptr(), B.data_ptr(), ref.data_ptr(), n))
    TF.pow(A, B, ours)
    _rel_close(to_np(ref), O.pow(a, b), dtype, f"reference pow<{dtype}> vs oracle")
    _rel_close(to_np(ours), to_np(ref), dtype, f"ours pow<{dtype}> vs reference")
    for s in (2.0, 2.5, -1.5, 0.5):
        R.check(lib.refcu_scalar(8, CODES[dtype], A.data_ptr(), s, int(s), ref.data_ptr(), n))
        TF.powscalar(A, s, ours)
        _rel_close(to_np(ref), O.powscalar(a, s), dtype, f"reference powscalar({s})<{dtype}> vs oracle")
        _rel_close(to_np(ours), to_np(ref), dtype, f"ours powscalar({s})<{dtype}> vs reference")
        R.check(lib.refcu_scalar(9, CODES[dtype], B.data_ptr(), abs(s), int(abs(s)), ref.data_ptr(), n))
        TF.rpowscalar(abs(s), B, ours)
        _rel_close(to_np(ref), O.rpowscalar(abs(s), b), dtype, f"reference rpowscalar({abs(s)})<{dtype}> vs oracle")
        _rel_close(to_np(ours), to_np(ref), dtype, f"ours rpowscalar({abs(s)})<{dtype}> vs reference")


@pytest.mark.parametrize("dtype", INTS)
def test_invert(R, mods, dtype):
    TF, O = mods
    lib = R.load()
    rng = np.random.default_rng(seed_of("refcu", "invert", dtype))
    for n in SIZES:
        a = make(rng, dtype, (n,))
        A = to_gpu(a)
        ref, ours = torch.empty_like(A), torch.empty_like(A)
        R.check(lib.refcu_unary(6, CODES[dtype], A.data_ptr(), ref.data_ptr(), n))
        TF.invert(A, ours)
        assert_bit_exact(to_np(ref), O.invert(a), f"reference invert<{dtype}> n={n} vs oracle")
        assert_bit_exact(to_np(ours), to_np(ref), f"ours invert<{dtype}> n={n} vs reference")


@pytest.mark.parametrize("dtype", ["float64", "float32", "int64", "int32", "int16", "int8"])
@pytest.mark.parametrize("op", ["equal", "notequal", "less", "greater"])
def test_compare(R, mods, op, dtype):
    TF, O = mods
    lib = R.load()
    code = {"equal": 0, "notequal": 1, "less": 2, "greater": 3}[op]
    rng = np.random.default_rng(seed_of("refcu", op, dtype))
    n = 70001
    a = make(rng, dtype, (n,))
    b = a.copy()
    flip = rng.random(n) < 0.5
    b[flip] = make(rng, dtype, (int(flip.sum()),))
    A, B = to_gpu(a), to_gpu(b)
    ref = torch.empty(n, dtype=torch.bool, device="cuda:0")
    ours = torch.empty_like(ref)
    epsilons = (0.0, 0.37) if (op in ("equal", "notequal") and dtype in ("float64", "float32")) else (0.0,)
    for eps in epsilons:
        R.check(lib.refcu_compare(code, CODES[dtype], A.data_ptr(), B.data_ptr(), eps, ref.data_ptr(), n))
        if op in ("equal", "notequal"):
            getattr(TF, op)(A, B, eps, ours)
            want = getattr(O, op)(a, b, eps)
        else:
            getattr(TF, op)(A, B, ours)
            want = getattr(O, op)(a, b)
        assert np.array_equal(to_np(ref), want), f"reference {op}<{dtype}> eps={eps} vs oracle"
        assert np.array_equal(to_np(ours), to_np(ref)), f"ours {op}<{dtype}> eps={eps} vs reference"
        sv = 3 if dtype in INTS else float(a[5])
        R.check(lib.refcu_compare_scalar(code, CODES[dtype], A.data_ptr(), float(sv), int(sv), eps, ref.data_ptr(), n))
        name = op + "scalar"
        if op in ("equal", "notequal"):
            getattr(TF, name)(A, sv, eps, ours)
            want = getattr(O, name)(a, sv, eps)
        else:
            getattr(TF, name)(A, sv, ours)
            want = getattr(O, name)(a, sv)
        assert np.array_equal(to_np(ref), want), f"reference {name}<{dtype}> eps={eps} vs oracle"
        assert np.array_equal(to_np(ours), to_np(ref)), f"ours {name}<{dtype}> eps={eps} vs reference"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "int64", "int8"])
def test_switch(R, mods, dtype):
    TF, O = mods
    lib = R.load()
    rng = np.random.default_rng(seed_of("refcu", "switch", dtype))
    n = 50021
    srcs = [make(rng, dtype, (n,)) for _ in range(3)]
    S = [to_gpu(s) for s in srcs]
    ref, ours = torch.empty_like(S[0]), torch.empty_like(S[0])
    for k, cases in ((3, rng.integers(0, 3, n).astype(np.int32)), (2, rng.integers(0, 2, n).astype(np.bool_))):
        Cs = to_gpu(cases)
        ptrs = (C.c_void_p * k)(*[S[i].data_ptr() for i in range(k)])
        R.check(lib.refcu_switch(CODES[dtype], ptrs, k, CODES["bool" if cases.dtype == np.bool_ else "int32"], Cs.data_ptr(), ref.data_ptr(), n))
        TF.Switch(S[:k], Cs, ours)
        assert_bit_exact(to_np(ref), O.Switch(srcs[:k], cases), f"reference switch<{dtype}> k={k} vs oracle")
        assert_bit_exact(to_np(ours), to_np(ref), f"ours switch<{dtype}> k={k} vs reference")


@pytest.mark.parametrize("src,dst", [("float32", "int32"), ("float32", "bfloat16"), ("float32", "float16"), ("float64", "float32"),
                                     ("int32", "float32"), ("int64", "int8"), ("bfloat16", "float32"), ("int8", "float64"),
                                     ("float16", "int16"), ("int16", "bfloat16")])
def test_todtype(R, mods, src, dst):
    TF, O = mods
    lib = R.load()
    rng = np.random.default_rng(seed_of("refcu", "cast", src, dst))
    n = 65539
    a = make(rng, src, (n,), -100.0, 100.0)
    A = to_gpu(a)
    ref = torch.empty(n, dtype=to_gpu(np.zeros(1, NP_DTYPES[dst])).dtype, device="cuda:0")
    ours = torch.empty_like(ref)
    R.check(lib.refcu_cast(CODES[src], A.data_ptr(), CODES[dst], ref.data_ptr(), n))
    TF.todtype(A, ours)
    assert_bit_exact(to_np(ref), O.todtype(a, NP_DTYPES[dst]), f"reference todtype {src}->{dst} vs oracle")
    assert_bit_exact(to_np(ours), to_np(ref), f"ours todtype {src}->{dst} vs reference")


@pytest.mark.parametrize("dims", [[0], [1], [2], [0, 1], [1, 2], [0, 2], [0, 1, 2]])
@pytest.mark.parametrize("keepdims", [False, True])
def test_sum(R, mods, dims, keepdims):
    TF, O = mods
    lib = R.load()
    rng = np.random.default_rng(seed_of("refcu", "sum", dims, keepdims))
    shape = (13, 33, 65)
    k = rng.integers(-100, 101, shape).astype(np.int32)
    x = rng.standard_normal(shape, dtype=np.float32)
    # Every axis reduced without keepdims: the reference's kernel then builds no output index at all and reads an
    # uninitialised one (reduce_miaobyte.cu:33-46 with result_dim 1 from reducedShape's [1]); that case is not run
    # on the reference, the oracle and this library are still compared with float64.
    run_reference = keepdims or len(dims) < 3
    for a, code, exact in ((k, CODES["int32"], True), (x, CODES["float32"], False)):
        want = O.sum(a, dims, keepdims)
        A = to_gpu(a)
        ref = torch.full(want.shape, 7, dtype=A.dtype, device="cuda:0")
        ours = torch.empty_like(ref)
        TF.sum(A, dims, keepdims, ours)
        if run_reference:
            R.check(lib.refcu_sum(code, A.data_ptr(), R.i64(shape), 3, R.i32(dims), len(dims), int(keepdims), ref.data_ptr()))
        else:
            ref.copy_(ours)
        if exact:
            assert_bit_exact(to_np(ref), want, f"reference sum<int32> {dims} vs oracle")
            assert_bit_exact(to_np(ours), want, f"ours sum<int32> {dims} vs oracle")
        else:
            scale = O.sum(np.abs(a), dims, keepdims).astype(np.float64)
            w64 = a.astype(np.float64).sum(axis=tuple(dims), keepdims=keepdims).reshape(want.shape)
            for got, who in ((to_np(ref), "reference"), (to_np(ours), "ours"), (want, "oracle")):
                assert (np.abs(got.astype(np.float64) - w64) <= 1e-5 * scale).all(), f"{who} sum<float32> {dims} outside 1e-5 of sum|x|"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "int64", "int8"])
def test_changeshape(R, mods, dtype):
    TF, O = mods
    lib = R.load()
    rng = np.random.default_rng(seed_of("refcu", "changeshape", dtype))
    code = CODES[dtype]
    a = make(rng, dtype, (6, 17, 5, 32))
    A = to_gpu(a)
    for order in ([0, 2, 1, 3], [3, 2, 1, 0], [1, 0, 3, 2]):
        want = O.transpose(a, order)
        ref = torch.empty(want.shape, dtype=A.dtype, device="cuda:0")
        ours = torch.empty_like(ref)
        R.check(lib.refcu_transpose(code, A.data_ptr(), R.i64(a.shape), 4, R.i32(order), ref.data_ptr()))
        TF.transpose(A, order, ours)
        assert_bit_exact(to_np(ref), want, f"reference transpose<{dtype}> {order} vs oracle")
        assert_bit_exact(to_np(ours), to_np(ref), f"ours transpose<{dtype}> {order} vs reference")
    for src_shape, to in (((1, 64), (33, 64)), ((7, 1, 5), (3, 7, 9, 5)), ((1,), (4, 100))):
        s = make(rng, dtype, src_shape)
        S = to_gpu(s)
        want = O.broadcastTo(s, to)
        ref = torch.empty(to, dtype=S.dtype, device="cuda:0")
        ours = torch.empty_like(ref)
        R.check(lib.refcu_broadcast_to(code, S.data_ptr(), R.i64(src_shape), len(src_shape), R.i64(to), len(to), ref.data_ptr()))
        TF.broadcastTo(S, list(to), ours)
        assert_bit_exact(to_np(ref), want, f"reference broadcastTo<{dtype}> {src_shape}->{to} vs oracle")
        assert_bit_exact(to_np(ours), to_np(ref), f"ours broadcastTo<{dtype}> {src_shape}->{to} vs reference")
    table = make(rng, dtype, (301, 48))
    T = to_gpu(table)
    for idx_dtype, axis, extent in ((np.int32, 0, 301), (np.int64, 1, 48)):
        idx = rng.integers(0, extent, (5, 11)).astype(idx_dtype)
        I = to_gpu(idx)
        want = O.indexselect(table, idx, axis)
        ref = torch.empty(want.shape, dtype=T.dtype, device="cuda:0")
        ours = torch.empty_like(ref)
        R.check(lib.refcu_indexselect(code, T.data_ptr(), R.i64(table.shape), 2, CODES[np.dtype(idx_dtype).name], I.data_ptr(), R.i64(idx.shape), 2,
                                      axis, ref.data_ptr()))
        TF.indexselect(T, I, axis, ours)
        assert_bit_exact(to_np(ref), want, f"reference indexselect<{dtype}> axis {axis} vs oracle")
        assert_bit_exact(to_np(ours), to_np(ref), f"ours indexselect<{dtype}> axis {axis} vs reference")


def test_matmul_float32(R, mods):
    """cuBLAS Sgemm as the reference calls it (matmul_cublas.hpp:16-80) against the oracle's GEMM and ours."""
    TF, O = mods
    lib = R.load()
    rng = np.random.default_rng(11)
    for shape_a, shape_b in (((64, 96), (96, 40)), ((3, 33, 20), (3, 20, 17))):
        a = rng.standard_normal(shape_a, dtype=np.float32)
        b = rng.standard_normal(shape_b, dtype=np.float32)
        A, B = to_gpu(a), to_gpu(b)
        want = O.matmul(a, b)
        ref = torch.empty(want.shape, dtype=torch.float32, device="cuda:0")
        ours = torch.empty_like(ref)
        R.check(lib.refcu_matmul(CODES["float32"], A.data_ptr(), B.data_ptr(), ref.data_ptr(), R.i64(shape_a), R.i64(shape_b), len(shape_a)))
        TF.matmul(A, B, ours)
        w64 = a.astype(np.float64) @ b.astype(np.float64)
        bound = 1e-5 * np.abs(w64) + 2e-6 * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64))
        for got, who in ((to_np(ref), "reference"), (to_np(ours), "ours"), (want, "oracle")):
            assert (np.abs(got.astype(np.float64) - w64) <= bound).all(), f"{who} matmul {shape_a}x{shape_b} outside the float32 bound"
