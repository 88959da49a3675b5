"""GPU parity: sum / prod / reducemax / reducemin through the C ABI vs the CPU oracle.

Bar: integer results and max/min bit-exact; float sum within 1e-5 (fp32), 1e-12 (fp64),
1e-2 (16-bit) of a float64 reference, relative to Σ|x| per output (a sum of mixed-sign
terms is ill-conditioned relative to |Σx|); float prod within the same relative bounds.
"""
import itertools

import numpy as np
import pytest
import torch

from helpers import ALL_NUMERIC, FLOATS, INTS, NP_DTYPES, assert_bit_exact, make, seed_of, to_gpu, to_np

pytestmark = pytest.mark.gpu

SUM_TOL = {"float64": 1e-12, "float32": 1e-5, "float16": 1e-2, "bfloat16": 1e-2}


@pytest.fixture(scope="module")
def mods():
    from deepx_b200 import tensorfunc as TF
    from oracle import oracle as O
    return TF, O


def run(TF, O, op, a, dims, keepdims):
    A = to_gpu(a)
    cd = O.checked_dims(a.shape, dims)
    out = torch.empty(O.reduced_shape(a.shape, cd, keepdims), dtype=A.dtype, device=A.device)
    getattr(TF, op)(A, dims, keepdims, out)
    return to_np(out)


def check(TF, O, op, a, dims, keepdims, dtype, what):
    got = run(TF, O, op, a, dims, keepdims)
    want = getattr(O, op)(a, dims, keepdims)
    if dtype in INTS or op in ("reducemax", "reducemin"):
        assert_bit_exact(got, want, what)
        return
    cd = tuple(O.checked_dims(a.shape, dims))
    a64 = a.astype(np.float64)
    if op == "sum":
        ref = a64.sum(axis=cd, keepdims=keepdims).reshape(want.shape)
        scale = np.abs(a64).sum(axis=cd, keepdims=keepdims).reshape(want.shape)
    else:
        ref = a64.prod(axis=cd, keepdims=keepdims).reshape(want.shape)
        scale = np.abs(ref)
    err = np.abs(got.astype(np.float64) - ref)
    tol = SUM_TOL[dtype]
    assert (err <= tol * scale + 1e-300).all(), f"{what}: max err/scale {np.max(err / np.maximum(scale, 1e-300))}"
    # and the oracle (sequential, same precision) sits inside the same band
    assert (np.abs(want.astype(np.float64) - ref) <= 10 * tol * scale + 1e-300).all()


@pytest.mark.parametrize("op", ["sum", "prod", "reducemax", "reducemin"])
def test_all_axis_subsets_3d(mods, op):
    """Every axis subset of a [3,4,5] tensor, keepdims on and off (the shape table of
    executor/op-ompsimd/test/tensorfunc/5_tensor_sum.cpp:21-50)."""
    TF, O = mods
    rng = np.random.default_rng(1)
    for dtype in ["float32", "int32"]:
        a = make(rng, dtype, (3, 4, 5), 0.5, 1.5)
        for r in range(0, 4):
            for dims in itertools.combinations(range(3), r):
                for keep in (False, True):
                    check(TF, O, op, a, list(dims), keep, dtype, f"{op}<{dtype}> dims={dims} keep={keep}")


SHAPE_CASES = [
    # (shape, dims): rows/team, rows/block, rows/split, cols, cols/split, mixed groups, odd extents
    ((1000, 7), [1]), ((1000, 896), [1]), ((64, 8192), [1]), ((3, 70001), [1]), ((1, 300000), [1]),
    ((300000,), [0]), ((2, 3, 50000), [1, 2]), ((8192, 16), [0]), ((5000, 129), [0]), ((37, 4096), [0]),
    ((7, 33, 65), [1]), ((7, 33, 64), [0, 2]), ((6, 5, 4, 3, 8), [1, 3]), ((6, 5, 4, 3, 8), [0, 2, 4]),
    ((4, 1, 9, 1, 16), [2]), ((2, 2, 2, 2, 2, 2, 2, 2, 2, 2, 2, 2), [0, 3, 5, 6, 11]), ((5,), []),
    ((17, 4), [0]), ((17, 4), [1]), ((1, 1), [0, 1]), ((9, 1), [1]),
]


@pytest.mark.parametrize("dtype", ["float32", "int32", "bfloat16", "int8", "float64", "int64"])
@pytest.mark.parametrize("case", SHAPE_CASES, ids=[f"{s}-{d}" for s, d in SHAPE_CASES])
def test_sum_shapes(mods, case, dtype):
    TF, O = mods
    shape, dims = case
    rng = np.random.default_rng(seed_of(shape, dims, dtype))
    a = make(rng, dtype, shape, -1.0, 1.0)
    check(TF, O, "sum", a, dims, False, dtype, f"sum<{dtype}> {shape} {dims}")


@pytest.mark.parametrize("dtype", ALL_NUMERIC)
@pytest.mark.parametrize("op", ["reducemax", "reducemin"])
def test_maxmin_dtypes(mods, op, dtype):
    TF, O = mods
    rng = np.random.default_rng(seed_of(op, dtype))
    for shape, dims in [((257, 1031), [1]), ((257, 1031), [0]), ((33, 9, 130), [0, 2]), ((100000,), [0])]:
        a = make(rng, dtype, shape, -1000.0, 1000.0)
        check(TF, O, op, a, dims, True, dtype, f"{op}<{dtype}> {shape} {dims}")


@pytest.mark.parametrize("dtype", ["float32", "float64", "int32", "int64", "int16"])
def test_prod(mods, dtype):
    TF, O = mods
    rng = np.random.default_rng(seed_of("prod", dtype))
    if dtype in INTS:
        a = rng.integers(-3, 4, (33, 40, 7)).astype(NP_DTYPES[dtype])  # wraps: modular product must still agree
    else:
        a = make(rng, dtype, (33, 40, 7), 0.95, 1.05)  # keeps a 9240-term product inside fp32 range
    for dims in ([1], [0, 2], [2], []):
        check(TF, O, "prod", a, dims, False, dtype, f"prod<{dtype}> {dims}")


def test_integer_wraparound_sum(mods):
    TF, O = mods
    a = np.full((4, 70000), 127, dtype=np.int8)
    check(TF, O, "sum", a, [1], False, "int8", "sum<int8> wraps")
    b = np.full((3, 5), 2**62, dtype=np.int64)
    check(TF, O, "sum", b, [1], False, "int64", "sum<int64> wraps")


def test_negative_and_duplicate_dims(mods):
    TF, O = mods
    rng = np.random.default_rng(3)
    a = make(rng, "int32", (5, 6, 7))
    check(TF, O, "sum", a, [-1, 2, -3], False, "int32", "sum dims [-1,2,-3]")
    with pytest.raises(ValueError):
        TF.sum(to_gpu(a), [3], False, torch.empty(1, dtype=torch.int32, device="cuda:0"))


def test_unaligned_input(mods):
    TF, O = mods
    rng = np.random.default_rng(4)
    a = make(rng, "float32", (64 * 1000 + 1,))
    A = to_gpu(a)[1:].view(64, 1000)
    out = torch.empty(64, dtype=torch.float32, device="cuda:0")
    TF.sum(A, [1], False, out)
    ref = a[1:].reshape(64, 1000).astype(np.float64)
    assert np.abs(to_np(out) - ref.sum(1)).max() <= 1e-5 * np.abs(ref).sum(1).max()
    out0 = torch.empty(1000, dtype=torch.float32, device="cuda:0")
    TF.sum(A, [0], False, out0)
    assert np.abs(to_np(out0) - ref.sum(0)).max() <= 1e-5 * np.abs(ref).sum(0).max()


def test_deterministic(mods):
    """Same input, same bits, every time (no atomics)."""
    TF, O = mods
    rng = np.random.default_rng(8)
    a = make(rng, "float32", (3, 1 << 20))
    first = run(TF, O, "sum", a, [1], False)
    for _ in range(3):
        assert_bit_exact(run(TF, O, "sum", a, [1], False), first, "repeat")
    first0 = run(TF, O, "sum", a.reshape(1 << 10, 3 << 10), [0], False)
    assert_bit_exact(run(TF, O, "sum", a.reshape(1 << 10, 3 << 10), [0], False), first0, "repeat cols")


def test_split_reduction_on_many_streams(mods):
    """A reduction split over several CTAs per output finishes itself on counters inside the library, one bank per
    stream; a stream beyond the banks takes the form with a finish kernel.  Ten streams at once, two shapes each (one
    output split 4000-fold, 300 outputs split a few times): every result has the bits of the default stream's."""
    TF, O = mods
    rng = np.random.default_rng(21)
    a = to_gpu(make(rng, "float32", (300, 1 << 19)))
    want_all = torch.empty(1, dtype=torch.float32, device="cuda:0")
    want_rows = torch.empty(300, dtype=torch.float32, device="cuda:0")
    TF.sum(a, [0, 1], False, want_all)
    TF.reducemax(a, [1], False, want_rows)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in range(10)]
    outs = [(torch.empty_like(want_all), torch.empty_like(want_rows)) for _ in streams]
    for _ in range(3):
        for st, (o_all, o_rows) in zip(streams, outs):
            with torch.cuda.stream(st):
                TF.sum(a, [0, 1], False, o_all)
                TF.reducemax(a, [1], False, o_rows)
    torch.cuda.synchronize()
    for i, (o_all, o_rows) in enumerate(outs):
        assert torch.equal(o_all, want_all) and torch.equal(o_rows, want_rows), f"stream {i}"
    assert_bit_exact(to_np(want_rows), O.reducemax(to_np(a), [1], False), "row max")


def test_config_reduce_suite(mods):
    """sum and max over the last axis and over axis 0 of float32 [8192,8192] ~ N(0,1);
    sum over axes (1,2) of int32 [64,1024,1024] in [-100,100] (bit-exact)."""
    TF, O = mods
    rng = np.random.default_rng(0)
    x = rng.standard_normal((8192, 8192), dtype=np.float32)
    for dims in ([1], [0]):
        check(TF, O, "sum", x, dims, False, "float32", f"sum f32 [8192,8192] {dims}")
        check(TF, O, "reducemax", x, dims, False, "float32", f"max f32 [8192,8192] {dims}")
    k = rng.integers(-100, 101, (64, 1024, 1024)).astype(np.int32)
    check(TF, O, "sum", k, [1, 2], False, "int32", "sum i32 [64,1024,1024] (1,2)")
