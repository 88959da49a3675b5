"""Randomised parity (hypothesis, derandomised so every run draws the same cases): shapes of rank
1–6 with extents that are odd, one, or zero; every axis subset and permutation; every dtype.
The CUDA result through the C ABI must equal the CPU oracle — bit for bit for data movement,
integer arithmetic, compares, max/min and IEEE float add/sub/mul/div; within the float-sum
tolerance for float sum.
"""
import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from helpers import ALL_NUMERIC, INTS, NP_DTYPES, TORCH_DTYPES, assert_bit_exact, make, to_gpu, to_np

pytestmark = pytest.mark.gpu
SETTINGS = dict(max_examples=60, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))


@pytest.fixture(scope="module")
def mods():
    from deepx_b200 import tensorfunc as TF
    from oracle import oracle as O
    return TF, O


def shapes(min_rank=1, max_rank=5, max_elems=60000, allow_zero=False):
    lo = 0 if allow_zero else 1
    return st.lists(st.sampled_from([lo, 1, 2, 3, 5, 7, 8, 16, 31, 33, 64, 100, 129]), min_size=min_rank, max_size=max_rank).filter(
        lambda s: int(np.prod(s)) <= max_elems)


@settings(**SETTINGS)
@given(shape=shapes(allow_zero=True), dtype=st.sampled_from(ALL_NUMERIC), op=st.sampled_from(["add", "sub", "mul", "max", "min"]),
       seed=st.integers(0, 2**31))
def test_binary_any_shape(mods, shape, dtype, op, seed):
    TF, O = mods
    rng = np.random.default_rng(seed)
    a, b = make(rng, dtype, shape), make(rng, dtype, shape)
    A, B = to_gpu(a), to_gpu(b)
    out = torch.empty_like(A)
    getattr(TF, op)(A, B, out)
    assert_bit_exact(to_np(out), getattr(O, op)(a, b), f"{op}<{dtype}> {shape}")


@settings(**SETTINGS)
@given(shape=shapes(allow_zero=True), dtype=st.sampled_from(ALL_NUMERIC), op=st.sampled_from(["less", "greater", "equal", "notequal"]),
       seed=st.integers(0, 2**31))
def test_compare_any_shape(mods, shape, dtype, op, seed):
    TF, O = mods
    rng = np.random.default_rng(seed)
    a = make(rng, dtype, shape)
    b = np.where(rng.random(a.shape) < 0.3, a, make(rng, dtype, shape)).astype(a.dtype)
    A, B = to_gpu(a), to_gpu(b)
    mask = torch.empty(a.shape, dtype=torch.bool, device=A.device)
    if op in ("equal", "notequal"):
        getattr(TF, op)(A, B, 0.0, mask)
        want = getattr(O, op)(a, b, 0.0)
    else:
        getattr(TF, op)(A, B, mask)
        want = getattr(O, op)(a, b)
    assert_bit_exact(to_np(mask), want, f"{op}<{dtype}> {shape}")


@settings(**SETTINGS)
@given(data=st.data(), shape=shapes(max_rank=6), dtype=st.sampled_from(ALL_NUMERIC), op=st.sampled_from(["sum", "reducemax", "reducemin", "prod"]),
       keepdims=st.booleans(), seed=st.integers(0, 2**31))
def test_reduce_any_axes(mods, data, shape, dtype, op, keepdims, seed):
    TF, O = mods
    rank = len(shape)
    dims = data.draw(st.lists(st.integers(-rank, rank - 1), min_size=0, max_size=rank, unique_by=lambda d: d % rank))
    if op == "prod" and int(np.prod(shape)) > 4096:
        op = "sum"  # a long float product leaves the normal range; the short ones cover prod
    rng = np.random.default_rng(seed)
    a = make(rng, dtype, shape, 0.9, 1.1) if op == "prod" and dtype not in INTS else make(rng, dtype, shape)
    if op == "prod" and dtype in INTS:
        a = np.where(a % 5 == 0, 2, 1).astype(a.dtype)
    A = to_gpu(a)
    cd = O.checked_dims(a.shape, dims)
    out = torch.empty(O.reduced_shape(a.shape, cd, keepdims), dtype=A.dtype, device=A.device)
    getattr(TF, op)(A, dims, keepdims, out)
    got, want = to_np(out), getattr(O, op)(a, dims, keepdims)
    if dtype in INTS or op in ("reducemax", "reducemin"):
        assert_bit_exact(got, want, f"{op}<{dtype}> {shape} dims {dims}")
    else:
        a64 = a.astype(np.float64)
        axes = tuple(cd)
        ref = (a64.sum(axis=axes, keepdims=keepdims) if op == "sum" else a64.prod(axis=axes, keepdims=keepdims)).reshape(want.shape)
        scale = (np.abs(a64).sum(axis=axes, keepdims=keepdims) if op == "sum" else np.abs(ref)).reshape(want.shape)
        tol = {"float64": 1e-12, "float32": 1e-5}.get(dtype, 1e-2)
        assert (np.abs(got.astype(np.float64) - ref) <= tol * scale + 1e-300).all(), f"{op}<{dtype}> {shape} dims {dims}"


@settings(**SETTINGS)
@given(data=st.data(), shape=shapes(max_rank=6, allow_zero=True), dtype=st.sampled_from(["float64", "float32", "bfloat16", "int16", "int8", "bool"]),
       seed=st.integers(0, 2**31))
def test_transpose_any_permutation(mods, data, shape, dtype, seed):
    TF, O = mods
    perm = data.draw(st.permutations(range(len(shape))))
    a = make(np.random.default_rng(seed), dtype, shape)
    A = to_gpu(a)
    out = torch.empty([shape[p] for p in perm], dtype=A.dtype, device=A.device)
    TF.transpose(A, list(perm), out)
    assert_bit_exact(to_np(out), O.transpose(a, list(perm)), f"transpose<{dtype}> {shape} {perm}")


@settings(**SETTINGS)
@given(data=st.data(), shape=shapes(max_rank=4, max_elems=20000), dtype=st.sampled_from(["float32", "bfloat16", "int64", "int8"]),
       seed=st.integers(0, 2**31))
def test_concat_and_broadcast(mods, data, shape, dtype, seed):
    TF, O = mods
    rng = np.random.default_rng(seed)
    axis = data.draw(st.integers(0, len(shape) - 1))
    k = data.draw(st.integers(1, 5))
    parts = []
    for _ in range(k):
        s = list(shape)
        s[axis] = data.draw(st.sampled_from([1, 2, 3, 8, 17]))
        parts.append(make(rng, dtype, s))
    want = O.concat(parts, axis)
    out = torch.empty(want.shape, dtype=TORCH_DTYPES[dtype], device="cuda:0")
    TF.concat([to_gpu(p) for p in parts], axis, out)
    assert_bit_exact(to_np(out), want, f"concat<{dtype}> {shape} axis {axis} x{k}")
    # broadcastTo: collapse a random subset of axes to 1, add leading axes, expand back
    src_shape = [1 if data.draw(st.booleans()) else d for d in shape]
    lead = data.draw(st.lists(st.sampled_from([1, 2, 3]), max_size=2))
    src = make(rng, dtype, src_shape)
    target = lead + list(shape)
    if int(np.prod(target)) <= 200000:
        bo = torch.empty(target, dtype=TORCH_DTYPES[dtype], device="cuda:0")
        TF.broadcastTo(to_gpu(src), target, bo)
        assert_bit_exact(to_np(bo), O.broadcastTo(src, target), f"broadcastTo<{dtype}> {src_shape} -> {target}")


@settings(**SETTINGS)
@given(data=st.data(), shape=shapes(max_rank=4, max_elems=20000), dtype=st.sampled_from(["float32", "bfloat16", "int8"]),
       itype=st.sampled_from(["int32", "int64"]), seed=st.integers(0, 2**31))
def test_indexselect_any_axis(mods, data, shape, dtype, itype, seed):
    TF, O = mods
    rng = np.random.default_rng(seed)
    axis = data.draw(st.integers(0, len(shape) - 1))
    ishape = data.draw(st.lists(st.sampled_from([1, 2, 3, 7]), min_size=1, max_size=2))
    a = make(rng, dtype, shape)
    idx = rng.integers(0, shape[axis], ishape).astype(NP_DTYPES[itype])
    want = O.indexselect(a, idx, axis)
    out = torch.empty(want.shape, dtype=TORCH_DTYPES[dtype], device="cuda:0")
    TF.indexselect(to_gpu(a), to_gpu(idx), axis, out)
    assert_bit_exact(to_np(out), want, f"indexselect<{dtype}> {shape} axis {axis} idx {ishape}")
