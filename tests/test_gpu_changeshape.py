"""GPU parity: transpose / concat / broadcastTo / indexselect / repeat vs the CPU oracle.
Pure data movement: bit-exact for every dtype."""
import itertools

import numpy as np
import pytest
import torch

from helpers import NP_DTYPES, TORCH_DTYPES, assert_bit_exact, make, seed_of, to_gpu, to_np

pytestmark = pytest.mark.gpu

MOVE_DTYPES = ["float64", "float32", "bfloat16", "int8", "bool"]


@pytest.fixture(scope="module")
def mods():
    from deepx_b200 import tensorfunc as TF
    from oracle import oracle as O
    return TF, O


def _transpose(TF, O, a, perm, what):
    A = to_gpu(a)
    out = torch.empty([a.shape[p] for p in perm], dtype=A.dtype, device=A.device)
    TF.transpose(A, perm, out)
    assert_bit_exact(to_np(out), O.transpose(a, perm), what)


@pytest.mark.parametrize("dtype", MOVE_DTYPES)
def test_transpose_all_perms_3d(mods, dtype):
    TF, O = mods
    rng = np.random.default_rng(seed_of("tr3", dtype))
    for shape in [(3, 4, 6), (33, 65, 17), (1, 70, 130)]:
        a = make(rng, dtype, shape)
        for perm in itertools.permutations(range(3)):
            _transpose(TF, O, a, list(perm), f"transpose<{dtype}> {shape} {perm}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_transpose_4d_5d(mods, dtype):
    TF, O = mods
    rng = np.random.default_rng(seed_of("tr4", dtype))
    a = make(rng, dtype, (5, 12, 7, 16))
    for perm in itertools.permutations(range(4)):
        _transpose(TF, O, a, list(perm), f"transpose<{dtype}> 4d {perm}")
    b = make(rng, dtype, (2, 3, 4, 5, 6))
    for perm in [(4, 3, 2, 1, 0), (0, 2, 1, 4, 3), (1, 0, 3, 2, 4), (3, 4, 0, 1, 2)]:
        _transpose(TF, O, b, list(perm), f"transpose<{dtype}> 5d {perm}")


def test_transpose_swap_last_two_large(mods):
    TF, O = mods
    rng = np.random.default_rng(21)
    a = make(rng, "float32", (3, 1000, 777))
    _transpose(TF, O, a, [0, 2, 1], "transpose swap last two")
    v = make(rng, "float32", (1000,))
    _transpose(TF, O, v, [0], "transpose 1d")
    # 2-byte elements, even moving extents: the paired-word tile kernel, with ragged tiles
    for shape, perm in [((3, 1000, 778), [0, 2, 1]), ((130, 258), [1, 0]), ((2, 66, 5, 130), [3, 2, 1, 0]), ((4, 64, 128), [2, 0, 1])]:
        for dt in ("bfloat16", "int16"):
            _transpose(TF, O, make(rng, dt, shape), perm, f"transpose<{dt}> {shape} {perm}")


def test_transpose_one_byte_quad_kernel(mods):
    """1-byte elements with moving extents that are multiples of 4 take the quad-word tile kernel:
    whole and ragged 128 x 128 patches, batch axes, and shapes that must fall back to the byte kernel."""
    TF, O = mods
    rng = np.random.default_rng(22)
    for shape, perm in [((128, 128), [1, 0]), ((256, 384), [1, 0]), ((132, 260), [1, 0]), ((4, 8), [1, 0]), ((3, 1000, 776), [0, 2, 1]),
                        ((2, 68, 4, 132), [3, 2, 1, 0]), ((8, 64, 128), [2, 0, 1]), ((5, 12, 100), [2, 1, 0]),
                        ((130, 258), [1, 0]), ((7, 64, 66), [0, 2, 1])]:
        for dt in ("int8", "bool"):
            _transpose(TF, O, make(rng, dt, shape), perm, f"transpose<{dt}> {shape} {perm}")
    # an unaligned base pointer must not take the word kernel
    a = make(rng, "int8", (129, 128))
    A = to_gpu(a.reshape(-1))[128:].view(128, 128)
    out = torch.empty((128, 128), dtype=torch.int8, device="cuda:0")
    TF.transpose(A.contiguous() if False else A, [1, 0], out)
    assert_bit_exact(to_np(out), O.transpose(a[1:], [1, 0]), "transpose<int8> from an offset view")


def test_transpose_errors(mods):
    TF, _ = mods
    a = torch.zeros(2, 3, device="cuda:0")
    with pytest.raises(ValueError):
        TF.transpose(a, [0], torch.zeros(3, 2, device="cuda:0"))
    with pytest.raises(Exception):
        TF.transpose(a, [0, 0], torch.zeros(2, 2, device="cuda:0"))
    with pytest.raises(Exception):
        TF.transpose(a, [1, 0], a.view(3, 2))  # aliasing is refused, not raced


@pytest.mark.parametrize("dtype", MOVE_DTYPES)
def test_concat(mods, dtype):
    TF, O = mods
    rng = np.random.default_rng(seed_of("cat", dtype))
    for shapes, axis in [
        ([(2, 3, 4)] * 3, 0), ([(2, 3, 4)] * 3, 1), ([(2, 3, 4)] * 3, 2),
        ([(5, 1, 9), (5, 4, 9), (5, 2, 9)], 1), ([(7, 3), (7, 5), (7, 1)], 1), ([(4, 8, 32), (4, 8, 32)], 1),
        ([(3, 0, 5), (3, 2, 5)], 1), ([(100, 37)], 0),
    ]:
        ts = [make(rng, dtype, s) for s in shapes]
        Ts = [to_gpu(t) for t in ts]
        oshape = list(shapes[0])
        oshape[axis] = sum(s[axis] for s in shapes)
        out = torch.empty(oshape, dtype=TORCH_DTYPES[dtype], device="cuda:0")
        TF.concat(Ts, axis, out)
        assert_bit_exact(to_np(out), O.concat(ts, axis), f"concat<{dtype}> {shapes} axis={axis}")


def test_concat_many_inputs(mods):
    """More inputs than one launch's pointer table holds."""
    TF, O = mods
    rng = np.random.default_rng(22)
    ts = [make(rng, "float32", (6, i % 5 + 1, 8)) for i in range(37)]
    out = torch.empty((6, sum(t.shape[1] for t in ts), 8), dtype=torch.float32, device="cuda:0")
    TF.concat([to_gpu(t) for t in ts], 1, out)
    assert_bit_exact(to_np(out), O.concat(ts, 1), "concat 37 inputs")


def test_concat_shape_error(mods):
    TF, _ = mods
    a = torch.zeros(2, 3, device="cuda:0")
    with pytest.raises(ValueError):
        TF.concat([a, a], 1, torch.zeros(2, 5, device="cuda:0"))
    with pytest.raises(ValueError):
        TF.concat([a, torch.zeros(3, 3, device="cuda:0")], 1, torch.zeros(2, 6, device="cuda:0"))


@pytest.mark.parametrize("dtype", MOVE_DTYPES)
def test_broadcast_to(mods, dtype):
    TF, O = mods
    rng = np.random.default_rng(seed_of("bc", dtype))
    for ashape, oshape in [
        ((3, 2), (4, 3, 2)), ((1, 4096), (64, 4096)), ((5, 1), (5, 130)), ((1,), (1000,)), ((7, 1, 3), (2, 7, 9, 3)),
        ((1, 6, 1, 4), (3, 6, 5, 4)), ((4, 1, 1), (4, 33, 17)), ((2, 3), (2, 3)), ((1, 1), (77, 5)), ((16,), (3, 5, 16)),
    ]:
        a = make(rng, dtype, ashape)
        out = torch.empty(oshape, dtype=TORCH_DTYPES[dtype], device="cuda:0")
        TF.broadcastTo(to_gpu(a), list(oshape), out)
        assert_bit_exact(to_np(out), O.broadcastTo(a, oshape), f"broadcastTo<{dtype}> {ashape}->{oshape}")
    with pytest.raises(ValueError):
        TF.broadcastTo(to_gpu(make(rng, dtype, (3, 2))), [4, 3, 3], torch.empty((4, 3, 3), dtype=TORCH_DTYPES[dtype], device="cuda:0"))


@pytest.mark.parametrize("dtype", MOVE_DTYPES)
@pytest.mark.parametrize("idt", ["int32", "int64"])
def test_indexselect(mods, dtype, idt):
    TF, O = mods
    rng = np.random.default_rng(seed_of("gather", dtype, idt))
    for ashape, ishape, axis in [
        ((50, 896), (8, 20), 0), ((7, 9, 5), (4,), 1), ((7, 9, 5), (2, 3), 2), ((7, 9, 5), (6,), -1),
        ((100, 3), (1000,), 0), ((4, 33), (5, 1, 2), 1), ((10,), (3, 3), 0),
        ((37, 100), (64,), 1), ((5, 6, 1000), (2, 16), 2), ((3, 70), (4, 8, 4), -1), ((9,), (32,), 0),  # innermost-axis vector kernel
        ((100, 100), (64,), 1), ((70, 3, 40), (2, 16), 2), ((65, 1000), (16,), 1), ((1000, 7), (48,), -1), ((333, 4096), (16,), 1),  # staged in shared memory
    ]:
        a = make(rng, dtype, ashape)
        g = axis + len(ashape) if axis < 0 else axis
        idx = rng.integers(0, ashape[g], ishape).astype(NP_DTYPES[idt])
        out = torch.empty(TF.indexselect_shape(ashape, ishape, g), dtype=TORCH_DTYPES[dtype], device="cuda:0")
        TF.indexselect(to_gpu(a), to_gpu(idx), axis, out)
        assert_bit_exact(to_np(out), O.indexselect(a, idx, axis), f"indexselect<{dtype},{idt}> {ashape} {ishape} {axis}")


def test_indexselect_out_of_range_is_flagged(mods):
    TF, O = mods
    a = np.arange(12, dtype=np.float32).reshape(4, 3)
    idx = np.array([0, 7, -1, 3], dtype=np.int32)
    out = torch.empty((4, 3), dtype=torch.float32, device="cuda:0")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    TF.indexselect(to_gpu(a), to_gpu(idx), 0, out, flag)
    assert_bit_exact(to_np(out), O.indexselect(a, idx, 0), "indexselect oob rows are zero")
    assert int(flag.item()) == 1
    # the same along the innermost axis (the vector kernel): 16 indices, three of them out of range
    idx2 = np.array([0, 2, 9, 1, -4, 2, 2, 1, 0, 0, 3, 1, 2, 0, 1, 2], dtype=np.int32)
    out2 = torch.empty((4, 16), dtype=torch.float32, device="cuda:0")
    flag.zero_()
    TF.indexselect(to_gpu(a), to_gpu(idx2), 1, out2, flag)
    assert_bit_exact(to_np(out2), O.indexselect(a, idx2, 1), "indexselect oob elements are zero")
    assert int(flag.item()) == 1
    big = np.arange(128 * 3, dtype=np.float32).reshape(128, 3)   # 128 rows: the staged kernel
    out3 = torch.empty((128, 16), dtype=torch.float32, device="cuda:0")
    flag.zero_()
    TF.indexselect(to_gpu(big), to_gpu(idx2), 1, out3, flag)
    assert_bit_exact(to_np(out3), O.indexselect(big, idx2, 1), "indexselect oob elements are zero (staged)")
    assert int(flag.item()) == 1


@pytest.mark.parametrize("dtype", ["float32", "int8"])
def test_repeat(mods, dtype):
    TF, O = mods
    rng = np.random.default_rng(seed_of("rep", dtype))
    for ashape, rep in [((3, 4), (2, 3)), ((5,), (7,)), ((2, 3, 4), (1, 1, 1)), ((2, 1, 5), (3, 4, 2)),
                        ((4, 8, 33, 64), (1, 4, 1, 1)),        # the KV-head repeat of grouped-query attention
                        ((4, 64), (1, 2)), ((3, 5, 32), (2, 1, 4)), ((2, 3, 4, 16), (3, 1, 2, 8)), ((7, 48), (1, 64)),  # innermost-repeat kernel
                        ((6, 130), (2, 1)), ((6, 130), (1, 3)), ((3, 5, 7), (2, 2, 2)), ((1, 1, 1), (2, 3, 4)),
                        ((2, 2, 2, 2, 2, 2), (2, 1, 2, 1, 2, 3)),  # 6 axes x 2 = 11 axis pairs: still word-wide
                        ((2, 1, 2, 1, 2, 1, 2), (2, 2, 2, 2, 2, 2, 2))]:  # 14 > 12: the per-element kernel
        a = make(rng, dtype, ashape)
        out = torch.empty([s * r for s, r in zip(ashape, rep)], dtype=TORCH_DTYPES[dtype], device="cuda:0")
        TF.repeat(to_gpu(a), list(rep), out)
        assert_bit_exact(to_np(out), O.repeat(a, rep), f"repeat<{dtype}> {ashape} {rep}")


def test_config_changeshape_suite(mods):
    """transpose perm [0,2,1,3] of bf16 [32,2048,32,128]; concat of four f32 [8,1024,4096] on axis 1;
    broadcastTo f32 [1,4096]→[8192,4096]; indexselect of f32 [151936,896] with int32 [8,2048]."""
    TF, O = mods
    rng = np.random.default_rng(0)
    t = rng.standard_normal((32, 2048, 32, 128), dtype=np.float32).astype(NP_DTYPES["bfloat16"])
    _transpose(TF, O, t, [0, 2, 1, 3], "transpose bf16 [32,2048,32,128]")
    del t
    parts = [np.random.default_rng(s).standard_normal((8, 1024, 4096), dtype=np.float32) for s in range(4)]
    out = torch.empty((8, 4096, 4096), dtype=torch.float32, device="cuda:0")
    TF.concat([to_gpu(p) for p in parts], 1, out)
    assert_bit_exact(to_np(out), O.concat(parts, 1), "concat 4x[8,1024,4096]")
    del parts, out
    r = rng.standard_normal((1, 4096), dtype=np.float32)
    out = torch.empty((8192, 4096), dtype=torch.float32, device="cuda:0")
    TF.broadcastTo(to_gpu(r), [8192, 4096], out)
    assert_bit_exact(to_np(out), O.broadcastTo(r, [8192, 4096]), "broadcastTo [1,4096]->[8192,4096]")
    del out
    table = (rng.standard_normal((151936, 896), dtype=np.float32) * np.float32(0.02))
    idx = rng.integers(0, 151936, (8, 2048)).astype(np.int32)
    out = torch.empty((8, 2048, 896), dtype=torch.float32, device="cuda:0")
    TF.indexselect(to_gpu(table), to_gpu(idx), 0, out)
    assert_bit_exact(to_np(out), O.indexselect(table, idx, 0), "indexselect [151936,896] x [8,2048]")
