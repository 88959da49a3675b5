"""CPU tests: the oracle, the IR parser, the op registry and the shape algebra against fixtures
generated from the REFERENCE's own code (tests/golden/reference_golden.json, made by
tests/golden/make_golden.py from oracle/_ref), against the known answers printed in the
reference's test sources, and — where oracle/_ref is present — live against that library."""
import ctypes as C
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle as O

GOLD = json.loads((Path(__file__).parent / "golden" / "reference_golden.json").read_text())


# ---- IR parser / dtype codec / registry (host C++ core, no GPU needed) ---------------------------
@pytest.fixture(scope="module")
def E():
    from deepx_b200 import executor
    return executor


def test_ir_parse_matches_reference(E):
    for case in GOLD["ir_parse"]:
        assert E.parse_ir(case["line"]) == case["parsed"], case["line"]


def test_ir_parse_missing_arrow_is_an_error(E):
    assert E.parse_ir("add(a,b)") == "!Invalid IR format: missing arrow"


def test_dtype_roundtrip_matches_reference(E):
    for case in GOLD["dtype"]:
        assert E.dtype_roundtrip(case["text"]) == case["out"], case["text"]


def test_registry_matching_matches_reference(E):
    reg = E.Registry()
    for sig in GOLD["registry"]["signatures"]:
        reg.add(sig)
    for case in GOLD["registry"]["calls"]:
        got = reg.get(case["call"])
        if case["author_known"]:
            assert got == case["index"], case["call"]
        else:
            # unknown author: the reference falls back to unordered_map::begin() (unspecified order);
            # here it is the first author registered for the op.  Either way one of them must match.
            assert got in (0, 1), case["call"]


def test_builtin_op_table(E):
    """Every op name / author the reference registers (executor/op-cuda/src/client/tfs.cpp) resolves."""
    reg = E.Registry(builtin=True)
    assert len(reg) == 63  # the 63 registrations of tfs.cpp
    calls = [
        "add(tensor<float32>:a, tensor<float32>:b)->(tensor<float32>:c) // author=miaobyte",
        "add(tensor<float32>:a, tensor<float32>:b)->(tensor<float32>:c) // author=cublas",
        "matmul(tensor<bfloat16>:a, tensor<bfloat16>:b)->(tensor<bfloat16>:c) // author=cublas",
        "sum(tensor<int32>:a, vector<int32>:[1 2], var<bool>:false)->(tensor<int32>:b) // author=miaobyte",
        "newtensor(vector<int32>:[3 4])->(tensor<float32>:t)",
        "deltensor()->(tensor<float32>:t)",
        "switch(listtensor<float32>:[a b], tensor<bool>:m)->(tensor<float32>:c) // author=miaobyte",
        "indexselect(tensor<float32>:A, tensor<int32>:i, var<int32>:0)->(tensor<float32>:B) // author=miaobyte",
        "powscalar(tensor<float32>:A, var<int32>:2)->(tensor<float32>:C) // author=miaobyte",
        "invert(tensor<bool>:a)->(tensor<bool>:c) // author=miaobyte",
        "print(tensor<float32>:t, var<string>:%.4f)->() // author=miaobyte",
    ]
    for c in calls:
        assert reg.get(c) == -2, c  # -2 = resolved to a built-in op
    for c in ["pow(tensor<int32>:a, tensor<int32>:b)->(tensor<int32>:c) // author=miaobyte",
              "sqrt(tensor<int32>:a)->(tensor<int32>:c) // author=miaobyte",
              "nosuchop(tensor<float32>:a)->(tensor<float32>:b)",
              "indexselect(tensor<float32>:A, tensor<float32>:i, var<int32>:0)->(tensor<float32>:B) // author=miaobyte"]:
        assert reg.get(c) == -1, c


# ---- shape algebra ------------------------------------------------------------------------------------
def test_shape_algebra_matches_reference():
    from deepx_b200 import tensorfunc as TF
    for s in GOLD["shapes"]:
        if s["fn"] == "reduced":
            if s["checked"] is None:
                with pytest.raises(ValueError):
                    TF.checked_dims(s["shape"], s["dims"])
                with pytest.raises(ValueError):
                    O.checked_dims(s["shape"], s["dims"])
                continue
            for impl in (TF, O):
                cd = impl.checked_dims(s["shape"], s["dims"])
                assert cd == s["checked"]
                assert impl.reduced_shape(s["shape"], cd, bool(s["keepdims"])) == s["out"]
        elif s["fn"] == "indexselect":
            assert TF.indexselect_shape(s["a"], s["idx"], s["axis"]) == s["out"]
        elif s["fn"] == "matmul":
            same_rank_ok = TF.check_matmul_shape(s["a"], s["b"])
            if s["out"] is None:
                assert not same_rank_ok
            else:
                assert same_rank_ok and s["a"][:-1] + [s["b"][-1]] == s["out"]
        elif s["fn"] == "transpose":
            assert [s["shape"][o] for o in s["order"]] == s["out"]
        elif s["fn"] == "broadcast":
            try:
                want = list(np.broadcast_shapes(tuple(s["a"]), tuple(s["b"])))
            except ValueError:
                want = []
            assert want == s["out"]
        elif s["fn"] == "repeat":
            assert [a * r for a, r in zip(s["shape"], s["repeats"])] == s["out"]


def test_sum_shape_table_of_reference_test():
    table = GOLD["known"]["sum_shapes_2x3x4"]  # 5_tensor_sum.cpp:41-48
    for dims_text, want in table.items():
        dims = json.loads(dims_text)
        # "[] => [2,3,4]" in that table is the identity row (no axis reduced); the executor treats an
        # empty dims vector as "all axes" (checkedDims), so it is the one row to skip.
        if not dims:
            continue
        assert O.reduced_shape([2, 3, 4], O.checked_dims([2, 3, 4], dims), False) == want


# ---- oracle vs fixtures made by the reference's changeshape code --------------------------------------------
def test_oracle_changeshape_matches_reference_outputs():
    for c in GOLD["changeshape"]:
        want = np.array(c["out"], dtype=np.int32)
        if c["op"] == "transpose":
            a = np.arange(int(np.prod(c["shape"])), dtype=np.int32).reshape(c["shape"])
            got = O.transpose(a, c["order"])
        elif c["op"] == "concat":
            ts = [(np.arange(int(np.prod(sh)), dtype=np.int32) + 100 * i).reshape(sh) for i, sh in enumerate(c["shapes"])]
            got = O.concat(ts, c["axis"])
        elif c["op"] == "broadcastTo":
            a = np.arange(int(np.prod(c["shape"])), dtype=np.int32).reshape(c["shape"])
            got = O.broadcastTo(a, c["new_shape"])
        elif c["op"] == "indexselect":
            a = np.arange(int(np.prod(c["shape"])), dtype=np.int32).reshape(c["shape"])
            idx = np.array(c["index"], dtype=np.int32).reshape(c["index_shape"])
            got = O.indexselect(a, idx, c["axis"])
        else:
            a = np.arange(int(np.prod(c["shape"])), dtype=np.int32).reshape(c["shape"])
            got = O.repeat(a, c["repeats"])
        assert np.array_equal(got.ravel(), want), c


def test_oracle_matmul_known_answer():
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    b = np.arange(40, dtype=np.float32).reshape(2, 4, 5)
    want = np.array(GOLD["known"]["matmul_arange_2x3x4_2x4x5"], dtype=np.float32).reshape(2, 3, 5)
    assert np.array_equal(O.matmul(a, b), want)


# ---- oracle vs numpy / float64 (the arithmetic the reference delegates to Highway, libm, OpenBLAS) ------------
@pytest.mark.parametrize("dtype", [np.float64, np.float32, np.int64, np.int32, np.int16, np.int8])
def test_oracle_elementwise_vs_numpy(dtype):
    rng = np.random.default_rng(1)
    if np.issubdtype(dtype, np.integer):
        a = rng.integers(-100, 101, 1000).astype(dtype)
        b = rng.integers(1, 50, 1000).astype(dtype)
    else:
        a = rng.uniform(-4, 4, 1000).astype(dtype)
        b = rng.uniform(0.5, 4, 1000).astype(dtype)
    with np.errstate(over="ignore"):
        assert np.array_equal(O.add(a, b), (a + b).astype(dtype))
        assert np.array_equal(O.sub(a, b), (a - b).astype(dtype))
        assert np.array_equal(O.mul(a, b), (a * b).astype(dtype))
    if np.issubdtype(dtype, np.integer):
        assert np.array_equal(O.div(a, b), np.trunc(a.astype(np.float64) / b).astype(dtype))  # C++ truncates
        assert np.array_equal(O.invert(a), ~a)
    else:
        assert np.array_equal(O.div(a, b), a / b)
        assert np.array_equal(O.sqrt(b), np.sqrt(b))
        assert np.allclose(O.exp(a), np.exp(a), rtol=1e-6)
        assert np.allclose(O.log(b), np.log(b), rtol=1e-6, atol=1e-7)
        assert np.allclose(O.pow(b, a), np.power(b, a), rtol=1e-6)
    assert np.array_equal(O.max(a, b), np.maximum(a, b))
    assert np.array_equal(O.min(a, b), np.minimum(a, b))
    assert np.array_equal(O.less(a, b), a < b)
    assert np.array_equal(O.greater(a, b), a > b)
    assert np.array_equal(O.equal(a, a.copy()), np.ones(1000, bool))
    s = dtype(3)
    assert np.array_equal(O.addscalar(a, 3), (a + s).astype(dtype))
    assert np.array_equal(O.rsubscalar(3, a), (s - a).astype(dtype))


def test_oracle_epsilon_rule_is_the_cpu_executors():
    a = np.array([0.0, 0.5, 1.0], dtype=np.float32)
    b = np.array([0.5, 0.5, 0.5], dtype=np.float32)
    assert O.equal(a, b, 0.5).tolist() == [True, True, True]        # |a-b| <= eps (op-ompsimd), not < (op-cuda)
    assert O.notequal(a, b, 0.5).tolist() == [False, False, False]
    assert O.equal(a, b, 0.0).tolist() == [False, True, False]


def test_oracle_16bit_rule():
    rng = np.random.default_rng(2)
    a = rng.uniform(-4, 4, 1000).astype(np.float32).astype(O.bfloat16)
    b = rng.uniform(-4, 4, 1000).astype(np.float32).astype(O.bfloat16)
    want = (a.astype(np.float32) * b.astype(np.float32)).astype(O.bfloat16)  # widen, fp32 op, one RNE
    assert np.array_equal(O.mul(a, b).view(np.uint16), want.view(np.uint16))
    h = a.astype(np.float16)
    assert np.array_equal(O.add(h, h).view(np.uint16), (h.astype(np.float32) * 2).astype(np.float16).view(np.uint16))
    d = rng.uniform(-100, 100, 2000)
    assert np.array_equal(O.todtype(d, O.bfloat16).view(np.uint16), d.astype(O.bfloat16).view(np.uint16))


def test_oracle_reduce_vs_numpy():
    rng = np.random.default_rng(3)
    k = rng.integers(-100, 101, (6, 7, 8)).astype(np.int32)
    for dims in ([0], [1], [2], [0, 1], [0, 2], [1, 2], [0, 1, 2]):
        assert np.array_equal(O.sum(k, dims), k.sum(tuple(dims)).reshape(O.reduced_shape(k.shape, dims, False)))
        assert np.array_equal(O.reducemax(k, dims, True), k.max(tuple(dims), keepdims=True))
        assert np.array_equal(O.reducemin(k, dims), k.min(tuple(dims)).reshape(O.reduced_shape(k.shape, dims, False)))
    x = rng.standard_normal((50, 60)).astype(np.float32)
    assert np.allclose(O.sum(x, [1]), x.astype(np.float64).sum(1), rtol=1e-5, atol=1e-5)
    assert np.array_equal(O.sum(np.full((3, 300), 127, np.int8), [1]), np.full(3, (127 * 300) % 256 - 256 * ((127 * 300) % 256 > 127), np.int8))


# ---- live against the reference's own library, where it was built ------------------------------------------------------
needs_ref = pytest.mark.skipif(O.ref_lib() is None, reason="oracle/_ref not built (no reference tree)")


@needs_ref
def test_oracle_changeshape_vs_reference_library_random():
    ref = O.ref_lib()
    rng = np.random.default_rng(4)

    def ia(v):
        return (C.c_int * max(len(v), 1))(*[int(x) for x in v])

    for _ in range(40):
        nd = int(rng.integers(1, 5))
        shp = [int(x) for x in rng.integers(1, 6, nd)]
        order = [int(x) for x in rng.permutation(nd)]
        for npdt in (np.int8, np.int16, np.int32, np.int64):
            a = rng.integers(-100, 100, shp).astype(npdt)
            out = np.empty([shp[o] for o in order], dtype=npdt)
            assert ref.ref_transpose(a.itemsize, C.c_void_p(a.ctypes.data), ia(shp), nd, ia(order), C.c_void_p(out.ctypes.data)) == 0
            assert np.array_equal(O.transpose(a, order), out)
        a = rng.integers(-100, 100, shp).astype(np.int32)
        lead = [int(x) for x in rng.integers(1, 4, int(rng.integers(0, 3)))]
        src = [1 if rng.random() < 0.4 else s for s in shp]
        a2 = rng.integers(-100, 100, src).astype(np.int32)
        oshape = lead + shp
        out = np.empty(oshape, dtype=np.int32)
        assert ref.ref_broadcast_to(4, C.c_void_p(a2.ctypes.data), ia(src), nd, ia(oshape), len(oshape), C.c_void_p(out.ctypes.data)) == 0
        assert np.array_equal(O.broadcastTo(a2, oshape), out)
        axis = int(rng.integers(0, nd))
        ishape = [int(x) for x in rng.integers(1, 4, int(rng.integers(1, 3)))]
        idx = rng.integers(0, shp[axis], ishape).astype(np.int64)
        oshape = shp[:axis] + ishape + shp[axis + 1:]
        out = np.empty(oshape, dtype=np.int32)
        assert ref.ref_indexselect(4, C.c_void_p(a.ctypes.data), ia(shp), nd, 8, C.c_void_p(idx.ctypes.data), ia(ishape), len(ishape), axis,
                                   C.c_void_p(out.ctypes.data)) == 0
        assert np.array_equal(O.indexselect(a, idx, axis), out)
        rep = [int(x) for x in rng.integers(1, 4, nd)]
        out = np.empty([s * r for s, r in zip(shp, rep)], dtype=np.int32)
        assert ref.ref_repeat(4, C.c_void_p(a.ctypes.data), ia(shp), nd, ia(rep), C.c_void_p(out.ctypes.data)) == 0
        assert np.array_equal(O.repeat(a, rep), out)


@needs_ref
def test_parser_vs_reference_library_fuzz(E):
    """Random IR-ish strings through both parsers."""
    ref = O.ref_lib()
    rng = np.random.default_rng(5)
    atoms = ["tensor<float32>:a", "var<int32>:3", "vector<int32>:[1 2 3]", "b", " c ", "listtensor<any>:[x y]", "var<bool>:True",
             "tensor:t", "<>", ":", "tensor<float16|float32>:h", "1.5", "", "var<string>:/p/q.r", "var|tensor<int>:m", "[ ]"]
    names = ["add", "newtensor ", "sum", "x y", "", "op2"]
    metas = ["", " // author=miaobyte", "// id=4 author=cublas benchmark.repeat=2", " //", "// created_at=1.5 sent_at=2.5 recv_at=3", "//bogus"]
    buf = C.create_string_buffer(1 << 16)
    for _ in range(600):
        na, nr = int(rng.integers(0, 4)), int(rng.integers(0, 3))
        line = str(rng.choice(names))
        args = ", ".join(str(rng.choice(atoms)) for _ in range(na))
        rets = ",".join(str(rng.choice(atoms)) for _ in range(nr))
        style = int(rng.integers(0, 4))
        if style == 0:
            line += f"({args})->({rets})"
        elif style == 1:
            line += f" ({args}) -> ({rets})"
        elif style == 2:
            line += f" {args} -> {rets}"
        else:
            line += f"({args}) ({rets})"  # no arrow
        line += str(rng.choice(metas))
        ref.ref_parse_ir(line.encode(), buf, len(buf))
        assert E.parse_ir(line) == buf.value.decode(), line


def test_integer_vectors_are_read_exactly_up_to_int64():
    """Extents in IR text: the reference's to<int> (int(std::stof(text)), dtype.hpp:15-25) rounds above 2^24
    and is undefined from 2^31; plain integer text is read exactly here, float text as the reference does."""
    from deepx_b200 import executor as E
    line = "newtensor(vector<int32>:[16777217 3000000000 7 2.0 1e3])->(tensor<float32>:t)"
    assert E.vector_i64(line, 0) == [16777217, 3000000000, 7, 2, 1000]
    assert E.vector_i64("reshape(tensor<float32>:a, vector<int32>:[2048 1048576])->(tensor<float32>:b)", 1) == [2048, 1048576]
    assert E.vector_i64("newtensor(vector<int32>:[-3 4])->(tensor<float32>:t)", 0) == [-3, 4]   # the op, not the parser, refuses it
    for bad in ("[99999999999999999999]", "[1e30]", "[nan]"):
        with pytest.raises(ValueError):
            E.vector_i64(f"newtensor(vector<int32>:{bad})->(tensor<float32>:t)", 0)


def test_print_format_is_checked_before_it_reaches_printf():
    """`print(t, format)` arrives in a datagram; only one numeric conversion that fits the dtype is let through."""
    from deepx_b200 import executor as E
    F32, I64, I32, BOOL = 1, 4, 5, 8
    assert E.check_print_format("%.4f", F32) == "%.4f"
    assert E.check_print_format("%8.3e", F32) == "%8.3e"
    assert E.check_print_format("%lf", F32) == "%f"
    assert E.check_print_format("%d", I32) == "%d"
    assert E.check_print_format("%d", I64) == "%lld"         # the argument is a long long: the modifier is supplied
    assert E.check_print_format("%ld", I32) == "%d"          # and removed where the argument is an int
    assert E.check_print_format("[%5x]", I32) == "[%5x]"
    assert E.check_print_format("%d%%", BOOL) == "%d%%"
    for fmt, code in (("%s", F32), ("%n", I32), ("%s%n%n%n", I32), ("%d %d", I32), ("%*d", I32), ("%c", I32), ("%p", I64),
                      ("%d", F32), ("%f", I32), ("no conversion", F32), ("%", F32), ("%.4", F32), ("%999999999999999999999d", I32)):
        with pytest.raises(ValueError):
            E.check_print_format(fmt, code)
