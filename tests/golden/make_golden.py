"""Generates tests/golden/reference_golden.json from the REFERENCE's own code.

Needs oracle/_ref/libdeepx_ref.so (built by oracle/Makefile from the reference tree: deepxcore's
tf.cpp, tffactory.cpp, shape_*.cpp and the CPU executor's changeshape header).  Everything in the
JSON is an output of that library, not of this repository's code:
  ir_parse      IR line -> what TF::parse understood
  dtype         type text -> dtype_str(dtype(text))
  registry      registered signatures + calls -> index TfFactory::get_tf resolves to
  shapes        transposeShape / broadcastShape / indexselectShape / reducedShape / repeatShape / matmul_shape
  changeshape   transpose / concat / broadcastTo / indexselect / repeat on small int32 tensors
Run in the build container:  python tests/golden/make_golden.py
"""
import ctypes as C
import glob
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402

ref = O.ref_lib()
assert ref is not None, "build oracle/_ref first (make -C oracle ref)"


def s(fn, *args):
    buf = C.create_string_buffer(1 << 16)
    fn(*args, buf, len(buf))
    return buf.value.decode()


def ia(v):
    return (C.c_int * max(len(v), 1))(*[int(x) for x in v])


def vec(fn, *args):
    out = (C.c_int * 32)()
    n = fn(*args, out, 32)
    return None if n < 0 else [out[i] for i in range(n)]


IR_LINES = [
    "add (tensor<float32>:a, tensor<float32>:b) -> (tensor<float32>:c) // author=miaobyte created_at=1744724799.0650852 sent_at=1744724799.0650952",
    "newtensor(vector<int32>:[3 4 5])->(tensor<float32>:t1) // id=7",
    "newtensor ( [3 4 5]) -> ( tensor_136144420556608) // id=1 created_at=1744724799.0650852",
    "matmul(float16|float32 a,float16|float32 b)->(float16|float32 c)",
    "matmul(float16,float16)->(float32)",
    "argset(1.34,2.34)->(float32 v1)",
    "argset(float32 1.34)->(float32 var1)",
    "sum(tensor<float32>:a, vector<int32>:[0 1], var<bool>:True)->(tensor<float32>:b) // author=miaobyte benchmark.repeat=10",
    "print(tensor<any>:t, var<string>:%.2f)->()",
    "deltensor()->(tensor<any>:t)",
    "noarrow(a,b)",
    "concat(listtensor<float32>:[a b c], var<int32>:1)->(tensor<float32>:d)//author=miaobyte",
    "x->y",
    "f a, b -> c",
    "  spaced (  tensor<int8> :  q  ) -> ( var|tensor<float> : z )",
    "switch(listtensor<float32>:[a b], tensor<bool>:m)->(tensor<float32>:c) // author= id=3",
    "g(tensor<bogus>:a)->(vector<int>:b, listtensor:c)",
    "h()->()",
    "k((a),(b))->((c))",
    "rsubscalar(var<float32>:1.5, tensor<bfloat16>:a)->(tensor<bfloat16>:c) // author=miaobyte id=12 benchmark.repeat=3",
    "vecset(vector<float64>:[1.5 2.5])->(vector<float64>:v)",
    "indexselect(tensor<float32>:A, tensor<int64>:idx, var<int32>:-1)->(tensor<float32>:B)",
    "equal(tensor<int8>:a, tensor<int8>:b, var<float32>:0.5)->(tensor<bool>:m) // weird=1 =x author=who",
    "save(tensor<any>:t, var<string>:/tmp/a b)->()",
]
for f in sorted(glob.glob(str(Path(__file__).parent / "frontend_ir" / "*.ir"))):
    IR_LINES += [ln for ln in Path(f).read_text().splitlines() if ln][:6]

DTYPES = ["tensor<float32>", "var<int32>", "vector<int32>", "listtensor<float16>", "tensor", "var", "tensor<any>",
          "tensor<int>", "tensor<float>", "tensor<float8>", "var|tensor<bool>", "tensor|vector|var|listtensor<string>",
          "tensor<float16|float32>", "tensor<bfloat16>", "tensor<float8e4m3>", "tensor<int4>", "bogus<float32>", "",
          "tensor<nonsense>", "vector<float64>", "tensor<float4e2m1>", "tensor<float8e5m2>", "tensor<int64>", "x<y"]

REG_SIGS = [
    "add(tensor<any>:a, tensor<any>:b)->(tensor<any>:c) // author=miaobyte",
    "add(tensor<any>:a, tensor<any>:b)->(tensor<any>:c) // author=cublas",
    "pow(tensor<float64|float32>:a, tensor<float32>:b)->(tensor<float32>:c) // author=miaobyte",
    "pow(tensor<float64>:a, tensor<float64>:b)->(tensor<float64>:c) // author=miaobyte",
    "newtensor(vector<int32>:shape)->(tensor<any>:t)",
    "newtensor(var<string>:shape)->(tensor<any>:t)",
    "invert(tensor<int>:a)->(tensor<int>:c) // author=miaobyte",
    "switch(listtensor<any>:ts, tensor<int32>:cases)->(tensor<any>:r) // author=miaobyte",
    "sum(tensor<any>:A, vector<int32>:dims, var<bool>:keepdims)->(tensor<any>:B) // author=miaobyte",
    "mixed(var|tensor<float32>:x)->(tensor<float32>:y) // author=miaobyte",
]
REG_CALLS = [
    "add(tensor<float32>:x, tensor<float32>:y)->(tensor<float32>:z) // author=miaobyte",
    "add(tensor<float32>:x, tensor<float32>:y)->(tensor<float32>:z) // author=cublas",
    "add(tensor<float32>:x, tensor<float32>:y)->(tensor<float32>:z)",
    "add(tensor<float32>:x)->(tensor<float32>:z) // author=miaobyte",
    "add(var<float32>:x, tensor<float32>:y)->(tensor<float32>:z) // author=miaobyte",
    "pow(tensor<float32>:x, tensor<float32>:y)->(tensor<float32>:z) // author=miaobyte",
    "pow(tensor<float64>:x, tensor<float64>:y)->(tensor<float64>:z) // author=miaobyte",
    "pow(tensor<float16>:x, tensor<float16>:y)->(tensor<float16>:z) // author=miaobyte",
    "pow(x, y)->(z) // author=miaobyte",
    "newtensor(vector<int32>:[2 3])->(tensor<float32>:t)",
    "newtensor(var<string>:shp)->(tensor<float32>:t)",
    "newtensor([2 3])->(t)",
    "invert(tensor<int32>:a)->(tensor<int32>:c) // author=miaobyte",
    "invert(tensor<bool>:a)->(tensor<bool>:c) // author=miaobyte",
    "switch(listtensor<float32>:[a b], tensor<int32>:c)->(tensor<float32>:r) // author=miaobyte",
    "switch(listtensor<float32>:[a b], tensor<bool>:c)->(tensor<float32>:r) // author=miaobyte",
    "sum(tensor<float32>:a, vector<int32>:[0], var<bool>:true)->(tensor<float32>:b) // author=miaobyte",
    "mixed(tensor<float32>:a)->(tensor<float32>:b) // author=miaobyte",
    "mixed(var<float32>:a)->(tensor<float32>:b) // author=miaobyte",
    "nosuchop(tensor<float32>:a)->(tensor<float32>:b)",
]


def main():
    g = {"ir_parse": [{"line": ln, "parsed": s(ref.ref_parse_ir, ln.encode())} for ln in IR_LINES],
         "dtype": [{"text": t, "out": s(ref.ref_dtype_roundtrip, t.encode())} for t in DTYPES]}
    h = ref.ref_factory_new()
    for sig in REG_SIGS:
        ref.ref_factory_add(h, sig.encode())
    # the unknown-author fallback of the reference picks unordered_map::begin(), which is not
    # specified; calls without a registered author are therefore recorded but flagged
    g["registry"] = {"signatures": REG_SIGS,
                     "calls": [{"call": c, "index": ref.ref_factory_get(h, c.encode()),
                                "author_known": ("author=miaobyte" in c or "author=cublas" in c or c.startswith("newtensor") or c.startswith("nosuch"))}
                               for c in REG_CALLS]}
    ref.ref_factory_free(h)

    shapes = []
    for shp, order in [([3, 4, 6], [0, 2, 1]), ([2, 3, 4, 5], [3, 1, 0, 2]), ([7], [0])]:
        shapes.append({"fn": "transpose", "shape": shp, "order": order, "out": vec(ref.ref_transpose_shape, ia(shp), len(shp), ia(order))})
    for a, b in [([3, 2], [4, 3, 2]), ([1, 4096], [8192, 4096]), ([3, 1], [1, 5]), ([2, 3], [4, 3]), ([5], [5]), ([1], [7, 7])]:
        shapes.append({"fn": "broadcast", "a": a, "b": b, "out": vec(ref.ref_broadcast_shape, ia(a), len(a), ia(b), len(b))})
    for a, i, ax in [([151936, 896], [8, 2048], 0), ([7, 9, 5], [2, 3], 1), ([7, 9, 5], [4], 2), ([10], [3, 3], 0)]:
        shapes.append({"fn": "indexselect", "a": a, "idx": i, "axis": ax, "out": vec(ref.ref_indexselect_shape, ia(a), len(a), ia(i), len(i), ax)})
    for shp, dims, keep in [([2, 3, 4], [], 0), ([2, 3, 4], [0], 0), ([2, 3, 4], [1], 0), ([2, 3, 4], [2], 0), ([2, 3, 4], [0, 1], 0),
                            ([2, 3, 4], [0, 2], 0), ([2, 3, 4], [1, 2], 0), ([2, 3, 4], [0, 1, 2], 0), ([2, 3, 4], [-1, 0], 1),
                            ([3, 4, 5], [2, 2, -1], 1), ([64, 1024, 1024], [1, 2], 0), ([4], [3], 0)]:
        shapes.append({"fn": "reduced", "shape": shp, "dims": dims, "keepdims": keep,
                       "checked": vec(ref.ref_checked_dims, ia(shp), len(shp), ia(dims), len(dims)),
                       "out": vec(ref.ref_reduced_shape, ia(shp), len(shp), ia(dims), len(dims), keep)})
    for shp, rep in [([3, 4], [2, 3]), ([2, 1, 5], [3, 4, 2])]:
        shapes.append({"fn": "repeat", "shape": shp, "repeats": rep, "out": vec(ref.ref_repeat_shape, ia(shp), len(shp), ia(rep))})
    for a, b in [([2, 3, 4], [2, 4, 5]), ([8192, 4096], [4096, 4096]), ([3, 4], [5, 6]), ([4], [4])]:
        shapes.append({"fn": "matmul", "a": a, "b": b, "out": vec(ref.ref_matmul_shape, ia(a), len(a), ia(b), len(b))})
    g["shapes"] = shapes

    cs = []
    rng = np.random.default_rng(0)
    for shp, order in [([3, 4, 6], [0, 2, 1]), ([2, 3, 4, 5], [3, 1, 0, 2]), ([4, 5], [1, 0]), ([2, 3, 4], [0, 1, 2]), ([3, 2, 2, 3], [0, 2, 1, 3])]:
        a = np.arange(int(np.prod(shp)), dtype=np.int32).reshape(shp)
        out = np.empty([shp[o] for o in order], dtype=np.int32)
        assert ref.ref_transpose(4, C.c_void_p(a.ctypes.data), ia(shp), len(shp), ia(order), C.c_void_p(out.ctypes.data)) == 0
        cs.append({"op": "transpose", "shape": shp, "order": order, "out": out.ravel().tolist()})
    for shapes_, axis in [([[2, 3, 4]] * 3, 0), ([[2, 3, 4]] * 3, 1), ([[2, 3, 4]] * 3, 2), ([[2, 1, 3], [2, 4, 3], [2, 2, 3]], 1)]:
        ts = [(np.arange(int(np.prod(sh)), dtype=np.int32) + 100 * i).reshape(sh) for i, sh in enumerate(shapes_)]
        oshape = list(shapes_[0])
        oshape[axis] = sum(sh[axis] for sh in shapes_)
        out = np.empty(oshape, dtype=np.int32)
        ptrs = (C.c_void_p * len(ts))(*[t.ctypes.data for t in ts])
        shp_arrs = [ia(sh) for sh in shapes_]
        shp_ptrs = (C.POINTER(C.c_int) * len(ts))(*[C.cast(x, C.POINTER(C.c_int)) for x in shp_arrs])
        assert ref.ref_concat(4, ptrs, shp_ptrs, len(ts), len(oshape), axis, C.c_void_p(out.ctypes.data)) == 0
        cs.append({"op": "concat", "shapes": shapes_, "axis": axis, "out": out.ravel().tolist()})
    for ashape, oshape in [([3, 2], [4, 3, 2]), ([1, 5], [4, 5]), ([3, 1], [3, 4]), ([2, 1, 3], [2, 2, 4, 3])]:
        a = np.arange(int(np.prod(ashape)), dtype=np.int32).reshape(ashape)
        out = np.empty(oshape, dtype=np.int32)
        assert ref.ref_broadcast_to(4, C.c_void_p(a.ctypes.data), ia(ashape), len(ashape), ia(oshape), len(oshape), C.c_void_p(out.ctypes.data)) == 0
        cs.append({"op": "broadcastTo", "shape": ashape, "new_shape": oshape, "out": out.ravel().tolist()})
    for ashape, ishape, axis in [([5, 4], [2, 3], 0), ([3, 6, 2], [4], 1), ([3, 2, 7], [2, 2], 2)]:
        a = np.arange(int(np.prod(ashape)), dtype=np.int32).reshape(ashape)
        idx = rng.integers(0, ashape[axis], ishape).astype(np.int32)
        oshape = ashape[:axis] + ishape + ashape[axis + 1:]
        out = np.empty(oshape, dtype=np.int32)
        assert ref.ref_indexselect(4, C.c_void_p(a.ctypes.data), ia(ashape), len(ashape), 4, C.c_void_p(idx.ctypes.data), ia(ishape), len(ishape), axis, C.c_void_p(out.ctypes.data)) == 0
        cs.append({"op": "indexselect", "shape": ashape, "index_shape": ishape, "index": idx.ravel().tolist(), "axis": axis,
                   "out": out.ravel().tolist()})
    for ashape, rep in [([3, 4], [2, 3]), ([2, 1, 5], [3, 4, 2])]:
        a = np.arange(int(np.prod(ashape)), dtype=np.int32).reshape(ashape)
        out = np.empty([x * r for x, r in zip(ashape, rep)], dtype=np.int32)
        assert ref.ref_repeat(4, C.c_void_p(a.ctypes.data), ia(ashape), len(ashape), ia(rep), C.c_void_p(out.ctypes.data)) == 0
        cs.append({"op": "repeat", "shape": ashape, "repeats": rep, "out": out.ravel().tolist()})
    g["changeshape"] = cs
    # known answers printed in the reference's own test sources
    g["known"] = {
        "matmul_arange_2x3x4_2x4x5": [70, 76, 82, 88, 94, 190, 212, 234, 256, 278, 310, 348, 386, 424, 462,
                                      1510, 1564, 1618, 1672, 1726, 1950, 2020, 2090, 2160, 2230, 2390, 2476, 2562, 2648, 2734],
        "matmul_source": "executor/op-ompsimd/test/tensorfunc/4_tensor_matmul.cpp:29-35",
        "sum_shapes_2x3x4": {"[]": [2, 3, 4], "[0]": [3, 4], "[1]": [2, 4], "[2]": [2, 3], "[0, 1]": [4], "[0, 2]": [3], "[1, 2]": [2], "[0, 1, 2]": [1]},
        "sum_shapes_source": "executor/op-ompsimd/test/tensorfunc/5_tensor_sum.cpp:41-48",
    }
    out = Path(__file__).parent / "reference_golden.json"
    out.write_text(json.dumps(g, indent=1))
    print("wrote", out, {k: len(v) for k, v in g.items()})


if __name__ == "__main__":
    main()
