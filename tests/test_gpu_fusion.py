"""GPU tests of program execution with chain fusion (Executor.run_program).

A program is run twice on fresh executors: line by line (what the reference does: one launch per
IR line) and as a program with the fusion pass on.  Every tensor that is still alive afterwards
must exist in both and hold the same values (the fused row sum may add in another order: 1e-5
relative for fp32, 1e-2 for 16-bit floats), the temporaries must be gone in both, and the fused
run must have launched fewer kernels and allocated less.
"""
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden" / "frontend_ir"
F = "tensor<float32>"

RMS_TEMPS = ["48", "49", "50", "51", "52", "53", "54", "56"]
SOFTMAX_TEMPS = ["58", "59", "60", "61", "62", "63", "64"]


@pytest.fixture(scope="module")
def O():
    from oracle import oracle
    return oracle


def fresh():
    from deepx_b200.executor import Executor
    return Executor(0)


def frontend_program(name, temps):
    lines = [l for l in (GOLDEN / name).read_text().splitlines() if l.strip()]
    return "\n".join(lines + [f"deltensor () -> ({F}:{t})" for t in temps])


def launches():
    """Kernel launches made so far by the executor library (it carries its own copy of the kernels)."""
    import ctypes
    from deepx_b200.executor import lib
    fn = lib().dx_launch_count
    fn.restype = ctypes.c_ulonglong
    return fn()


def run_both(program, inputs=None):
    """(line-by-line executor, fused executor, launches line by line, launches fused)."""
    a, b = fresh(), fresh()
    for ex in (a, b):
        for name, arr in (inputs or {}).items():
            ex.put(name, arr)
    n0 = launches()
    for line in program.splitlines():
        a.run(line)
    a.sync()
    n1 = launches()
    replies = b.run_program(program)
    b.sync()
    n2 = launches()
    assert len(replies) == len(program.splitlines())
    assert all(" ok" in r.split("//")[0] for r in replies)
    return a, b, n1 - n0, n2 - n1


def same_tensors(a, b, names, rtol):
    for n in names:
        x, y = a.download(n).astype(np.float64), b.download(n).astype(np.float64)
        assert x.shape == y.shape
        assert np.allclose(x, y, rtol=rtol, atol=rtol * 1e-2), n


@pytest.mark.parametrize("name,temps,out,kind", [
    ("chains__rmsnorm_forward.ir", RMS_TEMPS, "57", "rmsnorm_groups"),
    ("chains__softmax.ir", SOFTMAX_TEMPS, "65", "softmax_groups"),
])
def test_frontend_chain_fused_equals_line_by_line(name, temps, out, kind):
    program = frontend_program(name, temps)
    a, b, n_lines, n_fused = run_both(program)
    st = b.fusion_stats()
    assert st[kind] == 1 and st["programs"] == 1 and st["lines_absorbed"] > 20
    same_tensors(a, b, ["45", out], 1e-5)
    for t in temps:
        for ex in (a, b):
            with pytest.raises(KeyError):
                ex.info(t)
    assert n_fused < n_lines
    assert b.stats()["high_water"] < a.stats()["high_water"]
    a.close()
    b.close()


def test_fusion_off_runs_every_line():
    program = frontend_program("chains__softmax.ir", SOFTMAX_TEMPS)
    ex = fresh()
    ex.set_fusion(False)
    ex.run_program(program)
    assert ex.fusion_stats()["softmax_groups"] == 0
    ref = fresh()
    for line in program.splitlines():
        ref.run(line)
    assert np.array_equal(ex.download("65"), ref.download("65"))
    ex.close()
    ref.close()


def rms_program(shape, dtype="float32", sq="mul"):
    f = f"tensor<{dtype}>"
    full = " ".join(str(s) for s in shape)
    small = " ".join(str(s) for s in shape[:-1]) + " 1"
    p = [f"newtensor(vector<int32>:[{s}])->({f}:{n})" for n, s in
         [("sq", full), ("v", small), ("vb", full), ("y", full), ("wb", full), ("out", full)]]
    p.append(f"mul({f}:x, {f}:x)->({f}:sq)" if sq == "mul" else f"powscalar({f}:x, var<int32>:2)->({f}:sq)")
    p += [f"sum({f}:sq, vector<int32>:[{len(shape) - 1}], var<bool>:true)->({f}:v)",
          f"divscalar({f}:v, var<float32>:{shape[-1]})->({f}:v)",
          f"addscalar({f}:v, var<float32>:1e-6)->({f}:v)",
          f"sqrt({f}:v)->({f}:v)",
          f"rdivscalar(var<float32>:1, {f}:v)->({f}:v)",
          f"broadcastTo({f}:v, vector<int32>:[{full}])->({f}:vb)",
          f"mul({f}:x, {f}:vb)->({f}:y)",
          f"broadcastTo({f}:w, vector<int32>:[{full}])->({f}:wb)",
          f"mul({f}:y, {f}:wb)->({f}:out)"]
    p += [f"deltensor()->({f}:{n})" for n in ("sq", "v", "vb", "y", "wb")]
    return "\n".join(p)


def test_config_rmsnorm_program_at_full_size(O):
    """The benchmark's RMSNorm chain, f32 [16,2048,896], as one program: one launch instead of ten,
    117 MB of pool instead of 5 tensor-sized temporaries, and the oracle's result."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((16, 2048, 896), dtype=np.float32)
    w = (1 + 0.02 * rng.standard_normal(896)).astype(np.float32)
    a, b, n_lines, n_fused = run_both(rms_program(x.shape), {"x": x, "w": w})
    assert b.fusion_stats()["rmsnorm_groups"] == 1
    assert n_fused == 1 and n_lines >= 10
    same_tensors(a, b, ["out"], 1e-5)
    sq = O.mul(x, x)
    v = O.sum(sq, [2], True)
    v = O.rdivscalar(1.0, O.sqrt(O.addscalar(O.divscalar(v, 896.0), float(np.float32(1e-6)))))
    want = O.mul(O.mul(x, O.broadcastTo(v, x.shape)), O.broadcastTo(w, x.shape))
    assert np.allclose(b.download("out"), want, rtol=2e-5, atol=1e-6)
    tensor_bytes = x.nbytes
    assert a.stats()["high_water"] >= 6 * tensor_bytes       # x, sq, vb, y, wb, out
    assert b.stats()["high_water"] < 2.1 * tensor_bytes      # x, out, w
    a.close()
    b.close()


@pytest.mark.parametrize("dtype", ["float64", "float16", "bfloat16"])
def test_other_float_dtypes(dtype):
    import ml_dtypes
    npdt = {"float64": np.float64, "float16": np.float16, "bfloat16": ml_dtypes.bfloat16}[dtype]
    rng = np.random.default_rng(3)
    x = rng.uniform(-2, 2, (7, 33, 256)).astype(np.float32).astype(npdt)
    w = rng.uniform(0.5, 1.5, (256,)).astype(np.float32).astype(npdt)
    a, b, n_lines, n_fused = run_both(rms_program(x.shape, dtype), {"x": x, "w": w})
    assert b.fusion_stats()["rmsnorm_groups"] == 1
    same_tensors(a, b, ["out"], 1e-12 if dtype == "float64" else 1e-2)
    a.close()
    b.close()


def test_error_inside_a_program_is_reported_on_its_line():
    ex = fresh()
    ex.put("a", np.ones((2, 3), dtype=np.float32))
    replies = ex.run_program(f"newtensor(vector<int32>:[2 3])->({F}:c)\nadd({F}:a, {F}:missing)->({F}:c)\nmul({F}:a, {F}:a)->({F}:c)", check=False)
    assert len(replies) == 3
    assert " ok" in replies[0] and " error" in replies[1].split("//")[0] and " ok" in replies[2]
    assert np.array_equal(ex.download("c"), np.ones((2, 3), dtype=np.float32))
    ex.close()
