"""Compiled programs: a sequence of IR lines captured into a CUDA graph and replayed.

The replay must compute what running the lines one by one computes (same kernels, same order), refuse
what cannot be captured, and notice when a tensor it names has changed since compilation.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
F = "tensor<float32>"


@pytest.fixture()
def ex():
    from deepx_b200.executor import Executor
    e = Executor(0)
    yield e
    e.close()


def mlp_program():
    return "\n".join([
        f"matmul({F}:x, {F}:w1)->({F}:h)",
        f"add({F}:h, {F}:b1)->({F}:h)",
        f"maxscalar({F}:h, var<float32>:0)->({F}:h)",
        f"matmul({F}:h, {F}:w2)->({F}:y)",
        f"sum({F}:y, vector<int32>:[1], var<bool>:true)->({F}:s)",
        f"reducemax({F}:y, vector<int32>:[0 1], var<bool>:false)->({F}:m)",
        f"transpose({F}:y, vector<int32>:[1 0])->({F}:yt)",
        f"mulscalar({F}:x, var<float32>:1.5)->({F}:x)",   # the program updates its own input: replays differ
    ])


def setup_mlp(ex, rng):
    t = {"x": rng.standard_normal((64, 128), dtype=np.float32), "w1": rng.standard_normal((128, 256), dtype=np.float32) * 0.1,
         "b1": rng.standard_normal((64, 256), dtype=np.float32), "w2": rng.standard_normal((256, 32), dtype=np.float32) * 0.1}
    for k, v in t.items():
        ex.put(k, v)
    for name, shape in (("h", (64, 256)), ("y", (64, 32)), ("s", (64, 1)), ("m", (1,)), ("yt", (32, 64))):
        ex.new(name, "float32", shape)
    return t


def test_replay_equals_line_by_line(ex):
    from deepx_b200.executor import Executor
    rng = np.random.default_rng(0)
    setup_mlp(ex, rng)
    ref = Executor(0)
    setup_mlp(ref, np.random.default_rng(0))
    prog = ex.compile(mlp_program())            # runs the program once
    info = prog.info()
    assert info["lines"] == 8 and info["ops"] == 8 and info["graph_nodes"] >= 8
    for line in mlp_program().splitlines():
        ref.run(line)
    for _ in range(3):                          # three more passes each
        prog.run()
        for line in mlp_program().splitlines():
            ref.run(line)
    ex.sync()
    ref.sync()
    for name in ("x", "h", "y", "s", "m", "yt"):
        assert np.array_equal(ex.download(name), ref.download(name)), name
    prog.free()
    ref.close()


def test_fused_chain_inside_a_compiled_program(ex):
    """Temporaries of a chain the fusion pass absorbs never exist, so their newtensor / deltensor lines do not
    stop the program from being captured."""
    rng = np.random.default_rng(1)
    x = rng.standard_normal((32, 64, 256), dtype=np.float32)
    ex.put("x", x)
    ex.put("w", (1 + 0.1 * rng.standard_normal(256)).astype(np.float32))
    ex.new("out", "float32", x.shape)
    lines = [f"newtensor(vector<int32>:[{s}])->({F}:{n})" for n, s in (("sq", "32 64 256"), ("v", "32 64 1"), ("vb", "32 64 256"), ("y", "32 64 256"), ("wb", "32 64 256"))]
    lines += [f"mul({F}:x, {F}:x)->({F}:sq)", f"sum({F}:sq, vector<int32>:[2], var<bool>:true)->({F}:v)",
              f"divscalar({F}:v, var<float32>:256)->({F}:v)", f"addscalar({F}:v, var<float32>:1e-6)->({F}:v)", f"sqrt({F}:v)->({F}:v)",
              f"rdivscalar(var<float32>:1, {F}:v)->({F}:v)", f"broadcastTo({F}:v, vector<int32>:[32 64 256])->({F}:vb)",
              f"mul({F}:x, {F}:vb)->({F}:y)", f"broadcastTo({F}:w, vector<int32>:[32 64 256])->({F}:wb)", f"mul({F}:y, {F}:wb)->({F}:out)"]
    lines += [f"deltensor()->({F}:{n})" for n in ("sq", "v", "vb", "y", "wb")]
    prog = ex.compile("\n".join(lines))
    info = prog.info()
    assert info["fused_chains"] == 1 and info["ops"] == 1 and info["lines"] == 20
    ex.upload("out", np.zeros_like(x))
    prog.run()
    ex.sync()
    w = ex.download("w").astype(np.float64)
    x64 = x.astype(np.float64)
    ref = w * (x64 / np.sqrt((x64 * x64).mean(-1, keepdims=True) + 1e-6))
    assert np.allclose(ex.download("out"), ref, rtol=1e-5, atol=1e-6)
    prog.free()


def test_refusals(ex):
    from deepx_b200.executor import IRError
    ex.put("a", np.ones((4, 4), dtype=np.float32))
    for bad, why in [(f"newtensor(vector<int32>:[4])->({F}:t)", "newtensor"),
                     (f"print({F}:a)->()", "print"),
                     (f"add({F}:a, {F}:a)->({F}:a) // benchmark.repeat=3", "timed"),
                     (f"transpose({F}:a, vector<int32>:[1 0])->({F}:a)", "temporary"),
                     (f"add({F}:a, {F}:nope)->({F}:a)", "nope"),
                     ("this is not IR", "arrow"), ("", "empty")]:
        with pytest.raises(IRError, match=why):
            ex.compile(bad)
    # the executor is still usable after every refusal
    ex.run(f"addscalar({F}:a, var<float32>:1)->({F}:a)")
    assert np.array_equal(ex.download("a"), np.full((4, 4), 2, dtype=np.float32))


def test_stale_program_is_detected(ex):
    from deepx_b200.executor import IRError
    ex.put("a", np.ones((8,), dtype=np.float32))
    ex.put("b", np.ones((8,), dtype=np.float32))
    prog = ex.compile(f"add({F}:a, {F}:b)->({F}:a)\nmulscalar({F}:a, var<float32>:2)->({F}:b)")
    prog.run()
    ex.run(f"deltensor()->({F}:b)")
    with pytest.raises(IRError, match="stale"):
        prog.run()
    ex.put("b", np.ones((16,), dtype=np.float32))   # same name, other shape (and storage)
    with pytest.raises(IRError, match="stale"):
        prog.run()
    prog.free()


def test_k_split_matmul_and_self_finishing_reduction_inside_a_compiled_program(ex):
    """A program whose matmul takes the K split over cooperating CTA pairs (a cooperative launch, counters inside the
    library) and whose global sum finishes itself (last-CTA form): both must be capturable and replay to the same bits
    as the lines run one by one."""
    import ml_dtypes  # noqa: F401  (numpy bfloat16)
    from deepx_b200 import _native as N
    from deepx_b200.executor import Executor
    M, K, Nn = 256, 8192, 1024
    assert int(N.lib.dx_matmul_workspace_bytes(N.BF16, 1, M, Nn, K)) > 0, "this shape is meant to take the K-split path"
    B = "tensor<bfloat16>"
    program = "\n".join([
        f"matmul({B}:a, {B}:b)->({B}:c)",
        f"sum({B}:c, vector<int32>:[0 1], var<bool>:false)->({B}:s)",
        f"mulscalar({B}:a, var<float32>:0.5)->({B}:a)",
    ])
    rng = np.random.default_rng(5)
    a = (rng.standard_normal((M, K), dtype=np.float32) * 0.1).astype(ml_dtypes.bfloat16)
    b = (rng.standard_normal((K, Nn), dtype=np.float32) * 0.1).astype(ml_dtypes.bfloat16)
    ref = Executor(0)
    for e in (ex, ref):
        e.put("a", a)
        e.put("b", b)
        e.new("c", "bfloat16", (M, Nn))
        e.new("s", "bfloat16", (1,))
    for line in program.splitlines():   # once line by line on both: the executor's scratch has its size before the capture
        ex.run(line)
        ref.run(line)
    prog = ex.compile(program)          # runs the program once more
    for line in program.splitlines():
        ref.run(line)
    for _ in range(3):
        prog.run()
        for line in program.splitlines():
            ref.run(line)
    ex.sync()
    ref.sync()
    for name in ("a", "c", "s"):
        assert np.array_equal(ex.download(name).view(np.uint16), ref.download(name).view(np.uint16)), name
    assert np.abs(ex.download("c").astype(np.float32)).max() > 0
    prog.free()
    ref.close()
