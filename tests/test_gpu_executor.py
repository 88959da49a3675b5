"""GPU tests of the deepxIR text boundary: IR lines in, replies out, results checked with the oracle.

* transcripts of the IR that the reference's unmodified Python front end emits for its own
  examples (tests/golden/frontend_ir/*.ir) are replayed line by line; after every op the
  executor's output tensor is compared with the oracle applied to the executor's input tensors;
* the RMSNorm-shaped deepxIR sequence of the benchmark configs, at full size;
* error replies, aliasing rules, tensor lifetime, the on-disk tensor format, the UDP process.
"""
import glob
import os
import re
import socket
import subprocess
import time
from pathlib import Path

import numpy as np
import pytest

from helpers import assert_bit_exact

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


@pytest.fixture()
def ex():
    from deepx_b200.executor import Executor
    e = Executor(0)
    yield e
    e.close()


@pytest.fixture(scope="module")
def O():
    from oracle import oracle
    return oracle


# ---- a shadow interpreter: what each IR op should produce, via the oracle ----------------------------
def _stof(text):
    return float(np.float32(float(text)))


def _vec(text):
    return [int(np.float32(float(t))) for t in text.strip("[]").split(" ") if t != ""]


def parse_line(line):
    body = line.split("//")[0]
    left, right = body.split("->")
    name = left[:left.index("(")].strip()
    args = [a.strip() for a in left[left.index("(") + 1:left.rindex(")")].split(",") if a.strip()]
    rets = [a.strip() for a in right[right.index("(") + 1:right.rindex(")")].split(",") if a.strip()]
    split = lambda p: (p.split(":", 1)[0].strip(), p.split(":", 1)[1].strip()) if ":" in p else ("", p)
    return name, [split(a) for a in args], [split(r) for r in rets]


BINARY = {"add", "sub", "mul", "div", "max", "min", "pow"}
SCALAR = {"addscalar", "subscalar", "mulscalar", "divscalar", "maxscalar", "minscalar", "powscalar"}
RSCALAR = {"rsubscalar", "rdivscalar", "rpowscalar"}
UNARY = {"sqrt", "log", "exp", "sin", "cos", "tan", "invert"}
EXACT = {"add", "sub", "mul", "div", "max", "min", "sqrt", "invert", "addscalar", "subscalar", "mulscalar", "divscalar",
         "maxscalar", "minscalar", "rsubscalar", "rdivscalar"}


def expected(O, ex, name, args, rets):
    """Returns (array or None, exact?) for the op's output given the executor's current inputs."""
    get = lambda i: ex.download(args[i][1])
    sc = lambda a, i: (int(_stof(args[i][1])) if a.dtype.kind in "iu" else _stof(args[i][1]))
    if name in BINARY:
        return getattr(O, name)(get(0), get(1)), name in EXACT
    if name in SCALAR:
        a = get(0)
        return getattr(O, name)(a, sc(a, 1)), name in EXACT
    if name in RSCALAR:
        a = get(1)
        return getattr(O, name)(sc(a, 0), a), name in EXACT
    if name in UNARY:
        return getattr(O, name)(get(0)), name in EXACT
    if name in ("equal", "notequal"):
        return getattr(O, name)(get(0), get(1), _stof(args[2][1])), True
    if name in ("less", "greater"):
        return getattr(O, name)(get(0), get(1)), True
    if name in ("equalscalar", "notequalscalar"):
        a = get(0)
        return getattr(O, name)(a, sc(a, 1), _stof(args[2][1])), True
    if name in ("lessscalar", "greaterscalar"):
        a = get(0)
        return getattr(O, name)(a, sc(a, 1)), True
    if name == "switch":
        ts = [ex.download(n) for n in args[0][1].strip("[]").split(" ")]
        return O.Switch(ts, get(1)), True
    if name == "todtype":
        dst = ex.download(rets[0][1])
        return O.todtype(get(0), dst.dtype), True
    if name in ("sum", "prod", "reducemax", "reducemin"):
        a = get(0)
        return getattr(O, name)(a, _vec(args[1][1]), args[2][1].lower() == "true"), a.dtype.kind in "iu" or name.startswith("reduce")
    if name == "transpose":
        return O.transpose(get(0), _vec(args[1][1])), True
    if name == "concat":
        ts = [ex.download(n) for n in args[0][1].strip("[]").split(" ")]
        return O.concat(ts, int(_stof(args[1][1]))), True
    if name == "broadcastTo":
        return O.broadcastTo(get(0), _vec(args[1][1])), True
    if name == "indexselect":
        return O.indexselect(get(0), get(1), int(_stof(args[2][1]))), True
    if name == "repeat":
        return O.repeat(get(0), _vec(args[1][1])), True
    if name == "reshape":
        return get(0).reshape(_vec(args[1][1])), True
    if name == "matmul":
        return O.matmul(get(0), get(1)), False
    if name == "copytensor":
        return get(0), True
    if name == "constant":
        dst = ex.download(rets[0][1])
        v = args[0][1]
        val = (v.lower() == "true") if dst.dtype == np.bool_ else (int(_stof(v)) if dst.dtype.kind in "iu" else _stof(v))
        return np.full(dst.shape, val, dtype=dst.dtype), True
    if name == "arange":
        dst = ex.download(rets[0][1])
        i = np.arange(dst.size, dtype=np.float32)
        return (np.float32(_stof(args[0][1])) + np.float32(_stof(args[1][1])) * i).astype(dst.dtype).reshape(dst.shape), True
    return None, False


TRANSCRIPTS = sorted(glob.glob(str(HERE / "golden" / "frontend_ir" / "*.ir")))


@pytest.mark.parametrize("path", TRANSCRIPTS, ids=[Path(p).stem for p in TRANSCRIPTS])
def test_replay_reference_frontend_transcript(ex, O, path, capfd):
    checked = 0
    for line in Path(path).read_text().splitlines():
        if not line.strip():
            continue
        name, args, rets = parse_line(line)
        want, exact = (None, False)
        if name not in ("newtensor", "print", "deltensor", "renametensor", "uniform", "normal", "dropout", "save", "load"):
            want, exact = expected(O, ex, name, args, rets)
        rc, reply = ex.reply(line)
        assert rc == 0, f"{line}\n-> {reply}"
        assert re.match(r"^\d+ ok// recv_at=\d+ start_at=\d+ finish_at=\d+$", reply), reply
        if want is not None:
            got = ex.download(rets[0][1])
            if exact:
                assert_bit_exact(got.reshape(want.shape), want, line)
            else:
                assert np.allclose(got.astype(np.float64), want.astype(np.float64), rtol=1e-5, atol=1e-6), line
            checked += 1
        elif name in ("uniform", "normal"):
            got = ex.download(rets[0][1]).astype(np.float64)
            assert np.isfinite(got).all()
            if name == "uniform":
                lo, hi = _stof(args[0][1]), _stof(args[1][1])
                assert got.min() >= lo and got.max() <= hi
    out = capfd.readouterr().out
    if "print" in Path(path).read_text():
        assert "shape:[" in out  # the print op writes the tensor to the executor's stdout
    assert checked > 0 or "init" in path or "tensorlife" in path


# ---- the RMSNorm-shaped IR sequence of the benchmark configs ----------------------------------------------
def test_config_rmsnorm_ir_chain(ex, O):
    """x*x, sum over last axis, /896, +1e-6, sqrt, 1/., broadcast, mul, mul by weight on f32 [16,2048,896]."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((16, 2048, 896), dtype=np.float32)
    w = (1 + 0.02 * rng.standard_normal(896)).astype(np.float32)
    ex.put("x", x)
    ex.put("w", w)
    f = "tensor<float32>"
    for nm, shp in [("sq", "16 2048 896"), ("v", "16 2048 1"), ("vb", "16 2048 896"), ("y", "16 2048 896"), ("wb", "16 2048 896"), ("out", "16 2048 896")]:
        ex.run(f"newtensor(vector<int32>:[{shp}])->({f}:{nm})")
    A = "// author=miaobyte"
    ex.run(f"mul({f}:x, {f}:x)->({f}:sq) {A}")
    ex.run(f"sum({f}:sq, vector<int32>:[2], var<bool>:true)->({f}:v) {A}")
    ex.run(f"divscalar({f}:v, var<float32>:896)->({f}:v) {A}")
    ex.run(f"addscalar({f}:v, var<float32>:1e-6)->({f}:v) {A}")
    ex.run(f"sqrt({f}:v)->({f}:v) {A}")
    ex.run(f"rdivscalar(var<float32>:1, {f}:v)->({f}:v) {A}")
    ex.run(f"broadcastTo({f}:v, vector<int32>:[16 2048 896])->({f}:vb) {A}")
    ex.run(f"mul({f}:x, {f}:vb)->({f}:y) {A}")
    ex.run(f"broadcastTo({f}:w, vector<int32>:[16 2048 896])->({f}:wb) {A}")
    ex.run(f"mul({f}:y, {f}:wb)->({f}:out) {A}")
    got = ex.download("out")
    # the same sequence through the oracle, op by op
    sq = O.mul(x, x)
    v = O.sum(sq, [2], True)
    v = O.divscalar(v, float(np.float32(896)))
    v = O.addscalar(v, float(np.float32(1e-6)))
    v = O.sqrt(v)
    v = O.rdivscalar(1.0, v)
    want = O.mul(O.mul(x, O.broadcastTo(v, x.shape)), O.broadcastTo(w, x.shape))
    assert np.allclose(got, want, rtol=2e-5, atol=1e-6)  # only the 896-term sum may differ in order
    x64 = x.astype(np.float64)
    ref = x64 / np.sqrt((x64 * x64).mean(-1, keepdims=True) + 1e-6) * w
    assert np.allclose(got, ref, rtol=1e-4, atol=1e-5)


def test_error_replies_and_lifetime(ex):
    f = "tensor<float32>"
    rc, r = ex.reply(f"add({f}:nope, {f}:nope2)->({f}:c) // author=miaobyte id=5")
    assert rc == 1 and r.startswith("5 error//") and r.endswith("tensor not found: nope")
    rc, r = ex.reply("add(a,b)")
    assert rc == 1 and "Invalid IR format: missing arrow" in r
    rc, r = ex.reply("frobnicate(tensor<float32>:a)->(tensor<float32>:b)")
    assert rc == 1 and "opfrobnicate not found" in r
    ex.new("a", "float32", [4, 5])
    ex.new("b", "float64", [4, 5])
    ex.new("c", "float32", [4, 6])
    rc, r = ex.reply(f"add({f}:a, tensor<float64>:b)->({f}:a) // author=miaobyte")
    assert rc == 1 and "Type mismatch: float32 != float64 != float32" in r
    rc, r = ex.reply(f"add({f}:a, {f}:a)->({f}:c) // author=miaobyte")
    assert rc == 1 and "shape mismatch" in r
    rc, r = ex.reply(f"sum({f}:a, vector<int32>:[5], var<bool>:false)->({f}:c) // author=miaobyte")
    assert rc == 1 and "Dimension out of range" in r
    rc, r = ex.reply(f"sum({f}:a, vector<int32>:[0], var<bool>:maybe)->({f}:c) // author=miaobyte")
    assert rc == 1 and "Invalid bool value:maybe" in r
    rc, r = ex.reply("newtensor(vector<int32>:[2 2])->(tensor<float8e4m3>:q)")
    assert rc == 1 and "Float8E4M3 has not been implemented" in r
    # unknown author falls back to a registered one
    assert ex.reply(f"add({f}:a, {f}:a)->({f}:a) // author=somebody")[0] == 0
    # lifetime: rename, copy, delete
    ex.run(f"renametensor(var<string>:a2)->({f}:a)")
    with pytest.raises(KeyError):
        ex.info("a")
    assert ex.info("a2") == (1, [4, 5])
    ex.new("d", "float32", [4, 5])
    ex.upload("a2", np.arange(20, dtype=np.float32).reshape(4, 5))
    ex.run(f"copytensor({f}:a2)->({f}:d)")
    assert np.array_equal(ex.download("d"), np.arange(20, dtype=np.float32).reshape(4, 5))
    ex.run(f"deltensor()->({f}:d)")
    with pytest.raises(KeyError):
        ex.info("d")
    # the executor survived all of it
    assert ex.reply(f"mulscalar({f}:a2, var<float32>:2)->({f}:a2) // author=miaobyte")[0] == 0
    assert np.array_equal(ex.download("a2"), 2 * np.arange(20, dtype=np.float32).reshape(4, 5))


def test_aliased_changeshape_is_defined(ex, O):
    """transpose/broadcast with output == input are staged through a temporary (the reference races)."""
    a = np.arange(36, dtype=np.float32).reshape(6, 6)
    ex.put("t", a)
    ex.run("transpose(tensor<float32>:t, vector<int32>:[1 0])->(tensor<float32>:t) // author=miaobyte")
    assert np.array_equal(ex.download("t"), O.transpose(a, [1, 0]))
    ex.run("reshape(tensor<float32>:t, vector<int32>:[4 9])->(tensor<float32>:t) // author=miaobyte")
    assert ex.info("t") == (1, [4, 9])


def test_pool_recycles_blocks_and_enforces_its_limit():
    from deepx_b200.executor import Executor
    e = Executor(0, pool_limit_bytes=64 << 20)
    for i in range(20):
        e.new("t", "float32", [1024, 1024])  # 4 MiB each
        e.run("deltensor()->(tensor<float32>:t)")
    st = e.stats()
    assert st["driver_allocs"] == 1 and st["in_use"] == 0, st
    rc, r = e.reply("newtensor(vector<int32>:[8192 8192])->(tensor<float32>:big)")  # 256 MiB > limit
    assert rc == 1 and "pool limit" in r
    assert e.reply("newtensor(vector<int32>:[16])->(tensor<float32>:ok)")[0] == 0
    e.close()


def test_save_load_on_disk_format(ex, tmp_path):
    a = (np.arange(24, dtype=np.int32) - 7).reshape(2, 3, 4)
    ex.put("s", a)
    p = tmp_path / "s"
    ex.run(f"save(tensor<int32>:s, var<string>:{p})->()")
    text = (tmp_path / "s.shape").read_text()
    assert "dtype: int32" in text and "dim: 3" in text and "size: 24" in text
    assert np.array_equal(np.fromfile(tmp_path / "s.data", dtype=np.int32).reshape(2, 3, 4), a)
    ex.run("deltensor()->(tensor<int32>:s)")
    ex.run(f"load(var<string>:{p})->()")
    assert np.array_equal(ex.download("s"), a)
    # a file pair written the way the Python front end writes it (yaml.dump, keys sorted, block lists)
    (tmp_path / "q.shape").write_text("dim: 2\ndtype: float32\nshape:\n- 2\n- 3\nsize: 6\nstride:\n- 3\n- 1\n")
    np.arange(6, dtype=np.float32).tofile(tmp_path / "q.data")
    ex.run(f"load(var<string>:{tmp_path / 'q'})->()")
    assert np.array_equal(ex.download("q"), np.arange(6, dtype=np.float32).reshape(2, 3))


def test_udp_process_round_trip(tmp_path):
    """The executor binary behind its UDP socket, driven the way the front end drives it."""
    from deepx_b200.executor import BIN_PATH
    port = 19090 + os.getpid() % 1000
    env = dict(os.environ, DEEPX_PORT=str(port), DEEPX_OP_TABLE=str(tmp_path / "list.md"))
    proc = subprocess.Popen([str(BIN_PATH)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        assert "listening" in proc.stdout.readline()
        sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        sock.settimeout(20)

        def send(line):
            sock.sendto(line.encode(), ("127.0.0.1", port))
            return sock.recvfrom(65536)[0].decode()

        assert " ok//" in send("newtensor(vector<int32>:[3 4])->(tensor<float32>:u) // id=1")
        assert send("arange(var<int32>:0, var<int32>:1)->(tensor<float32>:u) // author=miaobyte id=2").startswith("2 ok//")
        assert " ok//" in send("newtensor(vector<int32>:[3])->(tensor<float32>:r) // id=3")
        # two lines in one datagram → two replies
        sock.sendto(b"sum(tensor<float32>:u, vector<int32>:[1], var<bool>:false)->(tensor<float32>:r) // author=miaobyte id=4\n"
                    b"print(tensor<float32>:r, var<string>:%.1f)->() // author=miaobyte id=5", ("127.0.0.1", port))
        assert sock.recvfrom(65536)[0].decode().startswith("4 ok//")
        assert sock.recvfrom(65536)[0].decode().startswith("5 ok//")
        assert send("sum(tensor<float32>:zzz, vector<int32>:[1], var<bool>:false)->(tensor<float32>:r) // id=6").startswith("6 error//")
    finally:
        proc.terminate()
        out = proc.communicate(timeout=20)[0]
    assert "[6.0 22.0 38.0]" in out, out
    assert "ops run" in out
    assert "| add | miaobyte |" in (tmp_path / "list.md").read_text()
