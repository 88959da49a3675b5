"""The executor PROCESS driven the way the reference's Python front end drives it.

front/py/deepx/scheduler/client/udpconn.py:6,17-44 sends one IR line per datagram to localhost:9090 and
blocks on the reply; front/py/deepx/nn/deepxir.py:161-204 parses it as "<id> ok|error // recv_at=… start_at=…
finish_at=… [message]".  The front end itself lives in the reference tree, which does not exist where the GPU
tests run, so what goes over the wire here is the front end's own text: the transcripts recorded from the
UNMODIFIED front end running its examples (tests/golden/record_frontend_ir.py).  Each line goes to a running
`deepx-op-b200` as its own datagram, the reply is awaited and parsed like the client does, and at the end every
tensor the transcript left alive is `save`d by the process and compared, bit for bit, with the same transcript
replayed in process through the C ABI (whose results tests/test_gpu_executor.py checks op by op against the
oracle).
"""
import glob
import os
import re
import socket
import subprocess
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent
TRANSCRIPTS = sorted(glob.glob(str(HERE / "golden" / "frontend_ir" / "*.ir")))
REPLY = re.compile(r"^(\d+) (ok|error)\s*// recv_at=(\d+) start_at=(\d+) finish_at=(\d+)(?: (.*))?$", re.S)
NP_OF = {"float64": np.float64, "float32": np.float32, "float16": np.float16, "int64": np.int64, "int32": np.int32, "int16": np.int16,
         "int8": np.int8, "bool": np.bool_}


class Client:
    """udpconn.py's protocol: sendto, then block on one reply."""

    def __init__(self, port):
        self.addr = ("127.0.0.1", port)
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        self.sock.settimeout(60)

    def send(self, ir: str):
        self.sock.sendto(ir.encode("utf-8"), self.addr)
        data, _ = self.sock.recvfrom(65536)
        m = REPLY.match(data.decode("utf-8"))
        assert m, data
        return {"id": int(m.group(1)), "result": m.group(2), "recv_at": int(m.group(3)), "start_at": int(m.group(4)),
                "finish_at": int(m.group(5)), "message": m.group(6) or ""}


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    import time
    from deepx_b200.executor import BIN_PATH
    port = 24000 + os.getpid() % 20000
    env = dict(os.environ, DEEPX_PORT=str(port))
    log = tmp_path_factory.mktemp("server") / "stdout.log"   # `print` ops write there: a file never fills up like a pipe nobody reads
    with open(log, "w") as out:
        proc = subprocess.Popen([str(BIN_PATH)], env=env, stdout=out, stderr=subprocess.STDOUT)
    deadline = time.time() + 120
    while "listening" not in log.read_text() and time.time() < deadline and proc.poll() is None:
        time.sleep(0.1)
    assert "listening on udp 127.0.0.1" in log.read_text()   # loopback unless DEEPX_BIND widens it
    yield Client(port)
    proc.terminate()
    try:
        proc.communicate(timeout=30)
    except Exception:
        proc.kill()


def _names_alive(lines):
    """name -> dtype text of the tensors a transcript leaves behind."""
    alive = {}
    for line in lines:
        body = line.split("//")[0]
        if "->" not in body:
            continue
        left, right = body.split("->")
        op = left[:left.index("(")].strip()
        rets = [r.strip() for r in right[right.index("(") + 1:right.rindex(")")].split(",") if r.strip()]
        args = [a.strip() for a in left[left.index("(") + 1:left.rindex(")")].split(",") if a.strip()]
        if op == "newtensor":
            ty, nm = rets[0].split(":", 1)
            alive[nm.strip()] = ty[ty.index("<") + 1:ty.index(">")]
        elif op == "deltensor":
            alive.pop(rets[0].split(":", 1)[-1].strip(), None)
        elif op == "renametensor":
            old = rets[0].split(":", 1)[-1].strip()
            new = args[0].split(":", 1)[-1].strip()
            if old in alive:
                alive[new] = alive.pop(old)
    return alive


@pytest.mark.parametrize("path", TRANSCRIPTS, ids=[Path(p).stem for p in TRANSCRIPTS])
def test_frontend_transcript_over_udp(server, path, tmp_path):
    from deepx_b200.executor import Executor
    lines = [l for l in Path(path).read_text().splitlines() if l.strip()]
    tag = Path(path).stem[:40] + "_"
    local = Executor(0)
    try:
        for line in lines:
            r = server.send(line)
            assert r["result"] == "ok", f"{line}\n-> {r}"
            assert r["recv_at"] <= r["start_at"] <= r["finish_at"]
            rc, reply = local.reply(line)
            assert rc == 0, reply
        alive = _names_alive(lines)
        assert alive, "a transcript that leaves no tensor behind proves nothing"
        checked = 0
        for name, dtype in alive.items():
            if dtype not in NP_OF:
                continue
            target = tmp_path / f"{tag}{checked}"
            r = server.send(f"save(tensor<{dtype}>:{name}, var<string>:{target})->() // id=77")
            assert r["result"] == "ok" and r["id"] == 77, r
            want = local.download(name)
            got = np.fromfile(str(target) + ".data", dtype=NP_OF[dtype]).reshape(want.shape)
            assert np.array_equal(got.view(np.uint8), np.ascontiguousarray(want).view(np.uint8)), f"{name} differs between the process and the C ABI"
            checked += 1
        assert checked > 0
        for name, dtype in alive.items():   # leave the shared process as it was found
            server.send(f"deltensor()->(tensor<{dtype}>:{name})")
    finally:
        local.close()


def test_error_reply_keeps_the_process_alive(server):
    r = server.send("add(tensor<float32>:nope1, tensor<float32>:nope2)->(tensor<float32>:nope3) // author=miaobyte id=5")
    assert r["result"] == "error" and r["id"] == 5 and "nope" in r["message"]
    r = server.send("print(tensor<float32>:nope1, var<string>:%s%n)->() // id=6")
    assert r["result"] == "error"
    r = server.send("newtensor(vector<int32>:[2 2])->(tensor<float32>:live_ok) // id=7")
    assert r["result"] == "ok" and r["id"] == 7
    r = server.send("print(tensor<float32>:live_ok, var<string>:%s)->() // author=miaobyte id=8")
    assert r["result"] == "error" and "not allowed" in r["message"]      # the format reaches printf only when it is a numeric conversion
    r = server.send("print(tensor<float32>:live_ok, var<string>:%.2f)->() // author=miaobyte id=9")
    assert r["result"] == "ok"
    server.send("deltensor()->(tensor<float32>:live_ok)")
