"""Records the deepxIR text that the reference's UNMODIFIED Python front end emits.

Runs in the build container only (needs the reference tree): imports the reference front end
from its own location, answers every datagram on UDP 9090 with an "ok" reply the way an executor
would, runs the reference's example scripts, and writes the IR lines each one sent, in order, to
tests/golden/frontend_ir/<example>.ir.  The GPU tests replay those transcripts through the
executor and check every op's result, so the executor is exercised with exactly the text the
real front end produces.

    python tests/golden/record_frontend_ir.py <path of the reference tree>
"""
import contextlib
import io
import runpy
import socket
import sys
import threading
from pathlib import Path

if len(sys.argv) < 2:
    raise SystemExit(__doc__)
REF = Path(sys.argv[1])
OUT = Path(__file__).resolve().parent / "frontend_ir"
EXAMPLES = [
    "2_ir/1_init_zeroones.py", "2_ir/2_elementwise_add.py", "2_ir/2_elementwise_operator.py", "2_ir/2_elementwise_sqrtlog.py",
    "2_ir/2_elementwise_minmax.py", "2_ir/2_elementwise_lessgreater.py", "2_ir/2_elementwise_switchwhere.py",
    "2_ir/2_elementwise_bit.py", "2_ir/4_changeshape_broadcast.py", "2_ir/4_changeshape_concat.py",
    "2_ir/4_changeshape_gather.py", "2_ir/4_changeshape_repeat.py", "2_ir/4_changeshape_reshape.py",
    "2_ir/4_changeshape_transpose.py", "2_ir/5_reduce_prod.py", "2_ir/5_reduce_sum.py", "2_ir/5_reduce_sum_keepdim.py",
    "2_ir/6_tensorlife_to.py", "3_functional/activite_relu.py", "3_functional/activite_sigmoid.py",
    "3_functional/activite_swish.py", "3_functional/changeshape_broadcast.py", "3_functional/elementwise_rsqrt.py",
    "3_functional/normalization_softmax.py", "3_functional/reduce_mean.py", "4_transformer/llama/1_llama_rmsnorm.py",
]


class FakeExecutor(threading.Thread):
    def __init__(self):
        super().__init__(daemon=True)
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        self.sock.bind(("127.0.0.1", 9090))
        self.lines = []

    def run(self):
        while True:
            data, addr = self.sock.recvfrom(65536)
            for line in data.decode().split("\n"):
                if line:
                    self.lines.append(line)
            self.sock.sendto(b"0 ok// recv_at=0 start_at=0 finish_at=0", addr)


def main():
    srv = FakeExecutor()
    srv.start()
    sys.path.insert(0, str(REF / "front" / "py"))
    # deepx/tensor/tensor.py:2 carries an unused `from triton.language.semantic import equal`; the
    # triton installed here has no such name.  Satisfy the import without touching the front end.
    import types
    for mod in ("triton", "triton.language", "triton.language.semantic"):
        sys.modules[mod] = types.ModuleType(mod)
    sys.modules["triton.language.semantic"].equal = None
    OUT.mkdir(exist_ok=True)
    for ex in EXAMPLES:
        path = REF / "front" / "py" / "examples" / ex
        if not path.exists():
            print("missing", ex)
            continue
        start = len(srv.lines)
        try:
            with contextlib.redirect_stdout(io.StringIO()):
                runpy.run_path(str(path), run_name="__main__")
        except BaseException as e:  # an example that needs files or a GPU: keep what it sent so far
            print(f"{ex}: stopped with {type(e).__name__}: {e}")
        lines = srv.lines[start:]
        name = ex.replace("/", "__").replace(".py", ".ir")
        if lines:
            (OUT / name).write_text("\n".join(lines) + "\n")
        print(f"{ex}: {len(lines)} IR lines")

    record_chains(srv)


def record_chains(srv):
    """The op chains of the two normalisation layers, as the front end's own functions emit them.

    softmax: deepx.nn.functional.softmax as it is (normalization.py:4-18).  RMSNorm: the three
    statements of T5LayerNorm.forward (t5layernorm.py:19-23) run one by one, because the module as
    written stops on its own asserts (mean(-1) wants a tuple, and weight * x wants equal ranks):
    the tuple and a reshape of the weight are supplied here, the ops sent are the front end's."""
    from deepx import arange, constant_, rsqrt, softmax
    from deepx.nn.modules.norm import RMSNorm
    start = len(srv.lines)
    x = arange(0, 48, 1, dtype="float32").reshape_((2, 3, 8))
    x.div_(10.0)
    x.sub_(2.0)
    norm = RMSNorm(8, eps=1e-6)
    constant_(norm.weight, 0.5)  # as examples/4_transformer/llama/1_llama_rmsnorm.py does
    setup = srv.lines[start:]
    start = len(srv.lines)
    variance = x.float().pow(2).mean((-1,), keepdim=True)
    xn = x * rsqrt(variance + norm.variance_epsilon)
    out = norm.weight.reshape((1, 1, 8)) * xn
    (OUT / "chains__rmsnorm_forward.ir").write_text("\n".join(setup + srv.lines[start:]) + "\n")
    print(f"chains/rmsnorm_forward: {len(setup)} setup + {len(srv.lines) - start} IR lines "
          f"(input tensor {x.name}, weight {norm.weight.name}, output {out.name})")
    start = len(srv.lines)
    sm = softmax(x, [-1])
    (OUT / "chains__softmax.ir").write_text("\n".join(setup + srv.lines[start:]) + "\n")
    print(f"chains/softmax: {len(setup)} setup + {len(srv.lines) - start} IR lines (input tensor {x.name}, output {sm.name})")

if __name__ == "__main__":
    main()
