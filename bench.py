#!/usr/bin/env python
"""Benchmark of the deepxIR op hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (``config.workload``): the sharded elementwise + reduce chain on float32
[2048, 1048576] (2^31 elements, U(-1,1)): t=exp(x); t=t*y; z=t+x; s=sum(z) over all axes;
m=reducemax(z) over axis 1.  The tensor is split on axis 0 over the ranks (total size fixed,
"strong" scaling); the global sum combines per-rank partials with one NCCL all-reduce.
One step = that chain once.  ``value`` = algorithmic bytes of the chain (each distinct input
read once + each output written once, all ranks) / step time, inputs resident in HBM.
``e2e`` = the same with host buffers: every step copies this rank's x and y rows from pinned
host memory and reads the two results back.

``--impl reference`` times the CPU restatement of the reference's op-ompsimd executor
(oracle/) on the host cores, on a bounded row sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS, COLS = 2048, 1 << 20
BLOCK_ROWS = 256            # data is generated per 256-row block, seed = block index
# dram__bytes_read.sum + dram__bytes_write.sum of ew2_kernel<mul,f32> on a 256-row slab, per row
MUL_TRAFFIC_PER_ROW = 3.180764e9 / 256
METRIC = "achieved HBM GB/s per op (chain: exp, mul, add, global sum, row max)"
UNIT = "GB/s"


def chain_bytes(rows: int) -> int:
    """Algorithmic bytes of one chain pass over `rows` rows of f32[.., 1048576]."""
    t = rows * COLS * 4
    return 2 * t + 3 * t + 3 * t + (t + 4) + (t + rows * 4)


def gen_block(block: int, which: str):
    import numpy as np
    rng = np.random.default_rng(block if which == "x" else 100000 + block)
    return rng.random((BLOCK_ROWS, COLS), dtype=np.float32) * np.float32(2) - np.float32(1)


def ctypes_ptr(ex) -> int:
    """The executor's CUDA stream handle as an integer."""
    from deepx_b200 import executor as E
    return int(E.lib().dx_exec_stream(ex._h) or 0)


def download_into(ex, name: str, out) -> None:
    """Device → the caller's (pinned) host array, through the executor's C ABI."""
    from deepx_b200 import executor as E
    rc = E.lib().dx_exec_download(ex._h, name.encode(), out.ctypes.data, out.nbytes)
    if rc != 0:
        raise RuntimeError(E.lib().dx_exec_last_error().decode())


def host_l3_note(working_set_bytes: int) -> str:
    """The sample's working set beside the host's last-level cache (a sample that fits it flatters the CPU)."""
    try:
        base = Path("/sys/devices/system/cpu")
        seen, total = set(), 0
        for idx in base.glob("cpu[0-9]*/cache/index3"):
            shared = (idx / "shared_cpu_list").read_text().strip()
            if shared in seen:
                continue
            seen.add(shared)
            txt = (idx / "size").read_text().strip()
            total += int(txt[:-1]) * (1 << 10 if txt.endswith("K") else 1 << 20) if txt[-1] in "KM" else int(txt)
        if total:
            return (f"working set {working_set_bytes / 2**20:.0f} MiB (x, y, t, z of the sample) against {total / 2**20:.0f} MiB of L3 "
                    f"in {len(seen)} slice(s): {'larger than' if working_set_bytes > total else 'WITHIN'} the cache")
    except Exception:
        pass
    return f"working set {working_set_bytes / 2**20:.0f} MiB; host L3 size not readable"


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 50 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())
        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
def run_reference(args) -> None:
    """CPU arm: the oracle port of op-ompsimd on the host cores, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torch.distributed.run pins OMP_NUM_THREADS to 1 for its workers; this arm is one process on all host cores
    # (the other ranks have exited), so give the OpenMP runtime the cores this process may run on before it loads
    if os.environ.get("WORLD_SIZE", "1") != "1" or "OMP_NUM_THREADS" not in os.environ:
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    import numpy as np
    from oracle import oracle as O
    O.build()
    threads = O.num_threads()
    rows = 32  # bounded sample: 32 of the 2048 rows (32 Mi elements per tensor)
    x = gen_block(0, "x")[:rows].copy()
    y = gen_block(0, "y")[:rows].copy()

    def step():
        t = O.exp(x)
        t = O.mul(t, y)
        z = O.add(t, x)
        s = O.reduce_all_parallel(O.SUM, z)
        m = O.reducemax(z, [1])
        return s, m

    for _ in range(max(args.warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    gbs = chain_bytes(rows) / dt / 1e9
    sample = f"{rows} of {ROWS} rows of the same chain per step (f32 [{rows},{COLS}]); " + host_l3_note(4 * rows * COLS * 4)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "exp,mul,add,sum(all),reducemax(axis 1) on f32 [2048,1048576] U(-1,1); CPU arm runs a row sample",
                   "rows": ROWS, "cols": COLS},
        "cpu_baseline": {"value": round(gbs, 3), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def udp_round_trip_us(ir_line: str, trips: int = 2000):
    """One IR line as one datagram to the executor process on loopback, reply awaited — what the
    reference's Python front end pays per op (front/py/deepx/scheduler/client/udpconn.py:31-44 blocks
    on the reply).  None when the process cannot be started; never raises."""
    import socket
    import subprocess
    proc = None
    try:
        from deepx_b200.executor import BIN_PATH
        port = 21000 + os.getpid() % 20000
        env = dict(os.environ, DEEPX_PORT=str(port), DEEPX_POOL_BYTES=str(256 << 20))
        proc = subprocess.Popen([str(BIN_PATH)], env=env, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        if "listening" not in proc.stdout.readline():
            return None
        sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        sock.settimeout(20)

        def send(line):
            sock.sendto(line.encode(), ("127.0.0.1", port))
            return sock.recvfrom(65536)[0]

        if b" ok" not in send("newtensor(vector<int32>:[16])->(tensor<float32>:tiny) // id=1"):
            return None
        payload = ir_line.encode()
        for _ in range(200):
            send(ir_line)
        t0 = time.perf_counter()
        for _ in range(trips):
            sock.sendto(payload, ("127.0.0.1", port))
            reply = sock.recvfrom(65536)[0]
        dt = time.perf_counter() - t0
        return dt / trips * 1e6 if b" ok" in reply else None
    except Exception:
        return None
    finally:
        if proc is not None:
            proc.terminate()
            try:
                proc.communicate(timeout=20)
            except Exception:
                proc.kill()


def cpu_baseline_leg() -> dict:
    """Bounded CPU baseline beside the GPU number (rank 0, N=1): ~10 s of oracle work."""
    import numpy as np
    from oracle import oracle as O
    O.build()
    rows = 32
    x = gen_block(0, "x")[:rows].copy()
    y = gen_block(0, "y")[:rows].copy()

    def step():
        t = O.exp(x)
        t = O.mul(t, y)
        z = O.add(t, x)
        O.reduce_all_parallel(O.SUM, z)
        O.reducemax(z, [1])

    step()
    t0 = time.perf_counter()
    n = 0
    while n < 3 or (time.perf_counter() - t0 < 8.0 and n < 200):
        step()
        n += 1
    dt = (time.perf_counter() - t0) / n
    return {"value": round(chain_bytes(rows) / dt / 1e9, 3), "unit": UNIT, "cores": O.num_threads(), "kind": "port",
            "sample": f"{n} passes over {rows} of {ROWS} rows of the same chain (f32 [{rows},{COLS}]); " + host_l3_note(4 * rows * COLS * 4)}


def cpu_ops_table(budget_s: float = 25.0) -> dict:
    """The CPU port of the reference (oracle, all host threads) on the same config shapes as the GPU
    per-op table, one to three passes each, stopping when the time budget is spent.  A baseline
    beside each GPU figure, not a target."""
    import numpy as np
    from oracle import oracle as O
    O.build()
    rng = np.random.default_rng(0)
    f32 = lambda *shape: rng.random(shape, dtype=np.float32) * 2 - 1
    cases = {}

    def case(name, make_inputs, fn, nbytes=None, flops=None):
        cases[name] = (make_inputs, fn, nbytes, flops)

    n44 = 4096 * 4096 * 4
    case("add_f32_4096x4096", lambda: (f32(4096, 4096), f32(4096, 4096)), lambda a, b: O.add(a, b), 3 * n44)
    n88 = 8192 * 8192 * 4
    case("sum_f32_8192x8192_last", lambda: (f32(8192, 8192),), lambda a: O.sum(a, [1]), n88 + 8192 * 4)
    case("sum_f32_8192x8192_axis0", lambda: (f32(8192, 8192),), lambda a: O.sum(a, [0]), n88 + 8192 * 4)
    case("max_f32_8192x8192_last", lambda: (f32(8192, 8192),), lambda a: O.reducemax(a, [1]), n88 + 8192 * 4)
    case("sum_i32_64x1024x1024_axes12", lambda: (rng.integers(-100, 101, (64, 1024, 1024)).astype(np.int32),),
         lambda a: O.sum(a, [1, 2]), 64 * 1024 * 1024 * 4 + 256)
    case("transpose_bf16_32x2048x32x128_0213", lambda: (rng.integers(0, 1 << 15, (32, 2048, 32, 128)).astype(np.int16),),
         lambda a: O.transpose(a, [0, 2, 1, 3]), 2 * 32 * 2048 * 32 * 128 * 2)
    case("concat_4x_f32_8x1024x4096_axis1", lambda: tuple(f32(8, 1024, 4096) for _ in range(4)),
         lambda *ts: O.concat(list(ts), 1), 2 * 4 * 8 * 1024 * 4096 * 4)
    case("broadcastTo_f32_1x4096_to_8192x4096", lambda: (f32(1, 4096),), lambda a: O.broadcastTo(a, [8192, 4096]), 8192 * 4096 * 4 + 4096 * 4)
    case("indexselect_f32_151936x896_by_8x2048", lambda: (f32(151936, 896), rng.integers(0, 151936, (8, 2048)).astype(np.int32)),
         lambda t, i: O.indexselect(t, i, 0), 2 * 8 * 2048 * 896 * 4 + 8 * 2048 * 4)
    case("matmul_f32_2048x4096x4096", lambda: (f32(2048, 4096) * 0.02, f32(4096, 4096) * 0.02), lambda a, b: O.matmul(a, b),
         flops=2 * 2048 * 4096 * 4096)

    def rms_chain(x, w):
        v = O.sum(O.mul(x, x), [2], True)
        v = O.rdivscalar(1.0, O.sqrt(O.addscalar(O.divscalar(v, 896.0), 1e-6)))
        return O.mul(O.mul(x, O.broadcastTo(v, x.shape)), O.broadcastTo(w, x.shape))
    nr, nv = 16 * 2048 * 896 * 4, 16 * 2048 * 4
    case("rmsnorm_ten_single_ops_f32_16x2048x896", lambda: (f32(16, 2048, 896), f32(1, 1, 896)), rms_chain,
         2 * nr + (nr + nv) + 4 * 2 * nv + (nv + nr) + 3 * nr + (896 * 4 + nr) + 3 * nr)

    out = {}
    t_start = time.perf_counter()
    for name, (make_inputs, fn, nbytes, flops) in cases.items():
        if time.perf_counter() - t_start > budget_s:
            out[name] = {"skipped": "time budget spent"}
            continue
        inputs = make_inputs()
        fn(*inputs)  # first touch of the output pages
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            fn(*inputs)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
            if time.perf_counter() - t_start > budget_s:
                break
        out[name] = {"ms": round(best * 1e3, 2), **({"gbs": round(nbytes / best / 1e9, 2)} if nbytes else {"tflops": round(flops / best / 1e12, 3)})}
        del inputs
    return {"kind": "port", "cores": O.num_threads(), "sample": "best of up to 3 passes per op at the config shape "
            "(matmul: 2048 of the 8192 rows, float32 — the CPU path has no bf16)", "ops": out}


# ------------------------------------------------------------------------------------------------
def reference_op_cuda_table(torch, peak: float) -> dict:
    """The reference's own op-cuda kernels as they are today (executor/op-cuda/src/deepx/tensorfunc/*.cu compiled
    unchanged for sm_100 into oracle/_ref/libdeepx_ref_cuda.so), timed at the config shapes beside ours: each
    call goes through the reference's launch_* wrapper (its small device vectors, default stream) and is
    synchronous; CUDA events around 3 calls after one warm-up.  A baseline row, not a target."""
    from oracle import ref_cuda as R
    lib = R.load()
    if lib is None:
        return {"unavailable": "oracle/_ref/libdeepx_ref_cuda.so was not built (no reference tree at build time)"}
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(0)
    out: dict[str, dict] = {}

    def timed(name, call, nbytes=None, flops=None):
        R.check(call())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            R.check(call())
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 3
        out[name] = {"us": round(ms * 1e3, 1), **({"gbs": round(nbytes / ms / 1e6, 1), "frac_hbm": round(nbytes / ms / 1e6 / peak, 3)}
                                                   if nbytes else {"tflops": round(flops / ms / 1e9, 1)})}

    a, b = torch.rand(4096, 4096, device=dev, generator=g), torch.rand(4096, 4096, device=dev, generator=g)
    c = torch.empty_like(a)
    timed("add_f32_4096x4096", lambda: lib.refcu_binary(0, 1, a.data_ptr(), b.data_ptr(), c.data_ptr(), a.numel()), 3 * a.numel() * 4)
    del a, b, c
    x = torch.randn(8192, 8192, device=dev, generator=g)
    o = torch.empty(8192, device=dev)
    timed("sum_f32_8192x8192_last", lambda: lib.refcu_sum(1, x.data_ptr(), R.i64(x.shape), 2, R.i32([1]), 1, 0, o.data_ptr()), x.numel() * 4 + 8192 * 4)
    timed("sum_f32_8192x8192_axis0", lambda: lib.refcu_sum(1, x.data_ptr(), R.i64(x.shape), 2, R.i32([0]), 1, 0, o.data_ptr()), x.numel() * 4 + 8192 * 4)
    del x, o
    t = torch.randn(32, 2048, 32, 128, device=dev, generator=g).to(torch.bfloat16)
    to = torch.empty(32, 32, 2048, 128, dtype=torch.bfloat16, device=dev)
    timed("transpose_bf16_32x2048x32x128_0213", lambda: lib.refcu_transpose(3, t.data_ptr(), R.i64(t.shape), 4, R.i32([0, 2, 1, 3]), to.data_ptr()),
          2 * t.numel() * 2)
    del t, to
    r = torch.randn(1, 4096, device=dev, generator=g)
    bo = torch.empty(8192, 4096, device=dev)
    timed("broadcastTo_f32_1x4096_to_8192x4096", lambda: lib.refcu_broadcast_to(1, r.data_ptr(), R.i64(r.shape), 2, R.i64(bo.shape), 2, bo.data_ptr()),
          bo.numel() * 4 + 4096 * 4)
    del r, bo
    table = torch.randn(151936, 896, device=dev, generator=g) * 0.02
    idx = torch.randint(0, 151936, (8, 2048), dtype=torch.int32, device=dev, generator=g)
    go = torch.empty(8, 2048, 896, device=dev)
    timed("indexselect_f32_151936x896_by_8x2048",
          lambda: lib.refcu_indexselect(1, table.data_ptr(), R.i64(table.shape), 2, 5, idx.data_ptr(), R.i64(idx.shape), 2, 0, go.data_ptr()),
          2 * go.numel() * 4 + idx.numel() * 4)
    del table, idx, go
    A, B = torch.randn(8192, 4096, device=dev, generator=g) * 0.02, torch.randn(4096, 4096, device=dev, generator=g) * 0.02
    Cm = torch.empty(8192, 4096, device=dev)
    timed("matmul_f32_8192x4096x4096_cublas_sgemm", lambda: lib.refcu_matmul(1, A.data_ptr(), B.data_ptr(), Cm.data_ptr(), R.i64(A.shape), R.i64(B.shape), 2),
          flops=2 * 8192 * 4096 * 4096)
    del A, B, Cm
    torch.cuda.empty_cache()
    return {"kind": "reference op-cuda kernels, unmodified, sm_100 build; bf16 matmul does not exist there (float32/float64 only)", "ops": out}


def op_cases(torch, TF, dev):
    """name -> builder returning (list of launch closures over rotating buffers, algorithmic bytes, flops or None).
    The ops of BASELINE configs 0-3 at their stated shapes, plus the chain ops on a 1 GiB slab."""
    g = torch.Generator(device=dev).manual_seed(0)
    R = 3

    def rnd(*shape, n=1, dtype=torch.float32):
        return [(torch.rand(*shape, device=dev, generator=g) * 2 - 1).to(dtype) for _ in range(n)]

    def nrm(*shape, n=1, dtype=torch.float32, scale=1.0):
        return [(torch.randn(*shape, device=dev, generator=g) * scale).to(dtype) for _ in range(n)]

    def add_f32():
        a, b = rnd(4096, 4096, n=R), rnd(4096, 4096, n=R)
        c = [torch.empty(4096, 4096, device=dev) for _ in range(R)]
        return [lambda i=i: TF.add(a[i], b[i], c[i]) for i in range(R)], 3 * 4096 * 4096 * 4, None

    def reduce_f32(op, dims):
        def build():
            x = nrm(8192, 8192, n=2)
            o = torch.empty(8192, device=dev)
            return [lambda i=i: getattr(TF, op)(x[i], dims, False, o) for i in range(2)], 8192 * 8192 * 4 + 8192 * 4, None
        return build

    def sum_i32():
        k = [torch.randint(-100, 101, (64, 1024, 1024), dtype=torch.int32, device=dev, generator=g) for _ in range(2)]
        o = torch.empty(64, dtype=torch.int32, device=dev)
        return [lambda i=i: TF.sum(k[i], [1, 2], False, o) for i in range(2)], 64 * 1024 * 1024 * 4 + 256, None

    def transpose_bf16():
        t = nrm(32, 2048, 32, 128, n=2, dtype=torch.bfloat16)
        o = torch.empty(32, 32, 2048, 128, dtype=torch.bfloat16, device=dev)
        return [lambda i=i: TF.transpose(t[i], [0, 2, 1, 3], o) for i in range(2)], 2 * o.numel() * 2, None

    def transpose_inner(dtype):
        def build():  # innermost axis moves: the shared-memory tile path
            t = nrm(8192, 8192, n=2, dtype=dtype)
            o = torch.empty(8192, 8192, dtype=dtype, device=dev)
            return [lambda i=i: TF.transpose(t[i], [1, 0], o) for i in range(2)], 2 * o.numel() * o.element_size(), None
        return build

    def concat_f32():
        parts = nrm(8, 1024, 4096, n=4)
        o = torch.empty(8, 4096, 4096, device=dev)
        return [lambda: TF.concat(parts, 1, o)], 2 * o.numel() * 4, None

    def broadcast_f32():
        r = nrm(1, 4096)[0]
        o = [torch.empty(8192, 4096, device=dev) for _ in range(R)]
        return [lambda i=i: TF.broadcastTo(r, [8192, 4096], o[i]) for i in range(R)], 8192 * 4096 * 4 + 4096 * 4, None

    def indexselect_f32():
        table = nrm(151936, 896, scale=0.02)[0]
        idx = [torch.randint(0, 151936, (8, 2048), dtype=torch.int32, device=dev, generator=g) for _ in range(R)]
        o = [torch.empty(8, 2048, 896, device=dev) for _ in range(R)]
        return [lambda i=i: TF.indexselect(table, idx[i], 0, o[i]) for i in range(R)], 2 * 8 * 2048 * 896 * 4 + 8 * 2048 * 4, None

    def matmul_bf16():
        A = nrm(8192, 4096, dtype=torch.bfloat16, scale=0.02)[0]
        B = nrm(4096, 4096, dtype=torch.bfloat16, scale=0.02)[0]
        Cm = torch.empty(8192, 4096, dtype=torch.bfloat16, device=dev)
        return [lambda: TF.matmul(A, B, Cm)], 0, 2 * 8192 * 4096 * 4096

    def matmul_f32():
        A = nrm(8192, 4096, scale=0.02)[0]
        B = nrm(4096, 4096, scale=0.02)[0]
        Cm = torch.empty(8192, 4096, device=dev)
        return [lambda: TF.matmul(A, B, Cm)], 0, 2 * 8192 * 4096 * 4096

    def pow_f32(kind):
        def build():  # 256 MiB per tensor, as in --sweep: what the profiler captures of the pow kernels are taken on
            n = (256 << 20) // 4
            a = [(torch.rand(n, device=dev, generator=g) * 1.5 + 0.5) for _ in range(R)]
            b = [(torch.rand(n, device=dev, generator=g) * 1.5 + 0.5) for _ in range(R)]
            c = [torch.empty(n, device=dev) for _ in range(R)]
            if kind == "pow":
                return [lambda i=i: TF.pow(a[i], b[i], c[i]) for i in range(R)], 3 * n * 4, None
            if kind == "powscalar":
                return [lambda i=i: TF.powscalar(a[i], 2.5, c[i]) for i in range(R)], 2 * n * 4, None
            return [lambda i=i: TF.rpowscalar(1.7, a[i], c[i]) for i in range(R)], 2 * n * 4, None
        return build

    def rms_fused():
        x = nrm(16, 2048, 896, n=R)
        w = nrm(896)[0]
        y = [torch.empty(16, 2048, 896, device=dev) for _ in range(R)]
        n = 16 * 2048 * 896 * 4
        return [lambda i=i: TF.rmsnorm(x[i], w, 896.0, 1e-6, y[i]) for i in range(R)], 2 * n + 896 * 4, None

    def rms_single_ops():
        """The ten IR ops of the RMSNorm chain, one launch each: what the fused kernel replaces."""
        x = nrm(16, 2048, 896, n=R)
        w = nrm(1, 1, 896)[0]
        sq, vb, y, wb, out = (torch.empty(16, 2048, 896, device=dev) for _ in range(5))
        v = torch.empty(16, 2048, 1, device=dev)
        n, nv, shp = 16 * 2048 * 896 * 4, 16 * 2048 * 4, [16, 2048, 896]

        def chain(i):
            TF.mul(x[i], x[i], sq)
            TF.sum(sq, [2], True, v)
            TF.divscalar(v, 896.0, v)
            TF.addscalar(v, 1e-6, v)
            TF.sqrt(v, v)
            TF.rdivscalar(1.0, v, v)
            TF.broadcastTo(v, shp, vb)
            TF.mul(x[i], vb, y)
            TF.broadcastTo(w, shp, wb)
            TF.mul(y, wb, out)
        total = 2 * n + (n + nv) + 4 * 2 * nv + (nv + n) + 3 * n + (896 * 4 + n) + 3 * n
        return [lambda i=i: chain(i) for i in range(R)], total, None

    def softmax_fused():
        x = nrm(32768, 2048, n=R)
        y = [torch.empty(32768, 2048, device=dev) for _ in range(R)]
        return [lambda i=i: TF.softmax(x[i], y[i]) for i in range(R)], 2 * 32768 * 2048 * 4, None

    def rms(opname):
        def build():
            x = nrm(16, 2048, 896, n=R)
            y = [torch.empty(16, 2048, 896, device=dev) for _ in range(R)]
            v = torch.empty(16, 2048, 1, device=dev)
            n = 16 * 2048 * 896 * 4
            if opname == "mul":
                return [lambda i=i: TF.mul(x[i], x[i], y[i]) for i in range(R)], 2 * n, None
            if opname == "sum":
                return [lambda i=i: TF.sum(x[i], [2], True, v) for i in range(R)], n + 16 * 2048 * 4, None
            if opname == "broadcast":
                return [lambda i=i: TF.broadcastTo(v, [16, 2048, 896], y[i]) for i in range(R)], n + 16 * 2048 * 4, None
            return [lambda i=i: TF.mul(x[i], y[(i + 1) % R], y[i]) for i in range(R)], 3 * n, None
        return build

    def chain(opname):
        def build():  # the bench chain on 256 of the 2048 rows (1 GiB per tensor): the size used for profiler captures
            x, y = rnd(256, 1 << 20)[0], rnd(256, 1 << 20)[0]
            t, z = torch.empty_like(x), torch.empty_like(x)
            s1, m = torch.empty(1, device=dev), torch.empty(256, device=dev)
            n = x.numel() * 4
            return {"exp": ([lambda: TF.exp(x, t)], 2 * n, None), "mul": ([lambda: TF.mul(x, y, t)], 3 * n, None),
                    "add": ([lambda: TF.add(x, y, z)], 3 * n, None), "sum": ([lambda: TF.sum(x, [0, 1], False, s1)], n + 4, None),
                    "rowmax": ([lambda: TF.reducemax(x, [1], False, m)], n + 1024, None)}[opname]
        return build

    return {
        "add_f32_4096x4096": add_f32,
        "sum_f32_8192x8192_last": reduce_f32("sum", [1]), "sum_f32_8192x8192_axis0": reduce_f32("sum", [0]),
        "max_f32_8192x8192_last": reduce_f32("reducemax", [1]), "max_f32_8192x8192_axis0": reduce_f32("reducemax", [0]),
        "sum_i32_64x1024x1024_axes12": sum_i32,
        "transpose_bf16_32x2048x32x128_0213": transpose_bf16,
        "transpose_f32_8192x8192_10": transpose_inner(torch.float32), "transpose_bf16_8192x8192_10": transpose_inner(torch.bfloat16), "concat_4x_f32_8x1024x4096_axis1": concat_f32,
        "broadcastTo_f32_1x4096_to_8192x4096": broadcast_f32, "indexselect_f32_151936x896_by_8x2048": indexselect_f32,
        "matmul_bf16_8192x4096x4096": matmul_bf16, "matmul_f32_8192x4096x4096": matmul_f32,
        "pow_f32_64Mi": pow_f32("pow"), "powscalar_2.5_f32_64Mi": pow_f32("powscalar"), "rpowscalar_1.7_f32_64Mi": pow_f32("rpowscalar"),
        "rmsnorm_fused_f32_16x2048x896": rms_fused, "softmax_fused_f32_32768x2048": softmax_fused,
        "rmsnorm_ten_single_ops_f32_16x2048x896": rms_single_ops,
        "rmsnorm_mul_xx_f32_16x2048x896": rms("mul"), "rmsnorm_sum_last_f32_16x2048x896": rms("sum"),
        "rmsnorm_broadcast_f32_16x2048x1": rms("broadcast"), "rmsnorm_mul_xy_f32_16x2048x896": rms("mul3"),
        "chain_exp_f32_256x1048576": chain("exp"), "chain_mul_f32_256x1048576": chain("mul"), "chain_add_f32_256x1048576": chain("add"),
        "chain_sum_f32_256x1048576": chain("sum"), "chain_rowmax_f32_256x1048576": chain("rowmax"),
    }


def time_case(torch, fns, nbytes, flops, peak, iters, warmup=1, graph=True):
    """Average time of one launch.  The launches are recorded once into a CUDA graph and the graph is
    replayed, so the figure is the kernels' (the host side of a 20 µs op — Python, ctypes — would
    otherwise be what is timed).  Buffers rotate between launches so L2 cannot hold an input."""
    for _ in range(max(warmup, 1)):
        for f in fns:
            f()
    torch.cuda.synchronize()
    replay = None
    if graph:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(iters):
                    fns[i % len(fns)]()
            replay = g.replay
            replay()
            torch.cuda.synchronize()
        except Exception:
            replay = None
            torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    if replay is not None:
        replay()
    else:
        for i in range(iters):
            fns[i % len(fns)]()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / iters
    how = "cuda-graph replay" if replay is not None else "direct launches"
    if flops is None:
        gbs = nbytes / ms / 1e6
        return {"us": round(ms * 1e3, 1), "gbs": round(gbs, 1), "frac_hbm": round(gbs / peak, 3), "timed": how}
    return {"us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1), "timed": how}


def per_op_table(torch, TF, N, peak: float) -> dict:
    """Single-GPU GB/s of each op of the other configs (rotating buffers so L2 cannot help)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    out: dict[str, dict] = {}
    for name, build in op_cases(torch, TF, dev).items():
        if name.startswith("chain_"):
            continue
        fns, nbytes, flops = build()
        out[name] = time_case(torch, fns, nbytes, flops, peak, iters=20 if flops else 12)
        del fns
        torch.cuda.empty_cache()
    N.check(N.lib.dx_matmul_status(None))
    return out


def run_one_op(args) -> None:
    """`--op NAME`: one op of the table on its own (what the profiler captures are taken on)."""
    import torch
    from deepx_b200 import _native as N
    from deepx_b200 import tensorfunc as TF
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    cases = op_cases(torch, TF, dev)
    if args.op not in cases:
        raise SystemExit("unknown --op; choose from: " + ", ".join(cases))
    fns, nbytes, flops = cases[args.op]()
    peak, kind = measured_peaks()
    res = time_case(torch, fns, nbytes, flops, peak, iters=args.steps, warmup=args.warmup, graph=not args.no_graph)
    res.update({"op": args.op, "steps": args.steps, "algorithmic_bytes": nbytes, "peak_source": kind})
    print(json.dumps(res), flush=True)


def run_ours(args) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from deepx_b200 import _native as N
    from deepx_b200.sharded import RowPartition, ShardedOps
    ops = ShardedOps(defer=True)  # the combine of the global sum runs after the row max: the skew between ranks is hidden
    part = RowPartition(ROWS, world)
    my_rows = part.count(rank)
    row0 = part.start(rank)

    # ---- this rank's rows, generated per 256-row block (seed = block index), pinned on the host
    hx = torch.empty((my_rows, COLS), dtype=torch.float32).pin_memory()
    hy = torch.empty((my_rows, COLS), dtype=torch.float32).pin_memory()
    pieces = []
    r = row0
    while r < row0 + my_rows:
        blk, off = divmod(r, BLOCK_ROWS)
        n = min(BLOCK_ROWS - off, row0 + my_rows - r)
        pieces.append((blk, off, n, r - row0))
        r += n

    def fill(job):
        (blk, off, n, dst), which = job
        host = hx if which == "x" else hy
        host[dst:dst + n].copy_(torch.from_numpy(gen_block(blk, which)[off:off + n]))

    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=min(8, max(1, (os.cpu_count() or 8) // max(world, 1)))) as ex:
        list(ex.map(fill, [(pc, w) for pc in pieces for w in ("x", "y")]))

    x = torch.empty((my_rows, COLS), dtype=torch.float32, device=dev)
    y = torch.empty_like(x)
    t = torch.empty_like(x)
    z = torch.empty_like(x)
    s = torch.empty(1, dtype=torch.float32, device=dev)
    m = torch.empty(my_rows, dtype=torch.float32, device=dev)
    hs = torch.empty(1, dtype=torch.float32).pin_memory()
    hm = torch.empty(my_rows, dtype=torch.float32).pin_memory()
    x.copy_(hx, non_blocking=True)
    y.copy_(hy, non_blocking=True)
    torch.cuda.synchronize()

    mul_events: list = []

    def chain(record_mul: bool = False):
        ops.exp(x, t)
        if record_mul:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        ops.mul(t, y, t)
        if record_mul:
            e1.record()
            mul_events.append((e0, e1))
        ops.add(t, x, z)
        ops.sum(z, [0, 1], False, s)
        ops.reducemax(z, [1], False, m)
        ops.flush()  # wait for the peers' partial sums and combine them: part of the step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- device-resident number ----------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        chain()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    if ops.peer is not None:
        ops.peer.wait_stats(reset=True)
    l0 = N.lib.dx_launch_count()
    # the dominant kernel is timed with a pair of events on a few of the timed steps (first, middle, last): an event
    # between two kernels costs their boundary the overlapped launch (a few µs), so not on every step
    sampled = sorted({0, args.steps // 2, args.steps - 1})
    step_no = [0]

    def timed_step():
        chain(step_no[0] in sampled)
        step_no[0] += 1

    ms_total = timed(timed_step, args.steps)
    launches = N.lib.dx_launch_count() - l0
    # what the rendezvous cost inside the timed region: the flag waits of this rank's combine CTAs (worst rank reported)
    exchange = None
    if ops.peer is not None:
        wait_us, waits = ops.peer.wait_stats(reset=True)
        w = torch.tensor([wait_us], dtype=torch.float64, device=dev)
        dist.all_reduce(w, op=dist.ReduceOp.MAX)
        exchange = {"flag_wait_us_per_step": round(float(w.item()) / args.steps, 2), "waits_per_step": waits / args.steps,
                    "what": "SM time the combine CTAs of the slowest-waiting rank spent polling peers' flags (dx_comm_wait_stats); "
                            "a wait that finds the flags set still counts the round trip of its acquire loads"}
    # nvidia-smi cannot sample faster than every few tens of ms; a short timed region (many GPUs, few
    # steps) may pass between two samples.  Keep the same chain running, untimed, until a few samples
    # exist, so that the clocks reported are clocks under this load.
    extra_passes = 0
    need_more = torch.tensor([1 if (sampler is not None and len(sampler.lines) < 3) else 0], device=dev)
    if world > 1:
        dist.broadcast(need_more, src=0)
    if int(need_more.item()):
        # the same count on every rank (the chain holds a collective): ~0.4 s worth, from the agreed timing
        extra_passes = int(min(2000, max(3, 400.0 / max(ms_total / args.steps, 1e-3))))
        for _ in range(extra_passes):
            chain()
        barrier()
    clocks = sampler.stop() if sampler else None
    if clocks is not None:
        clocks["window"] = "timed region" if extra_passes == 0 else f"timed region + {extra_passes} untimed passes of the same chain"
    ms_step = ms_total / args.steps
    total_bytes = chain_bytes(ROWS)
    value = total_bytes / ms_step / 1e6

    # parity guard on the outputs of the last timed step, over ALL of this rank's rows: the z the GPU holds
    # comes back in 256-row pieces; its row maxima must equal the device's bit for bit, its float64 sum
    # (all ranks together) must match the device's global sum within 1e-5 of sum|z|, and the first and
    # last 8 rows of the rank must match the chain recomputed on the host from x and y (rtol 1e-5).
    torch.cuda.synchronize()
    if ops.peer is not None:
        ops.peer.status()  # raises if a wait on a peer expired: a number with a skipped combine is not reported
    got_sum = float(s.item())
    got_m = m.cpu().numpy()
    part = np.zeros(2, dtype=np.float64)
    hz = torch.empty((min(BLOCK_ROWS, my_rows), COLS), dtype=torch.float32).pin_memory()
    for r0 in range(0, my_rows, BLOCK_ROWS):
        n = min(BLOCK_ROWS, my_rows - r0)
        hz[:n].copy_(z[r0:r0 + n])
        zb = hz[:n].numpy()
        if not np.array_equal(zb.max(axis=1).view(np.uint32), got_m[r0:r0 + n].view(np.uint32)):
            raise SystemExit(f"bench: row maxima of local rows {r0}..{r0 + n} are not those of z — refusing to report a number")
        part[0] += zb.sum(dtype=np.float64)
        part[1] += np.abs(zb).sum(dtype=np.float64)
        for lo in ({0, max(n - 8, 0)} if r0 in (0, (my_rows - 1) // BLOCK_ROWS * BLOCK_ROWS) else ()):
            hxr, hyr = hx[r0 + lo:r0 + lo + 8].numpy(), hy[r0 + lo:r0 + lo + 8].numpy()
            want = (np.exp(hxr.astype(np.float64)).astype(np.float32) * hyr + hxr)
            if not np.allclose(zb[lo:lo + 8], want, rtol=1e-5, atol=1e-6):
                raise SystemExit(f"bench: z of local rows {r0 + lo}..{r0 + lo + 8} disagrees with the host chain — refusing to report a number")
    del hz
    tot = torch.from_numpy(part).to(dev)
    if world > 1:
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    sum64, abs64 = (float(v) for v in tot.cpu())
    sum_rel_err = abs(got_sum - sum64) / max(abs64, 1e-300)
    if sum_rel_err > 1e-5:
        raise SystemExit(f"bench: global sum {got_sum} vs float64 {sum64} (sum|z| {abs64}) — refusing to report a number")
    parity_guard = {"rows_checked": ROWS, "row_max": "bit-exact against the max of the downloaded z, every row",
                    "z_rows_vs_host_chain": "first and last 8 rows of each rank, rtol 1e-5 + atol 1e-6",
                    "sum_rel_err": sum_rel_err, "sum_tolerance": "1e-5 of sum|z|, float64 over every element"}

    mul_ms = statistics.mean(a.elapsed_time(b) for a, b in mul_events)
    peak, peak_kind = measured_peaks()
    mul_bytes = 3 * my_rows * COLS * 4
    achieved = mul_bytes / mul_ms / 1e6

    # ---- end-to-end number: through the deepxIR executor (the reference-facing boundary), host buffers
    # in, results out, every step.  The device-resident tensors above are released first.  Every rank is one
    # executor of a world-of-N (dx_exec_set_shard): it gets the SAME IR lines with the GLOBAL shapes, holds its
    # rows of the partitioned tensors, and the global sum is combined by the executor itself over peer memory —
    # no torch.distributed call inside a step.
    del x, y, t, z
    torch.cuda.empty_cache()
    from deepx_b200.executor import Executor
    ex = Executor(local_rank)
    ex_comm = None
    if world > 1:
        from deepx_b200.comm import PeerComm
        ex_comm = PeerComm()  # set-up only: the IPC handles of the mailboxes travel through the process group
        ex.set_shard(rank, world, ex_comm._h, min_bytes=4096)
    f32 = "tensor<float32>"
    for nm, shp in (("x", (ROWS, COLS)), ("y", (ROWS, COLS)), ("t", (ROWS, COLS)), ("z", (ROWS, COLS)), ("s", (1,)), ("m", (ROWS,))):
        ex.new(nm, "float32", shp)
    if world > 1:
        assert ex.shard("x") == (True, row0, my_rows, ROWS) and ex.shard("m") == (True, row0, my_rows, ROWS) and not ex.shard("s")[0]
    ir = [f"exp({f32}:x)->({f32}:t) // author=miaobyte",
          f"mul({f32}:t, {f32}:y)->({f32}:t) // author=miaobyte",
          f"add({f32}:t, {f32}:x)->({f32}:z) // author=miaobyte",
          f"sum({f32}:z, vector<int32>:[0 1], var<bool>:false)->({f32}:s) // author=miaobyte",
          f"reducemax({f32}:z, vector<int32>:[1], var<bool>:false)->({f32}:m) // author=miaobyte"]
    hx_np, hy_np, hs_np, hm_np = hx.numpy(), hy.numpy(), hs.numpy(), hm.numpy()  # views of the pinned buffers
    ex_stream = torch.cuda.ExternalStream(ctypes_ptr(ex), device=dev)

    def e2e_step():
        ex.upload_async("x", hx_np)   # copy stream; exp waits for x only, so it runs while y is still on its way
        ex.upload_async("y", hy_np)
        for line in ir:
            ex.run(line)
        download_into(ex, "s", hs_np)  # completes the deferred combine of the partial sums first
        download_into(ex, "m", hm_np)

    def copies_only():
        ex.upload_async("x", hx_np)
        ex.upload_async("y", hy_np)
        ex.sync()

    def timed_ex(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ex_stream):
            e0.record()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        ex.sync()
        wall_ms = (time.perf_counter() - t0) * 1e3
        with torch.cuda.stream(ex_stream):
            e1.record()
        ex.sync()
        barrier()
        # the uploads run on the executor's copy stream: the step ends when the compute stream has consumed them, which
        # the events on the compute stream see; the host clock around the same region must agree with them
        ms = torch.tensor([max(e0.elapsed_time(e1), 0.0), wall_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms[0].item()), float(ms[1].item())

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    e2e_ms, e2e_wall_ms = (v / e2e_steps for v in timed_ex(e2e_step, e2e_steps))
    if abs(float(hs_np[0]) - got_sum) > 1e-4 * abs(got_sum) + 1e-3 or not np.array_equal(hm_np, got_m):
        raise SystemExit("bench: the executor path and the direct path disagree — refusing to report a number")
    # what the host can deliver: the same two uploads from the same pinned buffers and nothing else
    copies_only()
    h2d_ms, _ = (v / e2e_steps for v in timed_ex(copies_only, e2e_steps))
    h2d_bytes = 2 * my_rows * COLS * 4 * world
    executor_us = compiled_us = None
    tiny_ir = "addscalar(tensor<float32>:tiny, var<float32>:1)->(tensor<float32>:tiny) // author=miaobyte id=7"
    if world == 1:
        # what one IR line costs on the host side: parse, registry lookup, tensor lookup, one launch of a 16-element op
        ex.run("newtensor(vector<int32>:[16])->(tensor<float32>:tiny)")
        ex.run("constant(var<float32>:1)->(tensor<float32>:tiny)")
        for _ in range(100):
            ex.run(tiny_ir)
        ex.sync()
        t0 = time.perf_counter()
        for _ in range(3000):
            ex.run(tiny_ir)
        ex.sync()
        executor_us = (time.perf_counter() - t0) / 3000 * 1e6
        # the same line 200 times as one compiled program (CUDA graph): one launch call per replay
        prog = ex.compile("\n".join([tiny_ir] * 200))
        for _ in range(3):
            prog.run()
        ex.sync()
        t0 = time.perf_counter()
        for _ in range(50):
            prog.run()
        ex.sync()
        compiled_us = (time.perf_counter() - t0) / (50 * 200) * 1e6
        prog.free()
    ex.close()
    if ex_comm is not None:
        ex_comm.close()
    udp_us = udp_round_trip_us(tiny_ir) if world == 1 else None
    e2e_value = total_bytes / e2e_ms / 1e6

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "z=exp(x)*y+x, s=sum(z), m=reducemax(z,axis 1) on f32 [2048,1048576] U(-1,1) sharded on axis 0; "
                               "deepxIR ops exp,mul,add,sum,reducemax",
                   "rows": ROWS, "cols": COLS, "rows_per_gpu": my_rows, "parallelism": f"axis0-shard x{world}",
                   "l2": "inputs larger than L2 (8 GiB per tensor)", "algorithmic_bytes_per_step": total_bytes,
                   "combine": "none (1 GPU)" if world == 1 else ("peer-memory kernel (dx_comm)" if ops.peer is not None else "NCCL all-reduce")},
        "roofline": {"bound": "hbm", "kernel": "ew2_kernel<mul,f32> (t=t*y)", "achieved": round(achieved, 1), "peak": peak,
                     "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})", "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": round(MUL_TRAFFIC_PER_ROW * my_rows), "traffic_source": "ncu dram read+write of the same kernel on 256 rows "
                     "(profiles/ew2_mul_f32_chain_256x1048576.md), scaled by rows",
                     "bytes_per_launch": mul_bytes, "us_per_launch": round(mul_ms * 1e3, 2),
                     "timed_on": f"CUDA events around the kernel on {len(mul_events)} of the {args.steps} timed steps"},
        "e2e": {"value": round(e2e_value, 1), "unit": UNIT, "h2d_bytes_per_step": 2 * my_rows * COLS * 4 * world,
                "d2h_bytes_per_step": (4 + my_rows * 4) * world, "ms_per_step": round(e2e_ms, 3), "ms_per_step_host_clock": round(e2e_wall_ms, 3),
                "steps": e2e_steps,
                "h2d_bound_gbs": round(total_bytes / h2d_ms / 1e6, 1), "h2d_gbs_per_gpu": round(h2d_bytes / world / h2d_ms / 1e6, 1),
                "frac_of_h2d_bound": round(h2d_ms / e2e_ms, 3),
                "h2d_bound": "the same metric if a step were nothing but its two uploads (same pinned buffers, same copy stream, all ranks at once)",
                "path": "executor only: deepxIR text -> libdeepx_exec.so (dx_exec_upload_async / dx_exec_run / dx_exec_download), pinned host buffers; "
                        + ("one executor" if world == 1 else f"one executor per GPU as ranks of a world of {world} (dx_exec_set_shard): global shapes in the IR, "
                           "rows partitioned by the executor, partial sums combined by its own peer-memory exchange")},
        "executor": {"us_per_ir_line": None if executor_us is None else round(executor_us, 2),
                     "us_per_ir_line_compiled": None if compiled_us is None else round(compiled_us, 2),
                     "us_per_udp_round_trip": None if udp_us is None else round(udp_us, 2),
                     "what": "3000 addscalar lines on a 16-element tensor through dx_exec_run from Python (parse + dispatch + launch); "
                             "compiled: the same line 200x as one program captured into a CUDA graph (dx_exec_compile), 50 replays; "
                             "udp: the same line as one datagram to the deepx-op-b200 process on loopback, reply awaited, 2000 times"},
        "gpu_launches": int(launches),
        "exchange": exchange,
        "clocks": clocks,
        "global_sum": got_sum,
        "parity_guard": parity_guard,
    }
    if world == 1 and rank == 0:
        try:
            line["cpu_baseline"] = cpu_baseline_leg()
        except Exception as ex:  # the CPU leg must never take the GPU number down with it
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"failed: {ex}"}
        if not args.no_ops:
            torch.cuda.empty_cache()
            from deepx_b200 import tensorfunc as TF
            line["ops"] = per_op_table(torch, TF, N, peak)
            try:
                line["cpu_ops"] = cpu_ops_table()
            except Exception as ex:
                line["cpu_ops"] = {"failed": str(ex)}
            try:
                line["reference_op_cuda"] = reference_op_cuda_table(torch, peak)
            except Exception as ex:
                line["reference_op_cuda"] = {"failed": str(ex)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_sweep(args) -> None:
    """`--sweep`: every elementwise / compare / switch / cast / reduce / transpose op in every dtype on
    256 MiB tensors (CUDA-graph replay, rotating buffers), as a fraction of the measured HBM peak.
    Prints one JSON object: {"ops": {name: frac}, "below_0.8": {...}}."""
    import torch
    from deepx_b200 import tensorfunc as TF
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    peak, peak_kind = measured_peaks()
    R, BYTES = 3, 256 << 20
    DT = {"f64": torch.float64, "f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "i64": torch.int64,
          "i32": torch.int32, "i16": torch.int16, "i8": torch.int8}
    res: dict[str, float] = {}

    def run(name, fns, nbytes):
        res[name] = time_case(torch, fns, nbytes, None, peak, iters=9)["frac_hbm"]

    for dn, dt in DT.items():
        es = torch.empty(0, dtype=dt).element_size()
        n = BYTES // es

        def mk():
            if dt.is_floating_point:
                return (torch.rand(n, device=dev) * 1.5 + 0.5).to(dt)
            return torch.randint(1, 100, (n,), device=dev).to(dt)
        a, b = [mk() for _ in range(R)], [mk() for _ in range(R)]
        c = [torch.empty_like(a[0]) for _ in range(R)]
        m = [torch.empty(n, dtype=torch.bool, device=dev) for _ in range(R)]
        for op in ("add", "sub", "mul", "div", "max", "min"):
            run(f"{op}<{dn}>", [lambda i=i, op=op: getattr(TF, op)(a[i], b[i], c[i]) for i in range(R)], 3 * n * es)
        for op in ("addscalar", "subscalar", "rsubscalar", "mulscalar", "divscalar", "rdivscalar", "maxscalar", "minscalar"):
            run(f"{op}<{dn}>", [lambda i=i, op=op: (getattr(TF, op)(2, a[i], c[i]) if op.startswith("r") else getattr(TF, op)(a[i], 2, c[i]))
                               for i in range(R)], 2 * n * es)
        for op in ("less", "greater", "equal", "notequal"):
            if op in ("equal", "notequal"):
                run(f"{op}<{dn}>", [lambda i=i, op=op: getattr(TF, op)(a[i], b[i], 0.0, m[i]) for i in range(R)], n * (2 * es + 1))
            else:
                run(f"{op}<{dn}>", [lambda i=i, op=op: getattr(TF, op)(a[i], b[i], m[i]) for i in range(R)], n * (2 * es + 1))
        if dt.is_floating_point:
            for op in ["sqrt", "exp", "log", "sin", "cos"] + (["tan"] if dn in ("f64", "f32") else []):
                run(f"{op}<{dn}>", [lambda i=i, op=op: getattr(TF, op)(a[i], c[i]) for i in range(R)], 2 * n * es)
            if dn in ("f64", "f32"):
                run(f"pow<{dn}>", [lambda i=i: TF.pow(a[i], b[i], c[i]) for i in range(R)], 3 * n * es)
                run(f"powscalar(2)<{dn}>", [lambda i=i: TF.powscalar(a[i], 2, c[i]) for i in range(R)], 2 * n * es)
                run(f"powscalar(2.5)<{dn}>", [lambda i=i: TF.powscalar(a[i], 2.5, c[i]) for i in range(R)], 2 * n * es)
        else:
            run(f"invert<{dn}>", [lambda i=i: TF.invert(a[i], c[i]) for i in range(R)], 2 * n * es)
        cases = [torch.randint(0, 2, (n,), device=dev, dtype=torch.int32) for _ in range(R)]
        run(f"switch(2 sources, int32 cases)<{dn}>", [lambda i=i: TF.Switch([a[i], b[i]], cases[i], c[i]) for i in range(R)], n * (3 * es + 4))
        del cases
        run(f"switch(2 sources, bool cases)<{dn}>", [lambda i=i: TF.Switch([a[i], b[i]], m[i], c[i]) for i in range(R)], n * (3 * es + 1))
        for dn2 in ("f32", "bf16", "i32", "i8"):
            if dn2 != dn:
                o = [torch.empty(n, dtype=DT[dn2], device=dev) for _ in range(R)]
                run(f"todtype<{dn}->{dn2}>", [lambda i=i, o=o: TF.todtype(a[i], o[i]) for i in range(R)], n * (es + o[0].element_size()))
                del o
        x = [t.view(4096, n // 4096) for t in a]
        for op in ("sum", "prod", "reducemax", "reducemin"):
            for dims, oshape in (([1], (4096,)), ([0], (n // 4096,)), ([0, 1], (1,))):
                o = torch.empty(oshape, dtype=dt, device=dev)
                run(f"{op}<{dn}> [4096,{n // 4096}] dims{dims}", [lambda i=i, op=op, dims=dims, o=o: getattr(TF, op)(x[i], dims, False, o) for i in range(R)], n * es)
        t3 = [t.view(64, 512, n // 32768) for t in a]
        for perm in ([0, 2, 1], [1, 0, 2], [2, 0, 1]):
            o = [torch.empty([t3[0].shape[q] for q in perm], dtype=dt, device=dev) for _ in range(R)]
            run(f"transpose<{dn}> [64,512,{n // 32768}] {perm}", [lambda i=i, perm=perm, o=o: TF.transpose(t3[i], perm, o[i]) for i in range(R)], 2 * n * es)
            del o
        if dn in ("f32", "bf16", "i8"):
            # concat of four equal parts along each axis of a 3-d tensor (output 256 MiB)
            q3 = [t.view(64, 512, n // 32768) for t in a]
            for axis in (0, 1, 2):
                parts = [[q3[i].narrow(axis, k * (q3[i].shape[axis] // 4), q3[i].shape[axis] // 4).contiguous() for k in range(4)] for i in range(R)]
                o = [torch.empty_like(q3[0]) for _ in range(R)]
                run(f"concat<{dn}> 4 parts of [64,512,{n // 32768}] axis {axis}", [lambda i=i, axis=axis, parts=parts, o=o: TF.concat(parts[i], axis, o[i]) for i in range(R)], 2 * n * es)
                del parts, o
            # broadcastTo: a row repeated (inner axis kept), a column repeated (inner axis replicated), a scalar
            row, col = a[0][: n // 4096].view(1, n // 4096).contiguous(), a[0][:4096].view(4096, 1).contiguous()
            o = [torch.empty(4096, n // 4096, dtype=dt, device=dev) for _ in range(R)]
            run(f"broadcastTo<{dn}> [1,{n // 4096}] -> [4096,{n // 4096}]", [lambda i=i: TF.broadcastTo(row, [4096, n // 4096], o[i]) for i in range(R)], n * es + row.numel() * es)
            run(f"broadcastTo<{dn}> [4096,1] -> [4096,{n // 4096}]", [lambda i=i: TF.broadcastTo(col, [4096, n // 4096], o[i]) for i in range(R)], n * es + 4096 * es)
            del o
            # indexselect: rows of a [65536, n/65536] table by 2^16 random indices (axis 0), and along the inner axis
            table = [t.view(65536, n // 65536) for t in a]
            idx = torch.randint(0, 65536, (65536,), device=dev, dtype=torch.int32)
            o = [torch.empty_like(table[0]) for _ in range(R)]
            run(f"indexselect<{dn}> rows of [65536,{n // 65536}]", [lambda i=i: TF.indexselect(table[i], idx, 0, o[i]) for i in range(R)], 2 * n * es + 65536 * 4)
            wide = [t.view(n // 1024, 1024) for t in a]
            idx2 = torch.randint(0, 1024, (1024,), device=dev, dtype=torch.int32)
            o2 = [torch.empty_like(wide[0]) for _ in range(R)]
            run(f"indexselect<{dn}> inner axis of [{n // 1024},1024]", [lambda i=i: TF.indexselect(wide[i], idx2, 1, o2[i]) for i in range(R)], 2 * n * es + 4096)
            del table, o, wide, o2
            # repeat: [64,512,n/131072] x (1,2,2)
            src = a[0][: n // 4].view(64, 512, n // 131072)
            o = [torch.empty(64, 1024, n // 65536, dtype=dt, device=dev) for _ in range(R)]
            run(f"repeat<{dn}> [64,512,{n // 131072}] x (1,2,2)", [lambda i=i: TF.repeat(src, [1, 2, 2], o[i]) for i in range(R)], n * es + (n // 4) * es)
            del o, q3
        del a, b, c, m, x, t3
        torch.cuda.empty_cache()
    low = {k: v for k, v in res.items() if v < 0.8}
    print(json.dumps({"sweep": "256 MiB per tensor, cuda-graph replay", "peak_gbs": peak, "peak_source": peak_kind, "count": len(res),
                      "min": min(res.values()), "below_0.8": low, "ops": res}), flush=True)


def run_matmul_sweep(args) -> None:
    """`--matmul-sweep`: dx_matmul over a list of shapes (square, tall, wide, few rows, short K, batched) in bf16
    and float32, CUDA-graph replay over rotating buffers, with the library GEMM (torch.matmul: cuBLAS; float32 with
    TF32 off) timed the same way beside it as a yardstick.  Prints one JSON line per shape."""
    import torch
    from deepx_b200 import tensorfunc as TF
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    torch.backends.cuda.matmul.allow_tf32 = False
    shapes = [
        (1, 8192, 4096, 4096), (1, 4096, 4096, 4096), (1, 2048, 2048, 2048), (1, 1024, 1024, 1024), (1, 16384, 4096, 4096),
        (1, 8192, 8192, 8192), (1, 4096, 11008, 4096), (1, 4096, 4096, 11008), (1, 2048, 151936, 896), (1, 32768, 896, 896),
        (1, 32768, 4864, 896), (1, 32768, 896, 4864), (1, 1024, 4096, 4096), (1, 512, 4096, 4096), (1, 256, 4096, 4096),
        (1, 128, 4096, 4096), (1, 32, 4096, 4096), (1, 768, 2048, 8192), (32, 2048, 2048, 128), (32, 2048, 128, 2048),
        (224, 2048, 2048, 64), (16, 1024, 1024, 1024), (64, 512, 512, 512), (8, 4096, 4096, 512), (1, 4096, 4096, 256),
        (1, 1000, 1000, 1000), (1, 8192, 4104, 4096), (1, 3000, 5000, 7000),
    ]

    def replay_us(fns, iters=18):
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fns[i % len(fns)]()
        g.replay()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            g.replay()
            e.record()
            torch.cuda.synchronize()
            best = min(best, s.elapsed_time(e) / iters * 1e3)
        return best

    for name, dt in (("bf16", torch.bfloat16), ("f32", torch.float32)):
        for (b, M, N, K) in shapes:
            flop = 2.0 * b * M * N * K
            if name == "f32" and flop > 6e11:
                continue
            R = 3
            As = [torch.randn((b, M, K), device=dev).mul_(0.05).to(dt) for _ in range(R)]
            Bs = [torch.randn((b, K, N), device=dev).mul_(0.05).to(dt) for _ in range(R)]
            Cs = [torch.empty((b, M, N), device=dev, dtype=dt) for _ in range(R)]
            Cl = torch.empty((b, M, N), device=dev, dtype=dt)
            ours = replay_us([lambda i=i: TF.matmul(As[i], Bs[i], Cs[i]) for i in range(R)])
            lib = replay_us([lambda i=i: torch.matmul(As[i], Bs[i], out=Cl) for i in range(R)])
            torch.matmul(As[0], Bs[0], out=Cl)
            TF.matmul(As[0], Bs[0], Cs[0])
            err = float((Cs[0].double() - Cl.double()).abs().max() / (Cl.double().abs().max() + 1e-300))
            print(json.dumps({"dtype": name, "batch": b, "M": M, "N": N, "K": K, "us": round(ours, 1), "tflops": round(flop / ours / 1e6, 1),
                              "library_us": round(lib, 1), "library_tflops": round(flop / lib / 1e6, 1),
                              "speed_vs_library": round(lib / ours, 3), "max_diff_vs_library_rel": err}), flush=True)
            del As, Bs, Cs, Cl
    from deepx_b200 import _native as N_
    N_.check(N_.lib.dx_matmul_status(None))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-ops", action="store_true", help="skip the per-op table of the other configs")
    ap.add_argument("--no-graph", action="store_true", help="with --op: launch directly instead of replaying a CUDA graph")
    ap.add_argument("--op", default=None, help="time one named op of the per-op table alone (single GPU)")
    ap.add_argument("--sweep", action="store_true", help="every op x dtype on 256 MiB tensors as a fraction of the HBM peak (single GPU)")
    ap.add_argument("--matmul-sweep", action="store_true", help="dx_matmul over many shapes with the library GEMM beside it (single GPU)")
    args = ap.parse_args()
    if args.matmul_sweep:
        run_matmul_sweep(args)
    elif args.sweep:
        run_sweep(args)
    elif args.op:
        run_one_op(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
