"""The deepxIR executor as ranks of a multi-GPU world (dx_exec_set_shard), one process per GPU; skipped on a
one-GPU box.  Every rank is given the same IR lines with GLOBAL shapes; tensors above the threshold are split by
rows, ops run on the local rows, reductions over axis 0 are combined over NVLink peer memory by the executor
itself.  Each rank uploads its rows, and what comes back — assembled over the ranks — must be what the CPU oracle
computes on the whole tensors: bit for bit for elementwise ops, max/min and integer sums, within 1e-5 of
sum|x| for float sums.  NVLS plays no part (plain stores to peer memory).
"""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = textwrap.dedent("""
    import os, sys, tempfile
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, {root!r})
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepx_b200.comm import PeerComm, shard_rows
    from deepx_b200.executor import Executor, IRError
    from oracle import oracle as O
    comm = PeerComm()
    ex = Executor(rank)
    ex.set_shard(rank, world, comm._h, min_bytes=4096)
    f, i32, b = "tensor<float32>", "tensor<int32>", "tensor<bool>"
    R, Cn = 61, 300                      # 61 rows: an uneven split
    rng = np.random.default_rng(3)       # the same data on every rank; each uploads its rows
    X = rng.uniform(-1, 1, (R, Cn)).astype(np.float32)
    Y = rng.uniform(-1, 1, (R, Cn)).astype(np.float32)
    K = rng.integers(-100, 101, (R, Cn)).astype(np.int32)
    r0, n = shard_rows(R, rank, world)

    def new(name, dtype, shape):
        ex.run(f"newtensor(vector<int32>:[{{' '.join(map(str, shape))}}])->(tensor<{{dtype}}>:{{name}})")

    def put(name, full):
        part, a, cnt, g = ex.shard(name)
        ex.upload(name, np.ascontiguousarray(full[a:a + cnt]) if part else full)

    def whole(name):
        # the global tensor, assembled over the ranks where it is partitioned
        part, a, cnt, g = ex.shard(name)
        mine = ex.download(name)
        if not part:
            return mine
        blocks = [None] * world
        dist.all_gather_object(blocks, mine)
        return np.concatenate(blocks)

    for nm, dt in (("x", "float32"), ("y", "float32"), ("z", "float32"), ("k", "int32")):
        new(nm, dt, (R, Cn))
    assert ex.shard("x") == (True, r0, n, R)
    new("s", "float32", (1,)); new("m", "float32", (R,)); new("c", "float32", (Cn,)); new("ks", "int32", (Cn,)); new("mask", "bool", (R, Cn))
    assert not ex.shard("s")[0] and not ex.shard("m")[0] and not ex.shard("c")[0]      # below 4096 bytes: replicated
    put("x", X); put("y", Y); put("k", K)

    # elementwise by rows, then the three kinds of reduction
    ex.run(f"exp({{f}}:x)->({{f}}:z)")
    ex.run(f"mul({{f}}:z, {{f}}:y)->({{f}}:z)")
    ex.run(f"add({{f}}:z, {{f}}:x)->({{f}}:z)")
    Z = O.add(O.mul(O.exp(X), Y), X)
    got = whole("z")
    assert np.allclose(got, Z, rtol=1e-5, atol=1e-6)
    ex.run(f"sum({{f}}:z, vector<int32>:[0 1], var<bool>:false)->({{f}}:s)")          # deferred combine
    ex.run(f"reducemax({{f}}:z, vector<int32>:[1], var<bool>:false)->({{f}}:m)")      # rows + all-gather into the replicated m
    ex.run(f"reducemin({{f}}:z, vector<int32>:[0], var<bool>:false)->({{f}}:c)")      # second deferred combine: completes the first
    ex.run(f"sum({{i32}}:k, vector<int32>:[0], var<bool>:false)->({{i32}}:ks)")
    s = ex.download("s"); m = ex.download("m"); c = ex.download("c"); ks = ex.download("ks")
    assert abs(float(s[0]) - got.astype(np.float64).sum()) <= 1e-5 * np.abs(got).astype(np.float64).sum()
    assert np.array_equal(m, O.reducemax(got, [1])), "row max (all-gathered) differs"
    assert np.array_equal(c, O.reducemin(got, [0])), "column min (combined over ranks) differs"
    assert np.array_equal(ks, O.sum(K, [0])), "int32 column sum is not bit-exact"
    every = [None] * world
    dist.all_gather_object(every, (s.tobytes(), m.tobytes(), c.tobytes()))
    assert len(set(every)) == 1, "replicated results differ between ranks"

    # a replicated operand of the same global shape is used through its rows; a replicated output is completed by a gather
    new("xs", "float32", (R, 4)); new("ys", "float32", (R, 4))        # 976 bytes: replicated
    assert not ex.shard("xs")[0]
    XS = rng.uniform(-1, 1, (R, 4)).astype(np.float32)
    ex.upload("xs", XS)
    ex.run(f"mulscalar({{f}}:xs, var<float32>:2.5)->({{f}}:ys)")
    assert np.array_equal(ex.download("ys"), O.mulscalar(XS, 2.5))
    ex.run(f"less({{f}}:x, {{f}}:y)->({{b}}:mask)")                      # 18300 bytes of mask: partitioned like x and y
    assert ex.shard("mask")[0] and np.array_equal(whole("mask"), O.less(X, Y))

    # a reduction over axis 0 whose result is itself partitioned, and one whose result needs several rounds
    Rw, Cw = 2 * world + 1, 40000
    W = rng.uniform(-1, 1, (Rw, Cw)).astype(np.float32)
    new("w", "float32", (Rw, Cw)); new("wsum", "float32", (Cw,)); put("w", W)
    assert ex.shard("w")[0] and ex.shard("wsum")[0]                      # 160 KB output: partitioned by its own rows
    ex.run(f"sum({{f}}:w, vector<int32>:[0], var<bool>:false)->({{f}}:wsum)")
    ws = whole("wsum")
    assert np.all(np.abs(ws.astype(np.float64) - W.astype(np.float64).sum(0)) <= 1e-5 * np.abs(W).astype(np.float64).sum(0))
    new("wmax", "float32", (1, Cw))                                       # one row: replicated although 160 KB -> rounds
    assert not ex.shard("wmax")[0]
    ex.run(f"reducemax({{f}}:w, vector<int32>:[0], var<bool>:true)->({{f}}:wmax)")
    assert np.array_equal(ex.download("wmax"), O.reducemax(W, [0], True))

    # changeshape and matmul where the rows line up; a refusal where they do not
    T3 = rng.uniform(-1, 1, (R, 6, 50)).astype(np.float32)
    new("t3", "float32", (R, 6, 50)); new("t3t", "float32", (R, 50, 6)); put("t3", T3)
    ex.run(f"transpose({{f}}:t3, vector<int32>:[0 2 1])->({{f}}:t3t)")
    assert np.array_equal(whole("t3t"), O.transpose(T3, [0, 2, 1]))
    B = rng.uniform(-1, 1, (Cn, 64)).astype(np.float32)
    new("bm", "float32", (Cn, 64)); ex.run(f"deltensor()->({{f}}:bm)")
    ex.set_shard(rank, world, comm._h, min_bytes=1 << 20); new("bm", "float32", (Cn, 64)); ex.set_shard(rank, world, comm._h, min_bytes=4096)
    assert not ex.shard("bm")[0]                                           # created under a high threshold: replicated
    ex.upload("bm", B)
    new("xm", "float32", (R, 64))
    ex.run(f"matmul({{f}}:x, {{f}}:bm)->({{f}}:xm) // author=cublas")
    ref = X.astype(np.float64) @ B.astype(np.float64)
    bound = 1e-5 * np.abs(ref) + 2e-6 * (np.abs(X).astype(np.float64) @ np.abs(B).astype(np.float64))
    assert np.all(np.abs(whole("xm").astype(np.float64) - ref) <= bound)
    new("xt", "float32", (Cn, R))
    try:
        ex.run(f"transpose({{f}}:x, vector<int32>:[1 0])->({{f}}:xt)")
        raise SystemExit("a transpose that moves the partitioned axis was not refused")
    except IRError as e:
        assert "row-partitioned" in str(e)

    # save writes the file one GPU would write; load reads each rank's rows back
    tmp = [tempfile.mkdtemp() if rank == 0 else None]
    dist.broadcast_object_list(tmp, src=0)
    path = os.path.join(tmp[0], "zsaved")
    ex.run(f"save({{f}}:z, var<string>:{{path}})->()")
    ex.sync(); dist.barrier()
    if rank == 0:
        assert np.array_equal(np.fromfile(path + ".data", dtype=np.float32).reshape(R, Cn), got)
        assert "61" in open(path + ".shape").read()
    ex.run(f"deltensor()->({{f}}:z)")
    dist.barrier()
    ex.run(f"load(var<string>:{{path}})->()")
    assert ex.shard("zsaved") == (True, r0, n, R) and np.array_equal(whole("zsaved"), got)

    comm.status()
    dist.barrier()
    ex.close(); comm.close()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_executor_ranks_on_real_gpus():
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29633", WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, "-c", WORKER.format(root=str(ROOT))], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in o, f"rank {r}:\n{o}"


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_udp_process_over_two_devices(tmp_path):
    """deepx-op-b200 with DEEPX_DEVICES=0,1: one port, one reply per IR line, the tensors partitioned over two worker
    processes behind it.  The files `save` leaves are those a single GPU would write."""
    import socket
    import numpy as np
    from deepx_b200.executor import BIN_PATH
    port = 23000 + os.getpid() % 20000
    env = dict(os.environ, DEEPX_PORT=str(port), DEEPX_DEVICES="0,1", DEEPX_SHARD_MIN_BYTES="4096", NCCL_NVLS_ENABLE="0")
    proc = subprocess.Popen([str(BIN_PATH)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        first = proc.stdout.readline()
        assert "listening" in first and "devices 0,1" in first, first
        sock = socket.socket(socket.AF_INET, socket.SOCK_DGRAM)
        sock.settimeout(60)

        def send(text):
            sock.sendto(text.encode(), ("127.0.0.1", port))
            return [sock.recvfrom(65536)[0].decode() for _ in [l for l in text.split("\n") if l.strip()]]

        f = "tensor<float32>"
        replies = send("\n".join([
            f"newtensor(vector<int32>:[64 1000])->({f}:a) // id=1",
            f"newtensor(vector<int32>:[64 1000])->({f}:b) // id=2",
            f"newtensor(vector<int32>:[1])->({f}:s) // id=3",
            f"newtensor(vector<int32>:[1000])->({f}:c) // id=4",
            f"arange(var<float32>:0, var<float32>:1)->({f}:a) // author=miaobyte id=5",
            f"mulscalar({f}:a, var<float32>:0.5)->({f}:b) // author=miaobyte id=6",
            f"sum({f}:b, vector<int32>:[0 1], var<bool>:false)->({f}:s) // author=miaobyte id=7",
            f"reducemax({f}:b, vector<int32>:[0], var<bool>:false)->({f}:c) // author=miaobyte id=8",
            f"save({f}:b, var<string>:{tmp_path / 'b'})->() // id=9",
            f"save({f}:s, var<string>:{tmp_path / 's'})->() // id=10",
            f"save({f}:c, var<string>:{tmp_path / 'c'})->() // id=11"]))
        assert len(replies) == 11 and all(" ok" in r.split("//")[0] for r in replies), replies
        assert [int(r.split()[0]) for r in replies] == list(range(1, 12))
        want = (np.arange(64000, dtype=np.float32) * np.float32(0.5)).reshape(64, 1000)
        assert np.array_equal(np.fromfile(tmp_path / "b.data", dtype=np.float32).reshape(64, 1000), want)
        s = np.fromfile(tmp_path / "s.data", dtype=np.float32)
        assert abs(float(s[0]) - want.astype(np.float64).sum()) <= 1e-5 * want.astype(np.float64).sum()
        assert np.array_equal(np.fromfile(tmp_path / "c.data", dtype=np.float32), want.max(0))
        # an op without a row-wise form on a partitioned tensor: one error reply, and the process carries on
        bad = send(f"newtensor(vector<int32>:[1000 64])->({f}:bt) // id=20\ntranspose({f}:b, vector<int32>:[1 0])->({f}:bt) // author=miaobyte id=21")
        assert " ok" in bad[0].split("//")[0] and " error" in bad[1].split("//")[0] and "row-partitioned" in bad[1]
        assert " ok" in send(f"addscalar({f}:b, var<float32>:1)->({f}:b) // author=miaobyte id=22")[0].split("//")[0]
    finally:
        proc.terminate()
        try:
            proc.communicate(timeout=30)
        except Exception:
            proc.kill()
