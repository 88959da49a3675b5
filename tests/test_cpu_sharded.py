"""CPU tests of the multi-GPU host logic: the axis-0 partition and the combine step, run as
two gloo ranks.  Each rank reduces its row block with the oracle (standing in for the local GPU
kernel), the partials are combined with the same all-reduce the GPU path uses, and the result
is checked against the oracle on the whole tensor."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def test_row_partition_covers_all_rows_once():
    from deepx_b200.sharded import RowPartition
    for rows in (0, 1, 7, 8, 2048, 2049):
        for world in (1, 2, 3, 4, 8):
            p = RowPartition(rows, world)
            seen = []
            for r in range(world):
                s = p.slice(r)
                assert s.stop - s.start == p.count(r)
                seen += list(range(s.start, s.stop))
            assert seen == list(range(rows))
            assert max(p.count(r) for r in range(world)) - min(p.count(r) for r in range(world)) <= 1
    assert RowPartition(2048, 8).count(3) == 256


def test_shards_axis0_predicate():
    from deepx_b200.sharded import shards_axis0
    assert shards_axis0([0, 1], 2) and shards_axis0([0], 3)
    assert not shards_axis0([1], 2) and not shards_axis0([1, 2], 3)


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepx_b200.sharded import RowPartition, combine_partials, shards_axis0
    from oracle import oracle as O
    rng = np.random.default_rng(0)  # same data on every rank; each takes its rows
    x = rng.uniform(-1, 1, (37, 50)).astype(np.float32)
    k = rng.integers(-100, 101, (37, 6, 5)).astype(np.int32)
    part = RowPartition(37, world)
    sl = part.slice(rank)
    out = {}
    # global sum: local partial, then one all-reduce
    loc = torch.from_numpy(O.sum(x[sl], [0, 1]).copy())
    out["sum_all"] = combine_partials(loc, "sum").numpy()
    # axis-0 reductions of an int tensor: bit-exact whatever the split
    for op in ("sum", "reducemax", "reducemin"):
        loc = torch.from_numpy(getattr(O, op)(k[sl], [0]).copy())
        out[op + "_axis0"] = combine_partials(loc, op).numpy()
    loc = torch.from_numpy(O.prod(np.sign(k[sl]).astype(np.int32) + 2, [0, 2]).copy())
    out["prod_02"] = combine_partials(loc, "prod").numpy()
    # a reduction that does not touch axis 0 needs no exchange: rows stay where they are
    assert not shards_axis0([1], 2)
    out["rowmax_local"] = O.reducemax(x[sl], [1])
    if rank == 0:
        q.put(out)
    gathered = [None] * world
    dist.all_gather_object(gathered, out["rowmax_local"])
    if rank == 0:
        q.put(np.concatenate(gathered))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_combine_matches_whole_tensor():
    from oracle import oracle as O
    O.lib()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = q.get(timeout=120)
    rowmax = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, (37, 50)).astype(np.float32)
    k = rng.integers(-100, 101, (37, 6, 5)).astype(np.int32)
    ref = x.astype(np.float64).sum()
    assert abs(float(out["sum_all"][0]) - ref) <= 1e-5 * np.abs(x).astype(np.float64).sum()
    assert np.array_equal(out["sum_axis0"], O.sum(k, [0]))
    assert np.array_equal(out["reducemax_axis0"], O.reducemax(k, [0]))
    assert np.array_equal(out["reducemin_axis0"], O.reducemin(k, [0]))
    assert np.array_equal(out["prod_02"], O.prod(np.sign(k).astype(np.int32) + 2, [0, 2]))
    assert np.array_equal(rowmax, O.reducemax(x, [1]))


# ---- the executor's own partition decisions (dx_ir_shard_plan: the functions ops.cpp executes, without a device) ----
CHAIN = """
newtensor(vector<int32>:[2048 1048576])->(tensor<float32>:x)
newtensor(vector<int32>:[2048 1048576])->(tensor<float32>:y)
newtensor(vector<int32>:[2048 1048576])->(tensor<float32>:t)
newtensor(vector<int32>:[2048 1048576])->(tensor<float32>:z)
newtensor(vector<int32>:[1])->(tensor<float32>:s)
newtensor(vector<int32>:[2048])->(tensor<float32>:m)
exp(tensor<float32>:x)->(tensor<float32>:t)
mul(tensor<float32>:t, tensor<float32>:y)->(tensor<float32>:t)
add(tensor<float32>:t, tensor<float32>:x)->(tensor<float32>:z)
sum(tensor<float32>:z, vector<int32>:[0 1], var<bool>:false)->(tensor<float32>:s)
reducemax(tensor<float32>:z, vector<int32>:[1], var<bool>:false)->(tensor<float32>:m)
"""


def test_executor_partition_plan_of_the_sharded_chain():
    from deepx_b200 import executor as E
    big = ["newtensor %s: partitioned 2048 rows" % n for n in "xytz"]
    # m (8 KiB) is partitioned when the threshold is below it, replicated (and then all-gathered) otherwise
    assert E.shard_plan(CHAIN, 8, 4096) == big + ["newtensor s: whole", "newtensor m: partitioned 2048 rows",
                                                  "rows", "rows", "rows", "allreduce(deferred)", "rows"]
    assert E.shard_plan(CHAIN, 2, 1 << 20) == big + ["newtensor s: whole", "newtensor m: whole",
                                                     "rows", "rows", "rows", "allreduce(deferred)", "rows+allgather"]
    one = E.shard_plan(CHAIN, 1, 4096)
    assert one[:6] == ["newtensor %s: whole" % n for n in "xytzsm"] and set(one[6:]) == {"whole"}


def test_executor_partition_plan_cases():
    from deepx_b200 import executor as E
    f = "tensor<float32>"
    prog = f"""
newtensor(vector<int32>:[4096 4096])->({f}:a)
newtensor(vector<int32>:[4096])->({f}:colsum)
newtensor(vector<int32>:[1 4096])->({f}:colsum_keep)
newtensor(vector<int32>:[4096 4096])->(tensor<bool>:mask)
newtensor(vector<int32>:[3 5])->({f}:small)
newtensor(vector<int32>:[3])->({f}:small_rows)
newtensor(vector<int32>:[4096 1024])->({f}:narrow)
sum({f}:a, vector<int32>:[0], var<bool>:false)->({f}:colsum)
sum({f}:a, vector<int32>:[0], var<bool>:true)->({f}:colsum_keep)
less({f}:a, {f}:a)->(tensor<bool>:mask)
sum({f}:small, vector<int32>:[1], var<bool>:false)->({f}:small_rows)
add({f}:a, {f}:narrow)->({f}:a)
sum({f}:a, vector<int32>:[1], var<bool>:false)->({f}:small_rows)
transpose({f}:a, vector<int32>:[1 0])->({f}:a)
"""
    # threshold 8 KiB: a (64 MiB), mask (16 MiB), narrow, colsum (16 KiB) and colsum_keep... are sized against it
    plan = E.shard_plan(prog, 4, 8192)
    assert plan[:7] == ["newtensor a: partitioned 4096 rows", "newtensor colsum: partitioned 4096 rows", "newtensor colsum_keep: whole",
                        "newtensor mask: partitioned 4096 rows", "newtensor small: whole", "newtensor small_rows: whole",
                        "newtensor narrow: partitioned 4096 rows"]
    assert plan[7] == "allreduce(rounds)+keep-own-rows"      # axis 0 reduced into an output that is itself partitioned
    assert plan[8] == "allreduce(deferred)"                  # [1,4096] has one row: replicated, 16 KiB fits a mailbox slot
    assert plan[9] == "rows"                                 # a mask of one byte per element is partitioned like its inputs
    assert plan[10] == "whole"                               # nothing partitioned: the single-GPU path
    assert plan[11].startswith("refuse: shape mismatch")
    assert plan[12].startswith("refuse:")                    # 4096 row results into a 3-element tensor
    assert plan[13] == "rows-if-aligned"
    # a result too large for one mailbox slot, replicated because the threshold is high
    plan = E.shard_plan(prog, 4, 1 << 20)
    assert plan[1] == "newtensor colsum: whole" and plan[7] == "allreduce(deferred)"    # 16 KiB
    wide = f"""
newtensor(vector<int32>:[64 65536])->({f}:w)
newtensor(vector<int32>:[65536])->({f}:ws)
sum({f}:w, vector<int32>:[0], var<bool>:false)->({f}:ws)
"""
    assert E.shard_plan(wide, 2, 1 << 20) == ["newtensor w: partitioned 64 rows", "newtensor ws: whole", "allreduce(rounds)"]   # 256 KiB > 64 KiB slot


def test_row_blocks_agree_between_python_and_the_library():
    from deepx_b200.comm import shard_rows
    from deepx_b200.sharded import RowPartition
    for rows in (0, 1, 7, 8, 2048, 2049, 3 * 10 ** 9):
        for world in (1, 2, 3, 8, 16):
            p = RowPartition(rows, world)
            for r in range(world):
                assert shard_rows(rows, r, world) == (p.start(r), p.count(r))


def _plan_worker(rank, world, port, q):
    """Each rank plays the executor on the host: tensors are numpy arrays cut according to the plan text, row-wise ops
    run on the local rows, and the exchanges the plan names are gloo collectives.  The results must be those of one
    rank on the whole tensors."""
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepx_b200 import executor as E
    from deepx_b200.comm import shard_rows
    from oracle import oracle as O
    f = "tensor<float32>"
    prog = [f"newtensor(vector<int32>:[37 50])->({f}:x)", f"newtensor(vector<int32>:[37 50])->({f}:y)", f"newtensor(vector<int32>:[37 50])->({f}:z)",
            f"newtensor(vector<int32>:[1])->({f}:s)", f"newtensor(vector<int32>:[37])->({f}:m)", f"newtensor(vector<int32>:[50])->({f}:c)",
            f"exp({f}:x)->({f}:z)", f"mul({f}:z, {f}:y)->({f}:z)", f"add({f}:z, {f}:x)->({f}:z)",
            f"sum({f}:z, vector<int32>:[0 1], var<bool>:false)->({f}:s)", f"reducemax({f}:z, vector<int32>:[1], var<bool>:false)->({f}:m)",
            f"reducemin({f}:z, vector<int32>:[0], var<bool>:false)->({f}:c)"]
    plan = E.shard_plan("\n".join(prog), world, 1024)   # x, y, z (7400 bytes) are partitioned; s, m, c are not
    assert plan[:6] == ["newtensor x: partitioned 37 rows", "newtensor y: partitioned 37 rows", "newtensor z: partitioned 37 rows",
                        "newtensor s: whole", "newtensor m: whole", "newtensor c: whole"]
    assert plan[6:] == ["rows", "rows", "rows", "allreduce(deferred)", "rows+allgather", "allreduce(deferred)"]
    rng = np.random.default_rng(1)
    full = {"x": rng.uniform(-1, 1, (37, 50)).astype(np.float32), "y": rng.uniform(-1, 1, (37, 50)).astype(np.float32)}
    r0, n = shard_rows(37, rank, world)
    x, y = full["x"][r0:r0 + n], full["y"][r0:r0 + n]
    z = O.add(O.mul(O.exp(x), y), x)                                   # "rows": local, no exchange
    s = torch.from_numpy(O.sum(z, [0, 1]).copy())
    dist.all_reduce(s, op=dist.ReduceOp.SUM)                           # "allreduce(deferred)"
    m = np.full(37, -7.0, dtype=np.float32)
    m[r0:r0 + n] = O.reducemax(z, [1])                                 # "rows+allgather": own block, then everybody's
    blocks = [None] * world
    dist.all_gather_object(blocks, m[r0:r0 + n])
    m = np.concatenate(blocks)
    c = torch.from_numpy(O.reducemin(z, [0]).copy())
    dist.all_reduce(c, op=dist.ReduceOp.MIN)
    if rank == 0:
        q.put({"s": s.numpy(), "m": m, "c": c.numpy()})
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_following_the_executor_plan_match_one_rank():
    from oracle import oracle as O
    O.lib()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_plan_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    rng = np.random.default_rng(1)
    x, y = rng.uniform(-1, 1, (37, 50)).astype(np.float32), rng.uniform(-1, 1, (37, 50)).astype(np.float32)
    z = O.add(O.mul(O.exp(x), y), x)
    assert abs(float(out["s"][0]) - z.astype(np.float64).sum()) <= 1e-5 * np.abs(z).astype(np.float64).sum()
    assert np.array_equal(out["m"], O.reducemax(z, [1]))
    assert np.array_equal(out["c"], O.reducemin(z, [0]))
