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
