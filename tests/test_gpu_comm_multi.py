"""The peer-memory all-reduce between real GPUs (one process per GPU); skipped on a one-GPU box.

Each rank builds a PeerComm over a gloo group (the 64-byte IPC handles travel through the object
all-gather), combines small tensors with the peer kernel and checks them against the rank-order
combine computed on the host; ShardedOps then runs a global sum and an axis-0 max through it.
NVLS plays no part: plain stores to peer memory.
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
    import os, sys
    import numpy as np
    import torch
    import torch.distributed as dist
    sys.path.insert(0, {root!r})
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deepx_b200.comm import PeerComm
    from deepx_b200.sharded import ShardedOps
    comm = PeerComm()
    for round_ in range(5):
        for n in (1, 7, 1024, 1025, 16384):
            parts = [np.random.default_rng(1000 * round_ + 10 * r + n).uniform(-1, 1, n).astype(np.float32) for r in range(world)]
            t = torch.from_numpy(parts[rank]).cuda()
            comm.allreduce(t, "sum")
            comm.status()
            want = parts[0].copy()
            for p in parts[1:]:
                want = want + p
            assert np.array_equal(t.cpu().numpy(), want), (round_, n)
    k = torch.full((33,), rank + 1, dtype=torch.int32, device="cuda")
    comm.allreduce(k, "reducemax")
    assert (k == world).all()
    comm.close()
    ops = ShardedOps()
    assert ops.peer is not None
    rows = 64
    x = torch.from_numpy(np.random.default_rng(5).uniform(-1, 1, (rows * world, 512)).astype(np.float32))
    mine = x[rank * rows:(rank + 1) * rows].cuda().contiguous()
    s = torch.empty(1, device="cuda")
    ops.sum(mine, [0, 1], False, s)
    m = torch.empty(512, device="cuda")
    ops.reducemax(mine, [0], False, m)
    ops.peer.status()
    assert abs(s.item() - x.double().sum().item()) <= 1e-5 * x.double().abs().sum().item()
    assert torch.equal(m.cpu(), x.max(0).values)
    # a block big enough that the local sum is split over CTAs: its one-CTA finish kernel does the exchange itself
    big = torch.from_numpy(np.random.default_rng(6).uniform(-1, 1, (256 * world, 8192)).astype(np.float32))
    mine = big[rank * 256:(rank + 1) * 256].cuda().contiguous()
    ops.sum(mine, [0, 1], False, s)
    ops.peer.status()
    assert abs(s.item() - big.double().sum().item()) <= 1e-5 * big.double().abs().sum().item()
    every = [None] * world
    dist.all_gather_object(every, float(s.item()))
    assert len(set(every)) == 1   # identical bits on every rank
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_two_gpus():
    world = min(torch.cuda.device_count(), 4)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29611", WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, "-c", WORKER.format(root=str(ROOT))], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in o, f"rank {r}:\n{o}"
