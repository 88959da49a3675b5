"""The peer-memory all-reduce protocol (dx_comm_*), W ranks emulated on one GPU.

All ranks' thread blocks run in ONE launch with every mailbox local, so the exchange — publish into
every peer's slot, flag, bounded wait, combine in rank order — is the code the multi-GPU kernel runs,
minus NVLink.  Results must equal a rank-order combine on the host bit for bit, on every rank; the
failure path (a rank that never shows up) must end in a status report, not a hang.
"""
import numpy as np
import pytest
import torch

from helpers import NP_DTYPES, TORCH_DTYPES, make, seed_of, to_gpu, to_np

pytestmark = pytest.mark.gpu

NP_OPS = {"sum": np.add, "prod": np.multiply, "reducemax": np.maximum, "reducemin": np.minimum}


def rank_order_combine(parts, op, dtype):
    """What the kernel computes: accumulate in the reduce kernels' accumulation type, ranks 0..W-1."""
    acc_t = {"float16": np.float32, "bfloat16": np.float32, "int16": np.int32, "int8": np.int32}.get(dtype, NP_DTYPES[dtype])
    acc = parts[0].astype(acc_t)
    with np.errstate(over="ignore"):
        for p in parts[1:]:
            acc = NP_OPS[op](acc, p.astype(acc_t))
    return acc.astype(NP_DTYPES[dtype])


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("dtype", ["float32", "float64", "bfloat16", "float16", "int64", "int32", "int16", "int8"])
def test_emulated_ranks_all_ops(world, dtype):
    from deepx_b200.comm import EmulatedComm
    comm = EmulatedComm(world)
    rng = np.random.default_rng(seed_of("comm", world, dtype))
    es = np.dtype(NP_DTYPES[dtype]).itemsize
    sizes = [1, 5, 4096 // es, 4096 // es + 1, 3 * 4096 // es + 7]
    for round_, (op, n) in enumerate([(o, n) for o in ("sum", "reducemax", "prod", "reducemin", "sum") for n in sizes]):
        lo, hi = (0.9, 1.1) if op == "prod" else (-4.0, 4.0)
        parts = [make(rng, dtype, (n,), lo, hi) for _ in range(world)]
        if op == "prod" and dtype.startswith("int"):
            parts = [np.where(p % 3 == 0, 2, 1).astype(NP_DTYPES[dtype]) for p in parts]
        bufs = [to_gpu(p) for p in parts]
        comm.allreduce(bufs, op)
        comm.status()
        want = rank_order_combine(parts, op, dtype)
        for r in range(world):
            got = to_np(bufs[r])
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), f"{dtype} {op} n={n} round {round_} rank {r}"
    comm.close()


def test_full_slot_and_oversize():
    from deepx_b200 import _native as N
    from deepx_b200.comm import EmulatedComm
    comm = EmulatedComm(4)
    n = N.lib.dx_comm_max_bytes() // 4
    parts = [np.full(n, r + 1, dtype=np.float32) for r in range(4)]
    bufs = [to_gpu(p) for p in parts]
    comm.allreduce(bufs, "sum")
    comm.status()
    assert all(np.array_equal(to_np(b), np.full(n, 10, dtype=np.float32)) for b in bufs)
    big = [torch.zeros(n + 1, device="cuda:0") for _ in range(4)]
    with pytest.raises(N.DxError):
        comm.allreduce(big, "sum")
    comm.close()


def test_absent_rank_ends_in_a_status_report():
    """Three of four ranks run; their wait for the fourth expires (50 ms), the kernel returns, the local
    buffers are untouched and dx_comm_status names the rank.  The GPU stays usable."""
    from deepx_b200 import _native as N
    from deepx_b200.comm import EmulatedComm
    comm = EmulatedComm(4)
    comm.set_timeout_ms(50)
    parts = [np.full(100, r + 1, dtype=np.float32) for r in range(4)]
    bufs = [to_gpu(p) for p in parts]
    comm.allreduce(bufs, "sum", active=3)
    with pytest.raises(N.DxError, match="gave up waiting for rank 3"):
        comm.status()
    for r in range(4):
        assert np.array_equal(to_np(bufs[r]), parts[r])
    comm.close()
    # a fresh communicator works right after
    comm = EmulatedComm(2)
    a, b = to_gpu(np.ones(8, dtype=np.float32)), to_gpu(np.full(8, 2, dtype=np.float32))
    comm.allreduce([a, b], "sum")
    comm.status()
    assert np.array_equal(to_np(a), np.full(8, 3, dtype=np.float32)) and np.array_equal(to_np(b), to_np(a))
    comm.close()


def test_argument_errors():
    from deepx_b200 import _native as N
    assert N.lib.dx_comm_create(3, 2, 0) is None
    assert N.lib.dx_comm_emulate(0, 0) is None
    assert N.lib.dx_comm_emulate(99, 0) is None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "int32"])
def test_reduce_with_fused_exchange_on_one_rank(dtype):
    """A world of one: the reduce kernels that finish with the exchange run the whole protocol against
    their own mailbox, so the result must equal the plain reduction (every plan shape: one-CTA finish
    fused, many outputs followed by the exchange kernel, no finish step at all)."""
    from deepx_b200 import _native as N
    from deepx_b200 import tensorfunc as TF
    h = N.lib.dx_comm_create(0, 1, 0)
    assert h
    rng = np.random.default_rng(seed_of("fusedcomm", dtype))
    for shape, dims in [((512, 4096), [0, 1]), ((300, 1000), [0]), ((64, 200000), [0, 1]), ((8, 64, 4096), [0, 2]), ((5, 7), [0]),
                        ((4096, 8), [0]), ((3, 100000), [1])]:
        a = make(rng, dtype, shape, 0.0, 1.0)
        A = to_gpu(a)
        cd = TF.checked_dims(A.shape, dims)
        oshape = TF.reduced_shape(A.shape, cd, False)
        for op, code in (("sum", N.SUM), ("reducemax", N.RMAX)):
            plain = torch.empty(oshape, dtype=A.dtype, device=A.device)
            fused = torch.empty(oshape, dtype=A.dtype, device=A.device)
            getattr(TF, op)(A, dims, False, plain)
            TF._reduce(code, A, dims, False, fused, comm_handle=h)
            N.check(N.lib.dx_comm_status(h, None))
            assert np.array_equal(to_np(plain).view(np.uint8), to_np(fused).view(np.uint8)), (dtype, shape, dims, op)
    N.lib.dx_comm_destroy(h)
