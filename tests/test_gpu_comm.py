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


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "int64", "int8"])
def test_split_exchange_publish_then_combine(world, dtype):
    """The exchange as two launches — publish (stores + flags), then other work, then combine (bounded wait +
    rank-order combine): the form a deferred cross-rank reduction uses.  Same bits as the one-launch form, round
    after round (the epoch only advances in the combine), with a kernel on the stream in between."""
    from deepx_b200.comm import EmulatedComm
    comm = EmulatedComm(world)
    rng = np.random.default_rng(seed_of("split", world, dtype))
    es = np.dtype(NP_DTYPES[dtype]).itemsize
    other = torch.zeros(1 << 20, device="cuda:0")
    comm.wait_stats(reset=True)
    expected_waits = 0
    for round_, (op, n) in enumerate([(o, n) for o in ("sum", "reducemax", "reducemin") for n in (1, 4096 // es + 3, 2 * 4096 // es)]):
        expected_waits += 2 * -(-n * es // 4096)   # one wait per 4 KiB chunk and exchange (the split one and the one-launch one)
        parts = [make(rng, dtype, (n,), -4.0, 4.0) for _ in range(world)]
        bufs = [to_gpu(p) for p in parts]
        comm.publish(bufs, op)
        other.add_(1.0)                       # independent work between the two halves
        comm.combine(bufs, op)
        comm.status()
        want = rank_order_combine(parts, op, dtype)
        for r in range(world):
            assert np.array_equal(to_np(bufs[r]).view(np.uint8), want.view(np.uint8)), f"{dtype} {op} n={n} round {round_} rank {r}"
        # alternate with the one-launch form: both advance the same epochs
        bufs = [to_gpu(p) for p in parts]
        comm.allreduce(bufs, op)
        comm.status()
        assert np.array_equal(to_np(bufs[world - 1]).view(np.uint8), want.view(np.uint8))
    waited_us, waits = comm.wait_stats()
    assert waits == expected_waits and 0.0 < waited_us < 1e6, (waits, expected_waits, waited_us)   # the rendezvous is accounted for, per CTA
    assert comm.wait_stats() == (0.0, 0)
    comm.close()


def test_split_exchange_absent_rank_times_out_in_the_combine():
    from deepx_b200 import _native as N
    from deepx_b200.comm import EmulatedComm
    comm = EmulatedComm(4)
    comm.set_timeout_ms(50)
    parts = [np.full(100, r + 1, dtype=np.float32) for r in range(4)]
    bufs = [to_gpu(p) for p in parts]
    comm.publish(bufs, "sum", active=3)       # rank 3 never publishes
    comm.combine(bufs, "sum", active=3)
    with pytest.raises(N.DxError, match="gave up waiting for rank 3"):
        comm.status()
    for r in range(4):
        assert np.array_equal(to_np(bufs[r]), parts[r])   # nothing combined, local data untouched
    comm.close()


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("rows,row_elems,dtype", [(8, 5, "float32"), (17, 33, "int8"), (64, 4096, "float32"), (3, 100001, "bfloat16"),
                                                  (2048, 1, "float32"), (1, 7, "int64")])
def test_allgather_rows_on_emulated_ranks(world, rows, row_elems, dtype):
    """Every rank holds the whole tensor with only its own block of rows filled in (the rest poisoned); after the
    gather every rank holds every block, bit for bit.  Uneven splits (rows % world != 0), ranks without any row,
    unaligned row sizes and blocks larger than a mailbox slot (several rounds) included."""
    from deepx_b200.comm import EmulatedComm, shard_rows
    rng = np.random.default_rng(seed_of("gather", world, rows, row_elems, dtype))
    full = make(rng, dtype, (rows, row_elems))
    comm = EmulatedComm(world)
    bufs = []
    for r in range(world):
        r0, n = shard_rows(rows, r, world)
        mine = np.full_like(full, 99)
        mine[r0:r0 + n] = full[r0:r0 + n]
        bufs.append(to_gpu(mine))
    assert sum(shard_rows(rows, r, world)[1] for r in range(world)) == rows
    for _ in range(2):   # twice: epochs stay in step although ranks publish different numbers of chunks
        comm.allgather_rows(bufs)
        comm.status()
        for r in range(world):
            assert np.array_equal(to_np(bufs[r]).view(np.uint8), full.view(np.uint8)), f"rank {r}"
    # and the all-reduce still works on the same mailboxes afterwards
    parts = [np.full(10, r + 1, dtype=np.float32) for r in range(world)]
    ab = [to_gpu(p) for p in parts]
    comm.allreduce(ab, "sum")
    comm.status()
    assert np.array_equal(to_np(ab[0]), np.full(10, world * (world + 1) // 2, dtype=np.float32))
    comm.close()


@pytest.mark.parametrize("dtype", ["float32", "int32"])
def test_deferred_reduce_on_one_rank(dtype):
    """dx_reduce_allreduce_begin + dx_comm_allreduce_finish against the own mailbox (a world of one): the output is the
    plain reduction once finished; a second begin finishes the first by itself; dx_comm_pending tracks it."""
    import ctypes as C
    from deepx_b200 import _native as N
    from deepx_b200 import tensorfunc as TF
    h = N.lib.dx_comm_create(0, 1, 0)
    rng = np.random.default_rng(seed_of("defer", dtype))
    a = make(rng, dtype, (512, 4096), 0.0, 1.0)
    b = make(rng, dtype, (300, 1000), 0.0, 1.0)
    A, B = to_gpu(a), to_gpu(b)
    want_a, want_b = torch.empty(1, dtype=A.dtype, device="cuda:0"), torch.empty(1000, dtype=A.dtype, device="cuda:0")
    TF.sum(A, [0, 1], False, want_a)
    TF.reducemax(B, [0], False, want_b)
    out_a, out_b = torch.empty_like(want_a), torch.empty_like(want_b)
    TF._reduce(N.SUM, A, [0, 1], False, out_a, comm_handle=h, defer=True)        # one-CTA finish: published by the reduce kernel
    p = C.c_void_p()
    assert N.lib.dx_comm_pending(h, C.byref(p)) == 1 and p.value == out_a.data_ptr()
    TF._reduce(N.RMAX, B, [0], False, out_b, comm_handle=h, defer=True)          # finishes the first, begins the second
    assert N.lib.dx_comm_pending(h, C.byref(p)) == 1 and p.value == out_b.data_ptr()
    N.check(N.lib.dx_comm_allreduce_finish(h, torch.cuda.current_stream().cuda_stream))
    assert N.lib.dx_comm_pending(h, None) == 0
    N.check(N.lib.dx_comm_status(h, None))
    assert np.array_equal(to_np(out_a).view(np.uint8), to_np(want_a).view(np.uint8))
    assert np.array_equal(to_np(out_b).view(np.uint8), to_np(want_b).view(np.uint8))
    N.lib.dx_comm_destroy(h)
