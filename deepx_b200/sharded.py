"""Axis-0 sharding of deepxIR elementwise and reduce ops across the GPUs of one node.

One process per GPU (``torch.distributed``, NCCL over NVLink/NVSwitch).  A tensor is
partitioned into contiguous row blocks of its leading axis; every rank owns one block in
its own device pool.  Elementwise ops and reductions that do not touch axis 0 run on the
local block with no communication; a reduction that includes axis 0 reduces the local
block first and then combines the per-rank partials with ONE all-reduce (sum / product /
max / min) — 4 bytes for a global sum, one row for an axis-0 reduce.  Partials that fit a
mailbox slot (64 KiB) are combined by the GPUs themselves over NVLink peer memory
(:mod:`deepx_b200.comm`, one kernel per rank, no library collective); larger ones go to NCCL.
With ``defer=True`` the peer exchange is split: the reduction ends by publishing this rank's partial,
and the wait for the peers plus the combine run as a kernel of their own when ``flush()`` is called (or
just before the next op given to this object that touches the result, or the next cross-rank
reduction) — the ops issued in between hide the skew between the ranks.  Code that reads the output
tensor by other means must call ``flush()`` first, which is why it is off unless asked for.
Ops that do not shard this way (matmul, general transposes) stay single-GPU.

The reference has no multi-GPU code at all (no cudaSetDevice, streams or NCCL anywhere
under executor/); this module is the multi-GPU extension of its tensorfunc interface.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch
import torch.distributed as dist

REDUCE_OPS = {"sum": dist.ReduceOp.SUM, "prod": dist.ReduceOp.PRODUCT, "reducemax": dist.ReduceOp.MAX,
              "reducemin": dist.ReduceOp.MIN}


@dataclass(frozen=True)
class RowPartition:
    """Contiguous split of ``rows`` leading-axis indices over ``world`` ranks: the first
    ``rows % world`` ranks get one extra row."""
    rows: int
    world: int

    def count(self, rank: int) -> int:
        base, extra = divmod(self.rows, self.world)
        return base + (1 if rank < extra else 0)

    def start(self, rank: int) -> int:
        base, extra = divmod(self.rows, self.world)
        return rank * base + min(rank, extra)

    def slice(self, rank: int) -> slice:
        s = self.start(rank)
        return slice(s, s + self.count(rank))


def shards_axis0(dims: Sequence[int], ndim: int) -> bool:
    """True when a reduction over ``dims`` (checked, non-negative) crosses the sharded axis."""
    return ndim > 0 and 0 in set(int(d) for d in dims)


def combine_partials(partial: torch.Tensor, op: str, group=None, peer=None) -> torch.Tensor:
    """All-reduce per-rank partial results in place.  ``peer`` (a :class:`deepx_b200.comm.PeerComm`)
    takes the partials that fit its mailbox; everything else goes to the group's backend: NCCL on
    the GPUs, gloo on CPU tensors in the host-logic tests."""
    if op not in REDUCE_OPS:
        raise ValueError(f"unknown reduce op {op!r}")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        if peer is not None and peer.fits(partial):
            peer.allreduce(partial, op)
        else:
            dist.all_reduce(partial, op=REDUCE_OPS[op], group=group)
    return partial


class ShardedOps:
    """The tensorfunc interface on this rank's row block.

    Elementwise calls forward to :mod:`deepx_b200.tensorfunc` unchanged.  ``sum`` / ``prod`` /
    ``reducemax`` / ``reducemin`` take the LOCAL block and the output tensor; when axis 0 is
    reduced the output holds the global result on every rank after the call.
    """

    def __init__(self, group=None, peer_combine: bool | None = None, defer: bool | None = None):
        """``peer_combine``: combine small partials with the peer-memory kernel instead of NCCL
        (default: on when there is more than one rank, off with ``DX_PEER_COMBINE=0``).  Building
        it is collective: every rank of the group constructs its ShardedOps at the same point."""
        import os
        from . import tensorfunc  # needs the CUDA library; imported here so the partition logic is usable without it
        self.tf = tensorfunc
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if peer_combine is None:
            peer_combine = os.environ.get("DX_PEER_COMBINE", "1") != "0"
        self.defer = (os.environ.get("DX_PEER_DEFER", "0") == "1") if defer is None else bool(defer)
        self._pending = None
        self.peer = None
        if peer_combine and self.world > 1 and torch.cuda.is_available():
            from .comm import PeerComm
            try:
                self.peer = PeerComm(group)  # raises on every rank or on none
            except RuntimeError as e:
                # e.g. CUDA IPC not permitted in this container: the library all-reduce does the combine
                import sys
                if self.rank == 0:
                    print(f"deepx_b200.sharded: peer-memory combine unavailable ({e}); using the group's all-reduce", file=sys.stderr)
                self.peer = None

    def flush(self) -> None:
        """Completes a deferred exchange: after it the last cross-rank reduction's output is final."""
        if self.peer is not None and self._pending is not None:
            self._pending = None
            self.peer.finish()

    def _touches_pending(self, tensors) -> bool:
        if self._pending is None:
            return False
        lo, hi = self._pending
        for t in tensors:
            for u in (t if isinstance(t, (list, tuple)) else (t,)):
                if isinstance(u, torch.Tensor) and u.is_cuda and u.numel() and u.data_ptr() < hi and u.data_ptr() + u.numel() * u.element_size() > lo:
                    return True
        return False

    def __getattr__(self, name):
        fn = getattr(self.tf, name)
        if not callable(fn):
            return fn

        def call(*args, **kwargs):
            # an op that reads or writes the tensor whose exchange is still open waits for it first
            if self._touches_pending(args) or self._touches_pending(kwargs.values()):
                self.flush()
            return fn(*args, **kwargs)
        return call

    def _reduce(self, op: str, A: torch.Tensor, dims, keepdims: bool, B: torch.Tensor) -> None:
        cd = self.tf.checked_dims(A.shape, dims)
        crosses = shards_axis0(cd, A.dim())
        if self._touches_pending((A, B)):
            self.flush()
        if crosses and self.peer is not None and self.world > 1 and self.peer.fits(B):
            # reduce, publish (fused into the finish kernel where the plan allows); the combine is deferred
            self.peer.reduce_allreduce(op, A, dims, keepdims, B, defer=self.defer)
            self._pending = (B.data_ptr(), B.data_ptr() + B.numel() * B.element_size()) if self.defer and self.peer.pending() else None
            return
        getattr(self.tf, op)(A, dims, keepdims, B)
        if crosses:
            self.flush()
            combine_partials(B, op, self.group, self.peer)

    def sum(self, A, dims, keepdims, B): self._reduce("sum", A, dims, keepdims, B)  # noqa: A003
    def prod(self, A, dims, keepdims, B): self._reduce("prod", A, dims, keepdims, B)
    def reducemax(self, A, dims, keepdims, B): self._reduce("reducemax", A, dims, keepdims, B)
    def reducemin(self, A, dims, keepdims, B): self._reduce("reducemin", A, dims, keepdims, B)
