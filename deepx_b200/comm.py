"""Cross-GPU combine of small reduce partials over NVLink peer memory (C ABI ``dx_comm_*``).

``PeerComm`` is built collectively by the ranks of a ``torch.distributed`` group (one process per
GPU): every rank allocates a mailbox, the 64-byte IPC handles travel through the group's object
all-gather, and every rank maps its peers' mailboxes.  ``allreduce`` then combines a small CUDA
tensor in place with one kernel per rank — no library collective on the data path.  Tensors larger
than ``PeerComm.max_bytes`` should go to ``torch.distributed.all_reduce``.

``EmulatedComm`` runs the same protocol for W ranks on ONE GPU (all ranks' thread blocks in one
launch): the way to exercise it where fewer GPUs than ranks are available.
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import torch
import torch.distributed as dist

from . import _native as N

OPS = {"sum": N.SUM, "prod": N.PROD, "reducemax": N.RMAX, "reducemin": N.RMIN}


def _dtype_code(t: torch.Tensor) -> int:
    from .tensorfunc import dtype_code
    return dtype_code(t)


class PeerComm:
    def __init__(self, group=None, device: int | None = None):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("PeerComm needs an initialised torch.distributed process group")
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.cuda.current_device() if device is None else device
        # Every step that can fail locally is followed by an exchange of who succeeded, so that either
        # all ranks end up with a working communicator or all of them raise (nobody is left waiting).
        self._h = N.lib.dx_comm_create(self.rank, self.world, self.device)
        mine = None
        why = ""
        if self._h:
            buf = C.create_string_buffer(64)
            if N.lib.dx_comm_handle(self._h, buf) == N.OK:
                mine = bytes(buf.raw)
        if mine is None:
            why = N.lib.dx_last_error().decode()
        handles: list = [None] * self.world
        dist.all_gather_object(handles, (mine, why), group=group)
        if any(h is None for h, _ in handles):
            self.close()
            raise RuntimeError("PeerComm: mailbox set-up failed on rank(s) " +
                               ", ".join(f"{r}: {w}" for r, (h, w) in enumerate(handles) if h is None))
        rc = N.lib.dx_comm_connect(self._h, b"".join(h for h, _ in handles))
        status: list = [None] * self.world
        dist.all_gather_object(status, (rc, "" if rc == N.OK else N.lib.dx_last_error().decode()), group=group)
        if any(r != N.OK for r, _ in status):
            self.close()
            raise RuntimeError("PeerComm: mapping the peers' mailboxes failed on rank(s) " +
                               ", ".join(f"{i}: {w}" for i, (r, w) in enumerate(status) if r != N.OK))
        self.max_bytes = int(N.lib.dx_comm_max_bytes())
        # the second exchange also guarantees that nobody publishes into a mailbox a peer has not mapped yet

    def fits(self, t: torch.Tensor) -> bool:
        return t.is_cuda and t.is_contiguous() and t.dtype != torch.bool and t.numel() * t.element_size() <= self.max_bytes

    def allreduce(self, t: torch.Tensor, op: str = "sum") -> torch.Tensor:
        """In place; every rank must make the same sequence of calls."""
        if not self.fits(t):
            raise ValueError("tensor does not fit a mailbox slot (or is not a contiguous CUDA tensor)")
        with torch.cuda.device(t.device):
            st = torch.cuda.current_stream(t.device).cuda_stream
            N.check(N.lib.dx_comm_allreduce(self._h, OPS[op], _dtype_code(t), t.data_ptr(), t.numel(), st))
        return t

    def reduce_allreduce(self, op: str, A: torch.Tensor, dims, keepdims: bool, B: torch.Tensor, defer: bool = False) -> None:
        """sum / prod / reducemax / reducemin of this rank's block into B, combined over the ranks; where
        the local reduction ends in a one-CTA finish step, that kernel also does the exchange.  With
        `defer` the call stops once this rank's result is on its way to the peers: B is complete only
        after :meth:`finish` (or the next call on this communicator), and what the stream runs in
        between hides the skew between the ranks."""
        from . import tensorfunc as TF
        TF._reduce(OPS[op], A, dims, keepdims, B, comm_handle=self._h, defer=defer)

    def pending(self) -> int:
        """Address of the buffer whose exchange has been begun and not finished, or 0."""
        p = C.c_void_p()
        return int(p.value or 0) if N.lib.dx_comm_pending(self._h, C.byref(p)) else 0

    def finish(self, stream: int | None = None) -> None:
        """Completes a deferred exchange on the current stream of this communicator's device."""
        with torch.cuda.device(self.device):
            st = torch.cuda.current_stream().cuda_stream if stream is None else stream
            N.check(N.lib.dx_comm_allreduce_finish(self._h, st))

    def allgather_rows(self, t: torch.Tensor) -> torch.Tensor:
        """In place: every rank holds all of `t` and has filled its own block of leading-axis rows
        (``dx_shard_rows``); afterwards every rank holds every block."""
        if not (t.is_cuda and t.is_contiguous() and t.dim() >= 1):
            raise ValueError("allgather_rows needs a contiguous CUDA tensor with a leading axis")
        rows = t.shape[0]
        row_bytes = (t.numel() // rows if rows else 0) * t.element_size()
        with torch.cuda.device(t.device):
            N.check(N.lib.dx_comm_allgather_rows(self._h, t.data_ptr(), rows, row_bytes, torch.cuda.current_stream().cuda_stream))
        return t

    def set_timeout_ms(self, ms: int) -> None:
        N.check(N.lib.dx_comm_set_timeout_ms(self._h, ms))

    def status(self) -> None:
        """Raises DxError when a wait on a peer expired since the last call (synchronises)."""
        N.check(N.lib.dx_comm_status(self._h, None))

    def wait_stats(self, reset: bool = True) -> tuple[float, int]:
        """(microseconds this rank's CTAs spent waiting for peers' flags, number of waits) since the last reset."""
        import ctypes
        us, n = ctypes.c_double(0.0), ctypes.c_longlong(0)
        N.check(N.lib.dx_comm_wait_stats(self._h, ctypes.byref(us), ctypes.byref(n), 1 if reset else 0, None))
        return float(us.value), int(n.value)

    def close(self) -> None:
        if getattr(self, "_h", None) and N is not None and getattr(N, "lib", None) is not None:  # the module may be gone at interpreter exit
            N.lib.dx_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()


class EmulatedComm:
    def __init__(self, world: int, device: int = 0):
        self.world = world
        self._h = N.lib.dx_comm_emulate(world, device)
        if not self._h:
            raise N.DxError(N.E_CUDA, N.lib.dx_last_error().decode())

    def allreduce(self, bufs: Sequence[torch.Tensor], op: str = "sum", active: int | None = None) -> None:
        assert len(bufs) == self.world
        ptrs = (C.c_void_p * self.world)(*[b.data_ptr() for b in bufs])
        st = torch.cuda.current_stream(bufs[0].device).cuda_stream
        N.check(N.lib.dx_comm_emulated_allreduce(self._h, OPS[op], _dtype_code(bufs[0]), ptrs, self.world if active is None else active,
                                                 bufs[0].numel(), st))

    def _ptrs(self, bufs):
        assert len(bufs) == self.world
        return (C.c_void_p * self.world)(*[b.data_ptr() for b in bufs])

    def publish(self, bufs: Sequence[torch.Tensor], op: str = "sum", active: int | None = None) -> None:
        """First half of the exchange for all ranks (one launch): stores and flags, no waiting."""
        st = torch.cuda.current_stream(bufs[0].device).cuda_stream
        N.check(N.lib.dx_comm_emulated_publish(self._h, OPS[op], _dtype_code(bufs[0]), self._ptrs(bufs), self.world if active is None else active,
                                               bufs[0].numel(), st))

    def combine(self, bufs: Sequence[torch.Tensor], op: str = "sum", active: int | None = None) -> None:
        """Second half for all ranks (one launch): bounded wait for the flags, combine in rank order."""
        st = torch.cuda.current_stream(bufs[0].device).cuda_stream
        N.check(N.lib.dx_comm_emulated_combine(self._h, OPS[op], _dtype_code(bufs[0]), self._ptrs(bufs), self.world if active is None else active,
                                               bufs[0].numel(), st))

    def allgather_rows(self, bufs: Sequence[torch.Tensor]) -> None:
        """bufs[r] is rank r's copy of the whole tensor with rank r's row block filled in."""
        t = bufs[0]
        rows = t.shape[0]
        row_bytes = (t.numel() // rows if rows else 0) * t.element_size()
        st = torch.cuda.current_stream(t.device).cuda_stream
        N.check(N.lib.dx_comm_emulated_allgather_rows(self._h, self._ptrs(bufs), rows, row_bytes, st))

    def set_timeout_ms(self, ms: int) -> None:
        N.check(N.lib.dx_comm_set_timeout_ms(self._h, ms))

    def status(self) -> None:
        N.check(N.lib.dx_comm_status(self._h, None))

    def wait_stats(self, reset: bool = True) -> tuple[float, int]:
        """(microseconds rank 0's CTAs spent waiting for the other ranks' flags, number of waits) since the last reset."""
        import ctypes
        us, n = ctypes.c_double(0.0), ctypes.c_longlong(0)
        N.check(N.lib.dx_comm_wait_stats(self._h, ctypes.byref(us), ctypes.byref(n), 1 if reset else 0, None))
        return float(us.value), int(n.value)

    def close(self) -> None:
        if getattr(self, "_h", None) and N is not None and getattr(N, "lib", None) is not None:  # the module may be gone at interpreter exit
            N.lib.dx_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()


def shard_rows(global_rows: int, rank: int, world: int) -> tuple[int, int]:
    """(first row, row count) of `rank`'s block: the split every part of the library uses."""
    r0, n = C.c_int64(), C.c_int64()
    N.lib.dx_shard_rows(global_rows, rank, world, C.byref(r0), C.byref(n))
    return int(r0.value), int(n.value)
