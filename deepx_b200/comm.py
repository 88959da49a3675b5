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

    def reduce_allreduce(self, op: str, A: torch.Tensor, dims, keepdims: bool, B: torch.Tensor) -> None:
        """sum / prod / reducemax / reducemin of this rank's block into B, combined over the ranks; where
        the local reduction ends in a one-CTA finish step, that kernel also does the exchange."""
        from . import tensorfunc as TF
        TF._reduce(OPS[op], A, dims, keepdims, B, comm_handle=self._h)

    def set_timeout_ms(self, ms: int) -> None:
        N.check(N.lib.dx_comm_set_timeout_ms(self._h, ms))

    def status(self) -> None:
        """Raises DxError when a wait on a peer expired since the last call (synchronises)."""
        N.check(N.lib.dx_comm_status(self._h, None))

    def close(self) -> None:
        if getattr(self, "_h", None):
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

    def set_timeout_ms(self, ms: int) -> None:
        N.check(N.lib.dx_comm_set_timeout_ms(self._h, ms))

    def status(self) -> None:
        N.check(N.lib.dx_comm_status(self._h, None))

    def close(self) -> None:
        if getattr(self, "_h", None):
            N.lib.dx_comm_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()
