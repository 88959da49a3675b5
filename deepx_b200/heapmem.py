"""ctypes front of the heap-tensor service in ``libdeepx_exec.so`` (C ABI: ``include/dx_heapmem.h``).

Heap tensors are named device allocations that outlive a computation and are shared between
processes of one machine through CUDA IPC; the registry keeps, per tensor, the fields of the
reference's ``tensor:<name>`` hash and is driven by the JSON commands of its ``tensor_lifecycle``
list (executor/heapmem-cuda/README.md:13-40).
"""
from __future__ import annotations

import ctypes as C
import json

from .executor import lib as _exec_lib

_vp, _i, _sz, _cp = C.c_void_p, C.c_int, C.c_size_t, C.c_char_p
SIGNATURES = {
    "dx_heap_create": (_vp, [_cp, _i]),
    "dx_heap_create_redis": (_vp, [_cp, _i, _cp, _i]),
    "dx_heap_request": (_i, [_cp, _i, _cp]),
    "dx_heap_lookup": (_i, [_cp, _i, _cp, C.c_char_p, _sz]),
    "dx_heap_destroy": (None, [_vp]),
    "dx_heap_last_error": (_cp, []),
    "dx_heap_command": (_i, [_vp, _cp, C.c_char_p, _sz]),
    "dx_heap_push": (_i, [_vp, _cp]),
    "dx_heap_run_once": (_i, [_vp, _i]),
    "dx_heap_meta": (_i, [_vp, _cp, C.c_char_p, _sz]),
    "dx_heap_count": (_i, [_vp]),
    "dx_heap_ptr": (_vp, [_vp, _cp]),
    "dx_heap_gc_sweep": (C.c_int64, [_vp, _cp]),
    "dx_heap_open": (_vp, [_cp, _i]),
    "dx_heap_close": (_i, [_vp]),
    "dx_heap_copy": (_i, [_vp, _vp, _sz, _i]),
}
DEVICE, HOST_FAKE = 0, 1
_bound = False


def lib() -> C.CDLL:
    global _bound
    l = _exec_lib()
    if not _bound:
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype = res
            fn.argtypes = args
        _bound = True
    return l


class HeapError(RuntimeError):
    pass


def _err() -> str:
    return lib().dx_heap_last_error().decode()


class Heap:
    """The owner side: registry + allocations.  ``backing=HOST_FAKE`` runs the registry without a GPU."""

    def __init__(self, node: str | None = None, backing: int = DEVICE, redis: tuple[str, int] | None = None):
        """`redis` = (host, port): hashes and the command list live in that Redis server (the service side of a
        multi-process set-up, what the ``deepx-heapmem`` daemon is); None keeps them in this process."""
        if redis is None:
            self._h = lib().dx_heap_create(node.encode() if node else None, backing)
        else:
            self._h = lib().dx_heap_create_redis(node.encode() if node else None, backing, redis[0].encode(), int(redis[1]))
        if not self._h:
            raise HeapError(_err())
        self._buf = C.create_string_buffer(1 << 14)

    def close(self) -> None:
        if self._h:
            lib().dx_heap_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def command(self, cmd: dict | str) -> dict:
        text = cmd if isinstance(cmd, str) else json.dumps(cmd)
        if lib().dx_heap_command(self._h, text.encode(), self._buf, len(self._buf)) != 0:
            raise HeapError(_err())
        return json.loads(self._buf.value.decode())

    def create(self, name: str, dtype: str, shape, device: int = 0, pid: int = 0) -> dict:
        return self.command({"op": "create", "name": name, "dtype": dtype, "shape": list(shape), "device": device, "pid": pid})

    def get(self, name: str) -> dict:
        return self.command({"op": "get", "name": name})

    def delete(self, name: str) -> dict:
        return self.command({"op": "delete", "name": name})

    def push(self, cmd: dict | str) -> None:
        text = cmd if isinstance(cmd, str) else json.dumps(cmd)
        lib().dx_heap_push(self._h, text.encode())

    def run_once(self, timeout_ms: int = 0) -> bool:
        return lib().dx_heap_run_once(self._h, timeout_ms) == 1

    def meta(self, name: str) -> dict:
        if lib().dx_heap_meta(self._h, name.encode(), self._buf, len(self._buf)) != 0:
            raise KeyError(name)
        return json.loads(self._buf.value.decode())

    def __len__(self) -> int:
        return lib().dx_heap_count(self._h)

    def ptr(self, name: str) -> int:
        return int(lib().dx_heap_ptr(self._h, name.encode()) or 0)

    def gc_sweep(self, node: str | None = None) -> int:
        return int(lib().dx_heap_gc_sweep(self._h, node.encode() if node else None))


def request(redis: tuple[str, int], cmd: dict | str) -> None:
    """Client side: push one lifecycle command for the service process behind `redis` = (host, port)."""
    text = cmd if isinstance(cmd, str) else json.dumps(cmd)
    if lib().dx_heap_request(redis[0].encode(), int(redis[1]), text.encode()) != 0:
        raise HeapError(_err())


def lookup(redis: tuple[str, int], name: str) -> dict:
    """Client side: the tensor's hash (KeyError while the service has not created it yet)."""
    buf = C.create_string_buffer(1 << 14)
    rc = lib().dx_heap_lookup(redis[0].encode(), int(redis[1]), name.encode(), buf, len(buf))
    if rc == -1:
        raise KeyError(name)
    if rc != 0:
        raise HeapError(_err())
    return json.loads(buf.value.decode())


def open_handle(ipc_handle_hex: str, device: int = 0) -> int:
    """Consumer side (another process than the owner): device pointer of the shared allocation."""
    p = lib().dx_heap_open(ipc_handle_hex.encode(), device)
    if not p:
        raise HeapError(_err())
    return int(p)


def close_handle(ptr: int) -> None:
    if lib().dx_heap_close(ptr) != 0:
        raise HeapError(_err())


def copy_to_device(dst_ptr: int, host) -> None:
    if lib().dx_heap_copy(dst_ptr, host.ctypes.data, host.nbytes, 1) != 0:
        raise HeapError(_err())


def copy_to_host(host, src_ptr: int) -> None:
    if lib().dx_heap_copy(host.ctypes.data, src_ptr, host.nbytes, 0) != 0:
        raise HeapError(_err())
