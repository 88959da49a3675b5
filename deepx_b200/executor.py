"""ctypes front of ``libdeepx_exec.so`` (C ABI in ``include/dx_executor.h``): the deepxIR text
boundary.  ``Executor.run(ir_line)`` is what the reference's executor process does with one UDP
datagram line — parse, resolve in the op registry, run on the GPU, reply — in process.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libdeepx_exec.so"
BIN_PATH = _PKG / "deepx-op-b200"

_vp, _i, _sz, _cp = C.c_void_p, C.c_int, C.c_size_t, C.c_char_p
SIGNATURES = {
    "dx_exec_create": (_vp, [_i, _sz]),
    "dx_exec_destroy": (None, [_vp]),
    "dx_exec_last_error": (_cp, []),
    "dx_exec_run": (_i, [_vp, _cp, C.c_char_p, _sz]),
    "dx_exec_run_program": (_i, [_vp, _cp, C.c_char_p, _sz]),
    "dx_exec_set_fusion": (None, [_vp, _i]),
    "dx_exec_fusion_stats": (None, [_vp, C.POINTER(C.c_uint64)]),
    "dx_exec_compile": (_vp, [_vp, _cp]),
    "dx_program_run": (_i, [_vp]),
    "dx_program_info": (None, [_vp, C.POINTER(C.c_size_t)]),
    "dx_program_free": (None, [_vp]),
    "dx_exec_bind_tensor": (_i, [_vp, _cp, _i, C.POINTER(C.c_int64), _i, _vp]),
    "dx_exec_tensor_info": (_i, [_vp, _cp, C.POINTER(C.c_int), C.POINTER(C.c_int64), _i]),
    "dx_exec_tensor_ptr": (_vp, [_vp, _cp]),
    "dx_exec_set_shard": (_i, [_vp, _i, _i, _sz, _vp]),
    "dx_exec_tensor_shard": (_i, [_vp, _cp, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "dx_ir_shard_plan": (_i, [_cp, _i, _sz, C.c_char_p, _sz]),
    "dx_exec_upload": (_i, [_vp, _cp, _vp, _sz]),
    "dx_exec_upload_async": (_i, [_vp, _cp, _vp, _sz]),
    "dx_exec_download": (_i, [_vp, _cp, _vp, _sz]),
    "dx_exec_sync": (_i, [_vp]),
    "dx_exec_stream": (_vp, [_vp]),
    "dx_exec_op_table": (_sz, [_vp, C.c_char_p, _sz]),
    "dx_exec_stats": (None, [_vp, C.POINTER(C.c_size_t)]),
    "dx_ir_parse": (_i, [_cp, C.c_char_p, _sz]),
    "dx_ir_dtype_roundtrip": (_i, [_cp, C.c_char_p, _sz]),
    "dx_ir_vector_i64": (_i, [_cp, _i, C.POINTER(C.c_int64), _i]),
    "dx_ir_check_print_format": (_i, [_cp, _i, C.c_char_p, _sz]),
    "dx_ir_plan_fusion": (_i, [_cp, _cp, C.c_char_p, _sz]),
    "dx_registry_new": (_vp, [_i]),
    "dx_registry_free": (None, [_vp]),
    "dx_registry_add": (_i, [_vp, _cp]),
    "dx_registry_get": (_i, [_vp, _cp]),
    "dx_registry_size": (_i, [_vp]),
}

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m deepx_b200.build`. There is no CPU fallback.")
        _lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


_DX2NP = {0: np.float64, 1: np.float32, 2: np.float16, 3: None, 4: np.int64, 5: np.int32, 6: np.int16, 7: np.int8, 8: np.bool_}


def _bf16():
    import ml_dtypes
    return ml_dtypes.bfloat16


def parse_ir(line: str) -> str:
    """What the parser understood, as one canonical line ("!…" for a parse error)."""
    buf = C.create_string_buffer(1 << 16)
    lib().dx_ir_parse(line.encode(), buf, len(buf))
    return buf.value.decode()


def dtype_roundtrip(text: str) -> str:
    buf = C.create_string_buffer(4096)
    lib().dx_ir_dtype_roundtrip(text.encode(), buf, len(buf))
    return buf.value.decode()


def vector_i64(ir_line: str, arg_index: int) -> list[int]:
    """The integer vector argument `arg_index` of an IR line as the executor reads it (64-bit)."""
    out = (C.c_int64 * 64)()
    n = lib().dx_ir_vector_i64(ir_line.encode(), arg_index, out, 64)
    if n < 0:
        raise ValueError(lib().dx_exec_last_error().decode())
    return [int(out[i]) for i in range(n)]


def check_print_format(fmt: str, dtype_code: int) -> str:
    """The format `print` would use for a tensor of that dtype; ValueError when it is refused."""
    buf = C.create_string_buffer(256)
    rc = lib().dx_ir_check_print_format(fmt.encode(), dtype_code, buf, len(buf))
    if rc != 0:
        raise ValueError(lib().dx_exec_last_error().decode())
    return buf.value.decode()


def shard_plan(program: str, world: int, min_bytes: int = 1 << 20) -> list[str]:
    """What a rank of a `world`-GPU executor does with each line of `program` (no GPU needed): see
    ``dx_ir_shard_plan`` in include/dx_executor.h."""
    buf = C.create_string_buffer(max(1 << 16, 64 * (program.count("\n") + 2)))
    n = lib().dx_ir_shard_plan(program.encode(), world, min_bytes, buf, len(buf))
    if n < 0:
        raise ValueError("shard_plan: " + lib().dx_exec_last_error().decode())
    return buf.value.decode().split("\n") if n else []


def plan_fusion(program: str, existing: str = "") -> tuple[int, list[str]]:
    """The fusion pass alone (no GPU): (number of fused groups, one verdict per program line —
    "run", "absorbed <group>" or "fused <group> <op>").  `existing`: "<name> <dtype> <d0> <d1> …" lines."""
    buf = C.create_string_buffer(max(1 << 16, 4 * len(program) + 4096))
    n = lib().dx_ir_plan_fusion(program.encode(), existing.encode(), buf, len(buf))
    if n < 0:
        raise ValueError("plan_fusion: " + lib().dx_exec_last_error().decode())
    return n, buf.value.decode().splitlines()


class Registry:
    """An op registry on its own (no GPU): add signature lines, resolve calls."""

    def __init__(self, builtin: bool = False):
        self._h = lib().dx_registry_new(1 if builtin else 0)

    def add(self, signature_ir: str) -> int:
        return lib().dx_registry_add(self._h, signature_ir.encode())

    def get(self, call_ir: str) -> int:
        return lib().dx_registry_get(self._h, call_ir.encode())

    def __len__(self) -> int:
        return lib().dx_registry_size(self._h)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().dx_registry_free(self._h)
            self._h = None


class IRError(RuntimeError):
    pass


class Program:
    """A compiled program: its kernels captured into a CUDA graph (Executor.compile)."""

    def __init__(self, handle):
        self._h = handle

    def run(self) -> None:
        """Replays the graph on the executor's stream (asynchronous).  IRError when a tensor the
        program names was deleted, re-created or reshaped since compilation."""
        if lib().dx_program_run(self._h) != 0:
            raise IRError(lib().dx_exec_last_error().decode())

    def info(self) -> dict:
        st = (C.c_size_t * 4)()
        lib().dx_program_info(self._h, st)
        return {"lines": st[0], "ops": st[1], "graph_nodes": st[2], "fused_chains": st[3]}

    def free(self) -> None:
        if self._h:
            lib().dx_program_free(self._h)
            self._h = None

    def __del__(self):
        self.free()


class Executor:
    def __init__(self, device: int = 0, pool_limit_bytes: int = 0):
        self._h = lib().dx_exec_create(device, pool_limit_bytes)
        if not self._h:
            raise RuntimeError("cannot create executor: " + lib().dx_exec_last_error().decode())
        self._buf = C.create_string_buffer(1 << 16)

    def close(self):
        if self._h:
            lib().dx_exec_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def reply(self, ir_line: str) -> tuple[int, str]:
        rc = lib().dx_exec_run(self._h, ir_line.encode(), self._buf, len(self._buf))
        return rc, self._buf.value.decode()

    def run(self, ir_line: str) -> str:
        """Runs one IR line; raises IRError with the reply text when the executor answers `error`."""
        rc, text = self.reply(ir_line)
        if rc != 0:
            raise IRError(text)
        return text

    def run_program(self, program: str, check: bool = True) -> list[str]:
        """Runs several IR lines handed over together (chains of single ops in it may run fused);
        returns one reply per non-empty line.  With `check`, an error reply raises IRError."""
        buf = C.create_string_buffer(max(1 << 16, 256 * (program.count("\n") + 2)))
        rc = lib().dx_exec_run_program(self._h, program.encode(), buf, len(buf))
        if rc < 0:
            raise RuntimeError(lib().dx_exec_last_error().decode())
        replies = buf.value.decode().split("\n") if buf.value else []
        if check and rc != 0:
            raise IRError("\n".join(r for r in replies if " ok" not in r.split("//")[0]))
        return replies

    def compile(self, program: str) -> Program:
        """Runs `program` once and captures it into a CUDA graph (compute ops only)."""
        h = lib().dx_exec_compile(self._h, program.encode())
        if not h:
            raise IRError(lib().dx_exec_last_error().decode())
        return Program(h)

    def set_fusion(self, on: bool) -> None:
        lib().dx_exec_set_fusion(self._h, 1 if on else 0)

    def fusion_stats(self) -> dict:
        st = (C.c_uint64 * 4)()
        lib().dx_exec_fusion_stats(self._h, st)
        return {"programs": st[0], "rmsnorm_groups": st[1], "softmax_groups": st[2], "lines_absorbed": st[3]}

    def info(self, name: str):
        dt = C.c_int()
        shape = (C.c_int64 * 12)()
        nd = lib().dx_exec_tensor_info(self._h, name.encode(), C.byref(dt), shape, 12)
        if nd < 0:
            raise KeyError(name)
        return dt.value, [int(shape[i]) for i in range(nd)]

    def ptr(self, name: str) -> int:
        return int(lib().dx_exec_tensor_ptr(self._h, name.encode()) or 0)

    def new(self, name: str, dtype: str, shape) -> None:
        self.run(f"newtensor(vector<int32>:[{' '.join(str(int(s)) for s in shape)}])->(tensor<{dtype}>:{name})")

    def bind(self, name: str, dtype_code: int, shape, device_ptr: int) -> None:
        """Registers memory the executor does not own (e.g. a heap tensor) under `name`."""
        shp = (C.c_int64 * max(len(shape), 1))(*[int(s) for s in shape])
        if lib().dx_exec_bind_tensor(self._h, name.encode(), dtype_code, shp, len(shape), device_ptr) != 0:
            raise RuntimeError(lib().dx_exec_last_error().decode())

    def set_shard(self, rank: int, world: int, comm_handle, min_bytes: int = 1 << 20) -> None:
        """Makes this executor rank `rank` of `world` (one process per GPU, the same IR lines to every rank).
        `comm_handle` is a connected dx_comm (e.g. ``PeerComm(...)._h``) that must outlive the executor."""
        if lib().dx_exec_set_shard(self._h, rank, world, min_bytes, comm_handle) != 0:
            raise RuntimeError(lib().dx_exec_last_error().decode())

    def shard(self, name: str) -> tuple[bool, int, int, int]:
        """(partitioned, first row, rows held here, global rows) of a tensor."""
        r0, n, g = C.c_int64(), C.c_int64(), C.c_int64()
        rc = lib().dx_exec_tensor_shard(self._h, name.encode(), C.byref(r0), C.byref(n), C.byref(g))
        if rc < 0:
            raise KeyError(name)
        return bool(rc), int(r0.value), int(n.value), int(g.value)

    def upload(self, name: str, array: np.ndarray) -> None:
        a = np.ascontiguousarray(array)
        rc = lib().dx_exec_upload(self._h, name.encode(), a.ctypes.data, a.nbytes)
        if rc != 0:
            raise RuntimeError(lib().dx_exec_last_error().decode())

    def upload_async(self, name: str, array: np.ndarray) -> None:
        """Starts the copy and returns; `array` (contiguous, ideally page-locked) must stay alive until sync()."""
        if not array.flags["C_CONTIGUOUS"]:
            raise ValueError("upload_async needs a contiguous array (it is read after the call returns)")
        rc = lib().dx_exec_upload_async(self._h, name.encode(), array.ctypes.data, array.nbytes)
        if rc != 0:
            raise RuntimeError(lib().dx_exec_last_error().decode())

    def put(self, name: str, array: np.ndarray, dtype: str | None = None) -> None:
        """newtensor + upload."""
        a = np.ascontiguousarray(array)
        dtype = dtype or ("bfloat16" if a.dtype == np.dtype(_bf16()) else str(a.dtype))
        self.new(name, dtype, a.shape)
        self.upload(name, a)

    def download(self, name: str) -> np.ndarray:
        code, shape = self.info(name)
        npdt = _bf16() if code == 3 else _DX2NP[code]
        out = np.empty(shape, dtype=npdt)
        rc = lib().dx_exec_download(self._h, name.encode(), out.ctypes.data, out.nbytes)
        if rc != 0:
            raise RuntimeError(lib().dx_exec_last_error().decode())
        return out

    def sync(self) -> None:
        lib().dx_exec_sync(self._h)

    def op_table(self) -> str:
        n = lib().dx_exec_op_table(self._h, None, 0)
        buf = C.create_string_buffer(n)
        lib().dx_exec_op_table(self._h, buf, n)
        return buf.value.decode()

    def stats(self) -> dict:
        st = (C.c_size_t * 5)()
        lib().dx_exec_stats(self._h, st)
        return {"in_use": st[0], "reserved": st[1], "high_water": st[2], "driver_allocs": st[3], "ops_run": st[4]}
