"""Shared helpers of the GPU parity tests: numpy ↔ torch transfer that keeps 16-bit floats bit-exact."""
import zlib

import ml_dtypes
import numpy as np
import torch

NP_DTYPES = {
    "float64": np.float64, "float32": np.float32, "float16": np.float16, "bfloat16": ml_dtypes.bfloat16,
    "int64": np.int64, "int32": np.int32, "int16": np.int16, "int8": np.int8, "bool": np.bool_,
}
TORCH_DTYPES = {
    "float64": torch.float64, "float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
    "int64": torch.int64, "int32": torch.int32, "int16": torch.int16, "int8": torch.int8, "bool": torch.bool,
}
ALL_NUMERIC = ["float64", "float32", "float16", "bfloat16", "int64", "int32", "int16", "int8"]
FLOATS = ["float64", "float32", "float16", "bfloat16"]
INTS = ["int64", "int32", "int16", "int8"]


def to_gpu(a: np.ndarray, device="cuda:0") -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if a.dtype == np.dtype(ml_dtypes.bfloat16):
        return torch.from_numpy(a.view(np.int16).copy()).to(device).view(torch.bfloat16)
    return torch.from_numpy(a.copy()).to(device)


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(ml_dtypes.bfloat16)
    return t.numpy()


def bits(a: np.ndarray) -> np.ndarray:
    """Raw bit pattern view for exact comparison (distinguishes -0.0, compares NaNs by payload)."""
    a = np.ascontiguousarray(a)
    return a.view({1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[a.dtype.itemsize])


def assert_bit_exact(got: np.ndarray, want: np.ndarray, what=""):
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert got.dtype == want.dtype, f"{what}: dtype {got.dtype} != {want.dtype}"
    g, w = bits(got), bits(want)
    if not np.array_equal(g, w):
        bad = np.flatnonzero(g.ravel() != w.ravel())
        i = bad[0]
        raise AssertionError(f"{what}: {bad.size} of {g.size} elements differ; first at {i}: "
                             f"got {got.ravel()[i]!r} want {want.ravel()[i]!r}")


def make(rng: np.random.Generator, dtype: str, shape, lo=-4.0, hi=4.0, nonzero=False) -> np.ndarray:
    npdt = NP_DTYPES[dtype]
    if dtype == "bool":
        return rng.integers(0, 2, shape).astype(np.bool_)
    if dtype in INTS:
        info = np.iinfo(npdt)
        l, h = max(info.min, -100), min(info.max, 100)
        a = rng.integers(l, h + 1, shape).astype(npdt)
        if nonzero:
            a[a == 0] = 3
        return a
    a = rng.uniform(lo, hi, shape).astype(np.float32 if dtype in ("float16", "bfloat16") else npdt).astype(npdt)
    if nonzero:
        a[a == 0] = 1
    return a


def seed_of(*parts) -> int:
    """Stable across processes (str hash is salted)."""
    return zlib.crc32("|".join(str(p) for p in parts).encode())
