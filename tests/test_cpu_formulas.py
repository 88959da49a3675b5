"""The integer identities the small-integer division kernels rest on, checked on the CPU.

* division by a constant d (|d| >= 2) of an int8 / int16 value a:  trunc(a / d) ==
  sign * ((|a| * (floor(2^32 / |d|) + 1)) >> 32)                     (DivConstFn, ew_ops.cuh)
* division with a per-element divisor through fp32:  trunc(a / b) == int(fl32(a) / fl32(b)) with the
  IEEE-rounded quotient                                              (BinaryFn<DX_DIV>, ew_ops.cuh)
"""
import numpy as np


def test_multiply_high_division_every_int16_numerator():
    a = np.arange(-32768, 32768, dtype=np.int64)
    rng = np.random.default_rng(0)
    divisors = list(range(2, 600)) + [32767, 32768, 16384, 10923, 21845, 255, 257, 4097, 30000] + list(rng.integers(2, 32768, 300))
    for d in divisors:
        magic = (1 << 32) // int(d) + 1
        assert magic < (1 << 32)
        q = (np.abs(a) * magic) >> 32
        for sd in (int(d), -int(d)):
            got = np.where((a < 0) ^ (sd < 0), -q, q)
            assert np.array_equal(got, np.trunc(a / sd).astype(np.int64)), sd


def test_fp32_quotient_truncates_to_the_integer_quotient():
    # every int8 pair
    a8, b8 = np.meshgrid(np.arange(-128, 128), np.array([b for b in range(-128, 128) if b != 0]))
    got = np.trunc(a8.astype(np.float32) / b8.astype(np.float32)).astype(np.int64)
    assert np.array_equal(got, np.trunc(a8 / b8).astype(np.int64))
    # every int16 numerator against a spread of divisors (numpy's float32 division is IEEE-rounded)
    a = np.arange(-32768, 32768)
    rng = np.random.default_rng(1)
    for b in list(range(1, 400)) + [32767, -32768, 21845, 10923, -4097] + list(rng.integers(-32768, 32768, 400)):
        if b == 0:
            continue
        got = np.trunc(a.astype(np.float32) / np.float32(b)).astype(np.int64)
        assert np.array_equal(got, np.trunc(a / int(b)).astype(np.int64)), b
