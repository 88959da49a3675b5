"""The integer identities the small-integer division kernels rest on, checked on the CPU.

* division by a constant d (|d| >= 2) of an int8 / int16 value a:  trunc(a / d) ==
  sign * ((|a| * (floor(2^32 / |d|) + 1)) >> 32)                     (DivConstFn, ew_ops.cuh)
* division with a per-element divisor through fp32:  trunc(a / b) == int(fl32(a) / fl32(b)) with the
  IEEE-rounded quotient                                              (BinaryFn<DX_DIV>, ew_ops.cuh)
* the same without conversion instructions: int -> float through the bits of 1.5·2^23 + v, and the
  truncation as round-to-nearest of (q·(1 + p) − copysign(0.5, q)) + 1.5·2^23, with q the IEEE quotient
  and p = 2^-17 for int16, q an approximate quotient (up to 2 ulp off) and p = 2^-12 for int8
                                                                     (trunc_pushed, small_int_to_float)
* sin / cos of a 16-bit float in fp32 (quadrant by the magic number, three-constant reduction, Cephes
  polynomials): within 2 fp32 ulp, and the same f16 as the C library's float routine for every f16 input
                                                                     (trig_of_16bit, ew_ops.cuh)
* log of a 16-bit float in fp32 (exponent split on the bits, Cephes polynomial): within 0.75 fp32 ulp
                                                                     (log_of_16bit_x2, ew_ops.cuh)
* float32 pow as 2^(y·log2 x) with log2 x and the product carried as sums of two floats: within 4e-6
  relative of the exact power wherever the fast path applies              (pow_f32_x2, ew_ops.cuh)
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


def _trunc_pushed(q32, push):
    """The kernel's truncation (trunc_pushed, ew_ops.cuh) in numpy: fma(q, push, -copysign(0.5, q)) rounded once
    to fp32, plus 1.5·2^23 rounded to fp32, minus 1.5·2^23 as integers."""
    q32 = q32.astype(np.float32)
    half = np.copysign(np.float32(0.5), q32)
    u = (q32.astype(np.float64) * np.float64(np.float32(push)) - half.astype(np.float64)).astype(np.float32)  # one rounding, like fma
    f = (u + np.float32(12582912.0)).astype(np.float32)
    return f.view(np.int32).astype(np.int64) - 0x4B400000


def test_int8_approximate_quotient_pushed_away_from_zero_truncates_exactly():
    a8, b8 = np.meshgrid(np.arange(-128, 128), np.array([b for b in range(-128, 128) if b != 0]))
    want = np.trunc(a8 / b8).astype(np.int64)
    exact = a8.astype(np.float64) / b8.astype(np.float64)
    for ulps in (-2.5, -1.0, 0.0, 1.0, 2.5):  # the reciprocal unit's error bound is 2 ulp of the quotient
        approx = (exact * (1.0 + ulps * 2.0 ** -23)).astype(np.float32)
        assert np.array_equal(_trunc_pushed(approx, 1.000244140625), want), ulps
    # signed zeros (0 / negative gives -0.0): both must truncate to 0
    assert np.array_equal(_trunc_pushed(np.array([0.0, -0.0], dtype=np.float32), 1.000244140625), [0, 0])


def test_int16_ieee_quotient_pushed_away_from_zero_truncates_exactly():
    a = np.arange(-32768, 32768)
    rng = np.random.default_rng(2)
    for b in list(range(1, 600)) + [-1, -2, -3, -255, 32767, -32768, 21845, 10923, -4097, 16384, -16385] + list(rng.integers(-32768, 32768, 600)):
        if b == 0:
            continue
        q = a.astype(np.float32) / np.float32(b)  # IEEE-rounded, as __fdiv_rn
        assert np.array_equal(_trunc_pushed(q, 1.00000762939453125), np.trunc(a / int(b)).astype(np.int64)), b


def test_small_int_to_float_through_the_magic_number():
    v = np.arange(-32768, 32768, dtype=np.int32)
    f = (np.int32(0x4B400000) + v).view(np.float32) - np.float32(12582912.0)
    assert np.array_equal(f, v.astype(np.float32))


def _fma(a, b, c):
    """fp32 fused multiply-add of arrays: the exact product of two floats fits a double."""
    return (np.asarray(a, np.float32).astype(np.float64) * np.asarray(b, np.float32).astype(np.float64)
            + np.asarray(c, np.float32).astype(np.float64)).astype(np.float32)


def _trig_of_16bit(x, want_cos):
    """trig_of_16bit (ew_ops.cuh) in numpy, for |x| < 1e5."""
    f32 = np.float32
    x = x.astype(f32)
    magic = f32(12582912.0)
    j = _fma(x, f32(0.636619747), magic)
    n = j.view(np.int32).astype(np.int64) + int(want_cos)
    jf = (j - magic).astype(f32)
    r = _fma(jf, f32(-1.57079601e+00), x)
    r = _fma(jf, f32(-3.13916473e-07), r)
    r = _fma(jf, f32(-5.39030253e-15), r)
    r2 = (r * r).astype(f32)
    ps = _fma(r2, f32(-1.9515295891e-4), f32(8.3321608736e-3))
    ps = _fma(ps, r2, f32(-1.6666654611e-1))
    s = (r * _fma(r2, ps, f32(1.0))).astype(f32)
    pc = _fma(r2, f32(2.443315711809948e-5), f32(-1.388731625493765e-3))
    pc = _fma(pc, r2, f32(4.166664568298827e-2))
    pc = _fma(pc, r2, f32(-0.5))
    c = _fma(pc, r2, f32(1.0))
    v = np.where(n & 1, c, s)
    return np.where(n & 2, -v, v).astype(f32)


def test_trig_of_16bit_every_f16_argument():
    h = np.arange(0, 65536, dtype=np.uint16).view(np.float16)
    x = h[np.isfinite(h)].astype(np.float32)
    for want_cos, ref in ((0, np.sin), (1, np.cos)):
        got = _trig_of_16bit(x, want_cos)
        exact = ref(x.astype(np.float64))
        ulp = np.spacing(np.abs(exact).astype(np.float32)).astype(np.float64)
        assert (np.abs(got.astype(np.float64) - exact) <= 2.0 * ulp).all()
        assert np.array_equal(got.astype(np.float16).view(np.uint16), ref(x).astype(np.float16).view(np.uint16))  # the float routine, rounded


def test_trig_of_16bit_every_bf16_argument_below_1e5():
    b = (np.arange(0, 65536, dtype=np.uint32) << 16).view(np.float32)
    x = b[np.isfinite(b) & (np.abs(b) < 1e5)]
    for want_cos, ref in ((0, np.sin), (1, np.cos)):
        got = _trig_of_16bit(x, want_cos)
        exact = ref(x.astype(np.float64))
        ulp = np.spacing(np.abs(exact).astype(np.float32)).astype(np.float64)
        assert (np.abs(got.astype(np.float64) - exact) <= 2.0 * ulp).all()


def _log_of_16bit(x):
    """log_of_16bit_x2 (ew_ops.cuh) in numpy, for positive normal x."""
    f32 = np.float32
    x = x.astype(f32)
    b = x.view(np.uint32)
    eb = ((b - np.uint32(0x3f3504f3)) & np.uint32(0xff800000)).astype(np.uint32)
    m = (b - eb).view(f32)
    e = (eb.view(np.int32) >> 23).astype(f32)
    f = (m - f32(1)).astype(f32)
    z = (f * f).astype(f32)
    coef = [7.0376836292e-2, -1.1514610310e-1, 1.1676998740e-1, -1.2420140846e-1, 1.4249322787e-1, -1.6668057665e-1,
            2.0000714765e-1, -2.4999993993e-1, 3.3333331174e-1]
    y = np.full_like(f, f32(coef[0]))
    for c in coef[1:]:
        y = _fma(y, f, f32(c))
    y = ((y * f).astype(f32) * z).astype(f32)
    y = _fma(e, f32(-2.12194440e-4), y)
    y = _fma(z, f32(-0.5), y)
    return _fma(e, f32(0.693359375), (f + y).astype(f32))


def test_log_of_16bit_every_positive_argument():
    h = np.arange(0, 65536, dtype=np.uint16).view(np.float16)
    b = (np.arange(0, 65536, dtype=np.uint32) << 16).view(np.float32)
    for x in (h[np.isfinite(h) & (h > 0)].astype(np.float32), b[np.isfinite(b) & (b >= np.float32(1.1754944e-38))]):
        got = _log_of_16bit(x)
        exact = np.log(x.astype(np.float64))
        ulp = np.spacing(np.abs(exact).astype(np.float32)).astype(np.float64)
        assert (np.abs(got.astype(np.float64) - exact) <= 0.75 * np.maximum(ulp, 1e-45)).all()


# ---- pow_f32_x2 (ew_ops.cuh) in numpy: the same operations in the same order, FMAs through float64 ----------
_POW_Q = np.array([-7.213471532e-01, 4.808981419e-01, -3.607088029e-01, 2.885792851e-01, -2.393930554e-01, 2.042880207e-01,
                   -1.923508048e-01, 1.883963346e-01, -1.097617820e-01], dtype=np.float32)
_INVLN2_HI, _INVLN2_LO, _LN2 = np.float32(1.4426950216293335), np.float32(1.925963033500011e-08), np.float32(0.693147182)


def _fma(a, b, c):
    return (np.asarray(a, np.float32).astype(np.float64) * np.asarray(b, np.float32).astype(np.float64)
            + np.asarray(c, np.float32).astype(np.float64)).astype(np.float32)


def _pow_fast(x, y):
    """(result, fast) — `fast` marks the elements the kernel keeps; the others go to the library powf."""
    F = np.float32
    x, y = x.astype(F), y.astype(F)
    b = x.view(np.uint32)
    eb = (b - np.uint32(0x3f3504f3)) & np.uint32(0xff800000)
    f = (b - eb).view(F) - F(1)
    e = (eb.view(np.int32) >> 23).astype(F)
    q = np.full_like(f, _POW_Q[8])
    for i in range(7, -1, -1):
        q = _fma(q, f, np.full_like(f, _POW_Q[i]))
    ff = f * f
    p_hi = f * _INVLN2_HI
    p_lo = _fma(f, np.full_like(f, _INVLN2_HI), -p_hi)
    p_lo = _fma(f, np.full_like(f, _INVLN2_LO), p_lo)
    u = _fma(ff, q, p_lo)
    s1 = p_hi + u
    c1 = (p_hi - s1) + u
    s = e + s1
    c2 = (e - s) + s1
    l = c1 + c2
    with np.errstate(all="ignore"):
        t_hi = y * s
        t_lo = _fma(y, l, _fma(y, s, -t_hi))
        fast = ((b - np.uint32(0x00800000)) < np.uint32(0x7f000000)) & (np.abs(t_hi) < 125)
        p = np.exp2(np.where(fast, t_hi, 0).astype(np.float64)).astype(F)  # the hardware 2^t: at most 2^-22 off, allowed for below
        r = _fma(p, t_lo * _LN2, p)
    return r, fast


def test_fast_pow_is_within_tolerance_of_the_exact_power():
    rng = np.random.default_rng(0)
    n = 1_000_000
    cases = {
        "ordinary": (rng.uniform(0.1, 4, n), rng.uniform(-3, 3, n)),
        "wide x": (np.exp(rng.uniform(-80, 80, n)), rng.uniform(-1.5, 1.5, n)),
        "x near 1, huge y": (1 + rng.uniform(-1e-3, 1e-3, n), rng.uniform(-1e5, 1e5, n)),
        "every mantissa region, large y": (1 + rng.uniform(-0.3, 0.42, n), rng.uniform(-250, 250, n)),
        "integer y": (rng.uniform(0.5, 30, n), rng.integers(-12, 13, n).astype(np.float64)),
    }
    for name, (x, y) in cases.items():
        x, y = x.astype(np.float32), y.astype(np.float32)
        r, fast = _pow_fast(x, y)
        ref = np.power(x.astype(np.float64), y.astype(np.float64))
        rel = np.abs(r[fast].astype(np.float64) - ref[fast]) / ref[fast]
        assert fast.mean() > 0.9, name
        assert rel.max() + 2.0 ** -22 < 4e-6, (name, rel.max())   # 2^-22: the hardware exponential's own error


def test_fast_pow_hands_special_arguments_to_the_library():
    x = np.array([0.0, -2.0, np.inf, np.nan, 1e-40, 2.0, 2.0, 2.0, 1.0, 3.0, 1.5], dtype=np.float32)
    y = np.array([2.0, 3.0, 1.0, 1.0, 2.0, np.inf, np.nan, 200.0, np.nan, -90.0, 0.0], dtype=np.float32)
    r, fast = _pow_fast(x, y)
    assert fast.tolist() == [False, False, False, False, False, False, False, False, False, False, True]
    assert r[-1] == 1.0
    # exact cases stay exact: x = 1, y = 0, powers of two with integer exponents
    x = np.array([1.0, 7.3, 2.0, 4.0, 0.5, 8.0], dtype=np.float32)
    y = np.array([123.0, 0.0, 10.0, 0.5, 3.0, -1.0], dtype=np.float32)
    r, fast = _pow_fast(x, y)
    assert fast.all() and r.tolist() == [1.0, 1.0, 1024.0, 2.0, 0.125, 0.125]
