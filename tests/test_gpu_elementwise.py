"""GPU parity: elementwise kernels through the C ABI vs the CPU oracle.

Bar: bit-exact for integer dtypes, compares, invert, switch, todtype and for the IEEE
operations + - * / sqrt max min in every float dtype; exp/log/pow/sin/cos/tan within
rel 1e-5 (fp32), 1e-12 (fp64), one unit in the last place of the 16-bit formats.
"""
import numpy as np
import pytest
import torch

from helpers import (ALL_NUMERIC, FLOATS, INTS, NP_DTYPES, TORCH_DTYPES, assert_bit_exact, make, seed_of, to_gpu,
                     to_np)

pytestmark = pytest.mark.gpu

# sizes: empty, one element, odd (scalar tail), exactly one tile, tiles + ragged tail
SIZES = [0, 1, 7, 4096, 4096 * 3 + 5, 1 << 20]


@pytest.fixture(scope="module")
def mods():
    from deepx_b200 import tensorfunc as TF
    from oracle import oracle as O
    return TF, O


def _close(got, want, dtype, what):
    g, w = got.astype(np.float64), want.astype(np.float64)
    tol = {"float64": 1e-12, "float32": 1e-5, "float16": 2e-3, "bfloat16": 1.6e-2}[dtype]
    ok = np.isclose(g, w, rtol=tol, atol=0) | (np.isnan(g) & np.isnan(w)) | (g == w)
    assert ok.all(), f"{what}: max rel err {np.nanmax(np.abs(g - w) / np.maximum(np.abs(w), 1e-300))}"


@pytest.mark.parametrize("dtype", ALL_NUMERIC)
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div", "max", "min"])
def test_binary_exact(mods, op, dtype):
    TF, O = mods
    rng = np.random.default_rng(seed_of(op, dtype))
    for n in SIZES:
        a = make(rng, dtype, (n,))
        b = make(rng, dtype, (n,), nonzero=(op == "div"))
        A, B = to_gpu(a), to_gpu(b)
        Cc = torch.empty_like(A)
        getattr(TF, op)(A, B, Cc)
        assert_bit_exact(to_np(Cc), getattr(O, op)(a, b), f"{op}<{dtype}> n={n}")


@pytest.mark.parametrize("dtype", ["float32", "int32", "bfloat16"])
def test_binary_inplace_alias(mods, dtype):
    """out may be the same tensor as an input (front end's add_/mul_): identical indices only."""
    TF, O = mods
    rng = np.random.default_rng(5)
    a, b = make(rng, dtype, (70001,)), make(rng, dtype, (70001,))
    A, B = to_gpu(a), to_gpu(b)
    TF.add(A, B, A)
    assert_bit_exact(to_np(A), O.add(a, b), "add in place into a")
    A = to_gpu(a)
    TF.mul(A, A, A)
    assert_bit_exact(to_np(A), O.mul(a, a), "mul(a,a)->a")
    A, B = to_gpu(a), to_gpu(b)
    TF.sub(A, B, B)
    assert_bit_exact(to_np(B), O.sub(a, b), "sub in place into b")


def test_binary_unaligned_pointers(mods):
    """Views that start 4 bytes into an allocation take the scalar path and still match."""
    TF, O = mods
    rng = np.random.default_rng(6)
    a, b = make(rng, "float32", (10001,)), make(rng, "float32", (10001,))
    A, B = to_gpu(a)[1:], to_gpu(b)[1:]
    Cc = torch.empty(10001, dtype=torch.float32, device="cuda:0")[1:]
    TF.add(A, B, Cc)
    assert_bit_exact(to_np(Cc), O.add(a[1:], b[1:]), "add unaligned")


@pytest.mark.parametrize("dtype", ["float64", "float32"])
def test_pow(mods, dtype):
    TF, O = mods
    rng = np.random.default_rng(7)
    a = make(rng, dtype, (100003,), 0.1, 4.0)
    b = make(rng, dtype, (100003,), -3.0, 3.0)
    A, B = to_gpu(a), to_gpu(b)
    Cc = torch.empty_like(A)
    TF.pow(A, B, Cc)
    _close(to_np(Cc), O.pow(a, b), dtype, "pow")
    TF.powscalar(A, 2.5, Cc)
    _close(to_np(Cc), O.powscalar(a, 2.5), dtype, "powscalar")
    TF.rpowscalar(1.7, B, Cc)
    _close(to_np(Cc), O.rpowscalar(1.7, b), dtype, "rpowscalar")
    with pytest.raises(Exception):
        X = to_gpu(make(rng, "int32", (8,)))
        TF.pow(X, X, torch.empty_like(X))


def _pow_grid_check(got, want, what):
    """pow against the CPU's std::pow: the same class everywhere (NaN, ±inf, ±0), relative 1e-5 on normal results,
    and on subnormal results the same 1e-5 plus one unit of the subnormal grid (2^-149), which is all that is there."""
    assert np.array_equal(np.isnan(got), np.isnan(want)), what + ": NaN pattern"
    ok = ~np.isnan(want)
    assert np.array_equal(np.isinf(got[ok]), np.isinf(want[ok])), what + ": infinities"
    inf = np.isinf(want) & ok
    assert np.array_equal(np.signbit(got[inf]), np.signbit(want[inf])), what + ": sign of infinities"
    fin = np.isfinite(want)
    g, w = got[fin].astype(np.float64), want[fin].astype(np.float64)
    bad = np.abs(g - w) > 1e-5 * np.abs(w) + 2.0 ** -149
    assert not bad.any(), f"{what}: {int(bad.sum())} of {g.size} outside 1e-5; worst rel {np.max(np.abs(g - w) / np.maximum(np.abs(w), 1e-300))}"
    assert np.array_equal(np.signbit(got[fin]), np.signbit(want[fin])) or np.array_equal(np.signbit(g[w != 0]), np.signbit(w[w != 0])), what + ": signs"


def test_pow_float32_dense_grid(mods):
    """Every combination of a dense set of bases (subnormals, the whole normal range, values hugging 1, zero,
    negatives, inf, NaN) and exponents (fractions, integers, huge, ±inf, NaN, ±0) through pow, powscalar and
    rpowscalar: the fast path and the hand-over to the library routine must both stay within 1e-5."""
    TF, O = mods
    rng = np.random.default_rng(77)
    xs = np.concatenate([
        np.float32(2.0) ** np.arange(-149, 128, 3, dtype=np.float32),                  # powers of two, subnormals included
        np.exp(rng.uniform(-87, 88, 700)).astype(np.float32),                           # the normal range
        (1 + rng.uniform(-0.3, 0.42, 500)).astype(np.float32),                           # every mantissa region
        (1 + np.float32(2.0) ** -np.arange(1, 24, dtype=np.float32)), (1 - np.float32(2.0) ** -np.arange(1, 25, dtype=np.float32)),
        np.array([0.0, -0.0, 1.0, -1.0, -2.0, -0.5, -3.7, np.inf, -np.inf, np.nan, 1e-45, 1.1754944e-38, 3.4028235e38], dtype=np.float32),
    ]).astype(np.float32)
    ys = np.concatenate([
        rng.uniform(-4, 4, 300).astype(np.float32), rng.uniform(-200, 200, 300).astype(np.float32),
        np.arange(-12, 13, dtype=np.float32), np.float32(2.0) ** np.arange(-30, 40, 3, dtype=np.float32),
        np.array([0.0, -0.0, 0.5, -0.5, 1.0 / 3, 1e5, -1e5, 3e6, 1e30, -1e30, np.inf, -np.inf, np.nan, 1.0, 2.0, 3.0, -1.0], dtype=np.float32),
    ]).astype(np.float32)
    X, Y = np.meshgrid(xs, ys, indexing="ij")
    a, b = np.ascontiguousarray(X.ravel()), np.ascontiguousarray(Y.ravel())
    A, B = to_gpu(a), to_gpu(b)
    Cc = torch.empty_like(A)
    TF.pow(A, B, Cc)
    with np.errstate(all="ignore"):
        want = O.pow(a, b)
    _pow_grid_check(to_np(Cc), want, "pow<float32> grid")
    # the scalar tail (one element at a time) must give the very bits of the vector body
    odd = a.size - 3
    Cs = torch.empty(odd, dtype=torch.float32, device="cuda:0")
    TF.pow(A[3:], B[3:], Cs)   # starts 12 bytes into the allocation: the unaligned, element-wise kernel
    assert_bit_exact(to_np(Cs), to_np(Cc)[3:], "pow<float32>: element-wise path vs vector path")
    XA = to_gpu(xs)
    Cx = torch.empty_like(XA)
    for s in (2.5, -1.5, 0.5, 1.0 / 3, 7.0, -12.0, 100.0, 0.0):
        TF.powscalar(XA, s, Cx)
        with np.errstate(all="ignore"):
            _pow_grid_check(to_np(Cx), O.powscalar(xs, s), f"powscalar<float32>({s}) grid")
    YA = to_gpu(ys)
    Cy = torch.empty_like(YA)
    for s in (1.7, 2.0, 0.3, 10.0, 1e-30, 3e38, 1.0, 0.0, -2.0, 1e-45):
        TF.rpowscalar(s, YA, Cy)
        with np.errstate(all="ignore"):
            _pow_grid_check(to_np(Cy), O.rpowscalar(s, ys), f"rpowscalar<float32>({s}) grid")


@pytest.mark.parametrize("dtype", ["float64", "float32"])
@pytest.mark.parametrize("k", [2, 3, 1, -1])
def test_powscalar_small_integer_exponents(mods, dtype, k):
    """powscalar(x, 2|3|1|-1) runs as multiplications / one division (what x.pow(2) of a norm layer sends);
    against the CPU pow: negative, zero and huge bases included."""
    TF, O = mods
    rng = np.random.default_rng(70 + k)
    a = make(rng, dtype, (50001,), -30.0, 30.0)
    a[:6] = [0.0, -0.0, 1.0, -1.0, 1e18, -1e-18]
    A = to_gpu(a)
    Cc = torch.empty_like(A)
    TF.powscalar(A, k, Cc)
    got, want = to_np(Cc), O.powscalar(a, k)
    assert np.array_equal(np.isinf(got), np.isinf(want)) and np.array_equal(np.signbit(got), np.signbit(want))
    fin = np.isfinite(want)
    tol = 1e-12 if dtype == "float64" else 1e-5
    assert np.allclose(got[fin], want[fin], rtol=tol, atol=0.0)
    if k in (1, 2):  # x and x*x are correctly rounded: at least as close to the exact power as the CPU pow
        exact = a.astype(np.longdouble) ** k
        assert (np.abs(got[fin] - exact[fin]) <= np.abs(want[fin] - exact[fin])).all()


def test_small_integer_division_is_exact(mods):
    """int8 / int16 division goes through fp32: every int8 pair, and int16 numerators against small, large
    and extreme divisors, must give the truncated integer quotient bit for bit."""
    TF, O = mods
    a8, b8 = np.meshgrid(np.arange(-128, 128, dtype=np.int8), np.array([b for b in range(-128, 128) if b != 0], dtype=np.int8))
    a8, b8 = a8.ravel().copy(), b8.ravel().copy()
    out = torch.empty(a8.shape, dtype=torch.int8, device="cuda:0")
    TF.div(to_gpu(a8), to_gpu(b8), out)
    assert_bit_exact(to_np(out), O.div(a8, b8), "div<int8> all pairs")
    rng = np.random.default_rng(11)
    num = np.arange(-32768, 32768, dtype=np.int16)
    divisors = list(range(-300, 301)) + [-32768, -32767, 32767, 16384, -16385, 255, 257, 4097, 10923, 21845] + list(rng.integers(-32768, 32768, 200))
    for d in divisors:
        if d == 0:
            continue
        b = np.full(num.shape, d, dtype=np.int16)
        o16 = torch.empty(num.shape, dtype=torch.int16, device="cuda:0")
        TF.div(to_gpu(num), to_gpu(b), o16)
        assert_bit_exact(to_np(o16), O.div(num, b), f"div<int16> by {d}")
    for d in [7, -7, 2, -2, 3, 1, -1, 255, 10923, 32767, -32768, 30000]:
        o16 = torch.empty(num.shape, dtype=torch.int16, device="cuda:0")
        TF.divscalar(to_gpu(num), d, o16)
        assert_bit_exact(to_np(o16), O.divscalar(num, d), f"divscalar<int16> by {d}")
    n8 = np.arange(-128, 128, dtype=np.int8)
    for d in [5, -5, 2, 3, 1, -1, 127, -128, 100]:
        o8 = torch.empty(n8.shape, dtype=torch.int8, device="cuda:0")
        TF.divscalar(to_gpu(n8), d, o8)
        assert_bit_exact(to_np(o8), O.divscalar(n8, d), f"divscalar<int8> by {d}")
    nz = num[num != 0]
    o16 = torch.empty(nz.shape, dtype=torch.int16, device="cuda:0")
    TF.rdivscalar(30000, to_gpu(nz), o16)
    assert_bit_exact(to_np(o16), O.rdivscalar(30000, nz), "rdivscalar<int16>")


def test_int8_scalar_division_every_value_and_divisor(mods):
    """int8 divided by a scalar and a scalar divided by int8 run through a 256-entry table (whole tiles and the
    guarded tail of the kernel both): every value against every non-zero scalar, bit for bit."""
    TF, O = mods
    rng = np.random.default_rng(17)
    vals = np.concatenate([np.arange(-128, 128, dtype=np.int8), rng.integers(-128, 128, 20000 - 256 + 37).astype(np.int8)])
    nz = vals[vals != 0]
    A, NZ = to_gpu(vals), to_gpu(nz)
    out, outr = torch.empty_like(A), torch.empty_like(NZ)
    for d in range(-128, 128):
        if d == 0:
            continue
        TF.divscalar(A, d, out)
        assert_bit_exact(to_np(out), O.divscalar(vals, d), f"divscalar<int8> by {d}")
        TF.rdivscalar(d, NZ, outr)
        assert_bit_exact(to_np(outr), O.rdivscalar(d, nz), f"rdivscalar<int8> {d} / x")
    # in place, as the front end's div_ sends it
    B = to_gpu(vals)
    TF.divscalar(B, 7, B)
    assert_bit_exact(to_np(B), O.divscalar(vals, 7), "divscalar<int8> in place")


@pytest.mark.parametrize("dtype", ALL_NUMERIC)
@pytest.mark.parametrize("op", ["addscalar", "subscalar", "rsubscalar", "mulscalar", "divscalar", "rdivscalar",
                                "maxscalar", "minscalar"])
def test_scalar_exact(mods, op, dtype):
    TF, O = mods
    rng = np.random.default_rng(seed_of(op, dtype))
    s = 3 if dtype in INTS else 1.375
    for n in [0, 5, 4096 * 2 + 3]:
        a = make(rng, dtype, (n,), nonzero=True)
        A = to_gpu(a)
        Cc = torch.empty_like(A)
        if op.startswith("r"):
            getattr(TF, op)(s, A, Cc)
            want = getattr(O, op)(s, a)
        else:
            getattr(TF, op)(A, s, Cc)
            want = getattr(O, op)(a, s)
        assert_bit_exact(to_np(Cc), want, f"{op}<{dtype}> n={n}")


@pytest.mark.parametrize("dtype", FLOATS)
def test_sqrt_exact(mods, dtype):
    TF, O = mods
    rng = np.random.default_rng(11)
    a = make(rng, dtype, (300007,), 0.0, 1000.0)
    A = to_gpu(a)
    Cc = torch.empty_like(A)
    TF.sqrt(A, Cc)
    assert_bit_exact(to_np(Cc), O.sqrt(a), f"sqrt<{dtype}>")


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("op", ["exp", "log", "sin", "cos", "tan"])
def test_unary_math(mods, op, dtype):
    TF, O = mods
    if op == "tan" and dtype in ("float16", "bfloat16"):
        pytest.skip("tan is registered for float64/float32 only")
    rng = np.random.default_rng(12)
    lo, hi = {"exp": (-10, 10), "log": (1e-3, 1e3), "sin": (-6, 6), "cos": (-6, 6), "tan": (-1.4, 1.4)}[op]
    a = make(rng, dtype, (200003,), lo, hi)
    A = to_gpu(a)
    Cc = torch.empty_like(A)
    getattr(TF, op)(A, Cc)
    got, want = to_np(Cc), getattr(O, op)(a)
    if op in ("sin", "cos") and dtype in ("float32", "float64"):
        # near zeros of the function a relative bound is meaningless: absolute 1e-6 there
        g, w = got.astype(np.float64), want.astype(np.float64)
        assert (np.abs(g - w) <= 1e-6 + 1e-5 * np.abs(w)).all()
    else:
        _close(got, want, dtype, f"{op}<{dtype}>")


@pytest.mark.parametrize("op", ["sin", "cos"])
def test_trig_of_every_16bit_pattern(mods, op):
    """sin / cos of 16-bit floats run through the kernel's own fp32 routine: every finite float16 argument must
    give the float16 the CPU oracle gives (the C library's float routine, rounded), bit for bit; every bfloat16
    argument — huge ones, infinities and NaNs included, which take the library path — within one bfloat16 ulp
    near the function's zeros and exactly elsewhere in all but a handful of cases."""
    TF, O = mods
    h = np.arange(0, 65536, dtype=np.uint16).view(np.float16)
    h = h[np.isfinite(h)]
    out = torch.empty(h.shape, dtype=torch.float16, device="cuda:0")
    getattr(TF, op)(to_gpu(h), out)
    assert_bit_exact(to_np(out), getattr(O, op)(h), f"{op}<float16> every finite argument")
    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16).view(torch.bfloat16).cuda()
    outb = torch.empty_like(bits)
    getattr(TF, op)(bits, outb)
    x = bits.float().cpu().numpy()
    got = outb.float().cpu().numpy()
    with np.errstate(invalid="ignore"):
        exact = getattr(np, op)(x.astype(np.float64))
    fin = np.isfinite(x)
    assert np.isnan(got[~fin]).all()                      # sin(inf), sin(nan) are NaN
    err = np.abs(got[fin].astype(np.float64) - exact[fin])
    assert (err <= 2.0 ** -8 * np.abs(exact[fin]) + 1e-30).all()   # one bfloat16 ulp (half an ulp is the best possible)
    want = torch.from_numpy(exact[fin].astype(np.float32)).to(torch.bfloat16).float().numpy()
    assert (got[fin] != want).sum() <= 32                  # correctly rounded in all but a handful of cases


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_log_of_every_16bit_pattern(mods, dtype):
    """log of 16-bit floats runs through the kernel's own fp32 routine (0.71 fp32 ulp): every bit pattern — zeros,
    subnormals, negatives, infinities and NaNs included — must give the correctly rounded 16-bit result in all
    but a handful of cases and never be more than one 16-bit ulp away."""
    TF, O = mods
    tdt = TORCH_DTYPES[dtype]
    bits = torch.arange(0, 65536, dtype=torch.int32).to(torch.int16).view(tdt).cuda()
    out = torch.empty_like(bits)
    TF.log(bits, out)
    x = bits.float().cpu().numpy().astype(np.float64)
    got = out.float().cpu().numpy()
    with np.errstate(all="ignore"):
        exact = np.log(x)
    nan = np.isnan(exact)
    assert np.isnan(got[nan]).all() and not np.isnan(got[~nan]).any()
    inf = np.isinf(exact)
    assert np.array_equal(got[inf], exact[inf].astype(np.float32))          # log(0) = -inf, log(inf) = inf
    ok = ~nan & ~inf
    want = torch.from_numpy(exact[ok].astype(np.float32)).to(tdt).float().numpy()
    ulp = 2.0 ** (-10 if dtype == "float16" else -7)
    assert (np.abs(got[ok] - exact[ok]) <= ulp * np.abs(exact[ok]) + 1e-30).all()
    assert (got[ok] != want).sum() <= 16


@pytest.mark.parametrize("dtype", INTS + ["bool"])
def test_invert(mods, dtype):
    TF, O = mods
    rng = np.random.default_rng(13)
    a = make(rng, dtype, (50001,))
    A = to_gpu(a)
    Cc = torch.empty_like(A)
    TF.invert(A, Cc)
    assert_bit_exact(to_np(Cc), O.invert(a), f"invert<{dtype}>")


@pytest.mark.parametrize("dtype", ALL_NUMERIC)
@pytest.mark.parametrize("op", ["equal", "notequal", "less", "greater"])
def test_compare(mods, op, dtype):
    TF, O = mods
    rng = np.random.default_rng(seed_of(op, dtype))
    n = 4096 * 2 + 11
    a = make(rng, dtype, (n,))
    b = a.copy()
    flip = rng.random(n) < 0.5
    b[flip] = make(rng, dtype, (n,))[flip]
    A, B = to_gpu(a), to_gpu(b)
    M = torch.empty(n, dtype=torch.bool, device="cuda:0")
    s = 2 if dtype in INTS else 0.5
    if op in ("equal", "notequal"):
        for eps in (0.0, 0.75, 2.0):
            getattr(TF, op)(A, B, eps, M)
            assert_bit_exact(to_np(M), getattr(O, op)(a, b, eps), f"{op}<{dtype}> eps={eps}")
            getattr(TF, op + "scalar")(A, s, eps, M)
            assert_bit_exact(to_np(M), getattr(O, op + "scalar")(a, s, eps), f"{op}scalar<{dtype}> eps={eps}")
    else:
        getattr(TF, op)(A, B, M)
        assert_bit_exact(to_np(M), getattr(O, op)(a, b), f"{op}<{dtype}>")
        getattr(TF, op + "scalar")(A, s, M)
        assert_bit_exact(to_np(M), getattr(O, op + "scalar")(a, s), f"{op}scalar<{dtype}>")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16", "int64", "int8", "bool"])
def test_switch(mods, dtype):
    TF, O = mods
    rng = np.random.default_rng(17)
    for n in [1, 33, 4096 * 2 + 7]:
        ts = [make(rng, dtype, (n,)) for _ in range(3)]
        Ts = [to_gpu(t) for t in ts]
        out = torch.empty_like(Ts[0])
        cb = rng.integers(0, 2, n).astype(np.bool_)
        TF.Switch(Ts[:2], to_gpu(cb), out)
        assert_bit_exact(to_np(out), O.Switch(ts[:2], cb), f"switch bool<{dtype}> n={n}")
        ci = rng.integers(0, 3, n).astype(np.int32)
        TF.Switch(Ts, to_gpu(ci), out)
        assert_bit_exact(to_np(out), O.Switch(ts, ci), f"switch int32<{dtype}> n={n}")
    with pytest.raises(ValueError):
        TF.Switch(Ts, to_gpu(cb), out)  # bool cases need exactly two tensors


@pytest.mark.parametrize("src", ALL_NUMERIC)
@pytest.mark.parametrize("dst", ALL_NUMERIC)
def test_todtype(mods, src, dst):
    TF, O = mods
    rng = np.random.default_rng(19)
    a = make(rng, src, (4096 + 77,), -100.0, 100.0)
    A = to_gpu(a)
    Cc = torch.empty(a.shape, dtype=TORCH_DTYPES[dst], device="cuda:0")
    TF.todtype(A, Cc)
    assert_bit_exact(to_np(Cc), O.todtype(a, NP_DTYPES[dst]), f"todtype {src}->{dst}")


@pytest.mark.parametrize("dtype", ALL_NUMERIC + ["bool"])
def test_constant(mods, dtype):
    TF, _ = mods
    t = torch.empty(4096 * 2 + 3, dtype=TORCH_DTYPES[dtype], device="cuda:0")
    v = True if dtype == "bool" else (7 if dtype in INTS else 0.5)
    TF.constant(t, v)
    assert (to_np(t) == NP_DTYPES[dtype](v)).all()


def test_shape_and_dtype_errors(mods):
    TF, _ = mods
    a = torch.zeros(8, device="cuda:0")
    with pytest.raises(ValueError, match="shape mismatch"):
        TF.add(a, a, torch.zeros(9, device="cuda:0"))
    with pytest.raises(TypeError, match="Type mismatch"):
        TF.add(a, a, torch.zeros(8, device="cuda:0", dtype=torch.float64))
    with pytest.raises(ValueError):
        TF.add(a.cpu(), a.cpu(), a.cpu())


def test_config_add_4096x4096(mods):
    """deepxIR add on float32 [4096,4096], U(-1,1), seed 0 — element for element."""
    TF, O = mods
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (4096, 4096)).astype(np.float32)
    b = rng.uniform(-1, 1, (4096, 4096)).astype(np.float32)
    A, B = to_gpu(a), to_gpu(b)
    Cc = torch.empty_like(A)
    TF.add(A, B, Cc)
    assert_bit_exact(to_np(Cc), O.add(a, b), "add [4096,4096]")
