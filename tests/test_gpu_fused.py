"""GPU parity of the row-fused RMSNorm / softmax kernels.

Two checkers per case:
  * the CPU oracle running the op-by-op chain the front end sends
    (front/py/deepx/nn/modules/norm/t5layernorm.py:19-23, nn/functional/normalization.py:4-18);
  * the same chain run as single ops on the GPU through the C ABI.
The fused kernel applies the same arithmetic per step, so it may differ from either only by the
order of the additions in the row sum: 1e-5 relative for fp32, 1e-12 for fp64, 1e-2 for 16-bit
floats (one rounding step of the dtype on top of the sum tolerance).
"""
import numpy as np
import pytest
import torch

from helpers import FLOATS, NP_DTYPES, make, seed_of, to_gpu, to_np

pytestmark = pytest.mark.gpu

WIDE = ("float64", "float32")  # 16-bit chains round after every step: judged against the chain, not float64
TOL = {"float64": 1e-12, "float32": 1e-5, "float16": 1e-2, "bfloat16": 1e-2}

# rows x cols: one warp per row (8, 896, 1024), CTA per row (4096, 8192), 1024 threads (32768),
# rows too long for registers (40000), ragged / unaligned rows (7, 1001), a single column.
SHAPES = [(6, 8), (33, 896), (5, 1024), (9, 4096), (3, 8192), (2, 32768), (2, 40000), (11, 7), (4, 1001), (5, 1), (2, 3, 64)]


@pytest.fixture(scope="module")
def mods():
    from deepx_b200 import tensorfunc as TF
    from oracle import oracle as O
    return TF, O


def oracle_rmsnorm(O, x, w, divisor, eps, square):
    last = x.ndim - 1
    sq = O.powscalar(x, 2) if square == "powscalar" else O.mul(x, x)
    v = O.sum(sq, [last], True)
    v = O.divscalar(v, divisor)
    v = O.addscalar(v, eps)
    v = O.sqrt(v)
    v = O.rdivscalar(1, v)
    y = O.mul(x, O.broadcastTo(v, x.shape))
    if w is None:
        return y
    return O.mul(O.broadcastTo(w.reshape((1,) * last + (x.shape[-1],)), x.shape), y)


def gpu_chain_rmsnorm(TF, X, W, divisor, eps):
    last = X.dim() - 1
    sq = torch.empty_like(X)
    TF.mul(X, X, sq)
    v = torch.empty(X.shape[:-1] + (1,), dtype=X.dtype, device=X.device)
    TF.sum(sq, [last], True, v)
    TF.divscalar(v, divisor, v)
    TF.addscalar(v, eps, v)
    TF.sqrt(v, v)
    TF.rdivscalar(1, v, v)
    vb = torch.empty_like(X)
    TF.broadcastTo(v, list(X.shape), vb)
    y = torch.empty_like(X)
    TF.mul(X, vb, y)
    if W is None:
        return y
    wb = torch.empty_like(X)
    TF.broadcastTo(W.reshape((1,) * last + (X.shape[-1],)).contiguous(), list(X.shape), wb)
    out = torch.empty_like(X)
    TF.mul(wb, y, out)
    return out


def oracle_softmax(O, x):
    last = x.ndim - 1
    m = O.reducemax(x, [last], True)
    d = O.sub(x, O.broadcastTo(m, x.shape))
    e = O.exp(d)
    s = O.sum(e, [last], True)
    return O.div(e, O.broadcastTo(s, x.shape))


def gpu_chain_softmax(TF, X):
    last = X.dim() - 1
    m = torch.empty(X.shape[:-1] + (1,), dtype=X.dtype, device=X.device)
    TF.reducemax(X, [last], True, m)
    mb = torch.empty_like(X)
    TF.broadcastTo(m, list(X.shape), mb)
    d = torch.empty_like(X)
    TF.sub(X, mb, d)
    e = torch.empty_like(X)
    TF.exp(d, e)
    s = torch.empty_like(m)
    TF.sum(e, [last], True, s)
    sb = torch.empty_like(X)
    TF.broadcastTo(s, list(X.shape), sb)
    out = torch.empty_like(X)
    TF.div(e, sb, out)
    return out


def ref_rmsnorm(x, w, divisor, eps):
    x64 = x.astype(np.float64)
    y = x64 / np.sqrt((x64 * x64).sum(-1, keepdims=True) / divisor + float(np.float32(eps)))
    return y if w is None else y * w.astype(np.float64)


def ref_softmax(x):
    x64 = x.astype(np.float64)
    e = np.exp(x64 - x64.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def close(got, want, tol, what):
    g, w = got.astype(np.float64), want.astype(np.float64)
    err = np.abs(g - w)
    bound = tol * np.maximum(np.abs(w), np.abs(w).max() * 1e-3) + 1e-300
    assert (err <= bound).all(), f"{what}: max rel err {np.max(err / bound) * tol}"


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("shape", SHAPES)
def test_rmsnorm_matches_the_chain(mods, dtype, shape):
    TF, O = mods
    rng = np.random.default_rng(seed_of("rms", dtype, shape))
    x = make(rng, dtype, shape, -2.0, 2.0)
    w = make(rng, dtype, (shape[-1],), 0.5, 1.5)
    divisor, eps = float(shape[-1]), 1e-6
    X, W = to_gpu(x), to_gpu(w)
    out = torch.empty_like(X)
    TF.rmsnorm(X, W, divisor, eps, out)
    got = to_np(out)
    ref = ref_rmsnorm(x, w, divisor, eps)
    if dtype in WIDE:
        close(got, ref, TOL[dtype], f"rmsnorm<{dtype}> {shape} vs float64")
        close(oracle_rmsnorm(O, x, w, divisor, eps, "mul"), ref, 10 * TOL[dtype], f"oracle chain rmsnorm<{dtype}> {shape} vs float64")
    else:
        close(got, oracle_rmsnorm(O, x, w, divisor, eps, "mul"), TOL[dtype], f"rmsnorm<{dtype}> {shape} vs oracle chain")
    close(got, to_np(gpu_chain_rmsnorm(TF, X, W, divisor, eps)), TOL[dtype], f"rmsnorm<{dtype}> {shape} vs GPU chain")
    # without the weight multiply
    TF.rmsnorm(X, None, divisor, eps, out)
    if dtype in WIDE:
        close(to_np(out), ref_rmsnorm(x, None, divisor, eps), TOL[dtype], f"rmsnorm<{dtype}> {shape} no weight")
    close(to_np(out), oracle_rmsnorm(O, x, None, divisor, eps, "mul"), 10 * TOL[dtype], f"rmsnorm<{dtype}> {shape} no weight vs oracle chain")


def test_rmsnorm_powscalar_form_and_in_place(mods):
    """The front end squares with powscalar(x, 2); the fused kernel multiplies.  Same result within the
    sum tolerance.  And the output may be the input."""
    TF, O = mods
    rng = np.random.default_rng(5)
    x = make(rng, "float32", (64, 896), -3.0, 3.0)
    w = make(rng, "float32", (896,), 0.5, 1.5)
    X, W = to_gpu(x), to_gpu(w)
    TF.rmsnorm(X, W, 896.0, 1e-6, X)
    close(to_np(X), oracle_rmsnorm(O, x, w, 896.0, 1e-6, "powscalar"), 1e-5, "rmsnorm in place vs powscalar chain")


def test_rmsnorm_fp32_rows_agree_with_float64(mods):
    TF, O = mods
    rng = np.random.default_rng(6)
    x = make(rng, "float32", (16, 2048, 896)[1:], -1.0, 1.0)
    w = make(rng, "float32", (896,), 0.9, 1.1)
    X, W = to_gpu(x), to_gpu(w)
    out = torch.empty_like(X)
    TF.rmsnorm(X, W, 896.0, 1e-6, out)
    x64 = x.astype(np.float64)
    ref = w.astype(np.float64) * (x64 / np.sqrt((x64 * x64).sum(-1, keepdims=True) / 896.0 + 1e-6))
    close(to_np(out), ref, 1e-5, "rmsnorm vs float64")


@pytest.mark.parametrize("dtype", FLOATS)
@pytest.mark.parametrize("shape", SHAPES)
def test_softmax_matches_the_chain(mods, dtype, shape):
    TF, O = mods
    rng = np.random.default_rng(seed_of("softmax", dtype, shape))
    x = make(rng, dtype, shape, -6.0, 6.0)
    X = to_gpu(x)
    out = torch.empty_like(X)
    TF.softmax(X, out)
    got = to_np(out)
    ref = ref_softmax(x)
    if dtype in WIDE:
        close(got, ref, TOL[dtype], f"softmax<{dtype}> {shape} vs float64")
        close(oracle_softmax(O, x), ref, 10 * TOL[dtype], f"oracle chain softmax<{dtype}> {shape} vs float64")
        close(got, oracle_softmax(O, x), 10 * TOL[dtype], f"softmax<{dtype}> {shape} vs oracle chain")
    else:
        close(got, oracle_softmax(O, x), TOL[dtype], f"softmax<{dtype}> {shape} vs oracle chain")
    close(got, to_np(gpu_chain_softmax(TF, X)), TOL[dtype], f"softmax<{dtype}> {shape} vs GPU chain")
    sums = got.astype(np.float64).sum(-1)
    assert np.abs(sums - 1.0).max() <= (2e-2 if dtype in ("float16", "bfloat16") else 1e-5)


def test_softmax_in_place_and_large_values(mods):
    """Subtracting the row maximum keeps exp in range for inputs near the fp32 limit."""
    TF, O = mods
    x = np.array([[1e30, 1e30, -1e30, 0.0] * 64, [88.0, 89.0, -90.0, 87.5] * 64], dtype=np.float32)
    X = to_gpu(x)
    TF.softmax(X, X)
    got = to_np(X)
    assert np.isfinite(got).all()
    close(got, oracle_softmax(O, x), 1e-5, "softmax large values")


def test_fused_rejects_bad_arguments(mods):
    TF, O = mods
    from deepx_b200 import _native as N
    x = torch.zeros(4, 8, dtype=torch.int32, device="cuda:0")
    with pytest.raises(N.DxError):
        TF.softmax(x, torch.empty_like(x))
    with pytest.raises(N.DxError):
        TF.rmsnorm(x, None, 8.0, 1e-6, torch.empty_like(x))
    f = torch.zeros(4, 8, device="cuda:0")
    with pytest.raises(ValueError):
        TF.rmsnorm(f, torch.zeros(7, device="cuda:0"), 8.0, 1e-6, torch.empty_like(f))
    e = torch.zeros(0, 8, device="cuda:0")
    TF.softmax(e, torch.empty_like(e))  # empty: nothing to do, no error
