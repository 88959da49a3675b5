"""GPU parity: matmul through the C ABI vs the CPU oracle and a float64 reference.

Bar: bf16/f16 within 1e-2 relative (scaled by Σ|a||b| per output, fp32 accumulation, one
rounding), f32 within 1e-5, f64 within 1e-12, against a float64 GEMM of the same inputs.
"""
import numpy as np
import pytest
import torch

from helpers import NP_DTYPES, TORCH_DTYPES, make, seed_of, to_gpu, to_np

pytestmark = pytest.mark.gpu

TOL = {"float64": 1e-12, "float32": 1e-5, "float16": 2e-3, "bfloat16": 1e-2}


@pytest.fixture(scope="module")
def mods():
    from deepx_b200 import _native as N
    from deepx_b200 import tensorfunc as TF
    from oracle import oracle as O
    return TF, O, N


def check(TF, N, a, b, dtype, what):
    A, B = to_gpu(a), to_gpu(b)
    Cc = torch.empty(list(a.shape[:-1]) + [b.shape[-1]], dtype=TORCH_DTYPES[dtype], device="cuda:0")
    TF.matmul(A, B, Cc)
    N.check(N.lib.dx_matmul_status(None))
    got = to_np(Cc).astype(np.float64)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    ref = a64 @ b64
    scale = np.abs(a64) @ np.abs(b64)
    err = np.abs(got - ref)
    # one rounding of the result (relative to |ref|) + accumulation error (relative to Σ|a||b|)
    # float32 runs as three TF32 tensor-core products per product: the dropped lo·lo term and the tf32
    # truncation of the lo parts are each ~2^-21 of |a||b|, hence 2e-6 on the accumulation term
    acc_tol = {"float64": 1e-14, "float32": 2e-6}.get(dtype, 1e-6)
    bound = TOL[dtype] * np.abs(ref) + acc_tol * scale + 1e-300
    bad = err > bound
    assert not bad.any(), (f"{what}: {bad.sum()} of {bad.size} outside tolerance; max err {err.max():.3e}; "
                           f"first bad index {np.argwhere(bad)[0].tolist()} got {got[tuple(np.argwhere(bad)[0])]} "
                           f"ref {ref[tuple(np.argwhere(bad)[0])]}")
    return got


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("shape", [
    (128, 256, 64), (128, 256, 256), (256, 512, 128), (384, 768, 1024),   # whole tiles
    (100, 200, 72), (130, 264, 40), (1, 8, 8), (257, 1000, 520),          # ragged M/N/K (TMA path: N,K % 8 == 0)
    (64, 100, 30), (7, 5, 3),                                             # N or K not multiple of 8: SIMT path
])
def test_matmul_16bit(mods, shape, dtype):
    TF, O, N = mods
    M, Nn, K = shape
    rng = np.random.default_rng(seed_of("mm", shape, dtype))
    a = make(rng, dtype, (M, K), -1.0, 1.0)
    b = make(rng, dtype, (K, Nn), -1.0, 1.0)
    got = check(TF, N, a, b, dtype, f"matmul<{dtype}> {shape}")
    if M * Nn * K <= 64 * 1024 * 1024:
        want = O.matmul(a, b).astype(np.float64)
        # oracle: same fp32 accumulation + one rounding; may differ by the accumulation order only
        assert np.abs(got - want).max() <= 2 * TOL[dtype] * max(1.0, np.abs(want).max())


@pytest.fixture()
def force_pair(monkeypatch):
    """Forces the CTA-pair (cta_group::2) kernel regardless of problem size."""
    monkeypatch.setenv("DX_GEMM_CTA_PAIR", "1")
    yield
    monkeypatch.delenv("DX_GEMM_CTA_PAIR", raising=False)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("shape", [
    (256, 256, 64), (256, 256, 512), (512, 768, 128), (1024, 1024, 1024),   # whole 256×256 tiles
    (100, 200, 72), (130, 264, 40), (257, 1000, 520), (384, 520, 200), (1, 8, 8),  # ragged; second CTA partly or wholly past M
])
def test_matmul_16bit_cta_pair(mods, force_pair, shape, dtype):
    TF, O, N = mods
    M, Nn, K = shape
    rng = np.random.default_rng(seed_of("mm2", shape, dtype))
    a = make(rng, dtype, (M, K), -1.0, 1.0)
    b = make(rng, dtype, (K, Nn), -1.0, 1.0)
    check(TF, N, a, b, dtype, f"matmul pair<{dtype}> {shape}")


def test_matmul_cta_pair_identity_and_batched(mods, force_pair):
    TF, O, N = mods
    rng = np.random.default_rng(4)
    a = make(rng, "bfloat16", (512, 512), -2.0, 2.0)
    eye = np.eye(512, dtype=np.float32).astype(NP_DTYPES["bfloat16"])
    Cc = torch.empty((512, 512), dtype=torch.bfloat16, device="cuda:0")
    TF.matmul(to_gpu(a), to_gpu(eye), Cc)
    N.check(N.lib.dx_matmul_status(None))
    assert np.array_equal(to_np(Cc).view(np.uint16), a.view(np.uint16))
    a3 = make(rng, "bfloat16", (3, 300, 136), -1.0, 1.0)
    b3 = make(rng, "bfloat16", (3, 136, 264), -1.0, 1.0)
    check(TF, N, a3, b3, "bfloat16", "matmul pair batched [3,300,136]x[3,136,264]")


def test_matmul_both_forms_agree_bit_for_bit(mods, monkeypatch):
    """Same K order, same fp32 accumulation: the one-CTA and the CTA-pair kernels give identical bits."""
    TF, O, N = mods
    rng = np.random.default_rng(6)
    a = make(rng, "bfloat16", (1000, 520), -1.0, 1.0)
    b = make(rng, "bfloat16", (520, 776), -1.0, 1.0)
    A, B = to_gpu(a), to_gpu(b)
    outs = []
    for mode in ("0", "1"):
        monkeypatch.setenv("DX_GEMM_CTA_PAIR", mode)
        Cc = torch.empty((1000, 776), dtype=torch.bfloat16, device="cuda:0")
        TF.matmul(A, B, Cc)
        N.check(N.lib.dx_matmul_status(None))
        outs.append(to_np(Cc).view(np.uint16))
    monkeypatch.delenv("DX_GEMM_CTA_PAIR", raising=False)
    assert np.array_equal(outs[0], outs[1])


def test_matmul_identity_exact(mods):
    """A · I reproduces A bit for bit: exercises every (row, k) → (row, n) path of the tile."""
    TF, O, N = mods
    rng = np.random.default_rng(3)
    a = make(rng, "bfloat16", (256, 512), -2.0, 2.0)
    eye = np.eye(512, dtype=np.float32).astype(NP_DTYPES["bfloat16"])
    A, B = to_gpu(a), to_gpu(eye)
    Cc = torch.empty((256, 512), dtype=torch.bfloat16, device="cuda:0")
    TF.matmul(A, B, Cc)
    N.check(N.lib.dx_matmul_status(None))
    assert np.array_equal(to_np(Cc).view(np.uint16), a.view(np.uint16))


@pytest.mark.parametrize("dtype", ["bfloat16"])
def test_matmul_batched(mods, dtype):
    TF, O, N = mods
    rng = np.random.default_rng(5)
    a = make(rng, dtype, (2, 3, 130, 72), -1.0, 1.0)
    b = make(rng, dtype, (2, 3, 72, 264), -1.0, 1.0)
    check(TF, N, a, b, dtype, "matmul batched [2,3,130,72]x[2,3,72,264]")


@pytest.mark.parametrize("dtype", ["float32", "float64"])
def test_matmul_fp32_fp64(mods, dtype):
    TF, O, N = mods
    rng = np.random.default_rng(7)
    for M, Nn, K in [(2, 2, 3), (65, 130, 257), (256, 256, 512)]:
        a = make(rng, dtype, (M, K), -1.0, 1.0)
        b = make(rng, dtype, (K, Nn), -1.0, 1.0)
        check(TF, N, a, b, dtype, f"matmul<{dtype}> {(M, Nn, K)}")
    a = make(rng, dtype, (2, 3, 4, 5), -1.0, 1.0)
    b = make(rng, dtype, (2, 3, 5, 6), -1.0, 1.0)
    check(TF, N, a, b, dtype, "batched [2,3,4,5]x[2,3,5,6]")  # shapes of executor/op-cuda/test/tensorfunc/1_cublas_matmul.cpp:36-62


@pytest.mark.parametrize("shape", [(128, 128, 32), (256, 384, 96), (1000, 520, 264), (130, 36, 8), (2048, 1024, 512)])
def test_matmul_fp32_tensor_core_path(mods, shape):
    """float32 with K and N multiples of 4 takes the TF32x3 tcgen05 kernel; result within 1e-5."""
    TF, O, N = mods
    M, Nn, K = shape
    rng = np.random.default_rng(seed_of("mm32", shape))
    a = make(rng, "float32", (M, K), -1.0, 1.0)
    b = make(rng, "float32", (K, Nn), -1.0, 1.0)
    got = check(TF, N, a, b, "float32", f"matmul<float32 tf32x3> {shape}")
    ref = a.astype(np.float64) @ b.astype(np.float64)
    rel = np.abs(got - ref).max() / np.abs(ref).max()
    assert rel <= 1e-5, rel
    a3 = make(rng, "float32", (3, 200, 64), -1.0, 1.0)
    b3 = make(rng, "float32", (3, 64, 132), -1.0, 1.0)
    check(TF, N, a3, b3, "float32", "matmul<float32 tf32x3> batched")


@pytest.mark.parametrize("shape", [(256, 256, 32), (512, 768, 128), (1024, 1024, 1024), (100, 200, 72), (130, 264, 40),
                                   (257, 1000, 520), (384, 516, 200), (1, 8, 8)])
def test_matmul_fp32_cta_pair(mods, force_pair, shape):
    """The float32 CTA-pair kernel (256 x 256 tile per SM pair), forced on shapes of every raggedness."""
    TF, O, N = mods
    M, Nn, K = shape
    rng = np.random.default_rng(seed_of("mm32pair", shape))
    a = make(rng, "float32", (M, K), -1.0, 1.0)
    b = make(rng, "float32", (K, Nn), -1.0, 1.0)
    got = check(TF, N, a, b, "float32", f"matmul pair<float32 tf32x3> {shape}")
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-5
    a3 = make(rng, "float32", (3, 300, 136), -1.0, 1.0)
    b3 = make(rng, "float32", (3, 136, 264), -1.0, 1.0)
    check(TF, N, a3, b3, "float32", "matmul pair<float32 tf32x3> batched")


def test_matmul_fp32_both_forms_agree_bit_for_bit(mods, monkeypatch):
    """Same products in the same K order into fp32 accumulators: one-CTA and pair kernels give identical bits."""
    TF, O, N = mods
    rng = np.random.default_rng(9)
    a = make(rng, "float32", (1000, 520), -1.0, 1.0)
    b = make(rng, "float32", (520, 776), -1.0, 1.0)
    A, B = to_gpu(a), to_gpu(b)
    outs = []
    for mode in ("0", "1"):
        monkeypatch.setenv("DX_GEMM_CTA_PAIR", mode)
        Cc = torch.empty((1000, 776), dtype=torch.float32, device="cuda:0")
        TF.matmul(A, B, Cc)
        N.check(N.lib.dx_matmul_status(None))
        outs.append(to_np(Cc).view(np.uint32))
    monkeypatch.delenv("DX_GEMM_CTA_PAIR", raising=False)
    assert np.array_equal(outs[0], outs[1])


def test_matmul_fp32_simt_path_is_tighter(mods, monkeypatch):
    """The FMA kernel (shapes TMA cannot take, or DX_GEMM_F32_SIMT=1) accumulates in plain fp32."""
    TF, O, N = mods
    monkeypatch.setenv("DX_GEMM_F32_SIMT", "1")
    rng = np.random.default_rng(8)
    a = make(rng, "float32", (300, 256), -1.0, 1.0)
    b = make(rng, "float32", (256, 200), -1.0, 1.0)
    A, B = to_gpu(a), to_gpu(b)
    Cc = torch.empty((300, 200), dtype=torch.float32, device="cuda:0")
    TF.matmul(A, B, Cc)
    monkeypatch.delenv("DX_GEMM_F32_SIMT", raising=False)
    got = to_np(Cc).astype(np.float64)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    # sequential fp32 accumulation over K = 256: well inside K * 2^-24 of sum |a||b|
    assert (np.abs(got - a64 @ b64) <= 4e-6 * (np.abs(a64) @ np.abs(b64))).all()


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 16])
def test_matmul_few_rows_streaming_kernel(mods, dtype, m, monkeypatch):
    """Few rows (a decoding step): the weight-streaming kernel, forced here for every M <= 16 — K slices
    across a cluster, every N and K raggedness, batches; same tolerances as the tile kernels."""
    TF, O, N = mods
    monkeypatch.setenv("DX_GEMM_SKINNY_ROWS", "16")
    rng = np.random.default_rng(seed_of("skinny", dtype, m))
    for Nn, K in [(8, 8), (264, 100), (4104, 4096), (1000, 5000), (16384, 72), (256, 20000)]:
        a = make(rng, dtype, (m, K), -1.0, 1.0)
        b = make(rng, dtype, (K, Nn), -1.0, 1.0)
        check(TF, N, a, b, dtype, f"matmul skinny<{dtype}> {(m, Nn, K)}")
    a3 = make(rng, dtype, (3, m, 520), -1.0, 1.0)
    b3 = make(rng, dtype, (3, 520, 136), -1.0, 1.0)
    check(TF, N, a3, b3, dtype, f"matmul skinny<{dtype}> batched")


def test_matmul_few_rows_is_deterministic_and_matches_the_tile_kernel(mods, monkeypatch):
    TF, O, N = mods
    rng = np.random.default_rng(12)
    a = make(rng, "bfloat16", (4, 4096), -1.0, 1.0)
    b = make(rng, "bfloat16", (4096, 4096), -1.0, 1.0)
    A, B = to_gpu(a), to_gpu(b)
    outs = []
    for _ in range(3):
        Cc = torch.empty((4, 4096), dtype=torch.bfloat16, device="cuda:0")
        TF.matmul(A, B, Cc)
        outs.append(to_np(Cc).view(np.uint16).copy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    ref = a.astype(np.float64) @ b.astype(np.float64)
    got = to_np(Cc).astype(np.float64)
    assert np.abs(got - ref).max() <= 1e-2 * np.abs(ref).max()


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("m", [3, 16, 17, 64, 100, 128])
def test_matmul_one_tile_row_split_k(mods, dtype, m):
    """Up to 128 rows and few columns of tiles: the split-K cluster kernel (128 x 64 tiles, K divided over the
    CTAs of a cluster, partials combined through distributed shared memory)."""
    TF, O, N = mods
    rng = np.random.default_rng(seed_of("splitk", dtype, m))
    for Nn, K in [(8, 512), (264, 520), (4096, 4096), (4104, 1000), (1000, 11008), (64, 8192), (11008, 4096)]:
        a = make(rng, dtype, (m, K), -1.0, 1.0)
        b = make(rng, dtype, (K, Nn), -1.0, 1.0)
        check(TF, N, a, b, dtype, f"matmul split-K<{dtype}> {(m, Nn, K)}")
    a3 = make(rng, dtype, (3, m, 1032), -1.0, 1.0)
    b3 = make(rng, dtype, (3, 1032, 136), -1.0, 1.0)
    check(TF, N, a3, b3, dtype, f"matmul split-K<{dtype}> batched")


def test_matmul_split_k_is_deterministic(mods):
    TF, O, N = mods
    rng = np.random.default_rng(13)
    a = make(rng, "bfloat16", (32, 4096), -1.0, 1.0)
    b = make(rng, "bfloat16", (4096, 4096), -1.0, 1.0)
    A, B = to_gpu(a), to_gpu(b)
    outs = []
    for _ in range(3):
        Cc = torch.empty((32, 4096), dtype=torch.bfloat16, device="cuda:0")
        TF.matmul(A, B, Cc)
        N.check(N.lib.dx_matmul_status(None))
        outs.append(to_np(Cc).view(np.uint16).copy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])


@pytest.mark.parametrize("slices", ["auto", "2", "4"])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("m", [129, 256, 300, 512, 700])
def test_matmul_few_tile_rows_pair_split_k(mods, monkeypatch, dtype, m, slices):
    """Two to four rows of 256 x 256 tiles and a long K: the cluster kernel that splits K over CTA pairs
    (partials combined through distributed shared memory); ragged M, N and K, last K slice short.  By itself the
    kernel is chosen only for very long K; 2 and 4 slices are also forced on every shape that fits."""
    TF, O, N = mods
    if slices != "auto":
        monkeypatch.setenv("DX_GEMM_PAIR_SPLITK", slices)
    rng = np.random.default_rng(seed_of("pairsplitk", dtype, m))
    for Nn, K in [(256, 1024), (520, 2056), (4096, 4096), (1000, 1032), (264, 8192)]:
        a = make(rng, dtype, (m, K), -1.0, 1.0)
        b = make(rng, dtype, (K, Nn), -1.0, 1.0)
        check(TF, N, a, b, dtype, f"matmul pair split-K<{dtype}> {(m, Nn, K)}")
    a3 = make(rng, dtype, (2, m, 2048), -1.0, 1.0)
    b3 = make(rng, dtype, (2, 2048, 264), -1.0, 1.0)
    check(TF, N, a3, b3, dtype, f"matmul pair split-K<{dtype}> batched")


def test_matmul_pair_split_k_is_deterministic_and_close_to_the_tile_kernel(mods, monkeypatch):
    TF, O, N = mods
    monkeypatch.setenv("DX_GEMM_PAIR_SPLITK", "2")
    rng = np.random.default_rng(14)
    a = make(rng, "bfloat16", (512, 4096), -1.0, 1.0)
    b = make(rng, "bfloat16", (4096, 2048), -1.0, 1.0)
    A, B = to_gpu(a), to_gpu(b)
    outs = []
    for _ in range(3):
        Cc = torch.empty((512, 2048), dtype=torch.bfloat16, device="cuda:0")
        TF.matmul(A, B, Cc)
        N.check(N.lib.dx_matmul_status(None))
        outs.append(to_np(Cc).view(np.uint16).copy())
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[0], outs[2])
    # against the unsplit kernel: the K slices are added in a different order, so one 16-bit rounding apart at most
    ref = (a.astype(np.float64) @ b.astype(np.float64))
    got = to_np(Cc).astype(np.float64)
    assert np.abs(got - ref).max() <= 1e-2 * np.abs(ref).max()


@pytest.mark.parametrize("force", ["0", "1"])
def test_matmul_output_not_16_byte_aligned(mods, monkeypatch, force):
    """C starting 2 bytes past a 16-byte boundary: the tile kernels store each lane's own row with scalar stores
    instead of turning blocks round for 16-byte stores; same bits as the aligned result."""
    TF, O, N = mods
    monkeypatch.setenv("DX_GEMM_CTA_PAIR", force)
    rng = np.random.default_rng(21)
    a = make(rng, "bfloat16", (300, 520), -1.0, 1.0)
    b = make(rng, "bfloat16", (520, 264), -1.0, 1.0)
    A, B = to_gpu(a), to_gpu(b)
    aligned = torch.empty((300, 264), dtype=torch.bfloat16, device="cuda:0")
    TF.matmul(A, B, aligned)
    buf = torch.zeros(300 * 264 + 8, dtype=torch.bfloat16, device="cuda:0")
    off = buf[1:1 + 300 * 264].view(300, 264)
    assert off.data_ptr() % 16 == 2
    TF.matmul(A, B, off)
    N.check(N.lib.dx_matmul_status(None))
    assert np.array_equal(to_np(off).view(np.uint16), to_np(aligned).view(np.uint16))
    assert float(buf[0]) == 0.0 and float(buf[1 + 300 * 264:].abs().sum()) == 0.0  # nothing written outside C


def test_matmul_golden_arange(mods):
    """arange [2,3,4] x [2,4,5]: the worked example in executor/op-ompsimd/test/tensorfunc/4_tensor_matmul.cpp:22-35."""
    TF, O, N = mods
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    b = np.arange(40, dtype=np.float32).reshape(2, 4, 5)
    A, B = to_gpu(a), to_gpu(b)
    Cc = torch.empty((2, 3, 5), dtype=torch.float32, device="cuda:0")
    TF.matmul(A, B, Cc)
    assert np.array_equal(to_np(Cc), a @ b)  # small integers: exact in fp32
    assert np.array_equal(O.matmul(a, b), a @ b)


def test_matmul_shape_errors(mods):
    TF, O, N = mods
    a = torch.zeros(4, 5, device="cuda:0")
    with pytest.raises(ValueError):
        TF.matmul(a, torch.zeros(6, 7, device="cuda:0"), torch.zeros(4, 7, device="cuda:0"))
    with pytest.raises(Exception):
        i = torch.zeros(4, 4, dtype=torch.int32, device="cuda:0")
        TF.matmul(i, i, i.clone())


def test_config_matmul_bf16_8192x4096x4096(mods):
    """bf16 A[8192,4096] × B[4096,4096] ~ N(0,0.02), fp32 accumulate, bf16 out: sampled rows
    against float64, plus the size-independent identity (A·B)·1 = A·(B·1)."""
    TF, O, N = mods
    rng = np.random.default_rng(0)
    a = (rng.standard_normal((8192, 4096), dtype=np.float32) * np.float32(0.02)).astype(NP_DTYPES["bfloat16"])
    b = (rng.standard_normal((4096, 4096), dtype=np.float32) * np.float32(0.02)).astype(NP_DTYPES["bfloat16"])
    A, B = to_gpu(a), to_gpu(b)
    Cc = torch.empty((8192, 4096), dtype=torch.bfloat16, device="cuda:0")
    TF.matmul(A, B, Cc)
    N.check(N.lib.dx_matmul_status(None))
    got = to_np(Cc).astype(np.float64)
    rows = np.concatenate([np.arange(0, 8192, 517), [127, 128, 8191]])
    a64, b64 = a[rows].astype(np.float64), b.astype(np.float64)
    ref = a64 @ b64
    scale = np.abs(a64) @ np.abs(b64)
    err = np.abs(got[rows] - ref)
    assert (err <= 1e-2 * np.abs(ref) + 1e-6 * scale).all(), f"max err {err.max()}"
    lhs = got.sum(axis=1)
    rhs = a.astype(np.float64) @ b.astype(np.float64).sum(axis=1)
    # each of the 4096 outputs in a row carries ≤ 2^-9 relative rounding of |c|
    assert (np.abs(lhs - rhs) <= 2.0 ** -8 * np.abs(got).sum(axis=1) + 1e-9).all()


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("shape", [
    (1, 768, 2048, 8192), (1, 512, 4096, 8192), (1, 256, 1024, 16384),                           # few rows of tiles, long K
    (1, 300, 520, 8008), (1, 257, 264, 4096), (3, 260, 264, 4096), (1, 129, 8, 4096),            # ragged rows, columns, last K slice; batch
])
def test_matmul_16bit_k_split_through_workspace(mods, shape, dtype):
    """A few rows of 256 x 256 tiles: dx_matmul_ws splits each tile's K range over independent CTA pairs whose fp32
    partials meet in the caller's workspace; every pair finishes its share of the tile's columns, adding in slice
    order.  Against the float64 product; the same bits on every run (the arrival order must not show); the same answer
    from dx_matmul, which has no workspace, within the bound; and the counters the pairs meet on serve the next call,
    whatever its number of slices (the shapes of this list follow one another in one process)."""
    TF, O, N = mods
    batch, M, Nn, K = shape
    code = {"bfloat16": N.BF16, "float16": N.F16}[dtype]
    need = int(N.lib.dx_matmul_workspace_bytes(code, batch, M, Nn, K))
    assert need > 0, "this shape is meant to take the workspace path on this device"
    rng = np.random.default_rng(seed_of("mmws", shape, dtype))
    a = make(rng, dtype, (batch, M, K) if batch > 1 else (M, K), -1.0, 1.0)
    b = make(rng, dtype, (batch, K, Nn) if batch > 1 else (K, Nn), -1.0, 1.0)
    first = check(TF, N, a, b, dtype, f"matmul<{dtype}> {shape} (workspace)")       # tensorfunc.matmul passes a workspace
    again = check(TF, N, a, b, dtype, f"matmul<{dtype}> {shape} (workspace, second call)")
    assert np.array_equal(first, again), "two runs of the K-split kernel differ: the order of arrival shows in the result"
    A, B = to_gpu(a), to_gpu(b)
    plain = torch.empty(first.shape, dtype=TORCH_DTYPES[dtype], device="cuda:0")
    N.check(N.lib.dx_matmul(code, A.data_ptr(), B.data_ptr(), plain.data_ptr(), batch, M, Nn, K, None))   # no workspace: the other kernels
    small = torch.empty(1024, dtype=torch.uint8, device="cuda:0")
    short = torch.empty_like(plain)
    N.check(N.lib.dx_matmul_ws(code, A.data_ptr(), B.data_ptr(), short.data_ptr(), batch, M, Nn, K, small.data_ptr(), small.numel(), None))
    N.check(N.lib.dx_matmul_status(None))
    assert torch.equal(plain, short), "too small a workspace must fall back to what dx_matmul does"
    ref = a.astype(np.float64) @ b.astype(np.float64)
    scale = np.abs(a.astype(np.float64)) @ np.abs(b.astype(np.float64))
    assert (np.abs(to_np(plain).astype(np.float64) - ref) <= TOL[dtype] * np.abs(ref) + 1e-6 * scale + 1e-300).all()
    # an unrelated shape that takes the persistent kernels still works afterwards
    check(TF, N, make(rng, dtype, (384, 512), -1.0, 1.0), make(rng, dtype, (512, 2048), -1.0, 1.0), dtype, "after the K-split kernel")


def test_matmul_k_split_on_two_streams_at_once(mods):
    """Launches of the K-split kernel on different streams may overlap: each stream has its own workspace (the caller's)
    and its own set of counters (the library's), so both give the bits a launch alone gives."""
    TF, O, N = mods
    shapes = [(256, 1024, 8192), (300, 520, 8008)]
    rng = np.random.default_rng(77)
    jobs = []
    for M, Nn, K in shapes:
        assert int(N.lib.dx_matmul_workspace_bytes(N.BF16, 1, M, Nn, K)) > 0
        a, b = make(rng, "bfloat16", (M, K), -1.0, 1.0), make(rng, "bfloat16", (K, Nn), -1.0, 1.0)
        A, B = to_gpu(a), to_gpu(b)
        alone = torch.empty(M, Nn, dtype=torch.bfloat16, device="cuda:0")
        ws = torch.empty(int(N.lib.dx_matmul_workspace_bytes(N.BF16, 1, M, Nn, K)), dtype=torch.uint8, device="cuda:0")
        N.check(N.lib.dx_matmul_ws(N.BF16, A.data_ptr(), B.data_ptr(), alone.data_ptr(), 1, M, Nn, K, ws.data_ptr(), ws.numel(), None))
        jobs.append((A, B, alone, ws, torch.cuda.Stream(), [torch.empty_like(alone) for _ in range(8)], (M, Nn, K)))
    torch.cuda.synchronize()
    for i in range(8):
        for A, B, alone, ws, st, outs, (M, Nn, K) in jobs:
            N.check(N.lib.dx_matmul_ws(N.BF16, A.data_ptr(), B.data_ptr(), outs[i].data_ptr(), 1, M, Nn, K, ws.data_ptr(), ws.numel(), st.cuda_stream))
    torch.cuda.synchronize()
    N.check(N.lib.dx_matmul_status(None))
    for A, B, alone, ws, st, outs, shape in jobs:
        for o in outs:
            assert torch.equal(o, alone), f"{shape}: a launch that overlapped another stream's differs from a launch alone"


def test_matmul_k_split_more_streams_than_counter_banks(mods):
    """The library keeps eight banks of K-split counters per device; a stream that finds none left gets the kernels
    without a K split.  Twelve streams, each with its own workspace: every result within the bound of the float64
    product, whichever kernel the stream got."""
    TF, O, N = mods
    M, Nn, K = 256, 1024, 8192
    need = int(N.lib.dx_matmul_workspace_bytes(N.BF16, 1, M, Nn, K))
    assert need > 0
    rng = np.random.default_rng(78)
    a, b = make(rng, "bfloat16", (M, K), -1.0, 1.0), make(rng, "bfloat16", (K, Nn), -1.0, 1.0)
    A, B = to_gpu(a), to_gpu(b)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    scale = np.abs(a.astype(np.float64)) @ np.abs(b.astype(np.float64))
    jobs = [(torch.cuda.Stream(), torch.empty(need, dtype=torch.uint8, device="cuda:0"), torch.empty(M, Nn, dtype=torch.bfloat16, device="cuda:0"))
            for _ in range(12)]
    torch.cuda.synchronize()
    for _ in range(2):
        for st, ws, out in jobs:
            N.check(N.lib.dx_matmul_ws(N.BF16, A.data_ptr(), B.data_ptr(), out.data_ptr(), 1, M, Nn, K, ws.data_ptr(), ws.numel(), st.cuda_stream))
    torch.cuda.synchronize()
    N.check(N.lib.dx_matmul_status(None))
    for i, (st, ws, out) in enumerate(jobs):
        got = to_np(out).astype(np.float64)
        assert (np.abs(got - ref) <= TOL["bfloat16"] * np.abs(ref) + 1e-6 * scale + 1e-300).all(), f"stream {i}"
