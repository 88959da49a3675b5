"""dx_reduce_noalloc: the reduce entry point for callers that cannot allocate device memory
(a host whose memory budget lives in a pre-sized pool, code running inside another allocator's
callback, a service that bans cudaMalloc after start-up).  It must give exactly what dx_reduce
gives, call after call, although every call shares one scratch array that is never cleared.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  Passes alone in a fresh process and after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import assert_bit_exact, to_gpu, to_np

pytestmark = pytest.mark.gpu


def _both(N, op, A, dims, out_elems):
    """(dx_reduce with a caller workspace, dx_reduce_noalloc) on the same input."""
    shape = N.i64_array(A.shape)
    cd = N.i32_array(dims)
    code = {torch.float32: N.F32, torch.int32: N.I32}[A.dtype]
    need = N.lib.dx_reduce_workspace_bytes(op, code, shape, A.dim(), cd, len(dims))
    ws = torch.empty(max(int(need), 256), dtype=torch.uint8, device=A.device)
    ref = torch.empty(out_elems, dtype=A.dtype, device=A.device)
    got = torch.full((out_elems,), 7, dtype=A.dtype, device=A.device)
    N.check(N.lib.dx_reduce(op, code, A.data_ptr(), shape, A.dim(), cd, len(dims), ref.data_ptr(), ws.data_ptr(), ws.numel(), None))
    N.check(N.lib.dx_reduce_noalloc(op, code, A.data_ptr(), shape, A.dim(), cd, len(dims), got.data_ptr(), None))
    torch.cuda.synchronize()
    return need, to_np(ref), to_np(got)


def test_noalloc_matches_dx_reduce_on_consecutive_calls():
    from deepx_b200 import _native as N
    rng = np.random.default_rng(123)
    # call 1: few outputs, long rows -> several blocks per output, partials in the scratch
    a = to_gpu(rng.standard_normal((3, 1 << 20), dtype=np.float32))
    need, ref, got = _both(N, N.SUM, a, [1], 3)
    assert need > 0, "this case is meant to exercise the scratch"
    assert_bit_exact(got, ref, "noalloc sum rows, call 1")
    # call 2, straight after, other shape/op/dtype: what call 1 left in the scratch must not leak in
    b = to_gpu(rng.integers(-100, 101, (4096, 2048)).astype(np.int32))
    need, ref, got = _both(N, N.RMAX, b, [0], 2048)
    assert need > 0
    assert_bit_exact(got, ref, "noalloc max cols, call 2")
    # call 3: same as call 1 again -> same bits as before
    need, ref2, got2 = _both(N, N.SUM, a, [1], 3)
    assert_bit_exact(got2, ref2, "noalloc sum rows, call 3")
    # and a shape that needs no scratch at all still works
    c = to_gpu(rng.standard_normal((5000, 64), dtype=np.float32))
    need, ref, got = _both(N, N.SUM, c, [1], 5000)
    assert_bit_exact(got, ref, "noalloc sum, no scratch needed")


def test_noalloc_rejects_shapes_beyond_its_scratch():
    from deepx_b200 import _native as N
    # 151424 = 1183 column strips of 128 floats: too few strips to fill the GPU, so the rows are split
    # in two and the partials (2 x 151424 x 4 bytes) exceed the 1 MiB built-in scratch.
    a = torch.zeros((1024, 151424), dtype=torch.float32, device="cuda:0")
    shape, cd = N.i64_array(a.shape), N.i32_array([0])
    need = N.lib.dx_reduce_workspace_bytes(N.SUM, N.F32, shape, 2, cd, 1)
    if need <= (1 << 20):
        pytest.skip(f"this device's plan needs only {need} bytes here")
    out = torch.empty(151424, dtype=torch.float32, device="cuda:0")
    rc = N.lib.dx_reduce_noalloc(N.SUM, N.F32, a.data_ptr(), shape, 2, cd, 1, out.data_ptr(), None)
    assert rc == N.E_WORKSPACE
    msg = N.lib.dx_last_error().decode()
    assert "1048576" in msg and "scratch" in msg, msg
