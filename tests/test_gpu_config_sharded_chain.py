"""The sharded elementwise + reduce chain at its full size: float32 [2048, 1048576] (2^31 elements,
8 GiB per tensor), z = exp(x)*y + x, s = sum(z) over all axes, m = reducemax(z) over axis 1.

Rows above 1024 lie beyond byte offset 2^32 and the element count exceeds INT_MAX — the regime the
reference's 32-bit Shape (executor/deepxcore/src/deepx/shape.hpp:47-49) cannot describe, so the CPU
oracle works block by block (256 rows, seed = block index, the generator bench.py uses).

Checked, through the tensorfunc C ABI and through the deepxIR executor:
  * z of the first, a middle and the LAST block element for element against the oracle chain
    (exp is within 1e-5 relative of the C library's; the test allows rtol 1e-5 + atol 1e-6 on z);
  * all 2048 row maxima bit for bit against the oracle's reducemax of the z the GPU produced, and
    within the same tolerance against the oracle chain's;
  * the global sum against float64 block sums, within 1e-5 of sum(|z|);
  * the executor's z, s, m bit-equal to the direct path's.
"""
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
ROWS, COLS, BLOCK = 2048, 1 << 20, 256
NBLOCKS = ROWS // BLOCK


def _bench():
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))
    import bench
    return bench


def test_config_sharded_chain_full_size():
    from deepx_b200 import tensorfunc as TF
    from deepx_b200.executor import Executor
    from oracle import oracle as O
    bench = _bench()
    assert (bench.ROWS, bench.COLS, bench.BLOCK_ROWS) == (ROWS, COLS, BLOCK)
    free, _ = torch.cuda.mem_get_info()
    if free < 52 << 30:
        pytest.skip(f"needs 52 GiB of device memory, {free >> 30} GiB free")
    dev = torch.device("cuda:0")
    x = torch.empty((ROWS, COLS), dtype=torch.float32, device=dev)
    y = torch.empty_like(x)
    assert x.numel() == 1 << 31

    # host oracle per block while the data goes up
    want_max = np.empty(ROWS, dtype=np.float32)       # oracle chain
    keep = {}                                          # oracle z of the blocks compared element for element
    checked_blocks = (0, NBLOCKS // 2, NBLOCKS - 1)
    with ThreadPoolExecutor(max_workers=2) as pool:
        nxt = (pool.submit(bench.gen_block, 0, "x"), pool.submit(bench.gen_block, 0, "y"))
        for b in range(NBLOCKS):
            hx, hy = nxt[0].result(), nxt[1].result()
            if b + 1 < NBLOCKS:
                nxt = (pool.submit(bench.gen_block, b + 1, "x"), pool.submit(bench.gen_block, b + 1, "y"))
            x[b * BLOCK:(b + 1) * BLOCK].copy_(torch.from_numpy(hx))
            y[b * BLOCK:(b + 1) * BLOCK].copy_(torch.from_numpy(hy))
            z = O.add(O.mul(O.exp(hx), hy), hx)
            want_max[b * BLOCK:(b + 1) * BLOCK] = O.reducemax(z, [1])
            if b in checked_blocks:
                keep[b] = z
            del hx, hy, z

    # ---- direct path: tensorfunc → C ABI
    t = torch.empty_like(x)
    z = torch.empty_like(x)
    s = torch.empty(1, dtype=torch.float32, device=dev)
    m = torch.empty(ROWS, dtype=torch.float32, device=dev)
    TF.exp(x, t)
    TF.mul(t, y, t)
    TF.add(t, x, z)
    TF.sum(z, [0, 1], False, s)
    TF.reducemax(z, [1], False, m)
    torch.cuda.synchronize()
    del t

    got_m = m.cpu().numpy()
    got_s = float(s.item())
    sum64 = 0.0
    abs64 = 0.0
    for b in range(NBLOCKS):
        zb = z[b * BLOCK:(b + 1) * BLOCK].cpu().numpy()
        # reducemax at this size, bit for bit: the oracle's row max of the very z the GPU holds
        assert np.array_equal(got_m[b * BLOCK:(b + 1) * BLOCK].view(np.uint32), O.reducemax(zb, [1]).view(np.uint32)), \
            f"row maxima of block {b} are not bit-exact"
        sum64 += float(zb.astype(np.float64).sum())
        abs64 += float(np.abs(zb).astype(np.float64).sum())
        if b in keep:
            bad = ~np.isclose(zb, keep[b], rtol=1e-5, atol=1e-6)
            assert not bad.any(), f"z of block {b}: {int(bad.sum())} elements outside rtol 1e-5 + atol 1e-6"
        del zb
    assert np.allclose(got_m, want_max, rtol=1e-5, atol=1e-6), "row maxima differ from the oracle chain"
    assert abs(got_s - sum64) <= 1e-5 * abs64, f"global sum {got_s} vs float64 {sum64} (sum|z| = {abs64})"

    # ---- the same chain as deepxIR text through the executor, on the same x and y
    ex = Executor(0)
    f32 = "tensor<float32>"
    from deepx_b200 import _native as N
    ex.bind("x", N.F32, (ROWS, COLS), x.data_ptr())
    ex.bind("y", N.F32, (ROWS, COLS), y.data_ptr())
    ex.run(f"newtensor(vector<int32>:[{ROWS} {COLS}])->({f32}:t)")
    ex.run(f"newtensor(vector<int32>:[{ROWS} {COLS}])->({f32}:z)")
    ex.run(f"newtensor(vector<int32>:[1])->({f32}:s)")
    ex.run(f"newtensor(vector<int32>:[{ROWS}])->({f32}:m)")
    assert ex.info("z")[1] == [ROWS, COLS]
    for line in (f"exp({f32}:x)->({f32}:t) // author=miaobyte",
                 f"mul({f32}:t, {f32}:y)->({f32}:t) // author=miaobyte",
                 f"add({f32}:t, {f32}:x)->({f32}:z) // author=miaobyte",
                 f"sum({f32}:z, vector<int32>:[0 1], var<bool>:false)->({f32}:s) // author=miaobyte",
                 f"reducemax({f32}:z, vector<int32>:[1], var<bool>:false)->({f32}:m) // author=miaobyte"):
        ex.run(line)
    ex.sync()
    assert np.array_equal(ex.download("m").view(np.uint32), got_m.view(np.uint32)), "executor row maxima differ from the direct path"
    assert ex.download("s").view(np.uint32)[0] == np.float32(got_s).view(np.uint32), "executor global sum differs from the direct path"

    class _View:
        def __init__(self, ptr):
            self.__cuda_array_interface__ = {"shape": (ROWS, COLS), "typestr": "<f4", "data": (ptr, False), "version": 2}
    z_ex = torch.as_tensor(_View(ex.ptr("z")), device=dev)
    for b in range(NBLOCKS):  # block by block: a 2^31-element comparison in one go would need its own 2 GiB mask
        assert torch.equal(z_ex[b * BLOCK:(b + 1) * BLOCK], z[b * BLOCK:(b + 1) * BLOCK]), f"executor z differs in block {b}"
    del z_ex
    ex.close()
