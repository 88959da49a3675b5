"""Heap tensors on the GPU: allocation, CUDA-IPC export, and a second process mapping the memory.

The owner creates the tensor and fills it; a child process receives only the hash's `ipc_handle`
text, maps the allocation (cudaIpcOpenMemHandle), checks what it reads, writes something else and
unmaps; the owner then sees the child's bytes.  (executor/heapmem-cuda/README.md:25-40.)
"""
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHILD = textwrap.dedent("""
    import sys
    import numpy as np
    sys.path.insert(0, {root!r})
    from deepx_b200 import heapmem as H
    handle, n = sys.argv[1], int(sys.argv[2])
    ptr = H.open_handle(handle, 0)
    got = np.empty(n, dtype=np.float32)
    H.copy_to_host(got, ptr)
    assert np.array_equal(got, np.arange(n, dtype=np.float32) * 0.5), got[:8]
    H.copy_to_device(ptr, (got + 1000.0).astype(np.float32))
    H.close_handle(ptr)
    print("child ok")
""")


def test_second_process_maps_a_heap_tensor():
    from deepx_b200 import heapmem as H
    heap = H.Heap()
    n = 1 << 20
    meta = heap.create("kv_cache", "f32", [1024, 1024], device=0)
    assert meta["bytes"] == 4 * n and meta["state"] == "ready" and len(meta["ipc_handle"]) == 128
    src = np.arange(n, dtype=np.float32) * 0.5
    H.copy_to_device(heap.ptr("kv_cache"), src)
    got = heap.get("kv_cache")  # what a consumer does before mapping: refcount 2
    assert got["refcount"] == 2
    r = subprocess.run([sys.executable, "-c", CHILD.format(root=str(ROOT)), got["ipc_handle"], str(n)],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "child ok" in r.stdout, r.stdout + r.stderr
    back = np.empty(n, dtype=np.float32)
    H.copy_to_host(back, heap.ptr("kv_cache"))
    assert np.array_equal(back, src + 1000.0)
    assert heap.delete("kv_cache")["refcount"] == 1   # the consumer lets go
    assert heap.delete("kv_cache")["state"] == "deleted"
    assert len(heap) == 0
    heap.close()


def test_kernels_run_on_heap_tensors():
    """A heap tensor is plain device memory to the op kernels."""
    import torch
    from deepx_b200 import _native as N
    from deepx_b200 import heapmem as H
    heap = H.Heap()
    heap.create("a", "float32", [4096])
    heap.create("b", "float32", [4096])
    a = np.linspace(-1, 1, 4096, dtype=np.float32)
    H.copy_to_device(heap.ptr("a"), a)
    torch.cuda.synchronize()
    N.check(N.lib.dx_ew_scalar(N.MULS, N.F32, heap.ptr("a"), 3.0, 0, heap.ptr("b"), 4096, None))
    torch.cuda.synchronize()
    out = np.empty(4096, dtype=np.float32)
    H.copy_to_host(out, heap.ptr("b"))
    assert np.array_equal(out, a * np.float32(3.0))
    heap.close()


def test_executor_runs_ir_on_a_bound_heap_tensor():
    """A heap tensor registered in the executor under a name is an ordinary operand of IR ops; deleting
    the name does not free the heap allocation."""
    from deepx_b200 import heapmem as H
    from deepx_b200.executor import Executor
    heap = H.Heap()
    heap.create("weights", "float32", [8, 16])
    w = np.arange(128, dtype=np.float32).reshape(8, 16)
    H.copy_to_device(heap.ptr("weights"), w)
    ex = Executor(0)
    ex.bind("w", 1, [8, 16], heap.ptr("weights"))
    with pytest.raises(RuntimeError):
        ex.bind("w", 1, [8, 16], heap.ptr("weights"))
    ex.run("newtensor(vector<int32>:[8 16])->(tensor<float32>:y)")
    ex.run("mulscalar(tensor<float32>:w, var<float32>:2)->(tensor<float32>:y)")
    ex.run("addscalar(tensor<float32>:w, var<float32>:1)->(tensor<float32>:w)")   # in place, into the heap tensor
    assert np.array_equal(ex.download("y"), w * 2)
    ex.run("deltensor()->(tensor<float32>:w)")
    ex.sync()
    back = np.empty_like(w)
    H.copy_to_host(back, heap.ptr("weights"))
    assert np.array_equal(back, w + 1)
    ex.close()
    heap.close()


def test_bad_handle_is_an_error_not_a_fault():
    from deepx_b200 import heapmem as H
    with pytest.raises(H.HeapError):
        H.open_handle("zz", 0)
    with pytest.raises(H.HeapError):
        H.open_handle("12" * 10, 0)
