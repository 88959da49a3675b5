"""The heap-tensor registry and its lifecycle commands, without a GPU (host-backed allocations).

Follows the protocol of executor/heapmem-cuda/README.md:13-40: hash `tensor:<name>` with dtype,
shape, ctime, node, device, bytes, ipc_handle, refcount; commands create / get / delete.
"""
import json
import os
import subprocess
import sys

import pytest

from deepx_b200 import heapmem as H


@pytest.fixture()
def heap():
    h = H.Heap(node="n1", backing=H.HOST_FAKE)
    yield h
    h.close()


def test_create_get_delete_refcount(heap):
    m = heap.create("X", "f32", [2, 3], device=0, pid=123)
    assert m["name"] == "X" and m["dtype"] == "f32" and m["shape"] == [2, 3]
    assert m["bytes"] == 24 and m["refcount"] == 1 and m["state"] == "ready"
    assert m["node"] == "n1" and m["device"] == 0 and m["owner_pid"] == 123
    assert len(m["ipc_handle"]) == 128 and m["ctime"] > 0
    assert len(heap) == 1 and heap.ptr("X") != 0
    assert heap.get("X")["refcount"] == 2
    assert heap.meta("X")["refcount"] == 2
    assert heap.delete("X")["refcount"] == 1
    gone = heap.delete("X")
    assert gone["refcount"] == 0 and gone["state"] == "deleted" and gone["ipc_handle"] == ""
    assert len(heap) == 0 and heap.ptr("X") == 0
    with pytest.raises(KeyError):
        heap.meta("X")


def test_create_is_create_or_get(heap):
    a = heap.create("W", "bf16", [4, 8])
    b = heap.create("W", "bf16", [4, 8])
    assert b["refcount"] == 2 and b["ipc_handle"] == a["ipc_handle"] and len(heap) == 1
    with pytest.raises(H.HeapError):
        heap.create("W", "bf16", [4, 9])
    with pytest.raises(H.HeapError):
        heap.create("W", "f32", [4, 8])


def test_reference_command_text_and_long_dtype_names(heap):
    """The literal command of README.md:27 (shape as a JSON array), and the executor's dtype names."""
    m = heap.command('{"op":"create", "name":"X", "dtype":"f32", "shape":[2,3], "device":0, "pid":123, "node":"n1"}')
    assert m["bytes"] == 24
    assert heap.create("Y", "float16", [5])["bytes"] == 10
    assert heap.create("Z", "int64", [])["bytes"] == 8  # rank 0: one element
    assert heap.create("E", "i8", [0, 7])["bytes"] == 0


def test_errors(heap):
    for bad in ({"op": "get", "name": "nope"}, {"op": "delete", "name": "nope"}, {"op": "create", "name": "a", "dtype": "f33", "shape": [1]},
                {"op": "create", "name": "a", "dtype": "f32"}, {"op": "create", "name": "a", "dtype": "f32", "shape": [-1]},
                {"op": "grow", "name": "a"}, {"name": "a"}, {"op": "create"}):
        with pytest.raises(H.HeapError):
            heap.command(bad)
    assert len(heap) == 0


def test_command_list_worker(heap):
    """LPUSH tensor_lifecycle / BRPOP + handle, in order (LifecycleWorker::RunOnce, lifecycle.cpp:60-73)."""
    assert heap.run_once(10) is False  # empty list: times out
    heap.push({"op": "create", "name": "A", "dtype": "f32", "shape": [8]})
    heap.push({"op": "get", "name": "A"})
    heap.push("not json at all")
    heap.push({"op": "delete", "name": "A"})
    assert [heap.run_once(100) for _ in range(4)] == [True] * 4
    assert heap.run_once(0) is False
    assert heap.meta("A")["refcount"] == 1


def test_gc_sweep_drops_tensors_of_dead_owners():
    h = H.Heap(backing=H.HOST_FAKE)  # node = this host, so owner pids can be checked
    child = subprocess.Popen([sys.executable, "-c", "pass"])
    child.wait()
    h.create("orphan", "f32", [4], pid=child.pid)
    h.create("mine", "f32", [4], pid=os.getpid())
    h.create("elsewhere", "f32", [4], pid=child.pid)
    h.command({"op": "get", "name": "mine"})
    assert h.gc_sweep() == 2  # both tensors of the dead process
    assert h.gc_sweep() == 0
    assert len(h) == 1 and h.meta("mine")["refcount"] == 2
    h.close()


def test_gc_sweep_only_touches_the_named_node(heap):
    heap.command({"op": "create", "name": "a", "dtype": "f32", "shape": [1], "node": "n2", "pid": 1})
    heap.command({"op": "create", "name": "b", "dtype": "f32", "shape": [1], "node": "n1", "pid": os.getpid()})
    assert heap.gc_sweep("n3") == 0 and len(heap) == 2
    # a foreign node's owner pids cannot be checked from here: only non-positive refcounts go
    assert heap.gc_sweep("n2") == 0 and len(heap) == 2
