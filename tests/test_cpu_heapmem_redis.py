"""The heap-tensor service over the Redis wire protocol, without Redis and without a GPU.

An in-test server speaks RESP2 on a TCP socket and keeps hashes and lists in Python dicts (the commands the
service uses: PING, HSET, HGETALL, DEL, KEYS, LPUSH, BRPOP).  Against it run (a) the service as a library
(dx_heap_create_redis, host-backed allocations), (b) the `deepx-heapmem` daemon as a process, with clients that
push lifecycle commands and read hashes the way another process of the machine would (dx_heap_request /
dx_heap_lookup).  The keys, fields and commands are those of executor/heapmem-cuda/README.md:13-40 and
registry.cpp:11-86 / lifecycle.cpp:35-85.
"""
import os
import signal
import socket
import socketserver
import subprocess
import sys
import threading
import time

import pytest

from deepx_b200 import heapmem as H


class FakeRedis(socketserver.ThreadingTCPServer):
    allow_reuse_address = True
    daemon_threads = True

    def __init__(self):
        super().__init__(("127.0.0.1", 0), FakeRedisHandler)
        self.hashes, self.lists, self.log = {}, {}, []
        self.cond = threading.Condition()
        self.thread = threading.Thread(target=self.serve_forever, daemon=True)
        self.thread.start()

    @property
    def addr(self):
        return ("127.0.0.1", self.server_address[1])


class FakeRedisHandler(socketserver.StreamRequestHandler):
    def read_command(self):
        line = self.rfile.readline()
        if not line:
            return None
        assert line[:1] == b"*", line
        args = []
        for _ in range(int(line[1:])):
            n = int(self.rfile.readline()[1:])
            args.append(self.rfile.read(n + 2)[:-2].decode())
        return args

    @staticmethod
    def bulk(s):
        b = s.encode()
        return b"$%d\r\n%s\r\n" % (len(b), b)

    def handle(self):
        srv = self.server
        while True:
            args = self.read_command()
            if args is None:
                return
            cmd = args[0].upper()
            srv.log.append(args)
            with srv.cond:
                if cmd == "PING":
                    out = b"+PONG\r\n"
                elif cmd == "HSET":
                    h = srv.hashes.setdefault(args[1], {})
                    new = 0
                    for k, v in zip(args[2::2], args[3::2]):
                        new += k not in h
                        h[k] = v
                    out = b":%d\r\n" % new
                elif cmd == "HGETALL":
                    h = srv.hashes.get(args[1], {})
                    out = b"*%d\r\n" % (2 * len(h)) + b"".join(self.bulk(k) + self.bulk(v) for k, v in h.items())
                elif cmd == "DEL":
                    out = b":%d\r\n" % (1 if srv.hashes.pop(args[1], None) is not None else 0)
                elif cmd == "KEYS":
                    prefix = args[1].rstrip("*")
                    ks = [k for k in srv.hashes if k.startswith(prefix)]
                    out = b"*%d\r\n" % len(ks) + b"".join(self.bulk(k) for k in ks)
                elif cmd == "LPUSH":
                    srv.lists.setdefault(args[1], []).insert(0, args[2])
                    srv.cond.notify_all()
                    out = b":%d\r\n" % len(srv.lists[args[1]])
                elif cmd == "BRPOP":
                    deadline = time.time() + float(args[2])
                    while not srv.lists.get(args[1]) and time.time() < deadline:
                        srv.cond.wait(timeout=max(0.0, deadline - time.time()))
                    if srv.lists.get(args[1]):
                        out = b"*2\r\n" + self.bulk(args[1]) + self.bulk(srv.lists[args[1]].pop())
                    else:
                        out = b"*-1\r\n"
                else:
                    out = b"-ERR unknown command '%s'\r\n" % cmd.encode()
            self.wfile.write(out)
            self.wfile.flush()


@pytest.fixture()
def redis():
    srv = FakeRedis()
    yield srv
    srv.shutdown()
    srv.server_close()


def test_service_keeps_the_reference_keys_and_fields_in_the_store(redis):
    heap = H.Heap(node="n1", backing=H.HOST_FAKE, redis=redis.addr)
    m = heap.create("W", "f32", [4, 8], device=0, pid=4242)
    h = redis.hashes["tensor:W"]                                       # Registry::Key, registry.cpp:13-15
    assert {"dtype", "shape", "ctime", "node", "device", "bytes", "ipc_handle", "refcount", "state", "owner_pid"} <= set(h)
    assert h["dtype"] == "f32" and h["shape"] == "[4,8]" and h["bytes"] == "128" and h["refcount"] == "1" and h["state"] == "ready"
    assert h["node"] == "n1" and h["owner_pid"] == "4242" and len(h["ipc_handle"]) == 128 and m["ipc_handle"] == h["ipc_handle"]
    assert heap.get("W")["refcount"] == 2 and redis.hashes["tensor:W"]["refcount"] == "2"
    assert heap.create("W", "f32", [4, 8])["refcount"] == 3            # create-or-get
    with pytest.raises(H.HeapError):
        heap.create("W", "f32", [9, 9])
    for left in (2, 1):
        assert heap.delete("W")["refcount"] == left
    assert heap.delete("W")["state"] == "deleted" and "tensor:W" not in redis.hashes and len(heap) == 0
    # the command list: LPUSH by anybody, BRPOP + handle by the service (LifecycleWorker::RunOnce, lifecycle.cpp:60-73)
    H.request(redis.addr, {"op": "create", "name": "KV", "dtype": "bf16", "shape": [2, 16], "device": 0, "pid": os.getpid(), "node": "n1"})
    assert redis.lists["tensor_lifecycle"] and "KV" in redis.lists["tensor_lifecycle"][0]
    with pytest.raises(KeyError):
        H.lookup(redis.addr, "KV")                                     # not handled yet
    assert heap.run_once(1000) is True
    got = H.lookup(redis.addr, "KV")
    assert got["dtype"] == "bf16" and got["shape"] == [2, 16] and got["bytes"] == 64 and got["refcount"] == 1
    assert heap.run_once(200) is False                                 # BRPOP timed out: nil reply
    heap.push('{"op":"nonsense"}')                                     # a malformed command is dropped, not fatal
    assert heap.run_once(1000) is True and len(heap) == 1
    heap.close()
    assert "tensor:KV" not in redis.hashes                             # the service frees what it still held
    assert {a[0].upper() for a in redis.log} <= {"PING", "HSET", "HGETALL", "DEL", "KEYS", "LPUSH", "BRPOP"}


def test_unreachable_store_is_an_error_not_a_hang():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with pytest.raises(H.HeapError, match="cannot connect"):
        H.Heap(backing=H.HOST_FAKE, redis=("127.0.0.1", port))
    with pytest.raises(H.HeapError):
        H.request(("127.0.0.1", port), {"op": "get", "name": "x"})


def test_daemon_process_serves_clients_and_collects_dead_owners(redis):
    from deepx_b200.heapmem import lib  # noqa: F401  (loads the library, so the binary next to it exists)
    from deepx_b200.executor import BIN_PATH
    daemon = BIN_PATH.parent / "deepx-heapmem"
    env = dict(os.environ, HEAPMEM_REDIS="%s:%d" % redis.addr, HEAPMEM_NODE="n1", HEAPMEM_BACKING="host", HEAPMEM_GC_SECONDS="1")
    proc = subprocess.Popen([str(daemon)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    try:
        assert "serving tensor_lifecycle" in proc.stdout.readline()
        owner = subprocess.Popen([sys.executable, "-c", "import time; time.sleep(600)"])   # a client process that owns a tensor
        H.request(redis.addr, {"op": "create", "name": "weights", "dtype": "f16", "shape": [8, 8], "device": 0, "pid": owner.pid, "node": "n1"})
        H.request(redis.addr, {"op": "get", "name": "weights"})
        deadline = time.time() + 20
        meta = None
        while time.time() < deadline:
            try:
                meta = H.lookup(redis.addr, "weights")
                if meta["refcount"] == 2:
                    break
            except KeyError:
                pass
            time.sleep(0.05)
        assert meta and meta["refcount"] == 2 and meta["bytes"] == 128 and meta["owner_pid"] == owner.pid and meta["state"] == "ready"
        H.request(redis.addr, {"op": "delete", "name": "weights"})
        while time.time() < deadline and H.lookup(redis.addr, "weights")["refcount"] != 1:
            time.sleep(0.05)
        assert H.lookup(redis.addr, "weights")["refcount"] == 1
        owner.kill()                                                    # the owner dies without deleting: the sweep releases its tensor
        owner.wait()
        while time.time() < deadline + 10:
            try:
                H.lookup(redis.addr, "weights")
            except KeyError:
                break
            time.sleep(0.1)
        with pytest.raises(KeyError):
            H.lookup(redis.addr, "weights")
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            out, _ = proc.communicate(timeout=20)
        except Exception:
            proc.kill()
            out = ""
    assert "commands handled" in out
