// deepx-heapmem: the heap-tensor service as a process of its own, after the reference's heapmem-cuda daemon
// (executor/heapmem-cuda/src/runtime/lifecycle.cpp:75-85: a loop around BRPOP on `tensor_lifecycle`).
// It connects to a Redis server, pops lifecycle commands one at a time — create: allocate on the named
// device, export with CUDA IPC, write the `tensor:<name>` hash; get / delete: refcount up / down, at zero
// the memory is freed and the hash removed — and every few seconds drops the tensors whose owning process
// no longer exists (Registry::GcSweep, registry.cpp:61-66).  It is the only writer of the hashes, which
// makes each command atomic; clients push commands and read hashes (dx_heap_request / dx_heap_lookup).
//
// Environment: HEAPMEM_REDIS (host:port, default 127.0.0.1:6379), HEAPMEM_NODE (this machine's name in the
// `node` field; default the host name), HEAPMEM_BACKING (device | host; `host` runs the registry with host
// memory and made-up handles, for machines without a GPU), HEAPMEM_GC_SECONDS (5).  SIGINT / SIGTERM stop it;
// the tensors it still holds are freed and their hashes removed.
#include <csignal>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <iostream>
#include <string>

#include "dx_heapmem.h"

static volatile sig_atomic_t g_stop = 0;
static void on_signal(int) { g_stop = 1; }

int main() {
    const char *env;
    std::string host = "127.0.0.1";
    int port = 6379;
    if ((env = std::getenv("HEAPMEM_REDIS")) && *env) {
        const std::string s = env;
        const size_t colon = s.rfind(':');
        host = colon == std::string::npos ? s : s.substr(0, colon);
        if (colon != std::string::npos) port = std::atoi(s.c_str() + colon + 1);
    }
    const int backing = ((env = std::getenv("HEAPMEM_BACKING")) && std::strcmp(env, "host") == 0) ? DX_HEAP_HOST_FAKE : DX_HEAP_DEVICE;
    const int gc_seconds = (env = std::getenv("HEAPMEM_GC_SECONDS")) ? std::atoi(env) : 5;
    dx_heap *heap = dx_heap_create_redis(std::getenv("HEAPMEM_NODE"), backing, host.c_str(), port);
    if (!heap) {
        std::cerr << "deepx-heapmem: " << dx_heap_last_error() << std::endl;
        return 1;
    }
    std::signal(SIGINT, on_signal);
    std::signal(SIGTERM, on_signal);
    std::cout << "deepx-heapmem serving tensor_lifecycle at " << host << ":" << port << (backing == DX_HEAP_HOST_FAKE ? " (host memory)" : "") << std::endl;
    std::time_t last_gc = std::time(nullptr);
    unsigned long long handled = 0;
    while (!g_stop) {
        const int rc = dx_heap_run_once(heap, 1000);
        if (rc < 0) {
            std::cerr << "deepx-heapmem: " << dx_heap_last_error() << std::endl;
            break;
        }
        handled += rc > 0;
        if (gc_seconds > 0 && std::time(nullptr) - last_gc >= gc_seconds) {
            const long long dropped = dx_heap_gc_sweep(heap, nullptr);
            if (dropped > 0) std::cout << "deepx-heapmem: released " << dropped << " tensor(s) of processes that are gone" << std::endl;
            last_gc = std::time(nullptr);
        }
    }
    std::cout << "deepx-heapmem: " << handled << " commands handled, " << dx_heap_count(heap) << " tensors released at exit" << std::endl;
    dx_heap_destroy(heap);
    return 0;
}
