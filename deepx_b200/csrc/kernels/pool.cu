// dx_pool_*: per-device caching allocator for tensor storage.
//
// The reference allocates every tensor with its own cudaMalloc and releases it
// with cudaFree (executor/op-cuda/src/deepx/tensorfunc/tensorlife_miaobyte.hpp:16-40),
// both of which synchronise the device; its MemoryPool is an empty stub
// (new_mempool.hpp:6-37).  Every deepxIR op output is preceded by a `newtensor`,
// so allocation sits on the hot path.
//
// Here a freed block goes to a size-ordered free list and is handed out again to
// the next request it fits (best fit, at most 2× the request for blocks above
// 1 MiB so a large slab is not burnt on a small tensor).  Blocks are never split,
// which keeps every block a whole driver allocation and therefore exportable
// through CUDA IPC, the property the heap-tensor design asks for
// (executor/heapmem-cuda/README.md:42-46).  Reuse is safe for work submitted in
// order on one stream (the executor has one compute stream per device): a later
// kernel that writes a recycled block is ordered after every earlier kernel that
// read it.
#include <map>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

struct dx_pool {
    int device;
    size_t max_bytes;
    size_t in_use = 0, reserved = 0, high_water = 0, n_malloc = 0;
    std::multimap<size_t, void *> free_blocks;       // size → block
    std::unordered_map<void *, size_t> live;         // block → size
    std::mutex mu;
};

namespace {
using dx::DeviceGuard;

size_t round_size(size_t b) {
    if (b == 0) b = 1;
    if (b <= (1u << 20)) return (b + 511) / 512 * 512;          // small: 512-byte classes
    return (b + (2u << 20) - 1) / (2u << 20) * (2u << 20);      // large: 2 MiB granules
}

void release_cached(dx_pool *p) {
    for (auto &kv : p->free_blocks) {
        cudaFree(kv.second);
        p->reserved -= kv.first;
    }
    p->free_blocks.clear();
}

}  // namespace

extern "C" dx_pool *dx_pool_create(int device, size_t max_bytes) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) {
        dx::set_error("pool: device %d not available (%d visible)", device, n);
        cudaGetLastError();
        return nullptr;
    }
    dx_pool *p = new dx_pool();
    p->device = device;
    p->max_bytes = max_bytes;
    return p;
}

extern "C" void dx_pool_destroy(dx_pool *p) {
    if (!p) return;
    {
        std::lock_guard<std::mutex> lk(p->mu);
        DeviceGuard g(p->device);
        release_cached(p);
        for (auto &kv : p->live) cudaFree(kv.first);
        p->live.clear();
    }
    delete p;
}

extern "C" void *dx_pool_alloc(dx_pool *p, size_t bytes) {
    if (!p) {
        dx::set_error("pool: null pool");
        return nullptr;
    }
    const size_t sz = round_size(bytes);
    std::lock_guard<std::mutex> lk(p->mu);
    auto it = p->free_blocks.lower_bound(sz);
    if (it != p->free_blocks.end() && (sz <= (1u << 20) ? it->first == sz : it->first <= 2 * sz)) {
        void *ptr = it->second;
        const size_t got = it->first;
        p->free_blocks.erase(it);
        p->live[ptr] = got;
        p->in_use += got;
        if (p->in_use > p->high_water) p->high_water = p->in_use;
        return ptr;
    }
    DeviceGuard g(p->device);
    if (p->max_bytes && p->reserved + sz > p->max_bytes) {
        release_cached(p);  // give cached blocks back before refusing
        if (p->reserved + sz > p->max_bytes) {
            dx::set_error("pool: request of %zu bytes exceeds the pool limit (%zu reserved of %zu)", sz, p->reserved,
                          p->max_bytes);
            return nullptr;
        }
    }
    void *ptr = nullptr;
    cudaError_t e = cudaMalloc(&ptr, sz);
    if (e != cudaSuccess) {
        cudaGetLastError();
        release_cached(p);
        e = cudaMalloc(&ptr, sz);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        dx::set_error("pool: cudaMalloc(%zu) failed: %s", sz, cudaGetErrorString(e));
        return nullptr;
    }
    ++p->n_malloc;
    p->reserved += sz;
    p->live[ptr] = sz;
    p->in_use += sz;
    if (p->in_use > p->high_water) p->high_water = p->in_use;
    return ptr;
}

extern "C" int dx_pool_free(dx_pool *p, void *ptr) {
    if (!p) return dx::fail(DX_E_ARG, "pool: null pool");
    if (!ptr) return DX_OK;
    std::lock_guard<std::mutex> lk(p->mu);
    auto it = p->live.find(ptr);
    if (it == p->live.end()) return dx::fail(DX_E_ARG, "pool: pointer %p was not allocated from this pool", ptr);
    const size_t sz = it->second;
    p->live.erase(it);
    p->in_use -= sz;
    p->free_blocks.emplace(sz, ptr);
    return DX_OK;
}

extern "C" void dx_pool_stats(const dx_pool *p, size_t stats[4]) {
    if (!p || !stats) return;
    dx_pool *q = const_cast<dx_pool *>(p);
    std::lock_guard<std::mutex> lk(q->mu);
    stats[0] = p->in_use;
    stats[1] = p->reserved;
    stats[2] = p->high_water;
    stats[3] = p->n_malloc;
}

extern "C" void dx_pool_trim(dx_pool *p) {
    if (!p) return;
    std::lock_guard<std::mutex> lk(p->mu);
    DeviceGuard g(p->device);
    release_cached(p);
}
