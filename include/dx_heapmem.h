/*
 * dx_heapmem.h — C ABI of the heap-tensor service (part of libdeepx_exec.so).
 *
 * Heap tensors are the tensors that outlive one computation and are shared by several processes
 * on one machine (weights, KV caches), as opposed to the stack tensors an executor creates and
 * deletes while it runs a program.  The reference sketches this service in
 * executor/heapmem-cuda (README.md:1-46; registry/registry.h:11-51, registry.cpp:11-86;
 * runtime/lifecycle.h:10-35, lifecycle.cpp:35-85): per tensor a hash `tensor:<name>` with the
 * fields dtype, shape, ctime, node, device, bytes, ipc_handle, refcount (+ state, owner_pid), and
 * a command list `tensor_lifecycle` carrying JSON
 *     {"op":"create|get|delete","name":"X","dtype":"f32","shape":[2,3],"device":0,"pid":123,"node":"n1"}
 * with  create = allocate → cudaIpcGetMemHandle → hash(state=ready, refcount=1),
 *       get    = read hash → refcount+1 (the caller maps the memory with cudaIpcOpenMemHandle),
 *       delete = refcount-1, at 0 free the memory and drop the hash.
 * The reference keeps hash and list in a Redis server.  Two stores are offered here behind the same
 * operations: an in-process one (dx_heap_create: registry and its users in one process), and a Redis
 * server spoken to with the Redis wire protocol over a plain TCP socket (dx_heap_create_redis: no
 * client library is needed; redis++ and the reference's Lua scripts are not in its tree).  With a
 * server, ONE service process owns the allocations and is the only writer of the hashes — the
 * `deepx-heapmem` daemon, which pops commands off `tensor_lifecycle` one at a time — so create-or-get
 * and the refcount changes are atomic without scripts; every other process pushes commands
 * (dx_heap_request) and reads hashes (dx_heap_lookup), then maps the memory with dx_heap_open.
 * Every heap tensor is its own cudaMalloc allocation: CUDA IPC exports
 * whole allocations, so heap tensors never come from the sub-allocating pool (README.md:48-52).
 *
 * All functions return 0 (or a count) on success and a negative value on failure; the text of the
 * last failure on this thread is dx_heap_last_error().
 */
#ifndef DX_HEAPMEM_H
#define DX_HEAPMEM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct dx_heap dx_heap;

enum {
    DX_HEAP_DEVICE = 0, /* cudaMalloc + cudaIpcGetMemHandle */
    DX_HEAP_HOST_FAKE = 1 /* host malloc and a made-up handle: the registry logic without a GPU (tests) */
};

/* `node` is this machine's name as it appears in the `node` field (NULL = the host name). */
dx_heap *dx_heap_create(const char *node, int backing);
/* The same service with its hashes and its command list in a Redis server at host:port (NULL / 0 =
 * 127.0.0.1:6379).  NULL when the server cannot be reached (dx_heap_last_error). */
dx_heap *dx_heap_create_redis(const char *node, int backing, const char *host, int port);
void dx_heap_destroy(dx_heap *h); /* frees every tensor still registered */
const char *dx_heap_last_error(void);

/* Handles one lifecycle command (the JSON above) at once.  `reply` receives the tensor's hash as
 * one JSON object ({"name":…,"dtype":…,"shape":[…],"ctime":…,"node":…,"device":…,"bytes":…,
 * "ipc_handle":"<hex>","refcount":…,"state":"ready|deleted","owner_pid":…}).
 * create on an existing name is create-or-get (Registry::CreateOrGet, registry.cpp:24-45): the
 * refcount goes up and the existing tensor is returned; dtype/shape that differ are an error. */
int dx_heap_command(dx_heap *h, const char *json, char *reply, size_t cap);

/* The command list `tensor_lifecycle`: push a command (LPUSH), or pop one (BRPOP with a timeout in
 * milliseconds) and handle it as LifecycleWorker::RunOnce does (lifecycle.cpp:60-73).
 * dx_heap_run_once returns 1 when a command was handled, 0 on timeout. */
int dx_heap_push(dx_heap *h, const char *json);
int dx_heap_run_once(dx_heap *h, int timeout_ms);

/* HGETALL tensor:<name> as the same JSON object; -1 when there is no such tensor. */
int dx_heap_meta(dx_heap *h, const char *name, char *out, size_t cap);
/* Number of registered tensors. */
int dx_heap_count(dx_heap *h);
/* The owner's own device pointer of a tensor (NULL if absent). */
void *dx_heap_ptr(dx_heap *h, const char *name);
/* Registry::GcSweep (registry.cpp:61-66): drops the tensors of `node` (NULL = this node) whose
 * refcount is not positive or whose owning process no longer exists; returns how many. */
int64_t dx_heap_gc_sweep(dx_heap *h, const char *node);

/* Client side of a server-backed service: push one lifecycle command onto `tensor_lifecycle` (the daemon
 * handles it), and read a tensor's hash as the JSON object above (-1 when there is no such tensor yet). */
int dx_heap_request(const char *host, int port, const char *json);
int dx_heap_lookup(const char *host, int port, const char *name, char *out, size_t cap);

/* Consumer side, in ANOTHER process than the owner: map / unmap the memory behind an ipc_handle
 * (hex text from the hash) on `device` (cudaIpcOpenMemHandle / cudaIpcCloseMemHandle), and copy
 * between it and host memory (synchronous; for tests and small control data). */
void *dx_heap_open(const char *ipc_handle_hex, int device);
int dx_heap_close(void *ptr);
int dx_heap_copy(void *dst, const void *src, size_t bytes, int to_device);

#ifdef __cplusplus
}
#endif
#endif
