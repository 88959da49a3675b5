// The heap-tensor service: registry (hash `tensor:<name>`), lifecycle commands (list
// `tensor_lifecycle`) and CUDA-IPC export, after the sketch in executor/heapmem-cuda
// (registry/registry.h:11-51, registry.cpp:11-86, runtime/lifecycle.cpp:9-85, README.md:13-46).
// Interface and field list: include/dx_heapmem.h.
//
// The store below keeps exactly what the reference would keep in Redis — one string→string map per
// `tensor:<name>` key and one list of JSON commands — so the registry code reads like its
// Redis-backed counterpart (HSET/HGETALL/DEL, LPUSH/BRPOP) and only `Store` would change.
#include <cuda_runtime.h>
#include <signal.h>
#include <unistd.h>

#include <cctype>
#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "dx_heapmem.h"

namespace {

thread_local std::string g_err;
int fail(int code, const std::string &msg) {
    g_err = msg;
    return code;
}

using Hash = std::map<std::string, std::string>;

struct Store {  // the part Redis would play
    std::mutex mu;
    std::condition_variable cv;
    std::map<std::string, Hash> hashes;
    std::deque<std::string> list;  // tensor_lifecycle: pushed at the front, popped at the back
    void lpush(const std::string &v) {
        { std::lock_guard<std::mutex> lk(mu); list.push_front(v); }
        cv.notify_one();
    }
    bool brpop(int timeout_ms, std::string &out) {
        std::unique_lock<std::mutex> lk(mu);
        if (!cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return !list.empty(); })) return false;
        out = list.back();
        list.pop_back();
        return true;
    }
};

struct Command {  // LifecycleCommand, lifecycle.h:12-20, with the shape as numbers
    std::string op, name, dtype, node;
    std::vector<int64_t> shape;
    long long device = 0, pid = 0;
    bool has_shape = false;
};

// ---- a JSON reader for flat objects of strings, integers and one integer array ---------------------
size_t value_pos(const std::string &json, const std::string &key) {
    size_t pos = json.find("\"" + key + "\"");
    if (pos == std::string::npos) return pos;
    pos = json.find(':', pos + key.size() + 2);
    if (pos == std::string::npos) return pos;
    ++pos;
    while (pos < json.size() && std::isspace(static_cast<unsigned char>(json[pos]))) ++pos;
    return pos < json.size() ? pos : std::string::npos;
}
std::string get_string(const std::string &json, const std::string &key) {
    size_t pos = value_pos(json, key);
    if (pos == std::string::npos) return "";
    if (json[pos] == '"') {
        const size_t end = json.find('"', pos + 1);
        return end == std::string::npos ? "" : json.substr(pos + 1, end - pos - 1);
    }
    size_t end = pos;
    while (end < json.size() && json[end] != ',' && json[end] != '}' && !std::isspace(static_cast<unsigned char>(json[end]))) ++end;
    return json.substr(pos, end - pos);
}
long long get_int(const std::string &json, const std::string &key) {
    const std::string s = get_string(json, key);
    if (s.empty()) return 0;
    char *end = nullptr;
    const long long v = std::strtoll(s.c_str(), &end, 10);
    return end == s.c_str() ? 0 : v;
}
// "shape":[2,3] or "shape":"[2,3]" (the hash stores it as text, README.md:18)
bool get_shape(const std::string &json, std::vector<int64_t> &out) {
    size_t pos = value_pos(json, "shape");
    if (pos == std::string::npos) return false;
    if (json[pos] == '"') ++pos;
    if (pos >= json.size() || json[pos] != '[') return false;
    const size_t end = json.find(']', pos);
    if (end == std::string::npos) return false;
    std::string body = json.substr(pos + 1, end - pos - 1);
    for (char &c : body)
        if (c == ',') c = ' ';
    const char *p = body.c_str();
    while (*p) {
        char *q = nullptr;
        const long long v = std::strtoll(p, &q, 10);
        if (q == p) {
            while (*p && std::isspace(static_cast<unsigned char>(*p))) ++p;
            if (*p) return false;
            break;
        }
        out.push_back(v);
        p = q;
    }
    return true;
}

int dtype_bytes(const std::string &d) {
    static const std::map<std::string, int> sizes = {
        {"f64", 8}, {"float64", 8}, {"f32", 4}, {"float32", 4}, {"f16", 2}, {"float16", 2}, {"bf16", 2}, {"bfloat16", 2},
        {"i64", 8}, {"int64", 8}, {"i32", 4}, {"int32", 4}, {"i16", 2}, {"int16", 2}, {"i8", 1}, {"int8", 1}, {"u8", 1},
        {"bool", 1}};
    auto it = sizes.find(d);
    return it == sizes.end() ? 0 : it->second;
}

std::string shape_text(const std::vector<int64_t> &s) {
    std::string t = "[";
    for (size_t i = 0; i < s.size(); ++i) t += (i ? "," : "") + std::to_string(s[i]);
    return t + "]";
}

std::string to_hex(const void *p, size_t n) {
    static const char *digits = "0123456789abcdef";
    std::string s;
    const unsigned char *b = static_cast<const unsigned char *>(p);
    for (size_t i = 0; i < n; ++i) {
        s += digits[b[i] >> 4];
        s += digits[b[i] & 15];
    }
    return s;
}
bool from_hex(const std::string &s, void *p, size_t n) {
    if (s.size() != 2 * n) return false;
    auto nib = [](char c) { return c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : -1; };
    unsigned char *b = static_cast<unsigned char *>(p);
    for (size_t i = 0; i < n; ++i) {
        const int hi = nib(s[2 * i]), lo = nib(s[2 * i + 1]);
        if (hi < 0 || lo < 0) return false;
        b[i] = static_cast<unsigned char>(hi * 16 + lo);
    }
    return true;
}

}  // namespace

struct dx_heap {
    std::string node;
    int backing;
    Store store;
    std::map<std::string, void *> ptrs;  // owner-side pointers; guarded by store.mu

    static std::string key(const std::string &name) { return "tensor:" + name; }  // Registry::Key, registry.cpp:13-15

    std::string render(const std::string &name, const Hash &h) const {
        auto f = [&](const char *k) { auto it = h.find(k); return it == h.end() ? std::string() : it->second; };
        auto num = [&](const char *k) { const std::string v = f(k); return v.empty() ? std::string("0") : v; };
        return "{\"name\":\"" + name + "\",\"dtype\":\"" + f("dtype") + "\",\"shape\":" + (f("shape").empty() ? "[]" : f("shape")) +
               ",\"ctime\":" + num("ctime") + ",\"node\":\"" + f("node") + "\",\"device\":" + num("device") + ",\"bytes\":" + num("bytes") +
               ",\"ipc_handle\":\"" + f("ipc_handle") + "\",\"refcount\":" + num("refcount") + ",\"state\":\"" + f("state") +
               "\",\"owner_pid\":" + num("owner_pid") + "}";
    }

    int allocate(long long device, size_t bytes, void **ptr, std::string *handle_hex) {
        if (backing == DX_HEAP_HOST_FAKE) {
            *ptr = std::malloc(bytes ? bytes : 1);
            if (!*ptr) return fail(-4, "out of host memory");
            unsigned char fake[64] = {0};
            std::memcpy(fake, ptr, sizeof(void *));
            *handle_hex = to_hex(fake, sizeof(fake));
            return 0;
        }
        cudaError_t e = cudaSetDevice(int(device));
        if (e == cudaSuccess) e = cudaMalloc(ptr, bytes ? bytes : 1);
        if (e != cudaSuccess) return fail(-4, std::string("cudaMalloc: ") + cudaGetErrorString(e));
        cudaIpcMemHandle_t hd;
        e = cudaIpcGetMemHandle(&hd, *ptr);
        if (e != cudaSuccess) {
            cudaFree(*ptr);
            *ptr = nullptr;
            return fail(-4, std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
        }
        *handle_hex = to_hex(&hd, sizeof(hd));
        return 0;
    }
    void release(void *ptr, long long device) {
        if (!ptr) return;
        if (backing == DX_HEAP_HOST_FAKE) {
            std::free(ptr);
            return;
        }
        cudaSetDevice(int(device));
        cudaFree(ptr);
    }

    // drop hash + memory; store.mu held
    void drop_locked(const std::string &name) {
        auto it = store.hashes.find(key(name));
        long long device = 0;
        if (it != store.hashes.end()) {
            device = std::atoll(it->second["device"].c_str());
            store.hashes.erase(it);
        }
        auto p = ptrs.find(name);
        if (p != ptrs.end()) {
            release(p->second, device);
            ptrs.erase(p);
        }
    }

    // Names, dtypes and node names go into JSON replies and hash keys as they are: refuse the
    // characters that would need escaping there instead of emitting text a client mis-parses.
    static bool plain_text(const std::string &s) {
        for (unsigned char ch : s)
            if (ch < 0x20 || ch == '"' || ch == '\\' || ch == 0x7f) return false;
        return true;
    }

    int handle(const Command &c, std::string *reply) {
        if (!plain_text(c.name) || !plain_text(c.dtype) || !plain_text(c.node))
            return fail(-3, "name, dtype and node must not contain quotes, backslashes or control characters");
        std::lock_guard<std::mutex> lk(store.mu);
        auto it = store.hashes.find(key(c.name));
        if (c.op == "create") {
            if (it != store.hashes.end()) {  // create-or-get
                Hash &h = it->second;
                if ((!c.dtype.empty() && dtype_bytes(c.dtype) != dtype_bytes(h["dtype"])) || (c.has_shape && shape_text(c.shape) != h["shape"]))
                    return fail(-2, "tensor " + c.name + " exists as " + h["dtype"] + h["shape"] + ", asked for " + c.dtype + shape_text(c.shape));
                h["refcount"] = std::to_string(std::atoll(h["refcount"].c_str()) + 1);
                if (reply) *reply = render(c.name, h);
                return 0;
            }
            const int es = dtype_bytes(c.dtype);
            if (es == 0) return fail(-1, "create: unknown dtype '" + c.dtype + "'");
            if (!c.has_shape) return fail(-2, "create: shape missing");
            size_t n = 1;
            for (auto d : c.shape) {
                if (d < 0) return fail(-2, "create: negative extent");
                if (__builtin_mul_overflow(n, size_t(d), &n)) return fail(-2, "create: shape " + shape_text(c.shape) + " overflows the address space");
            }
            size_t nbytes = 0;
            if (__builtin_mul_overflow(n, size_t(es), &nbytes)) return fail(-2, "create: shape " + shape_text(c.shape) + " overflows the address space");
            void *ptr = nullptr;
            std::string hex;
            if (int e = allocate(c.device, nbytes, &ptr, &hex)) return e;
            Hash h;
            h["dtype"] = c.dtype;
            h["shape"] = shape_text(c.shape);
            h["ctime"] = std::to_string(std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count());
            h["node"] = c.node.empty() ? node : c.node;
            h["device"] = std::to_string(c.device);
            h["bytes"] = std::to_string(nbytes);
            h["ipc_handle"] = hex;
            h["refcount"] = "1";
            h["state"] = "ready";
            h["owner_pid"] = std::to_string(c.pid ? c.pid : (long long)getpid());
            store.hashes[key(c.name)] = h;
            ptrs[c.name] = ptr;
            if (reply) *reply = render(c.name, h);
            return 0;
        }
        if (it == store.hashes.end()) return fail(-1, c.op + ": no tensor named " + c.name);
        Hash &h = it->second;
        if (c.op == "get") {  // Registry::RefInc, registry.cpp:47-52
            h["refcount"] = std::to_string(std::atoll(h["refcount"].c_str()) + 1);
            if (reply) *reply = render(c.name, h);
            return 0;
        }
        if (c.op == "delete") {  // Registry::RefDec, registry.cpp:54-59; at zero the memory goes
            const long long left = std::atoll(h["refcount"].c_str()) - 1;
            h["refcount"] = std::to_string(left);
            if (left <= 0) {
                h["state"] = "deleted";
                h["ipc_handle"] = "";
                if (reply) *reply = render(c.name, h);
                drop_locked(c.name);
            } else if (reply) *reply = render(c.name, h);
            return 0;
        }
        return fail(-3, "unknown op '" + c.op + "' (create|get|delete)");
    }
};

namespace {
bool parse_command(const std::string &json, Command &c) {  // LifecycleWorker::Parse, lifecycle.cpp:38-47
    c.op = get_string(json, "op");
    c.name = get_string(json, "name");
    c.dtype = get_string(json, "dtype");
    c.node = get_string(json, "node");
    c.device = get_int(json, "device");
    c.pid = get_int(json, "pid");
    c.has_shape = get_shape(json, c.shape);
    return !c.op.empty() && !c.name.empty();
}
int put(const std::string &s, char *out, size_t cap) {
    if (!out || cap == 0) return 0;
    if (s.size() + 1 > cap) return fail(-5, "reply does not fit");
    std::memcpy(out, s.c_str(), s.size() + 1);
    return 0;
}
}  // namespace

extern "C" {

dx_heap *dx_heap_create(const char *node, int backing) {
    if (backing != DX_HEAP_DEVICE && backing != DX_HEAP_HOST_FAKE) {
        fail(-3, "unknown backing");
        return nullptr;
    }
    auto *h = new dx_heap();
    h->backing = backing;
    if (node && *node) h->node = node;
    else {
        char buf[256] = {0};
        gethostname(buf, sizeof(buf) - 1);
        h->node = buf;
    }
    return h;
}

void dx_heap_destroy(dx_heap *h) {
    if (!h) return;
    {
        std::lock_guard<std::mutex> lk(h->store.mu);
        std::vector<std::string> names;
        for (auto &p : h->ptrs) names.push_back(p.first);
        for (auto &n : names) h->drop_locked(n);
    }
    delete h;
}

const char *dx_heap_last_error(void) { return g_err.c_str(); }

int dx_heap_command(dx_heap *h, const char *json, char *reply, size_t cap) {
    if (!h || !json) return fail(-3, "null heap or command");
    Command c;
    if (!parse_command(json, c)) return fail(-3, "command needs \"op\" and \"name\"");
    std::string text;
    if (int e = h->handle(c, &text)) return e;
    return put(text, reply, cap);
}

int dx_heap_push(dx_heap *h, const char *json) {
    if (!h || !json) return fail(-3, "null heap or command");
    h->store.lpush(json);
    return 0;
}

int dx_heap_run_once(dx_heap *h, int timeout_ms) {
    if (!h) return fail(-3, "null heap");
    std::string msg;
    if (!h->store.brpop(timeout_ms < 0 ? 0 : timeout_ms, msg)) return 0;
    Command c;
    if (parse_command(msg, c)) h->handle(c, nullptr);  // a worker has nobody to report to: bad commands are dropped (lifecycle.cpp:68-71)
    return 1;
}

int dx_heap_meta(dx_heap *h, const char *name, char *out, size_t cap) {
    if (!h || !name) return fail(-3, "null heap or name");
    std::lock_guard<std::mutex> lk(h->store.mu);
    auto it = h->store.hashes.find(dx_heap::key(name));
    if (it == h->store.hashes.end()) return fail(-1, std::string("no tensor named ") + name);
    return put(h->render(name, it->second), out, cap);
}

int dx_heap_count(dx_heap *h) {
    if (!h) return 0;
    std::lock_guard<std::mutex> lk(h->store.mu);
    return int(h->store.hashes.size());
}

void *dx_heap_ptr(dx_heap *h, const char *name) {
    if (!h || !name) return nullptr;
    std::lock_guard<std::mutex> lk(h->store.mu);
    auto it = h->ptrs.find(name);
    return it == h->ptrs.end() ? nullptr : it->second;
}

int64_t dx_heap_gc_sweep(dx_heap *h, const char *node) {
    if (!h) return 0;
    const std::string which = node && *node ? node : h->node;
    std::lock_guard<std::mutex> lk(h->store.mu);
    std::vector<std::string> dead;
    for (auto &kv : h->store.hashes) {
        Hash &f = kv.second;
        if (f["node"] != which) continue;
        const long long pid = std::atoll(f["owner_pid"].c_str());
        const bool owner_gone = which == h->node && pid > 0 && kill(pid_t(pid), 0) != 0 && errno == ESRCH;
        if (std::atoll(f["refcount"].c_str()) <= 0 || owner_gone) dead.push_back(kv.first.substr(7));
    }
    for (auto &n : dead) h->drop_locked(n);
    return int64_t(dead.size());
}

void *dx_heap_open(const char *ipc_handle_hex, int device) {
    cudaIpcMemHandle_t hd;
    if (!ipc_handle_hex || !from_hex(ipc_handle_hex, &hd, sizeof(hd))) {
        fail(-3, "ipc handle must be " + std::to_string(2 * sizeof(hd)) + " hex digits");
        return nullptr;
    }
    void *ptr = nullptr;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaIpcOpenMemHandle(&ptr, hd, cudaIpcMemLazyEnablePeerAccess);
    if (prev >= 0 && prev != device) cudaSetDevice(prev);  // the caller's current device is left as it was
    if (e != cudaSuccess) {
        fail(-4, std::string("cudaIpcOpenMemHandle: ") + cudaGetErrorString(e));
        return nullptr;
    }
    return ptr;
}

int dx_heap_close(void *ptr) {
    if (!ptr) return 0;
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? 0 : fail(-4, std::string("cudaIpcCloseMemHandle: ") + cudaGetErrorString(e));
}

int dx_heap_copy(void *dst, const void *src, size_t bytes, int to_device) {
    if (!dst || !src) return fail(-3, "null pointer");
    const cudaError_t e = cudaMemcpy(dst, src, bytes, to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost);
    return e == cudaSuccess ? 0 : fail(-4, std::string("cudaMemcpy: ") + cudaGetErrorString(e));
}
}
