// The heap-tensor service: registry (hash `tensor:<name>`), lifecycle commands (list
// `tensor_lifecycle`) and CUDA-IPC export, after the sketch in executor/heapmem-cuda
// (registry/registry.h:11-51, registry.cpp:11-86, runtime/lifecycle.cpp:9-85, README.md:13-46).
// Interface and field list: include/dx_heapmem.h.
//
// What the reference keeps in Redis — one string→string map per `tensor:<name>` key and one list of
// JSON commands — sits behind `Store` (HSET/HGETALL/DEL/KEYS, LPUSH/BRPOP).  Two stores exist: an
// in-process one, and a Redis server reached with the Redis wire protocol (RESP2) over a plain TCP socket
// (no client library).  With the server between them, the SERVICE process (`deepx-heapmem`, or any
// process that calls dx_heap_run_once in a loop) is the only writer of the hashes: it pops commands off
// the list one at a time, so create-or-get, refcount+1 and refcount-1 are atomic without the Lua scripts
// the reference's registry evaluates (registry.cpp:24-66; the scripts themselves are not in its tree).
// Clients in other processes push commands (dx_heap_request) and read hashes (dx_heap_lookup).
#include <cuda_runtime.h>
#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cctype>
#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
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

struct Store {  // the part Redis plays
    virtual ~Store() = default;
    virtual bool hgetall(const std::string &key, Hash &out) = 0;  // false: no such key
    virtual void hset(const std::string &key, const Hash &fields) = 0;
    virtual void del(const std::string &key) = 0;
    virtual std::vector<std::string> keys(const std::string &prefix) = 0;
    virtual void lpush(const std::string &list, const std::string &v) = 0;
    virtual bool brpop(const std::string &list, int timeout_ms, std::string &out) = 0;
};

struct LocalStore : Store {
    std::mutex mu;
    std::condition_variable cv;
    std::map<std::string, Hash> hashes;
    std::map<std::string, std::deque<std::string>> lists;  // pushed at the front, popped at the back
    bool hgetall(const std::string &key, Hash &out) override {
        std::lock_guard<std::mutex> lk(mu);
        auto it = hashes.find(key);
        if (it == hashes.end()) return false;
        out = it->second;
        return true;
    }
    void hset(const std::string &key, const Hash &fields) override {
        std::lock_guard<std::mutex> lk(mu);
        Hash &h = hashes[key];
        for (auto &kv : fields) h[kv.first] = kv.second;
    }
    void del(const std::string &key) override {
        std::lock_guard<std::mutex> lk(mu);
        hashes.erase(key);
    }
    std::vector<std::string> keys(const std::string &prefix) override {
        std::lock_guard<std::mutex> lk(mu);
        std::vector<std::string> out;
        for (auto &kv : hashes)
            if (kv.first.compare(0, prefix.size(), prefix) == 0) out.push_back(kv.first);
        return out;
    }
    void lpush(const std::string &list, const std::string &v) override {
        { std::lock_guard<std::mutex> lk(mu); lists[list].push_front(v); }
        cv.notify_one();
    }
    bool brpop(const std::string &list, int timeout_ms, std::string &out) override {
        std::unique_lock<std::mutex> lk(mu);
        auto &q = lists[list];
        if (!cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return !q.empty(); })) return false;
        out = q.back();
        q.pop_back();
        return true;
    }
};

// ---- RESP2 over TCP: the subset the registry needs (PING, HSET, HGETALL, DEL, KEYS, LPUSH, BRPOP) --------------
struct RespReply {
    enum Kind { NIL, TEXT, INTEGER, ARRAY, ERROR } kind = NIL;
    std::string text;
    long long integer = 0;
    std::vector<RespReply> items;
};

class RespClient {
  public:
    RespClient(const std::string &host, int port, int timeout_ms) : timeout_ms_(timeout_ms) {
        addrinfo hints{}, *res = nullptr;
        hints.ai_family = AF_UNSPEC;
        hints.ai_socktype = SOCK_STREAM;
        if (getaddrinfo(host.c_str(), std::to_string(port).c_str(), &hints, &res) != 0 || !res) throw std::runtime_error("cannot resolve " + host);
        for (addrinfo *a = res; a; a = a->ai_next) {
            fd_ = socket(a->ai_family, a->ai_socktype, a->ai_protocol);
            if (fd_ < 0) continue;
            if (connect(fd_, a->ai_addr, a->ai_addrlen) == 0) break;
            close(fd_);
            fd_ = -1;
        }
        freeaddrinfo(res);
        if (fd_ < 0) throw std::runtime_error("cannot connect to " + host + ":" + std::to_string(port));
        int one = 1;
        setsockopt(fd_, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        set_timeout(timeout_ms_);
    }
    ~RespClient() { if (fd_ >= 0) close(fd_); }
    RespClient(const RespClient &) = delete;
    RespClient &operator=(const RespClient &) = delete;

    // `extra_wait_ms`: a blocking command may take that much longer than the usual reply
    RespReply command(const std::vector<std::string> &args, int extra_wait_ms = 0) {
        std::string out = "*" + std::to_string(args.size()) + "\r\n";
        for (const auto &a : args) out += "$" + std::to_string(a.size()) + "\r\n" + a + "\r\n";
        size_t done = 0;
        while (done < out.size()) {
            const ssize_t n = send(fd_, out.data() + done, out.size() - done, MSG_NOSIGNAL);
            if (n <= 0) throw std::runtime_error("connection to the store lost while sending");
            done += size_t(n);
        }
        if (extra_wait_ms) set_timeout(timeout_ms_ + extra_wait_ms);
        RespReply r;
        try {
            r = read_reply();
        } catch (...) {
            if (extra_wait_ms) set_timeout(timeout_ms_);
            throw;
        }
        if (extra_wait_ms) set_timeout(timeout_ms_);
        if (r.kind == RespReply::ERROR) throw std::runtime_error("store: " + r.text);
        return r;
    }

  private:
    int fd_ = -1, timeout_ms_;
    std::string buf_;
    size_t pos_ = 0;
    void set_timeout(int ms) {
        timeval tv{ms / 1000, (ms % 1000) * 1000};
        setsockopt(fd_, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    }
    void fill() {
        if (pos_ > 0 && pos_ == buf_.size()) { buf_.clear(); pos_ = 0; }
        char tmp[4096];
        ssize_t n;
        do n = recv(fd_, tmp, sizeof(tmp), 0);
        while (n < 0 && errno == EINTR);
        if (n <= 0) throw std::runtime_error(n == 0 ? "the store closed the connection" : "no reply from the store in time");
        buf_.append(tmp, size_t(n));
    }
    std::string line() {
        for (;;) {
            const size_t e = buf_.find("\r\n", pos_);
            if (e != std::string::npos) {
                std::string l = buf_.substr(pos_, e - pos_);
                pos_ = e + 2;
                return l;
            }
            fill();
        }
    }
    RespReply read_reply() {
        const std::string l = line();
        if (l.empty()) throw std::runtime_error("malformed reply from the store");
        RespReply r;
        const std::string rest = l.substr(1);
        switch (l[0]) {
            case '+': r.kind = RespReply::TEXT; r.text = rest; return r;
            case '-': r.kind = RespReply::ERROR; r.text = rest; return r;
            case ':': r.kind = RespReply::INTEGER; r.integer = std::atoll(rest.c_str()); return r;
            case '$': {
                const long long n = std::atoll(rest.c_str());
                if (n < 0) return r;  // nil
                while (buf_.size() - pos_ < size_t(n) + 2) fill();
                r.kind = RespReply::TEXT;
                r.text = buf_.substr(pos_, size_t(n));
                pos_ += size_t(n) + 2;
                return r;
            }
            case '*': {
                const long long n = std::atoll(rest.c_str());
                if (n < 0) return r;  // nil array (BRPOP timeout)
                r.kind = RespReply::ARRAY;
                for (long long i = 0; i < n; ++i) r.items.push_back(read_reply());
                return r;
            }
            default: throw std::runtime_error("malformed reply from the store");
        }
    }
};

struct RedisStore : Store {
    RespClient client;
    RedisStore(const std::string &host, int port) : client(host, port, 5000) {
        const RespReply r = client.command({"PING"});
        if (r.text != "PONG") throw std::runtime_error("the store did not answer PING with PONG");
    }
    bool hgetall(const std::string &key, Hash &out) override {
        const RespReply r = client.command({"HGETALL", key});
        out.clear();
        for (size_t i = 0; i + 1 < r.items.size(); i += 2) out[r.items[i].text] = r.items[i + 1].text;
        return !out.empty();
    }
    void hset(const std::string &key, const Hash &fields) override {
        std::vector<std::string> cmd{"HSET", key};
        for (auto &kv : fields) {
            cmd.push_back(kv.first);
            cmd.push_back(kv.second);
        }
        if (cmd.size() > 2) client.command(cmd);
    }
    void del(const std::string &key) override { client.command({"DEL", key}); }
    std::vector<std::string> keys(const std::string &prefix) override {
        const RespReply r = client.command({"KEYS", prefix + "*"});
        std::vector<std::string> out;
        for (auto &it : r.items) out.push_back(it.text);
        return out;
    }
    void lpush(const std::string &list, const std::string &v) override { client.command({"LPUSH", list, v}); }
    bool brpop(const std::string &list, int timeout_ms, std::string &out) override {
        // BRPOP counts in seconds (0 = for ever): at least one, rounded up
        const int secs = timeout_ms <= 0 ? 1 : (timeout_ms + 999) / 1000;
        const RespReply r = client.command({"BRPOP", list, std::to_string(secs)}, secs * 1000);
        if (r.kind != RespReply::ARRAY || r.items.size() < 2) return false;
        out = r.items[1].text;
        return true;
    }
};

const char *const LIFECYCLE_LIST = "tensor_lifecycle";  // executor/heapmem-cuda/README.md:13

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
    std::unique_ptr<Store> store;
    std::mutex mu;                       // one command at a time in this process
    std::map<std::string, void *> ptrs;  // owner-side pointers; guarded by mu

    static std::string key(const std::string &name) { return "tensor:" + name; }  // Registry::Key, registry.cpp:13-15

    static std::string render(const std::string &name, const Hash &h) {
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
        int prev = -1;
        cudaGetDevice(&prev);
        cudaError_t e = cudaSetDevice(int(device));
        if (e == cudaSuccess) e = cudaMalloc(ptr, bytes ? bytes : 1);
        cudaIpcMemHandle_t hd;
        if (e == cudaSuccess) {
            e = cudaIpcGetMemHandle(&hd, *ptr);
            if (e != cudaSuccess) {
                cudaFree(*ptr);
                *ptr = nullptr;
            }
        }
        if (prev >= 0 && prev != int(device)) cudaSetDevice(prev);
        if (e != cudaSuccess) return fail(-4, std::string("heap tensor allocation: ") + cudaGetErrorString(e));
        *handle_hex = to_hex(&hd, sizeof(hd));
        return 0;
    }

    void release(void *ptr, long long device) {
        if (!ptr) return;
        if (backing == DX_HEAP_HOST_FAKE) {
            std::free(ptr);
            return;
        }
        int prev = -1;
        cudaGetDevice(&prev);
        cudaSetDevice(int(device));
        cudaFree(ptr);
        if (prev >= 0 && prev != int(device)) cudaSetDevice(prev);
    }

    // drop hash + memory; mu held
    void drop_locked(const std::string &name) {
        Hash h;
        long long device = 0;
        if (store->hgetall(key(name), h)) {
            device = std::atoll(h["device"].c_str());
            store->del(key(name));
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
        std::lock_guard<std::mutex> lk(mu);
        Hash h;
        const bool exists = store->hgetall(key(c.name), h);
        if (c.op == "create") {
            if (exists) {  // create-or-get (Registry::CreateOrGet, registry.cpp:24-45)
                if ((!c.dtype.empty() && dtype_bytes(c.dtype) != dtype_bytes(h["dtype"])) || (c.has_shape && shape_text(c.shape) != h["shape"]))
                    return fail(-2, "tensor " + c.name + " exists as " + h["dtype"] + h["shape"] + ", asked for " + c.dtype + shape_text(c.shape));
                h["refcount"] = std::to_string(std::atoll(h["refcount"].c_str()) + 1);
                store->hset(key(c.name), {{"refcount", h["refcount"]}});
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
            h.clear();
            h["dtype"] = c.dtype;
            h["shape"] = shape_text(c.shape);
            h["ctime"] = std::to_string(std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count());
            h["node"] = c.node.empty() ? node : c.node;
            h["device"] = std::to_string(c.device);
            h["bytes"] = std::to_string(nbytes);
            h["ipc_handle"] = hex;
            h["refcount"] = "1";
            h["state"] = "ready";
            h["owner_pid"] = std::to_string(c.pid ? c.pid : (long long)getpid());  // whose death releases the tensor (dx_heap_gc_sweep)
            store->hset(key(c.name), h);
            ptrs[c.name] = ptr;
            if (reply) *reply = render(c.name, h);
            return 0;
        }
        if (!exists) return fail(-1, c.op + ": no tensor named " + c.name);
        if (c.op == "get") {  // Registry::RefInc, registry.cpp:47-52
            h["refcount"] = std::to_string(std::atoll(h["refcount"].c_str()) + 1);
            store->hset(key(c.name), {{"refcount", h["refcount"]}});
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
            } else {
                store->hset(key(c.name), {{"refcount", h["refcount"]}});
                if (reply) *reply = render(c.name, h);
            }
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

static std::string host_name() {
    char buf[256] = {0};
    gethostname(buf, sizeof(buf) - 1);
    return buf;
}

extern "C" {

dx_heap *dx_heap_create(const char *node, int backing) {
    if (backing != DX_HEAP_DEVICE && backing != DX_HEAP_HOST_FAKE) {
        fail(-3, "unknown backing");
        return nullptr;
    }
    auto *h = new dx_heap();
    h->backing = backing;
    h->store = std::make_unique<LocalStore>();
    h->node = node && *node ? node : host_name();
    return h;
}

dx_heap *dx_heap_create_redis(const char *node, int backing, const char *host, int port) {
    if (backing != DX_HEAP_DEVICE && backing != DX_HEAP_HOST_FAKE) {
        fail(-3, "unknown backing");
        return nullptr;
    }
    try {
        auto store = std::make_unique<RedisStore>(host && *host ? host : "127.0.0.1", port > 0 ? port : 6379);
        auto *h = new dx_heap();
        h->backing = backing;
        h->store = std::move(store);
        h->node = node && *node ? node : host_name();
        return h;
    } catch (const std::exception &e) {
        fail(-4, e.what());
        return nullptr;
    }
}

void dx_heap_destroy(dx_heap *h) {
    if (!h) return;
    try {
        std::lock_guard<std::mutex> lk(h->mu);
        std::vector<std::string> names;
        for (auto &p : h->ptrs) names.push_back(p.first);
        for (auto &n : names) h->drop_locked(n);
    } catch (const std::exception &) {
        // the store is unreachable: the memory is released with the process
    }
    delete h;
}

const char *dx_heap_last_error(void) { return g_err.c_str(); }

int dx_heap_command(dx_heap *h, const char *json, char *reply, size_t cap) {
    if (!h || !json) return fail(-3, "null heap or command");
    Command c;
    if (!parse_command(json, c)) return fail(-3, "command needs \"op\" and \"name\"");
    std::string text;
    try {
        if (int e = h->handle(c, &text)) return e;
    } catch (const std::exception &e) {
        return fail(-4, e.what());
    }
    return put(text, reply, cap);
}

int dx_heap_push(dx_heap *h, const char *json) {
    if (!h || !json) return fail(-3, "null heap or command");
    try {
        h->store->lpush(LIFECYCLE_LIST, json);
    } catch (const std::exception &e) {
        return fail(-4, e.what());
    }
    return 0;
}

int dx_heap_run_once(dx_heap *h, int timeout_ms) {
    if (!h) return fail(-3, "null heap");
    std::string msg;
    try {
        if (!h->store->brpop(LIFECYCLE_LIST, timeout_ms < 0 ? 0 : timeout_ms, msg)) return 0;
        Command c;
        if (parse_command(msg, c)) h->handle(c, nullptr);  // a worker has nobody to report to: bad commands are dropped (lifecycle.cpp:68-71)
    } catch (const std::exception &e) {
        return fail(-4, e.what());
    }
    return 1;
}

int dx_heap_meta(dx_heap *h, const char *name, char *out, size_t cap) {
    if (!h || !name) return fail(-3, "null heap or name");
    try {
        std::lock_guard<std::mutex> lk(h->mu);
        Hash f;
        if (!h->store->hgetall(dx_heap::key(name), f)) return fail(-1, std::string("no tensor named ") + name);
        return put(dx_heap::render(name, f), out, cap);
    } catch (const std::exception &e) {
        return fail(-4, e.what());
    }
}

int dx_heap_count(dx_heap *h) {
    if (!h) return 0;
    try {
        std::lock_guard<std::mutex> lk(h->mu);
        return int(h->store->keys("tensor:").size());
    } catch (const std::exception &) {
        return 0;
    }
}

void *dx_heap_ptr(dx_heap *h, const char *name) {
    if (!h || !name) return nullptr;
    std::lock_guard<std::mutex> lk(h->mu);
    auto it = h->ptrs.find(name);
    return it == h->ptrs.end() ? nullptr : it->second;
}

int64_t dx_heap_gc_sweep(dx_heap *h, const char *node) {
    if (!h) return 0;
    const std::string which = node && *node ? node : h->node;
    try {
        std::lock_guard<std::mutex> lk(h->mu);
        std::vector<std::string> dead;
        for (const auto &k : h->store->keys("tensor:")) {
            Hash f;
            if (!h->store->hgetall(k, f) || f["node"] != which) continue;
            const long long pid = std::atoll(f["owner_pid"].c_str());
            const bool owner_gone = which == h->node && pid > 0 && kill(pid_t(pid), 0) != 0 && errno == ESRCH;
            if (std::atoll(f["refcount"].c_str()) <= 0 || owner_gone) dead.push_back(k.substr(7));
        }
        for (auto &n : dead) h->drop_locked(n);
        return int64_t(dead.size());
    } catch (const std::exception &e) {
        return fail(-4, e.what());
    }
}

// ---- the client side of a store-backed service: other processes of the machine -------------------------------
int dx_heap_request(const char *host, int port, const char *json) {
    if (!json) return fail(-3, "null command");
    Command c;
    if (!parse_command(json, c)) return fail(-3, "command needs \"op\" and \"name\"");
    try {
        RedisStore store(host && *host ? host : "127.0.0.1", port > 0 ? port : 6379);
        store.lpush(LIFECYCLE_LIST, json);
        return 0;
    } catch (const std::exception &e) {
        return fail(-4, e.what());
    }
}

int dx_heap_lookup(const char *host, int port, const char *name, char *out, size_t cap) {
    if (!name) return fail(-3, "null name");
    try {
        RedisStore store(host && *host ? host : "127.0.0.1", port > 0 ? port : 6379);
        Hash f;
        if (!store.hgetall(dx_heap::key(name), f)) return fail(-1, std::string("no tensor named ") + name);
        return put(dx_heap::render(name, f), out, cap);
    } catch (const std::exception &e) {
        return fail(-4, e.what());
    }
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
