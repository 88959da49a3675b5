// dx_comm: the exchange step of a reduction that crosses the sharded axis, done by the GPUs
// themselves over NVLink peer memory instead of by a library collective.
//
// Each rank (one process per GPU) owns a MAILBOX in its own device memory, exported with CUDA IPC
// and mapped by every peer.  An all-reduce of a small buffer (the per-rank partials of a global
// sum, a few KB at most for an axis-0 reduce of a narrow tensor) is ONE kernel per rank:
//   1. every CTA takes one 4 KiB chunk, reads it from the local buffer and stores it into slot
//      [parity][my rank] of EVERY rank's mailbox (plain 16-byte st.global to peer memory; no TMA,
//      no multicast, no library call on peer pointers);
//   2. fence, then one thread per peer publishes flag[parity][my rank][chunk] = epoch there
//      (st.release.sys);
//   3. one thread per peer waits (ld.acquire.sys, clock-bounded) until its own mailbox shows this
//      epoch from that peer;
//   4. the CTA combines the W slots in rank order 0..W-1 (so every rank computes the same bits)
//      and writes the result back over the local buffer.
// Slots and flags are double-buffered by epoch parity: a rank can start epoch e+1 while a peer
// still reads epoch e, and cannot reach e+2 before every peer has published e+1, i.e. finished
// reading e.  The epoch of a chunk lives in the mailbox and is advanced by the kernel itself, so a
// captured launch can be replayed.
//
// The exchange comes in two halves (comm.cuh): publish (steps 1–2) and combine (steps 3–4).  One kernel can
// do both, or a reduction can end with the publish (dx_reduce_allreduce_begin) and the combine runs as a
// kernel of its own later on the stream (dx_comm_allreduce_finish): the kernels in between hide the skew
// between the ranks, which otherwise shows up as a wait in every step.  Buffers larger than a slot take
// several rounds of the same kernel.  dx_comm_allgather_rows moves row blocks instead of combining values:
// every rank fills its own rows of a buffer that all ranks hold, and fetches the others'.
//
// Every wait is bounded (default 2 s, dx_comm_set_timeout_ms); when one expires the kernel records
// which (chunk, peer) it gave up on, skips the combine and returns, and dx_comm_status reports it.
// The reference has no multi-GPU code at all; the alternative here is an NCCL all-reduce of the
// same partial, which deepx_b200/sharded.py uses for buffers larger than a mailbox slot.
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "comm.cuh"

namespace dx {
namespace {

// One launch per rank: blockIdx.x = chunk.
template <int OP, typename T>
__global__ void __launch_bounds__(COMM_THREADS) peer_allreduce_kernel(Peers peers, int rank, T *buf, int64_t n, long long wait_cycles) {
    exchange_chunk<OP, T>(peers, rank, blockIdx.x, buf, n, wait_cycles);
}

template <typename T>
__global__ void __launch_bounds__(COMM_THREADS) peer_publish_kernel(Peers peers, int rank, const T *buf, int64_t n, T pad) {
    exchange_publish<T>(peers, rank, blockIdx.x, buf, n, pad);
}
template <int OP, typename T>
__global__ void __launch_bounds__(COMM_THREADS) peer_combine_kernel(Peers peers, int rank, T *buf, int64_t n, long long wait_cycles) {
    griddep_wait_cta();
    exchange_combine<OP, T>(peers, rank, blockIdx.x, buf, n, wait_cycles);
}
__global__ void __launch_bounds__(COMM_THREADS) peer_gather_kernel(Peers peers, int rank, unsigned char *buf, GatherPlan plan, long long wait_cycles) {
    gather_chunk(peers, rank, blockIdx.x, buf, plan, wait_cycles);
}

// All ranks in ONE launch on one GPU (blockIdx.y = rank), every mailbox local: the same protocol
// where there are fewer GPUs than ranks.  Ranks >= `active` are left out, so that the others'
// waits run into their limit (the failure path, without a second process that misbehaves).
struct Bufs {
    void *buf[COMM_MAX_WORLD];
};
template <int OP, typename T>
__global__ void __launch_bounds__(COMM_THREADS) emulated_allreduce_kernel(Peers peers, Bufs bufs, int active, int64_t n, long long wait_cycles) {
    if (int(blockIdx.y) >= active) return;
    exchange_chunk<OP, T>(peers, blockIdx.y, blockIdx.x, static_cast<T *>(bufs.buf[blockIdx.y]), n, wait_cycles);
}

template <typename T>
__global__ void __launch_bounds__(COMM_THREADS) emulated_publish_kernel(Peers peers, Bufs bufs, int active, int64_t n, T pad) {
    if (int(blockIdx.y) >= active) return;
    exchange_publish<T>(peers, blockIdx.y, blockIdx.x, static_cast<const T *>(bufs.buf[blockIdx.y]), n, pad);
}
template <int OP, typename T>
__global__ void __launch_bounds__(COMM_THREADS) emulated_combine_kernel(Peers peers, Bufs bufs, int active, int64_t n, long long wait_cycles) {
    if (int(blockIdx.y) >= active) return;
    exchange_combine<OP, T>(peers, blockIdx.y, blockIdx.x, static_cast<T *>(bufs.buf[blockIdx.y]), n, wait_cycles);
}
__global__ void __launch_bounds__(COMM_THREADS) emulated_gather_kernel(Peers peers, Bufs bufs, GatherPlan plan, long long wait_cycles) {
    gather_chunk(peers, blockIdx.y, blockIdx.x, static_cast<unsigned char *>(bufs.buf[blockIdx.y]), plan, wait_cycles);
}

}  // namespace
}  // namespace dx

struct dx_comm {
    int rank = 0, world = 1, device = 0;
    dx::Mailbox *mine = nullptr;
    dx::Peers peers{};
    bool opened[dx::COMM_MAX_WORLD] = {};
    bool connected = false;
    long long wait_cycles = 4000000000ll;
    std::vector<dx::Mailbox *> emulated;  // dx_comm_emulate: all mailboxes local
    // an exchange that has been published and still waits for its combine
    bool pending = false;
    int pending_op = 0, pending_dtype = 0;
    void *pending_buf = nullptr;
    int64_t pending_n = 0;
};

namespace dx {
namespace {

template <int OP, typename T> int launch_real(dx_comm *c, void *buf, int64_t n, cudaStream_t st) {
    constexpr int PER = COMM_CHUNK / int(sizeof(T));
    const int chunks = int((n + PER - 1) / PER);
    peer_allreduce_kernel<OP, T><<<chunks, COMM_THREADS, 0, st>>>(c->peers, c->rank, static_cast<T *>(buf), n, c->wait_cycles);
    return check_launch("comm allreduce");
}
template <int OP, typename T> int launch_emulated(dx_comm *c, void *const *bufs, int active, int64_t n, cudaStream_t st) {
    constexpr int PER = COMM_CHUNK / int(sizeof(T));
    const int chunks = int((n + PER - 1) / PER);
    Bufs b{};
    for (int r = 0; r < c->world; ++r) b.buf[r] = bufs[r];
    emulated_allreduce_kernel<OP, T><<<dim3(chunks, c->world), COMM_THREADS, 0, st>>>(c->peers, b, active, n, c->wait_cycles);
    return check_launch("comm allreduce (emulated ranks)");
}

template <int OP, typename T> int launch_publish(dx_comm *c, void *buf, int64_t n, cudaStream_t st) {
    constexpr int PER = COMM_CHUNK / int(sizeof(T));
    const int chunks = int((n + PER - 1) / PER);
    peer_publish_kernel<T><<<chunks, COMM_THREADS, 0, st>>>(c->peers, c->rank, static_cast<const T *>(buf), n, narrow<T>(identity<OP, T>()));
    return check_launch("comm publish");
}
template <int OP, typename T> int launch_combine(dx_comm *c, void *buf, int64_t n, cudaStream_t st) {
    constexpr int PER = COMM_CHUNK / int(sizeof(T));
    const int chunks = int((n + PER - 1) / PER);
    launch_pdl(peer_combine_kernel<OP, T>, dim3(chunks), dim3(COMM_THREADS), 0, st, c->peers, c->rank, static_cast<T *>(buf), n, c->wait_cycles);
    return check_launch("comm combine");
}
template <int OP, typename T> int launch_emulated_publish(dx_comm *c, void *const *bufs, int active, int64_t n, cudaStream_t st) {
    constexpr int PER = COMM_CHUNK / int(sizeof(T));
    const int chunks = int((n + PER - 1) / PER);
    Bufs b{};
    for (int r = 0; r < c->world; ++r) b.buf[r] = bufs[r];
    emulated_publish_kernel<T><<<dim3(chunks, c->world), COMM_THREADS, 0, st>>>(c->peers, b, active, n, narrow<T>(identity<OP, T>()));
    return check_launch("comm publish (emulated ranks)");
}
template <int OP, typename T> int launch_emulated_combine(dx_comm *c, void *const *bufs, int active, int64_t n, cudaStream_t st) {
    constexpr int PER = COMM_CHUNK / int(sizeof(T));
    const int chunks = int((n + PER - 1) / PER);
    Bufs b{};
    for (int r = 0; r < c->world; ++r) b.buf[r] = bufs[r];
    emulated_combine_kernel<OP, T><<<dim3(chunks, c->world), COMM_THREADS, 0, st>>>(c->peers, b, active, n, c->wait_cycles);
    return check_launch("comm combine (emulated ranks)");
}

#define DX_COMM_BY_OP(FN, T, ...)                                             \
    switch (op) {                                                             \
        case DX_SUM: return FN<DX_SUM, T>(__VA_ARGS__);                       \
        case DX_PROD: return FN<DX_PROD, T>(__VA_ARGS__);                     \
        case DX_RMAX: return FN<DX_RMAX, T>(__VA_ARGS__);                     \
        case DX_RMIN: return FN<DX_RMIN, T>(__VA_ARGS__);                     \
        default: return fail(DX_E_ARG, "comm: unknown reduce op %d", op);     \
    }
#define DX_COMM_DISPATCH(FN, ...)                                             \
    switch (dtype) {                                                          \
        case DX_F64: DX_COMM_BY_OP(FN, double, __VA_ARGS__)                   \
        case DX_F32: DX_COMM_BY_OP(FN, float, __VA_ARGS__)                    \
        case DX_F16: DX_COMM_BY_OP(FN, f16, __VA_ARGS__)                      \
        case DX_BF16: DX_COMM_BY_OP(FN, bf16, __VA_ARGS__)                    \
        case DX_I64: DX_COMM_BY_OP(FN, int64_t, __VA_ARGS__)                  \
        case DX_I32: DX_COMM_BY_OP(FN, int32_t, __VA_ARGS__)                  \
        case DX_I16: DX_COMM_BY_OP(FN, int16_t, __VA_ARGS__)                  \
        case DX_I8: DX_COMM_BY_OP(FN, int8_t, __VA_ARGS__)                    \
        default: return fail(DX_E_DTYPE, "comm: unsupported dtype code %d", dtype); \
    }

int real_dispatch(dx_comm *c, int op, int dtype, void *buf, int64_t n, cudaStream_t st) { DX_COMM_DISPATCH(launch_real, c, buf, n, st) }
int emulated_dispatch(dx_comm *c, int op, int dtype, void *const *bufs, int active, int64_t n, cudaStream_t st) {
    DX_COMM_DISPATCH(launch_emulated, c, bufs, active, n, st)
}

int publish_dispatch(dx_comm *c, int op, int dtype, void *buf, int64_t n, cudaStream_t st) { DX_COMM_DISPATCH(launch_publish, c, buf, n, st) }
int combine_dispatch(dx_comm *c, int op, int dtype, void *buf, int64_t n, cudaStream_t st) { DX_COMM_DISPATCH(launch_combine, c, buf, n, st) }
int emulated_publish_dispatch(dx_comm *c, int op, int dtype, void *const *bufs, int active, int64_t n, cudaStream_t st) {
    DX_COMM_DISPATCH(launch_emulated_publish, c, bufs, active, n, st)
}
int emulated_combine_dispatch(dx_comm *c, int op, int dtype, void *const *bufs, int active, int64_t n, cudaStream_t st) {
    DX_COMM_DISPATCH(launch_emulated_combine, c, bufs, active, n, st)
}

int check_size(int dtype, int64_t n) {
    const int es = dx_dtype_size(dtype);
    if (es == 0 || dtype == DX_BOOL) return fail(DX_E_DTYPE, "comm: unsupported dtype code %d", dtype);
    if (n < 0) return fail(DX_E_SHAPE, "comm: negative count");
    if (n * es > COMM_SLOT) return fail(DX_E_WORKSPACE, "comm: %lld bytes exceed the %d-byte mailbox slot (use a library all-reduce)", (long long)(n * es), COMM_SLOT);
    return DX_OK;
}

int new_mailbox(Mailbox **out) {
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, sizeof(Mailbox));
    if (e == cudaSuccess) e = cudaMemset(p, 0, sizeof(Mailbox));
    if (e != cudaSuccess) return fail(DX_E_CUDA, "comm: mailbox allocation: %s", cudaGetErrorString(e));
    *out = static_cast<Mailbox *>(p);
    return DX_OK;
}

}  // namespace
}  // namespace dx

namespace dx {
bool comm_device_view(dx_comm *c, Peers *peers, int *rank, long long *wait_cycles) {
    if (!c || !c->connected || !c->emulated.empty()) return false;
    *peers = c->peers;
    *rank = c->rank;
    *wait_cycles = c->wait_cycles;
    return true;
}
void comm_set_pending(dx_comm *c, int op, int dtype, void *buf, int64_t n) {
    c->pending = true;
    c->pending_op = op;
    c->pending_dtype = dtype;
    c->pending_buf = buf;
    c->pending_n = n;
}
int comm_flush_pending(dx_comm *c, cudaStream_t st) {
    if (!c || !c->pending) return DX_OK;
    c->pending = false;
    return combine_dispatch(c, c->pending_op, c->pending_dtype, c->pending_buf, c->pending_n, st);
}
}  // namespace dx

using namespace dx;

extern "C" size_t dx_comm_max_bytes(void) { return COMM_SLOT; }

extern "C" dx_comm *dx_comm_create(int rank, int world, int device) {
    if (world < 1 || world > COMM_MAX_WORLD || rank < 0 || rank >= world) {
        fail(DX_E_ARG, "comm: rank %d of %d (at most %d ranks)", rank, world, COMM_MAX_WORLD);
        return nullptr;
    }
    DeviceGuard guard(device);  // the caller's current device is left as it was
    int now = -1;
    if (cudaGetDevice(&now) != cudaSuccess || now != device) {
        fail(DX_E_CUDA, "comm: cannot make device %d current: %s", device, cudaGetErrorString(cudaGetLastError()));
        return nullptr;
    }
    dx_comm *c = new (std::nothrow) dx_comm();
    if (!c) return nullptr;
    c->rank = rank;
    c->world = world;
    c->device = device;
    if (new_mailbox(&c->mine) != DX_OK) {
        delete c;
        return nullptr;
    }
    c->peers.world = world;
    c->peers.box[rank] = c->mine;
    c->connected = world == 1;
    return c;
}

extern "C" int dx_comm_handle(dx_comm *c, unsigned char out[64]) {
    if (!c || !out) return fail(DX_E_ARG, "comm: null argument");
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "IPC handle size");
    const cudaError_t e = cudaIpcGetMemHandle(&h, c->mine);
    if (e != cudaSuccess) return fail(DX_E_CUDA, "comm: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    std::memcpy(out, &h, 64);
    return DX_OK;
}

extern "C" int dx_comm_connect(dx_comm *c, const unsigned char *handles) {
    if (!c || !handles) return fail(DX_E_ARG, "comm: null argument");
    DeviceGuard guard(c->device);
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank || c->opened[r]) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + size_t(r) * 64, 64);
        void *p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return fail(DX_E_CUDA, "comm: cannot map the mailbox of rank %d: %s", r, cudaGetErrorString(e));
        c->peers.box[r] = static_cast<Mailbox *>(p);
        c->opened[r] = true;
    }
    c->connected = true;
    return DX_OK;
}

extern "C" int dx_comm_set_timeout_ms(dx_comm *c, int ms) {
    if (!c || ms <= 0) return fail(DX_E_ARG, "comm: timeout must be positive");
    int khz = 0;
    if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device) != cudaSuccess || khz <= 0) khz = 1965000;
    c->wait_cycles = (long long)ms * khz;
    return DX_OK;
}

extern "C" int dx_comm_allreduce(dx_comm *c, int op, int dtype, void *buf, int64_t n, void *stream) {
    if (!c || !buf) return fail(DX_E_ARG, "comm: null argument");
    if (!c->connected) return fail(DX_E_ARG, "comm: dx_comm_connect has not been called");
    if (!c->emulated.empty()) return fail(DX_E_ARG, "comm: this communicator emulates its ranks on one GPU; use dx_comm_emulated_allreduce");
    const int es = dx_dtype_size(dtype);
    if (es == 0 || dtype == DX_BOOL) return fail(DX_E_DTYPE, "comm: unsupported dtype code %d", dtype);
    if (n < 0) return fail(DX_E_SHAPE, "comm: negative count");
    if (n == 0) return DX_OK;
    if (int e = comm_flush_pending(c, as_stream(stream))) return e;
    // a buffer larger than a slot goes in rounds of one slot each (the parity double-buffering lets round k+1
    // start while a peer still reads round k, and nobody can get two rounds ahead)
    const int64_t per_round = COMM_SLOT / es;
    for (int64_t first = 0; first < n; first += per_round) {
        const int64_t count = n - first < per_round ? n - first : per_round;
        if (int e = real_dispatch(c, op, dtype, static_cast<unsigned char *>(buf) + first * es, count, as_stream(stream))) return e;
    }
    return DX_OK;
}

extern "C" int dx_comm_rank(dx_comm *c) { return c ? c->rank : -1; }
extern "C" int dx_comm_world(dx_comm *c) { return c ? c->world : 0; }

extern "C" void dx_shard_rows(int64_t global_rows, int rank, int world, int64_t *row0, int64_t *rows) {
    if (world < 1) world = 1;
    const int64_t base = global_rows / world, extra = global_rows % world;
    if (rows) *rows = base + (rank < extra ? 1 : 0);
    if (row0) *row0 = rank * base + (rank < extra ? rank : extra);
}

extern "C" int dx_comm_allreduce_begin(dx_comm *c, int op, int dtype, void *buf, int64_t n, void *stream) {
    if (!c || !buf) return fail(DX_E_ARG, "comm: null argument");
    if (!c->connected) return fail(DX_E_ARG, "comm: dx_comm_connect has not been called");
    if (!c->emulated.empty()) return fail(DX_E_ARG, "comm: this communicator emulates its ranks on one GPU");
    if (int e = check_size(dtype, n)) return e;
    if (int e = comm_flush_pending(c, as_stream(stream))) return e;
    if (n == 0) return DX_OK;
    if (int e = publish_dispatch(c, op, dtype, buf, n, as_stream(stream))) return e;
    comm_set_pending(c, op, dtype, buf, n);
    return DX_OK;
}

extern "C" int dx_comm_allreduce_finish(dx_comm *c, void *stream) {
    if (!c) return fail(DX_E_ARG, "comm: null argument");
    return comm_flush_pending(c, as_stream(stream));
}

extern "C" int dx_comm_pending(dx_comm *c, void **buf) {
    if (!c || !c->pending) return 0;
    if (buf) *buf = c->pending_buf;
    return 1;
}

namespace {
// the per-round byte ranges of an all-gather of row blocks; false when nothing is left to move
bool gather_round(int world, int64_t global_rows, int64_t row_bytes, int64_t round, GatherPlan *g, int *chunks) {
    int64_t longest = 0;
    for (int r = 0; r < world; ++r) {
        int64_t row0, rows;
        dx_shard_rows(global_rows, r, world, &row0, &rows);
        const int64_t len = rows * row_bytes - round * COMM_SLOT;
        g->off[r] = row0 * row_bytes + round * COMM_SLOT;
        g->len[r] = len <= 0 ? 0 : (len < COMM_SLOT ? len : COMM_SLOT);
        longest = g->len[r] > longest ? g->len[r] : longest;
    }
    *chunks = int((longest + COMM_CHUNK - 1) / COMM_CHUNK);
    return longest > 0;
}
}  // namespace

extern "C" int dx_comm_allgather_rows(dx_comm *c, void *buf, int64_t global_rows, int64_t row_bytes, void *stream) {
    if (!c || !buf) return fail(DX_E_ARG, "comm: null argument");
    if (!c->connected) return fail(DX_E_ARG, "comm: dx_comm_connect has not been called");
    if (!c->emulated.empty()) return fail(DX_E_ARG, "comm: this communicator emulates its ranks on one GPU; use dx_comm_emulated_allgather_rows");
    if (global_rows < 0 || row_bytes < 0) return fail(DX_E_SHAPE, "comm: negative extent");
    if (c->world == 1) return DX_OK;
    if (int e = comm_flush_pending(c, as_stream(stream))) return e;
    GatherPlan g;
    int chunks;
    for (int64_t round = 0; gather_round(c->world, global_rows, row_bytes, round, &g, &chunks); ++round) {
        peer_gather_kernel<<<chunks, COMM_THREADS, 0, as_stream(stream)>>>(c->peers, c->rank, static_cast<unsigned char *>(buf), g, c->wait_cycles);
        if (int e = check_launch("comm allgather")) return e;
    }
    return DX_OK;
}

extern "C" int dx_comm_wait_stats(dx_comm *c, double *microseconds, long long *waits, int reset, void *stream) {
    if (!c || !microseconds || !waits) return fail(DX_E_ARG, "comm: null argument");
    cudaStream_t st = as_stream(stream);
    Mailbox *m = c->emulated.empty() ? c->mine : c->emulated[0];
    struct { unsigned int waits; unsigned long long cycles; } h = {0u, 0ull};
    if (cudaMemcpyAsync(&h.waits, &m->waits, sizeof(unsigned int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaMemcpyAsync(&h.cycles, &m->waited_cycles, sizeof(unsigned long long), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess)
        return fail(DX_E_CUDA, "comm: cannot read the wait counters: %s", cudaGetErrorString(cudaGetLastError()));
    if (reset) {
        cudaMemsetAsync(&m->waits, 0, sizeof(unsigned int), st);
        cudaMemsetAsync(&m->waited_cycles, 0, sizeof(unsigned long long), st);
        cudaStreamSynchronize(st);
    }
    int khz = 0;
    if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c->device) != cudaSuccess || khz <= 0) khz = 1965000;
    *microseconds = double(h.cycles) * 1000.0 / double(khz);
    *waits = (long long)h.waits;
    return DX_OK;
}

extern "C" int dx_comm_status(dx_comm *c, void *stream) {
    if (!c) return fail(DX_E_ARG, "comm: null argument");
    cudaStream_t st = as_stream(stream);
    int worst = 0;
    auto check = [&](Mailbox *m, int r) -> int {
        int h = 0;
        if (cudaMemcpyAsync(&h, &m->status, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess)
            return fail(DX_E_CUDA, "comm: cannot read the status word: %s", cudaGetErrorString(cudaGetLastError()));
        if (h != 0) {
            cudaMemsetAsync(&m->status, 0, sizeof(int), st);
            cudaStreamSynchronize(st);
            worst = fail(DX_E_CUDA, "comm: rank %d gave up waiting for rank %d (chunk %d): peer absent or late", r, (h - 1) % 64, (h - 1) / 64);
        }
        return DX_OK;
    };
    if (c->emulated.empty()) {
        if (int e = check(c->mine, c->rank)) return e;
    } else {
        for (int r = c->world - 1; r >= 0; --r)
            if (int e = check(c->emulated[r], r)) return e;
    }
    return worst;
}

extern "C" void dx_comm_destroy(dx_comm *c) {
    if (!c) return;
    DeviceGuard guard(c->device);
    for (int r = 0; r < c->world; ++r)
        if (c->opened[r]) cudaIpcCloseMemHandle(c->peers.box[r]);
    if (c->emulated.empty()) cudaFree(c->mine);
    for (Mailbox *m : c->emulated) cudaFree(m);
    delete c;
}

extern "C" dx_comm *dx_comm_emulate(int world, int device) {
    if (world < 1 || world > COMM_MAX_WORLD) {
        fail(DX_E_ARG, "comm: %d ranks (at most %d)", world, COMM_MAX_WORLD);
        return nullptr;
    }
    DeviceGuard guard(device);
    int now = -1;
    if (cudaGetDevice(&now) != cudaSuccess || now != device) {
        fail(DX_E_CUDA, "comm: cannot make device %d current", device);
        return nullptr;
    }
    dx_comm *c = new (std::nothrow) dx_comm();
    if (!c) return nullptr;
    c->world = world;
    c->device = device;
    c->peers.world = world;
    for (int r = 0; r < world; ++r) {
        Mailbox *m = nullptr;
        if (new_mailbox(&m) != DX_OK) {
            for (Mailbox *x : c->emulated) cudaFree(x);
            delete c;
            return nullptr;
        }
        c->emulated.push_back(m);
        c->peers.box[r] = m;
    }
    c->mine = c->emulated[0];
    c->connected = true;
    return c;
}

extern "C" int dx_comm_emulated_allreduce(dx_comm *c, int op, int dtype, void *const *bufs, int active_ranks, int64_t n, void *stream) {
    if (!c || !bufs) return fail(DX_E_ARG, "comm: null argument");
    if (c->emulated.empty()) return fail(DX_E_ARG, "comm: not an emulating communicator (dx_comm_emulate)");
    if (active_ranks < 1 || active_ranks > c->world) return fail(DX_E_ARG, "comm: %d active ranks of %d", active_ranks, c->world);
    if (int e = check_size(dtype, n)) return e;
    if (n == 0) return DX_OK;
    // every CTA of the launch must be resident at once, since they wait on one another
    const int es = dx_dtype_size(dtype);
    const int64_t chunks = (n * es + COMM_CHUNK - 1) / COMM_CHUNK;
    if (chunks * c->world > sm_count()) return fail(DX_E_UNSUPPORTED, "comm: %lld CTAs would not all be resident", (long long)(chunks * c->world));
    return emulated_dispatch(c, op, dtype, bufs, active_ranks, n, as_stream(stream));
}

// The two halves as separate launches (what dx_reduce_allreduce_begin / dx_comm_allreduce_finish do on real ranks).
extern "C" int dx_comm_emulated_publish(dx_comm *c, int op, int dtype, void *const *bufs, int active_ranks, int64_t n, void *stream) {
    if (!c || !bufs) return fail(DX_E_ARG, "comm: null argument");
    if (c->emulated.empty()) return fail(DX_E_ARG, "comm: not an emulating communicator (dx_comm_emulate)");
    if (active_ranks < 1 || active_ranks > c->world) return fail(DX_E_ARG, "comm: %d active ranks of %d", active_ranks, c->world);
    if (int e = check_size(dtype, n)) return e;
    if (n == 0) return DX_OK;
    return emulated_publish_dispatch(c, op, dtype, bufs, active_ranks, n, as_stream(stream));
}
extern "C" int dx_comm_emulated_combine(dx_comm *c, int op, int dtype, void *const *bufs, int active_ranks, int64_t n, void *stream) {
    if (!c || !bufs) return fail(DX_E_ARG, "comm: null argument");
    if (c->emulated.empty()) return fail(DX_E_ARG, "comm: not an emulating communicator (dx_comm_emulate)");
    if (active_ranks < 1 || active_ranks > c->world) return fail(DX_E_ARG, "comm: %d active ranks of %d", active_ranks, c->world);
    if (int e = check_size(dtype, n)) return e;
    if (n == 0) return DX_OK;
    return emulated_combine_dispatch(c, op, dtype, bufs, active_ranks, n, as_stream(stream));
}
// All ranks' row blocks gathered in one launch per round (every CTA of a round must be resident at once).
extern "C" int dx_comm_emulated_allgather_rows(dx_comm *c, void *const *bufs, int64_t global_rows, int64_t row_bytes, void *stream) {
    if (!c || !bufs) return fail(DX_E_ARG, "comm: null argument");
    if (c->emulated.empty()) return fail(DX_E_ARG, "comm: not an emulating communicator (dx_comm_emulate)");
    if (global_rows < 0 || row_bytes < 0) return fail(DX_E_SHAPE, "comm: negative extent");
    Bufs b{};
    for (int r = 0; r < c->world; ++r) b.buf[r] = bufs[r];
    GatherPlan g;
    int chunks;
    for (int64_t round = 0; gather_round(c->world, global_rows, row_bytes, round, &g, &chunks); ++round) {
        if (int64_t(chunks) * c->world > sm_count()) return fail(DX_E_UNSUPPORTED, "comm: %lld CTAs would not all be resident", (long long)chunks * c->world);
        emulated_gather_kernel<<<dim3(chunks, c->world), COMM_THREADS, 0, as_stream(stream)>>>(c->peers, b, g, c->wait_cycles);
        if (int e = check_launch("comm allgather (emulated ranks)")) return e;
    }
    return DX_OK;
}
