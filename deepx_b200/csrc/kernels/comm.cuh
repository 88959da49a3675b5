// Device side of the peer-memory all-reduce, shared by the stand-alone exchange kernel and by the
// reduce kernels that finish with the exchange (comm.cu explains the protocol).
#pragma once
#include "common.cuh"
#include "reduce_ops.cuh"

struct dx_comm;

namespace dx {

constexpr int COMM_MAX_WORLD = 16;
constexpr int COMM_CHUNK = 4096;                  // bytes per CTA
constexpr int COMM_CHUNKS = 16;                   // chunks per slot
constexpr int COMM_SLOT = COMM_CHUNK * COMM_CHUNKS;  // 64 KiB per (parity, rank)
constexpr int COMM_THREADS = 256;

struct Mailbox {
    unsigned int flag[2][COMM_MAX_WORLD][COMM_CHUNKS];  // epoch last published by (rank, chunk)
    unsigned int epoch[COMM_CHUNKS];                    // epochs this rank has completed per chunk
    int status;                                         // 0, or 1 + chunk * 64 + peer of the wait that expired
    unsigned int waits;                                 // flag waits done by this rank's CTAs, and
    unsigned long long waited_cycles;                   // the SM cycles they took (the longest thread of each CTA)
    int pad[12];
    alignas(256) unsigned char slot[2][COMM_MAX_WORLD][COMM_SLOT];
};

struct Peers {
    Mailbox *box[COMM_MAX_WORLD];
    int world;
};

__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// 16-bit __ldcg overloads do not exist for the float wrappers: go through the bit pattern.
template <typename T> __device__ __forceinline__ T ldcg_any(const T *p) {
    if constexpr (sizeof(T) == 2) {
        const unsigned short u = __ldcg(reinterpret_cast<const unsigned short *>(p));
        return *reinterpret_cast<const T *>(&u);
    } else if constexpr (sizeof(T) == 1) {
        const unsigned char u = __ldcg(reinterpret_cast<const unsigned char *>(p));
        return *reinterpret_cast<const T *>(&u);
    } else return __ldcg(p);
}

// The exchange for one rank and one chunk, in two halves so that independent work can run between them:
//   publish: this rank's chunk goes into slot [parity][rank] of every mailbox, then the flags (st.release.sys);
//   combine: wait (bounded) for every peer's flag in the own mailbox, combine the W slots in rank order
//            0..W-1 (the same bits on every rank), write the result over the local data, advance the epoch.
// A kernel may do both (exchange_chunk) or end after publishing and leave the combine to a later kernel on
// the same stream: whatever the stream runs in between hides the skew between the ranks.  Only one exchange
// per chunk may be outstanding at a time (the parity double-buffering covers one, not two).
template <typename T>
__device__ void exchange_publish(const Peers &peers, int rank, int chunk, const T *buf, int64_t n, T pad) {
    constexpr int PER = COMM_CHUNK / int(sizeof(T));  // elements per chunk
    constexpr int VEC = 16 / int(sizeof(T));
    Mailbox *mine = peers.box[rank];
    const int W = peers.world;
    const int64_t first = int64_t(chunk) * PER;
    const int count = int(n - first < PER ? n - first : PER);  // elements of this chunk
    const unsigned int e = mine->epoch[chunk] + 1;  // only the CTA of this chunk ever touches its epoch
    const int par = int(e & 1u);
    // my chunk → slot [par][rank] of every mailbox (16-byte vectors; the tail of the last one is padding)
    const T *src = buf + first;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    for (int v = threadIdx.x; v * VEC < count; v += COMM_THREADS) {
        Pack<T, VEC> pk;
        if (vec_ok && (v + 1) * VEC <= count) pk = ld_cached<T, VEC>(src + v * VEC);
        else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) pk.v[k] = (v * VEC + k < count) ? src[v * VEC + k] : pad;
        }
        for (int p = 0; p < W; ++p) {
            T *dst = reinterpret_cast<T *>(peers.box[p]->slot[par][rank] + size_t(chunk) * COMM_CHUNK);
            *reinterpret_cast<Pack<T, VEC> *>(dst + v * VEC) = pk;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < W) st_release_sys(&peers.box[threadIdx.x]->flag[par][rank][chunk], e);
}

// Waits for every peer's flag of this chunk's current exchange; returns false (and records who was missing)
// when a wait ran into its limit.  All threads of the CTA call it and get the same answer.
__device__ __forceinline__ bool exchange_wait(const Peers &peers, int rank, int chunk, long long wait_cycles, unsigned int *epoch_out) {
    __shared__ int gave_up;
    __shared__ unsigned long long longest;
    Mailbox *mine = peers.box[rank];
    const unsigned int e = mine->epoch[chunk] + 1;
    const int par = int(e & 1u);
    if (threadIdx.x == 0) { gave_up = 0; longest = 0ull; }
    __syncthreads();
    if (threadIdx.x < peers.world) {
        const int p = threadIdx.x;
        const long long t0 = clock64();
        while (ld_acquire_sys(&mine->flag[par][p][chunk]) != e) {
            if (clock64() - t0 > wait_cycles) {
                atomicCAS(&mine->status, 0, 1 + chunk * 64 + p);
                gave_up = 1;
                break;
            }
        }
        atomicMax(&longest, (unsigned long long)(clock64() - t0));
    }
    __syncthreads();
    if (threadIdx.x == 0) {  // what the rendezvous cost this CTA: dx_comm_wait_stats adds these up
        atomicAdd(&mine->waited_cycles, longest);
        atomicAdd(&mine->waits, 1u);
    }
    *epoch_out = e;
    return gave_up == 0;
}

template <int OP, typename T>
__device__ void exchange_combine(const Peers &peers, int rank, int chunk, T *buf, int64_t n, long long wait_cycles) {
    constexpr int PER = COMM_CHUNK / int(sizeof(T));
    using A = acc_t<T>;
    Mailbox *mine = peers.box[rank];
    const int W = peers.world;
    const int64_t first = int64_t(chunk) * PER;
    const int count = int(n - first < PER ? n - first : PER);
    unsigned int e;
    const bool complete = exchange_wait(peers, rank, chunk, wait_cycles, &e);
    const int par = int(e & 1u);
    // combine in rank order; on a timeout leave the local data as it was
    if (complete) {
        T *dst = buf + first;
        for (int i = threadIdx.x; i < count; i += COMM_THREADS) {
            A acc = widen<T>(ldcg_any(reinterpret_cast<const T *>(mine->slot[par][0] + size_t(chunk) * COMM_CHUNK) + i));
            for (int r = 1; r < W; ++r)
                acc = combine<OP, A>(acc, widen<T>(ldcg_any(reinterpret_cast<const T *>(mine->slot[par][r] + size_t(chunk) * COMM_CHUNK) + i)));
            dst[i] = narrow<T>(acc);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) mine->epoch[chunk] = e;  // advanced even after a timeout: the ranks stay in step
}

template <int OP, typename T>
__device__ void exchange_chunk(const Peers &peers, int rank, int chunk, T *buf, int64_t n, long long wait_cycles) {
    exchange_publish<T>(peers, rank, chunk, buf, n, narrow<T>(identity<OP, T>()));
    exchange_combine<OP, T>(peers, rank, chunk, buf, n, wait_cycles);
}

// All-gather of row blocks: every rank holds the whole buffer and has filled its own byte range
// [off[rank], off[rank] + len[rank]); afterwards every rank holds every range.  Same mailbox, flags and
// epochs as the all-reduce (one chunk = 4 KiB of a rank's range; every rank launches the same number of
// CTAs, a CTA beyond the end of its rank's range publishes nothing but still flags, so epochs stay in step).
struct GatherPlan {
    long long off[COMM_MAX_WORLD];
    long long len[COMM_MAX_WORLD];  // this round: at most COMM_SLOT bytes per rank
};
__device__ __forceinline__ void copy_bytes(unsigned char *dst, const unsigned char *src, int count) {
    if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
        const int vecs = count >> 4;
        for (int v = threadIdx.x; v < vecs; v += COMM_THREADS) reinterpret_cast<uint4 *>(dst)[v] = reinterpret_cast<const uint4 *>(src)[v];
        for (int i = (vecs << 4) + threadIdx.x; i < count; i += COMM_THREADS) dst[i] = src[i];
    } else {
        for (int i = threadIdx.x; i < count; i += COMM_THREADS) dst[i] = src[i];
    }
}
__device__ __forceinline__ int gather_count(const GatherPlan &g, int p, int chunk) {
    const long long left = g.len[p] - (long long)chunk * COMM_CHUNK;
    return left <= 0 ? 0 : (left < COMM_CHUNK ? int(left) : COMM_CHUNK);
}
__device__ inline void gather_chunk(const Peers &peers, int rank, int chunk, unsigned char *buf, const GatherPlan &g, long long wait_cycles) {
    Mailbox *mine = peers.box[rank];
    const int W = peers.world;
    const unsigned int e0 = mine->epoch[chunk] + 1;
    const int par0 = int(e0 & 1u);
    const int mine_count = gather_count(g, rank, chunk);
    if (mine_count > 0) {
        const unsigned char *src = buf + g.off[rank] + (long long)chunk * COMM_CHUNK;
        for (int p = 0; p < W; ++p)
            if (p != rank) copy_bytes(peers.box[p]->slot[par0][rank] + size_t(chunk) * COMM_CHUNK, src, mine_count);
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < W) st_release_sys(&peers.box[threadIdx.x]->flag[par0][rank][chunk], e0);
    unsigned int e;
    const bool complete = exchange_wait(peers, rank, chunk, wait_cycles, &e);
    if (complete) {
        for (int p = 0; p < W; ++p) {
            const int count = gather_count(g, p, chunk);
            if (p == rank || count == 0) continue;
            // written by a peer over NVLink: read past L1 (the flag's acquire orders it)
            const volatile unsigned char *src = mine->slot[par0][p] + size_t(chunk) * COMM_CHUNK;
            unsigned char *dst = buf + g.off[p] + (long long)chunk * COMM_CHUNK;
            if (((reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
                const int vecs = count >> 4;
                for (int v = threadIdx.x; v < vecs; v += COMM_THREADS) reinterpret_cast<uint4 *>(dst)[v] = __ldcg(reinterpret_cast<const uint4 *>(const_cast<const unsigned char *>(src)) + v);
                for (int i = (vecs << 4) + threadIdx.x; i < count; i += COMM_THREADS) dst[i] = src[i];
            } else {
                for (int i = threadIdx.x; i < count; i += COMM_THREADS) dst[i] = src[i];
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) mine->epoch[chunk] = e;
}

// What a kernel needs from a connected communicator; false if it is not usable for a real exchange.
bool comm_device_view(dx_comm *c, Peers *peers, int *rank, long long *wait_cycles);
// Book-keeping of an exchange that has been published but not yet combined (see dx_comm_allreduce_finish).
void comm_set_pending(dx_comm *c, int op, int dtype, void *buf, int64_t n);
int comm_flush_pending(dx_comm *c, cudaStream_t st);

}  // namespace dx
