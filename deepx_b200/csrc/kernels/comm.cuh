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
    int pad[15];
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

// The exchange for one rank and one chunk; `buf` is that rank's local data.
template <int OP, typename T>
__device__ void exchange_chunk(const Peers &peers, int rank, int chunk, T *buf, int64_t n, long long wait_cycles) {
    constexpr int PER = COMM_CHUNK / int(sizeof(T));  // elements per chunk
    constexpr int VEC = 16 / int(sizeof(T));
    using A = acc_t<T>;
    __shared__ int gave_up;
    Mailbox *mine = peers.box[rank];
    const int W = peers.world;
    const int64_t first = int64_t(chunk) * PER;
    const int count = int(n - first < PER ? n - first : PER);  // elements of this chunk
    if (threadIdx.x == 0) gave_up = 0;
    const unsigned int e = mine->epoch[chunk] + 1;  // only this CTA ever touches this chunk's epoch
    const int par = int(e & 1u);

    // 1. my chunk → slot [par][rank] of every mailbox (16-byte vectors; the tail of the last one is padding)
    T *src = buf + first;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    for (int v = threadIdx.x; v * VEC < count; v += COMM_THREADS) {
        Pack<T, VEC> pk;
        if (vec_ok && (v + 1) * VEC <= count) pk = ld_cached<T, VEC>(src + v * VEC);
        else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) pk.v[k] = (v * VEC + k < count) ? src[v * VEC + k] : narrow<T>(identity<OP, T>());
        }
        for (int p = 0; p < W; ++p) {
            T *dst = reinterpret_cast<T *>(peers.box[p]->slot[par][rank] + size_t(chunk) * COMM_CHUNK);
            *reinterpret_cast<Pack<T, VEC> *>(dst + v * VEC) = pk;
        }
    }
    __threadfence_system();
    __syncthreads();
    // 2. publish, 3. wait: thread p talks to peer p
    if (threadIdx.x < W) {
        const int p = threadIdx.x;
        st_release_sys(&peers.box[p]->flag[par][rank][chunk], e);
        const long long t0 = clock64();
        while (ld_acquire_sys(&mine->flag[par][p][chunk]) != e) {
            if (clock64() - t0 > wait_cycles) {
                atomicCAS(&mine->status, 0, 1 + chunk * 64 + p);
                gave_up = 1;
                break;
            }
        }
    }
    __syncthreads();
    // 4. combine in rank order; on a timeout leave the local data as it was
    if (!gave_up) {
        for (int i = threadIdx.x; i < count; i += COMM_THREADS) {
            A acc = widen<T>(ldcg_any(reinterpret_cast<const T *>(mine->slot[par][0] + size_t(chunk) * COMM_CHUNK) + i));
            for (int r = 1; r < W; ++r)
                acc = combine<OP, A>(acc, widen<T>(ldcg_any(reinterpret_cast<const T *>(mine->slot[par][r] + size_t(chunk) * COMM_CHUNK) + i)));
            src[i] = narrow<T>(acc);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) mine->epoch[chunk] = e;  // advanced even after a timeout: the ranks stay in step
}


// What a kernel needs from a connected communicator; false if it is not usable for a real exchange.
bool comm_device_view(dx_comm *c, Peers *peers, int *rank, long long *wait_cycles);

}  // namespace dx
