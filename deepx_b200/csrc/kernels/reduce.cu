// dx_reduce: sum / prod / max / min over an arbitrary subset of axes.
//
// Host side: size-1 axes are dropped and neighbouring axes of the same class
// (kept / reduced) are merged, which leaves an alternating list of groups.  Two
// device strategies cover every case:
//
//   rows  (innermost group is REDUCED, contiguous run of L elements per output):
//         a team of threads (1..32 lanes of a warp, or a whole 256-thread CTA,
//         or several CTAs when there are few outputs) streams the run(s) of one
//         output with 16-byte loads, then combines with warp shuffles and shared
//         memory.
//   cols  (innermost group is KEPT, Kin contiguous outputs): a CTA owns a strip
//         of 32 column vectors and walks the reduced rows 8 at a time (coalesced
//         512-byte row segments), combines the 8 row lanes through shared memory.
//
// When one launch cannot fill the machine (few outputs), the reduced range is
// split over several CTAs which write partials to caller-provided scratch, and a
// small second kernel combines them in a fixed order.  No atomics anywhere, so a
// given (shape, dims, device) always produces the same bits.
//
// The reference does this with one thread per INPUT element and a global atomic
// per element (executor/op-cuda/src/deepx/tensorfunc/reduce_miaobyte.cu:22-48),
// and its max/min are racy read-modify-writes (:230-256, :339-365).
#include <algorithm>
#include <limits>
#include <mutex>
#include <vector>

#include "comm.cuh"
#include "common.cuh"
#include "reduce_ops.cuh"

namespace dx {
namespace {

constexpr int RB = 256;      // threads per CTA
constexpr int RUNROLL = 4;   // independent 16-byte loads per thread per step
constexpr int MAXG = 6;      // ≤ 12 axes → ≤ 6 groups of each class
constexpr int TEAM_UNROLL = 8;  // vectors a lane of the team kernel keeps in flight

template <typename A> __device__ __forceinline__ A shfl_down(A v, int delta, int width) {
    if constexpr (sizeof(A) == 8) {
        long long t = __shfl_down_sync(0xffffffffu, *reinterpret_cast<long long *>(&v), delta, width);
        return *reinterpret_cast<A *>(&t);
    } else {
        int t = __shfl_down_sync(0xffffffffu, *reinterpret_cast<int *>(&v), delta, width);
        return *reinterpret_cast<A *>(&t);
    }
}

// ---- parameter blocks (by value in the launch, no device-side tables) --------------
struct Groups {
    int n;
    FastDiv fd[MAXG];       // group extents, outermost first
    int64_t stride[MAXG];   // input stride of each group, in elements
};

__device__ __forceinline__ int64_t unravel(uint32_t idx, const Groups &g) {
    // idx is a row-major index over the groups; returns Σ coord·stride.
    int64_t off = 0;
#pragma unroll 1
    for (int i = g.n - 1; i > 0; --i) {
        uint32_t q = fd_div(idx, g.fd[i]);
        off += int64_t(idx - q * g.fd[i].d) * g.stride[i];
        idx = q;
    }
    if (g.n > 0) off += int64_t(idx) * g.stride[0];
    return off;
}

struct RowsParams {
    Groups kept;      // all kept groups → base offset of an output's data
    Groups rout;      // reduced groups other than the innermost run
    FastDiv lv;       // vectors per innermost run (L / VEC)
    uint32_t units;   // vectors per output = Π rout · lv
    uint32_t split;   // CTAs per output (block kernel only)
    uint32_t chunk;   // vectors per CTA
    uint32_t nout;    // outputs
    int team;         // lanes per output (team kernel only)
};

struct ColsParams {
    Groups kouter;    // kept groups other than the innermost run
    Groups red;       // all reduced groups
    FastDiv ctiles;   // column tiles per kept-outer index
    FastDiv kouter_n; // number of kept-outer indices
    uint32_t kv;      // column vectors in the innermost run (Kin / VEC)
    int64_t kin;      // Kin
    uint32_t rows;    // Π red
    uint32_t split, chunk;
    int64_t nout;     // Π kept
    int tx;           // threads across columns (power of two ≤ 32); RB/tx rows in flight
};

// ---- a split reduction that finishes itself -------------------------------------------------------------
// A reduction split over several CTAs per output leaves partials; adding them up used to be a second, one-CTA
// launch: a launch boundary (≈3 µs) plus 3–5 µs of a kernel that is all latency.  Instead every CTA counts itself in
// on its output's counter after its partial is stored and fenced, and the CTA that finds the count complete adds
// the partials — in index order, so the same bits whichever CTA it is — writes the output and puts the counter
// back to zero.  When the result is one value that has to be combined across GPUs, that CTA also publishes it to
// the peers (and combines, unless that is deferred).  The counters are the library's (zero between launches), one
// bank per stream that uses them.
constexpr int RED_BANKS = 8, RED_COUNTERS = 2048;
__device__ unsigned int g_reduce_counters[RED_BANKS][RED_COUNTERS];
struct PeerTail {
    Peers peers;
    int rank;
    long long wait_cycles;
    int combine_now;  // 0: the kernel ends after publishing; the combine runs later on the stream (dx_comm_allreduce_finish)
};
struct FuseTail {
    unsigned int *counters;  // one per output
    int peer;                // 1: the finished value (one output) goes into the exchange
    PeerTail tail;
};

// One output whose partials are many (a single output split over several waves of CTAs): the whole CTA adds them,
// thread t taking partials t, t + RB, ..., then lanes, then warps, always in the same order.  The value is in thread 0.
constexpr uint32_t FINISH_WIDE_FROM = 128;  // partials per output from which a CTA, not a warp, finishes an output
template <int OP, typename T>
__device__ __forceinline__ acc_t<T> cta_combine_partials(const acc_t<T> *__restrict__ p, uint32_t split) {
    using A = acc_t<T>;
    __shared__ A wide_part[RB / 32];
    A r = identity<OP, T>();
    // L2 loads (other CTAs of this launch may have written them), eight in flight per thread; added in index order
    for (uint32_t c0 = threadIdx.x; c0 < split; c0 += 8 * RB) {
        A v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = (c0 + k * RB < split) ? __ldcg(p + c0 + k * RB) : identity<OP, T>();
#pragma unroll
        for (int k = 0; k < 8; ++k) r = combine<OP>(r, v[k]);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) r = combine<OP>(r, shfl_down(r, d, 32));
    __syncthreads();  // a previous output's wide_part has been read
    if ((threadIdx.x & 31) == 0) wide_part[threadIdx.x >> 5] = r;
    __syncthreads();
    if (threadIdx.x == 0) {
        r = wide_part[0];
#pragma unroll
        for (int w = 1; w < RB / 32; ++w) r = combine<OP>(r, wide_part[w]);
    }
    return r;
}
// ---- rows: one CTA (or 1/split of the work) per output ----------------------------------
template <int OP, typename T, int VEC, bool FUSE = false>
__global__ void __launch_bounds__(RB) rows_block_kernel(const T *__restrict__ in, T *out, acc_t<T> *partial, RowsParams p, FuseTail ft) {
    griddep_wait_cta();
    using A = acc_t<T>;
    const uint32_t o = blockIdx.x / p.split;
    const uint32_t c = blockIdx.x - o * p.split;
    const T *base = in + unravel(o, p.kept);
    const uint32_t u0 = c * p.chunk;
    const uint32_t u1 = min(p.units, u0 + p.chunk);

    A acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = identity<OP, T>();

    auto addr = [&](uint32_t u) -> const T * {
        if (p.rout.n == 0) return base + int64_t(u) * VEC;
        uint32_t seg = fd_div(u, p.lv);
        uint32_t pos = u - seg * p.lv.d;
        return base + unravel(seg, p.rout) + int64_t(pos) * VEC;
    };

    uint32_t u = u0 + threadIdx.x;
    // u0 + chunk ≤ 2^31 is guaranteed by the host, so u + k·RB cannot wrap.
    for (; u + (RUNROLL - 1) * RB < u1; u += RUNROLL * RB) {
        Pack<T, VEC> v[RUNROLL];
#pragma unroll
        for (int k = 0; k < RUNROLL; ++k) v[k] = ld_stream<T, VEC>(addr(u + k * RB));
#pragma unroll
        for (int k = 0; k < RUNROLL; ++k)
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = combine<OP>(acc[i], widen<T>(v[k].v[i]));
    }
    for (; u < u1; u += RB) {
        Pack<T, VEC> v = ld_stream<T, VEC>(addr(u));
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = combine<OP>(acc[i], widen<T>(v.v[i]));
    }
    A r = acc[0];
#pragma unroll
    for (int i = 1; i < VEC; ++i) r = combine<OP>(r, acc[i]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) r = combine<OP>(r, shfl_down(r, d, 32));
    __shared__ A warp_part[RB / 32];
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = r;
    __syncthreads();
    if (threadIdx.x == 0) {
        r = warp_part[0];
#pragma unroll
        for (int w = 1; w < RB / 32; ++w) r = combine<OP>(r, warp_part[w]);
        if (p.split == 1) out[o] = narrow<T>(r);
        else partial[size_t(o) * p.split + c] = r;
    }
    if constexpr (FUSE) {
        __shared__ int last;
        if (threadIdx.x == 0) {
            __threadfence();  // the partial is visible device-wide before this CTA counts itself in
            last = atomicAdd(ft.counters + o, 1u) == p.split - 1 ? 1 : 0;
        }
        __syncthreads();
        if (last) {
            __threadfence();
            const A total = cta_combine_partials<OP, T>(partial + size_t(o) * p.split, p.split);
            if (threadIdx.x == 0) {
                out[o] = narrow<T>(total);
                ft.counters[o] = 0u;  // ready for the next launch on this stream
            }
            if (ft.peer) {
                __syncthreads();  // this CTA's own store to `out` is visible to all its threads
                exchange_publish<T>(ft.tail.peers, ft.tail.rank, 0, out, 1, narrow<T>(identity<OP, T>()));
                if (ft.tail.combine_now) exchange_combine<OP, T>(ft.tail.peers, ft.tail.rank, 0, out, 1, ft.tail.wait_cycles);
            }
        }
    }
}

// ---- rows: a team of 1..32 lanes per output -------------------------------------------------
template <int OP, typename T, int VEC>
__global__ void __launch_bounds__(RB) rows_team_kernel(const T *__restrict__ in, T *__restrict__ out, RowsParams p) {
    using A = acc_t<T>;
    const int team = p.team;
    const uint32_t teams_per_cta = RB / team;
    const uint64_t o64 = uint64_t(blockIdx.x) * teams_per_cta + threadIdx.x / team;
    const int lane = threadIdx.x & (team - 1);
    const bool live = o64 < p.nout;
    const uint32_t o = live ? uint32_t(o64) : 0;
    const T *base = in + unravel(o, p.kept);

    A acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = identity<OP, T>();
    auto addr = [&](uint32_t u) -> const T * {
        if (p.rout.n == 0) return base + int64_t(u) * VEC;
        uint32_t seg = fd_div(u, p.lv);
        uint32_t pos = u - seg * p.lv.d;
        return base + unravel(seg, p.rout) + int64_t(pos) * VEC;
    };
    if (live) {
        // Short runs: a lane owns at most a handful of vectors, so issue up to TEAM_UNROLL of them
        // (predicated) before the first use instead of a 4-wide body plus a serial remainder.
#pragma unroll 1
        for (uint32_t u0 = lane; u0 < p.units; u0 += TEAM_UNROLL * team) {
            Pack<T, VEC> v[TEAM_UNROLL];
#pragma unroll
            for (int k = 0; k < TEAM_UNROLL; ++k)
                if (u0 + k * team < p.units) v[k] = ld_stream<T, VEC>(addr(u0 + k * team));
#pragma unroll
            for (int k = 0; k < TEAM_UNROLL; ++k)
                if (u0 + k * team < p.units) {
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[i] = combine<OP>(acc[i], widen<T>(v[k].v[i]));
                }
        }
    }
    A r = acc[0];
#pragma unroll
    for (int i = 1; i < VEC; ++i) r = combine<OP>(r, acc[i]);
    for (int d = team >> 1; d > 0; d >>= 1) r = combine<OP>(r, shfl_down(r, d, team));
    if (live && lane == 0) out[o] = narrow<T>(r);
}

template <int OP, typename T>
__global__ void __launch_bounds__(RB) rows_finish_wide_kernel(const acc_t<T> *__restrict__ partial, T *__restrict__ out, uint32_t split) {
    griddep_wait_cta();
    const acc_t<T> r = cta_combine_partials<OP, T>(partial + size_t(blockIdx.x) * split, split);
    if (threadIdx.x == 0) out[blockIdx.x] = narrow<T>(r);
}

// partial[nout][split] → out[nout]; one warp per output, fixed order.
template <int OP, typename T>
__global__ void __launch_bounds__(RB) rows_finish_kernel(const acc_t<T> *__restrict__ partial, T *__restrict__ out,
                                                         uint32_t nout, uint32_t split) {
    griddep_wait_cta();
    using A = acc_t<T>;
    const uint32_t o = blockIdx.x * (RB / 32) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (o >= nout) return;  // whole warp exits together
    A r = identity<OP, T>();
    for (uint32_t c = lane; c < split; c += 32) r = combine<OP>(r, partial[size_t(o) * split + c]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) r = combine<OP>(r, shfl_down(r, d, 32));
    if (lane == 0) out[o] = narrow<T>(r);
}

// ---- cols: innermost group kept ------------------------------------------------------------------
template <int OP, typename T, int VEC>
__global__ void __launch_bounds__(RB) cols_kernel(const T *__restrict__ in, T *__restrict__ out,
                                                  acc_t<T> *__restrict__ partial, ColsParams p) {
    using A = acc_t<T>;
    // blockIdx.x = ((ko * split) + c) * ctiles + ct
    uint32_t b = blockIdx.x;
    uint32_t q = fd_div(b, p.ctiles);
    const uint32_t ct = b - q * p.ctiles.d;
    const uint32_t ko = q / p.split;
    const uint32_t c = q - ko * p.split;

    const int tx = threadIdx.x & (p.tx - 1);
    const int ty = threadIdx.x / p.tx;
    const int ny = RB / p.tx;
    const uint32_t cv = ct * p.tx + tx;  // column vector index
    const bool live = cv < p.kv;
    const T *base = in + unravel(ko, p.kouter) + int64_t(cv) * VEC;

    const uint32_t r0 = c * p.chunk;
    const uint32_t r1 = min(p.rows, r0 + p.chunk);

    A acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = identity<OP, T>();

    auto addr = [&](uint32_t r) -> const T * {
        if (p.red.n == 1) return base + int64_t(r) * p.red.stride[0];
        return base + unravel(r, p.red);
    };
    if constexpr (sizeof(T) == 1 && VEC % 4 == 0 && (OP == DX_RMAX || OP == DX_RMIN)) {
        // int8 max / min: four elements per 32-bit word with the byte-wise SIMD max / min, instead of unpacking
        // sixteen bytes of every vector one by one (which made this the one instruction-bound column reduction)
        if (live) {
            uint32_t pk[VEC / 4];
#pragma unroll
            for (int j = 0; j < VEC / 4; ++j) pk[j] = OP == DX_RMAX ? 0x80808080u : 0x7f7f7f7fu;
            uint32_t r = r0 + ty;
            for (; r + (RUNROLL - 1) * ny < r1; r += RUNROLL * ny) {
                Pack<T, VEC> v[RUNROLL];
#pragma unroll
                for (int k = 0; k < RUNROLL; ++k) v[k] = ld_stream<T, VEC>(addr(r + k * ny));
#pragma unroll
                for (int k = 0; k < RUNROLL; ++k) {
                    const uint32_t *w = reinterpret_cast<const uint32_t *>(&v[k]);
#pragma unroll
                    for (int j = 0; j < VEC / 4; ++j) pk[j] = OP == DX_RMAX ? __vmaxs4(pk[j], w[j]) : __vmins4(pk[j], w[j]);
                }
            }
            for (; r < r1; r += ny) {
                Pack<T, VEC> v = ld_stream<T, VEC>(addr(r));
                const uint32_t *w = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
                for (int j = 0; j < VEC / 4; ++j) pk[j] = OP == DX_RMAX ? __vmaxs4(pk[j], w[j]) : __vmins4(pk[j], w[j]);
            }
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = static_cast<A>(static_cast<int8_t>((pk[i / 4] >> (8 * (i % 4))) & 0xffu));
        }
    } else if (live) {
        uint32_t r = r0 + ty;
        for (; r + (RUNROLL - 1) * ny < r1; r += RUNROLL * ny) {
            Pack<T, VEC> v[RUNROLL];
#pragma unroll
            for (int k = 0; k < RUNROLL; ++k) v[k] = ld_stream<T, VEC>(addr(r + k * ny));
#pragma unroll
            for (int k = 0; k < RUNROLL; ++k)
#pragma unroll
                for (int i = 0; i < VEC; ++i) acc[i] = combine<OP>(acc[i], widen<T>(v[k].v[i]));
        }
        for (; r < r1; r += ny) {
            Pack<T, VEC> v = ld_stream<T, VEC>(addr(r));
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = combine<OP>(acc[i], widen<T>(v.v[i]));
        }
    }
    // combine the ny row lanes of each column through shared memory (fixed order)
    __shared__ A sm[RB * VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) sm[(ty * p.tx + tx) * VEC + i] = acc[i];
    __syncthreads();
    if (ty == 0 && live) {
#pragma unroll 1
        for (int y = 1; y < ny; ++y)
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = combine<OP>(acc[i], sm[(y * p.tx + tx) * VEC + i]);
        const int64_t o = int64_t(ko) * p.kin + int64_t(cv) * VEC;
        if (p.split == 1) {
            Pack<T, VEC> w;
#pragma unroll
            for (int i = 0; i < VEC; ++i) w.v[i] = narrow<T>(acc[i]);
            *reinterpret_cast<Pack<T, VEC> *>(out + o) = w;
        } else {
            A *dst = partial + int64_t(c) * p.nout + o;
#pragma unroll
            for (int i = 0; i < VEC; ++i) dst[i] = acc[i];
        }
    }
}

// partial[split][nout] → out[nout]; one thread per output, coalesced across threads.
template <int OP, typename T>
__global__ void __launch_bounds__(RB) cols_finish_kernel(const acc_t<T> *__restrict__ partial, T *__restrict__ out,
                                                         int64_t nout, uint32_t split) {
    griddep_wait_cta();
    using A = acc_t<T>;
    const int64_t o = int64_t(blockIdx.x) * RB + threadIdx.x;
    if (o >= nout) return;
    A r = partial[o];
    for (uint32_t c = 1; c < split; ++c) r = combine<OP>(r, partial[int64_t(c) * nout + o]);
    out[o] = narrow<T>(r);
}

// ---- the finish step and the cross-GPU exchange in one kernel ------------------------------------
// When a reduction crosses the axis the tensor is sharded along, the per-rank result is a partial
// that has to be combined over the ranks.  If the local reduction ends in a finish step that one CTA
// can do (a handful of outputs: the global sum of the sharded chain is one), that CTA goes straight
// on to the peer exchange (comm.cuh): combine this rank's partials, store the result into every
// peer's mailbox, wait for theirs, combine in rank order, write `out`.  One launch is both the tail
// of the reduction and the all-reduce.
static_assert(RB == COMM_THREADS, "the exchange is written for the reduce kernels' CTA size");
template <int OP, typename T>
__global__ void __launch_bounds__(RB) rows_finish_peer_kernel(const acc_t<T> *__restrict__ partial, T *out, uint32_t nout, uint32_t split,
                                                              PeerTail tail) {
    griddep_wait_cta();
    using A = acc_t<T>;
    const uint32_t o = threadIdx.x >> 5;  // one CTA, one warp per output
    const int lane = threadIdx.x & 31;
    if (split >= FINISH_WIDE_FROM) {  // many partials per output: the CTA takes the outputs one after the other
        for (uint32_t w = 0; w < nout; ++w) {
            const A r = cta_combine_partials<OP, T>(partial + size_t(w) * split, split);
            if (threadIdx.x == 0) out[w] = narrow<T>(r);
        }
    } else if (o < nout) {
        A r = identity<OP, T>();
        for (uint32_t c = lane; c < split; c += 32) r = combine<OP>(r, partial[size_t(o) * split + c]);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) r = combine<OP>(r, shfl_down(r, d, 32));
        if (lane == 0) out[o] = narrow<T>(r);
    }
    __syncthreads();  // this CTA's own stores to `out` are visible to all its threads
    exchange_publish<T>(tail.peers, tail.rank, 0, out, nout, narrow<T>(identity<OP, T>()));
    if (tail.combine_now) exchange_combine<OP, T>(tail.peers, tail.rank, 0, out, nout, tail.wait_cycles);
}
template <int OP, typename T>
__global__ void __launch_bounds__(RB) cols_finish_peer_kernel(const acc_t<T> *__restrict__ partial, T *out, int64_t nout, uint32_t split,
                                                              PeerTail tail) {
    griddep_wait_cta();
    using A = acc_t<T>;
    const int64_t o = threadIdx.x;  // one CTA, one thread per output
    if (o < nout) {
        A r = partial[o];
        for (uint32_t c = 1; c < split; ++c) r = combine<OP>(r, partial[int64_t(c) * nout + o]);
        out[o] = narrow<T>(r);
    }
    __syncthreads();
    exchange_publish<T>(tail.peers, tail.rank, 0, out, nout, narrow<T>(identity<OP, T>()));
    if (tail.combine_now) exchange_combine<OP, T>(tail.peers, tail.rank, 0, out, nout, tail.wait_cycles);
}

template <typename T> __global__ void fill_kernel(T *out, int64_t n, T v) {
    int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = v;
}

// ---- host-side plan -----------------------------------------------------------------------------
enum PlanKind { PLAN_EMPTY_OUT, PLAN_IDENTITY, PLAN_COPY, PLAN_ROWS_TEAM, PLAN_ROWS_BLOCK, PLAN_COLS };

struct Plan {
    PlanKind kind;
    int vec;  // elements per vector the kernels will use (before the pointer-alignment check)
    RowsParams rows;
    ColsParams cols;
    int64_t nout, nin;
    size_t workspace;  // bytes
    unsigned grid;
};

// CTAs of the split kernels that fit on one SM, per (op, element type): the register count differs
// (32 for float32 rows, 47 for 16-bit columns, 61 for 8-bit columns), and a grid sized for more
// CTAs than fit leaves a few stragglers that run alone after the first wave.
struct Residency {
    int rows_block, cols;
};
template <int OP, typename T> Residency residency_t() {
    static Residency r{0, 0};
    static std::once_flag once;
    std::call_once(once, [] {
        constexpr int FULL = 16 / sizeof(T);
        int n = 0;
        r.rows_block = (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, rows_block_kernel<OP, T, FULL, true>, RB, 0) == cudaSuccess && n > 0) ? n : 8;
        r.cols = (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, cols_kernel<OP, T, FULL>, RB, 0) == cudaSuccess && n > 0) ? n : 6;
        cudaGetLastError();  // no device (a host-only build check): the defaults stand
    });
    return r;
}
template <typename T> Residency residency_op(int op) {
    switch (op) {
        case DX_SUM: return residency_t<DX_SUM, T>();
        case DX_PROD: return residency_t<DX_PROD, T>();
        case DX_RMAX: return residency_t<DX_RMAX, T>();
        default: return residency_t<DX_RMIN, T>();
    }
}
Residency residency(int op, int dtype) {
    switch (dtype) {
        case DX_F64: return residency_op<double>(op);
        case DX_F32: return residency_op<float>(op);
        case DX_F16: return residency_op<f16>(op);
        case DX_BF16: return residency_op<bf16>(op);
        case DX_I64: return residency_op<int64_t>(op);
        case DX_I32: return residency_op<int32_t>(op);
        case DX_I16: return residency_op<int16_t>(op);
        case DX_I8: return residency_op<int8_t>(op);
        default: return Residency{8, 6};
    }
}

int pow2_ceil(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

int make_plan(int dtype, const int64_t *shape, int ndim, const int32_t *dims, int ndims, int sms, Residency res, Plan *pl) {
    if (ndim < 0 || ndim > DX_MAX_DIMS) return fail(DX_E_SHAPE, "reduce: rank %d outside [0, %d]", ndim, DX_MAX_DIMS);
    if ((ndim > 0 && !shape) || (ndims > 0 && !dims)) return fail(DX_E_ARG, "reduce: null shape or dims");
    bool red[DX_MAX_DIMS] = {false};
    for (int i = 0; i < ndims; ++i) {
        if (dims[i] < 0 || dims[i] >= ndim) return fail(DX_E_SHAPE, "reduce: axis %d out of range for rank %d", dims[i], ndim);
        if (red[dims[i]]) return fail(DX_E_SHAPE, "reduce: axis %d listed twice", dims[i]);
        red[dims[i]] = true;
    }
    const int es = dx_dtype_size(dtype);
    const int acc_size = (es == 8) ? 8 : 4;
    int64_t nin = 1, nout = 1;
    for (int i = 0; i < ndim; ++i) {
        if (shape[i] < 0) return fail(DX_E_SHAPE, "reduce: negative extent");
        nin *= shape[i];
        if (!red[i]) nout *= shape[i];
    }
    pl->nin = nin;
    pl->nout = nout;
    pl->workspace = 0;
    pl->grid = 0;
    if (nout == 0) { pl->kind = PLAN_EMPTY_OUT; return DX_OK; }
    if (nin == 0) { pl->kind = PLAN_IDENTITY; return DX_OK; }
    if (nin == nout) { pl->kind = PLAN_COPY; return DX_OK; }

    // merge: drop extent-1 axes, fuse neighbours of the same class
    struct G { int64_t size, stride; bool red; };
    std::vector<G> g;
    int64_t stride = 1;
    for (int i = ndim - 1; i >= 0; --i) {
        if (shape[i] != 1) {
            if (!g.empty() && g.back().red == red[i]) g.back().size *= shape[i];  // g is built innermost-first
            else g.push_back({shape[i], stride, red[i]});
        }
        stride *= shape[i];
    }
    std::reverse(g.begin(), g.end());  // outermost first
    auto fill_groups = [&](Groups &dst, bool want_red, size_t skip_last) -> int {
        dst.n = 0;
        for (size_t i = 0; i + skip_last < g.size(); ++i)
            if (g[i].red == want_red) {
                if (g[i].size >= (1ll << 31)) return fail(DX_E_SHAPE, "reduce: merged axis of %lld elements is too long", (long long)g[i].size);
                dst.fd[dst.n] = make_fastdiv((uint32_t)g[i].size);
                dst.stride[dst.n] = g[i].stride;
                ++dst.n;
            }
        return DX_OK;
    };
    const int64_t inner = g.back().size;
    int vec = 16 / es;  // full 16-byte vectors when the contiguous run allows it, else scalar
    if (inner % vec != 0) vec = 1;
    pl->vec = vec;
    // one wave: as many CTAs as can be resident at once for this kernel and element type
    const int target_ctas = sms * (g.back().red ? res.rows_block : res.cols);

    if (g.back().red) {
        RowsParams &p = pl->rows;
        if (int e = fill_groups(p.kept, false, 0)) return e;
        if (int e = fill_groups(p.rout, true, 1)) return e;
        if (nout >= (1ll << 31)) return fail(DX_E_SHAPE, "reduce: %lld outputs exceed the 2^31 limit", (long long)nout);
        const int64_t units = (nin / nout) / vec;
        if (units >= (1ll << 31)) return fail(DX_E_SHAPE, "reduce: %lld elements per output exceed the limit", (long long)(nin / nout));
        p.lv = make_fastdiv((uint32_t)(inner / vec));
        p.units = (uint32_t)units;
        p.nout = (uint32_t)nout;
        p.split = 1;
        p.chunk = p.units;
        p.team = 32;
        if (units <= 512 && nout >= 64) {
            pl->kind = PLAN_ROWS_TEAM;
            p.team = std::min(32, pow2_ceil((int)((units + 3) / 4)));
            const int64_t teams_per_cta = RB / p.team;
            pl->grid = (unsigned)((nout + teams_per_cta - 1) / teams_per_cta);
        } else {
            pl->kind = PLAN_ROWS_BLOCK;
            int64_t split = 1;
            if (nout < target_ctas) {
                // Too few outputs for one CTA each to fill the GPU: split every output — over about FOUR waves of
                // CTAs, not one.  CTAs of a single wave all end at about the same time and the slowest decides
                // (measured on [256, 1048576] float32: sum 175 µs, row max 161 µs against 154 / 147 µs at the
                // bandwidth the same kernels reach on 8 times the rows); with several short waves the hardware
                // scheduler evens that out, like it does for the elementwise kernels' grids.
                // ... as long as a CTA keeps at least 128 KiB to read (below that the partials to add at the end outweigh
                // the smoother finish), and in WHOLE waves: 1.7 waves of equal CTAs end with a 0.7 wave of stragglers
                // (a 256 MiB input: 0.96 of the copy rate with 1184 CTAs, 0.92 with 2048, 0.89 with 4736).
                const int64_t by_work = std::max<int64_t>(1, units * vec * es / (128 << 10));
                const int64_t waves = std::max<int64_t>(1, std::min<int64_t>(4, by_work * nout / target_ctas));
                split = std::max<int64_t>(1, std::min(waves * target_ctas / nout, by_work));
            }
            int64_t chunk = (units + split - 1) / split;
            chunk = (chunk + RB - 1) / RB * RB;  // keeps every CTA's vectors 16-byte·RB aligned
            split = (units + chunk - 1) / chunk;
            p.split = (uint32_t)split;
            p.chunk = (uint32_t)chunk;
            if (nout * split >= (1ll << 31)) return fail(DX_E_SHAPE, "reduce: grid too large");
            pl->grid = (unsigned)(nout * split);
            if (split > 1) pl->workspace = size_t(nout) * split * acc_size;
        }
    } else {
        pl->kind = PLAN_COLS;
        ColsParams &p = pl->cols;
        if (int e = fill_groups(p.kouter, false, 1)) return e;
        if (int e = fill_groups(p.red, true, 0)) return e;
        const int64_t rows = nin / nout;
        const int64_t nko = nout / inner;
        if (rows >= (1ll << 31) || nko >= (1ll << 31) || inner / vec >= (1ll << 31))
            return fail(DX_E_SHAPE, "reduce: extent too large");
        p.kin = inner;
        p.kv = (uint32_t)(inner / vec);
        p.rows = (uint32_t)rows;
        p.nout = nout;
        p.tx = std::min(32, pow2_ceil((int)std::min<int64_t>(p.kv, 32)));
        const int ny = RB / p.tx;
        const int64_t ctiles = (p.kv + p.tx - 1) / p.tx;
        p.ctiles = make_fastdiv((uint32_t)ctiles);
        p.kouter_n = make_fastdiv((uint32_t)nko);
        int64_t split = 1;
        const int64_t ctas = ctiles * nko;
        if (ctas < target_ctas) {
            const int64_t by_target = target_ctas / ctas;  // floor: one wave, no straggler CTAs
            const int64_t by_work = std::max<int64_t>(1, rows / (ny * RUNROLL * 2));
            split = std::max<int64_t>(1, std::min(by_target, by_work));
        }
        int64_t chunk = (rows + split - 1) / split;
        split = (rows + chunk - 1) / chunk;
        p.split = (uint32_t)split;
        p.chunk = (uint32_t)chunk;
        if (ctas * split >= (1ll << 31)) return fail(DX_E_SHAPE, "reduce: grid too large");
        pl->grid = (unsigned)(ctas * split);
        if (split > 1) pl->workspace = size_t(nout) * split * acc_size;
    }
    return DX_OK;
}

// The counter bank of a stream on the current device (nullptr: all banks belong to other streams, or no device).
unsigned int *fuse_counters(cudaStream_t st) {
    static std::mutex mu;
    static unsigned int *base[64] = {};
    static std::vector<cudaStream_t> owners[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return nullptr; }
    std::lock_guard<std::mutex> lk(mu);
    if (!base[dev]) {
        void *sym = nullptr;
        if (cudaGetSymbolAddress(&sym, g_reduce_counters) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        base[dev] = static_cast<unsigned int *>(sym);
    }
    auto &v = owners[dev];
    size_t i = 0;
    while (i < v.size() && v[i] != st) ++i;
    if (i == v.size()) {
        if (v.size() >= size_t(RED_BANKS)) return nullptr;
        v.push_back(st);
    }
    return base[dev] + i * RED_COUNTERS;
}

template <int OP, typename T>
int run_plan(const Plan &pl, const T *in, T *out, void *ws, size_t ws_bytes, cudaStream_t st, const PeerTail *tail = nullptr,
             bool *exchanged = nullptr) {
    using A = acc_t<T>;
    switch (pl.kind) {
        case PLAN_EMPTY_OUT: return DX_OK;
        case PLAN_IDENTITY: {
            const unsigned grid = (unsigned)((pl.nout + 255) / 256);
            fill_kernel<T><<<grid, 256, 0, st>>>(out, pl.nout, narrow<T>(identity<OP, T>()));
            return check_launch("reduce(identity)");
        }
        case PLAN_COPY: {
            cudaError_t e = cudaMemcpyAsync(out, in, size_t(pl.nin) * sizeof(T), cudaMemcpyDeviceToDevice, st);
            if (e != cudaSuccess) return fail(DX_E_CUDA, "reduce(copy): %s", cudaGetErrorString(e));
            return DX_OK;
        }
        default: break;
    }
    if (pl.workspace > 0) {
        if (!ws || ws_bytes < pl.workspace)
            return fail(DX_E_WORKSPACE, "reduce: needs %zu bytes of workspace, got %zu", pl.workspace, ws_bytes);
        if (!aligned_to(ws, 16)) return fail(DX_E_WORKSPACE, "reduce: workspace must be 16-byte aligned");
    }
    A *partial = static_cast<A *>(ws);
    constexpr int FULL = 16 / sizeof(T);
    // The plan's vector width holds only if the pointers allow it; otherwise scalar.
    int vec = pl.vec;
    if (vec > 1 && !aligned_to(in, 16)) vec = 1;
    if (pl.kind == PLAN_COLS && vec > 1 && !aligned_to(out, 16)) vec = 1;
    Plan q = pl;
    if (vec != pl.vec) {
        const int f = pl.vec;  // pl.vec → 1
        if (pl.kind == PLAN_COLS) {
            ColsParams &p = q.cols;
            p.kv = pl.cols.kv * f;
            p.tx = std::min(32, pow2_ceil((int)std::min<uint32_t>(p.kv, 32)));
            const int64_t ctiles = (int64_t(p.kv) + p.tx - 1) / p.tx;
            p.ctiles = make_fastdiv((uint32_t)ctiles);
            const int64_t nko = pl.nout / pl.cols.kin;
            if (ctiles * nko * p.split >= (1ll << 31)) return fail(DX_E_SHAPE, "reduce: grid too large");
            q.grid = (unsigned)(ctiles * nko * p.split);
        } else {
            RowsParams &p = q.rows;
            if (uint64_t(pl.rows.units) * f >= (1ull << 31)) return fail(DX_E_SHAPE, "reduce: unaligned input too large");
            p.units = pl.rows.units * f;
            p.lv = make_fastdiv(pl.rows.lv.d * f);
            p.chunk = pl.rows.chunk * f;
        }
    }

#define LAUNCH_VEC(KERNEL, ...)                                                  \
    do {                                                                         \
        if (vec == FULL) KERNEL<OP, T, FULL><<<q.grid, RB, 0, st>>>(__VA_ARGS__); \
        else KERNEL<OP, T, 1><<<q.grid, RB, 0, st>>>(__VA_ARGS__);                \
    } while (0)

    if (pl.kind == PLAN_ROWS_TEAM) {
        LAUNCH_VEC(rows_team_kernel, in, out, q.rows);
        return check_launch("reduce(rows/team)");
    }
    if (pl.kind == PLAN_ROWS_BLOCK) {
        // a split reduction finishes itself when there are counters for it: few enough outputs, a bank for this stream,
        // and — if the result goes on into the exchange — a single output
        FuseTail ft = {};
        bool fuse = false;
        if (q.rows.split > 1 && q.rows.nout <= uint32_t(RED_COUNTERS) && (!tail || q.rows.nout == 1)) {
            if (unsigned int *bank = fuse_counters(st)) {
                fuse = true;
                ft.counters = bank;
                if (tail) { ft.peer = 1; ft.tail = *tail; }
            }
        }
        if (fuse) {
            if (vec == FULL) launch_pdl(rows_block_kernel<OP, T, FULL, true>, dim3(q.grid), dim3(RB), 0, st, in, out, partial, q.rows, ft);
            else launch_pdl(rows_block_kernel<OP, T, 1, true>, dim3(q.grid), dim3(RB), 0, st, in, out, partial, q.rows, ft);
            if (tail && exchanged) *exchanged = true;
            return check_launch("reduce(rows/block, finishing itself)");
        }
        if (vec == FULL) launch_pdl(rows_block_kernel<OP, T, FULL, false>, dim3(q.grid), dim3(RB), 0, st, in, out, partial, q.rows, ft);
        else launch_pdl(rows_block_kernel<OP, T, 1, false>, dim3(q.grid), dim3(RB), 0, st, in, out, partial, q.rows, ft);
        if (int e = check_launch("reduce(rows/block)")) return e;
        if (q.rows.split > 1) {
            const unsigned grid = (q.rows.nout + RB / 32 - 1) / (RB / 32);
            if (tail && grid == 1) {
                launch_pdl(rows_finish_peer_kernel<OP, T>, dim3(1), dim3(RB), 0, st, partial, out, q.rows.nout, q.rows.split, *tail);
                if (exchanged) *exchanged = true;
                return check_launch("reduce(rows/finish + exchange)");
            }
            if (q.rows.split >= FINISH_WIDE_FROM) launch_pdl(rows_finish_wide_kernel<OP, T>, dim3(q.rows.nout), dim3(RB), 0, st, partial, out, q.rows.split);
            else launch_pdl(rows_finish_kernel<OP, T>, dim3(grid), dim3(RB), 0, st, partial, out, q.rows.nout, q.rows.split);
            return check_launch("reduce(rows/finish)");
        }
        return DX_OK;
    }
    LAUNCH_VEC(cols_kernel, in, out, partial, q.cols);
    if (int e = check_launch("reduce(cols)")) return e;
    if (q.cols.split > 1) {
        const unsigned grid = (unsigned)((q.cols.nout + RB - 1) / RB);
        if (tail && grid == 1) {
            cols_finish_peer_kernel<OP, T><<<1, RB, 0, st>>>(partial, out, q.cols.nout, q.cols.split, *tail);
            if (exchanged) *exchanged = true;
            return check_launch("reduce(cols/finish + exchange)");
        }
        cols_finish_kernel<OP, T><<<grid, RB, 0, st>>>(partial, out, q.cols.nout, q.cols.split);
        return check_launch("reduce(cols/finish)");
    }
    return DX_OK;
#undef LAUNCH_VEC
}

template <typename T>
int run_op(int op, const Plan &pl, const void *a, void *out, void *ws, size_t wsb, cudaStream_t st, const PeerTail *tail = nullptr,
           bool *exchanged = nullptr) {
    switch (op) {
        case DX_SUM: return run_plan<DX_SUM, T>(pl, (const T *)a, (T *)out, ws, wsb, st, tail, exchanged);
        case DX_PROD: return run_plan<DX_PROD, T>(pl, (const T *)a, (T *)out, ws, wsb, st, tail, exchanged);
        case DX_RMAX: return run_plan<DX_RMAX, T>(pl, (const T *)a, (T *)out, ws, wsb, st, tail, exchanged);
        case DX_RMIN: return run_plan<DX_RMIN, T>(pl, (const T *)a, (T *)out, ws, wsb, st, tail, exchanged);
        default: return fail(DX_E_ARG, "reduce: unknown op code %d", op);
    }
}

}  // namespace
}  // namespace dx

using namespace dx;

extern "C" size_t dx_reduce_workspace_bytes(int op, int dtype, const int64_t *shape, int ndim, const int32_t *dims,
                                            int ndims) {
    Plan pl;
    if (dx_dtype_size(dtype) == 0 || dtype == DX_BOOL) return 0;
    if (make_plan(dtype, shape, ndim, dims, ndims, sm_count(), residency(op, dtype), &pl) != DX_OK) return 0;
    return (pl.workspace + 255) / 256 * 256;
}

extern "C" int dx_reduce(int op, int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims,
                         int ndims, void *out, void *workspace, size_t workspace_bytes, void *stream) {
    cudaStream_t st = as_stream(stream);
    if (dx_dtype_size(dtype) == 0 || dtype == DX_BOOL)
        return fail(DX_E_DTYPE, "reduce: unsupported dtype code %d", dtype);
    Plan pl;
    if (int e = make_plan(dtype, shape, ndim, dims, ndims, sm_count(), residency(op, dtype), &pl)) return e;
    if (pl.nout > 0 && !out) return fail(DX_E_ARG, "reduce: null output");
    if (pl.nin > 0 && !a) return fail(DX_E_ARG, "reduce: null input");
    if (a == out && pl.nin > 0 && pl.kind != PLAN_COPY) return fail(DX_E_ALIAS, "reduce: output aliases input");
    switch (dtype) {
        case DX_F64: return run_op<double>(op, pl, a, out, workspace, workspace_bytes, st);
        case DX_F32: return run_op<float>(op, pl, a, out, workspace, workspace_bytes, st);
        case DX_F16: return run_op<f16>(op, pl, a, out, workspace, workspace_bytes, st);
        case DX_BF16: return run_op<bf16>(op, pl, a, out, workspace, workspace_bytes, st);
        case DX_I64: return run_op<int64_t>(op, pl, a, out, workspace, workspace_bytes, st);
        case DX_I32: return run_op<int32_t>(op, pl, a, out, workspace, workspace_bytes, st);
        case DX_I16: return run_op<int16_t>(op, pl, a, out, workspace, workspace_bytes, st);
        case DX_I8: return run_op<int8_t>(op, pl, a, out, workspace, workspace_bytes, st);
        default: return fail(DX_E_DTYPE, "reduce: unsupported dtype code %d", dtype);
    }
}

// Local reduction followed by the combine over the ranks of `comm`, result on every rank.  When the
// local reduction ends in a one-CTA finish step that CTA also publishes this rank's result to the peers
// (one launch less, and the collective is part of the reduce kernel); otherwise a publish kernel follows on
// the same stream.  `combine_now` = 0 stops there: the wait for the peers and the combine are left to
// dx_comm_allreduce_finish (or to the next call on the communicator), so that whatever the stream runs in
// between hides the skew between the ranks.  The combined output must fit a mailbox slot (dx_comm_max_bytes).
static int reduce_allreduce(dx_comm *comm, int op, int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims, int ndims,
                            void *out, void *workspace, size_t workspace_bytes, void *stream, int combine_now) {
    cudaStream_t st = as_stream(stream);
    if (dx_dtype_size(dtype) == 0 || dtype == DX_BOOL)
        return fail(DX_E_DTYPE, "reduce: unsupported dtype code %d", dtype);
    PeerTail tail;
    if (!comm_device_view(comm, &tail.peers, &tail.rank, &tail.wait_cycles))
        return fail(DX_E_ARG, "reduce+allreduce: the communicator is not connected (or emulates its ranks)");
    tail.combine_now = combine_now;
    Plan pl;
    if (int e = make_plan(dtype, shape, ndim, dims, ndims, sm_count(), residency(op, dtype), &pl)) return e;
    if (pl.nout > 0 && !out) return fail(DX_E_ARG, "reduce: null output");
    if (pl.nin > 0 && !a) return fail(DX_E_ARG, "reduce: null input");
    if (a == out && pl.nin > 0 && pl.kind != PLAN_COPY) return fail(DX_E_ALIAS, "reduce: output aliases input");
    if (size_t(pl.nout) * dx_dtype_size(dtype) > dx_comm_max_bytes())
        return fail(DX_E_WORKSPACE, "reduce+allreduce: %lld output bytes exceed the mailbox slot; reduce locally and use dx_comm_allreduce",
                    (long long)(pl.nout * dx_dtype_size(dtype)));
    if (int e = comm_flush_pending(comm, st)) return e;  // an earlier exchange still waiting for its combine goes first
    bool exchanged = false;
    int rc;
    switch (dtype) {
        case DX_F64: rc = run_op<double>(op, pl, a, out, workspace, workspace_bytes, st, &tail, &exchanged); break;
        case DX_F32: rc = run_op<float>(op, pl, a, out, workspace, workspace_bytes, st, &tail, &exchanged); break;
        case DX_F16: rc = run_op<f16>(op, pl, a, out, workspace, workspace_bytes, st, &tail, &exchanged); break;
        case DX_BF16: rc = run_op<bf16>(op, pl, a, out, workspace, workspace_bytes, st, &tail, &exchanged); break;
        case DX_I64: rc = run_op<int64_t>(op, pl, a, out, workspace, workspace_bytes, st, &tail, &exchanged); break;
        case DX_I32: rc = run_op<int32_t>(op, pl, a, out, workspace, workspace_bytes, st, &tail, &exchanged); break;
        case DX_I16: rc = run_op<int16_t>(op, pl, a, out, workspace, workspace_bytes, st, &tail, &exchanged); break;
        case DX_I8: rc = run_op<int8_t>(op, pl, a, out, workspace, workspace_bytes, st, &tail, &exchanged); break;
        default: return fail(DX_E_DTYPE, "reduce: unsupported dtype code %d", dtype);
    }
    if (rc != DX_OK || pl.nout == 0) return rc;
    if (exchanged) {
        if (!combine_now) comm_set_pending(comm, op, dtype, out, pl.nout);  // published by the finish kernel
        return DX_OK;
    }
    if (combine_now) return dx_comm_allreduce(comm, op, dtype, out, pl.nout, stream);
    return dx_comm_allreduce_begin(comm, op, dtype, out, pl.nout, stream);
}

extern "C" int dx_reduce_allreduce(dx_comm *comm, int op, int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims,
                                   int ndims, void *out, void *workspace, size_t workspace_bytes, void *stream) {
    return reduce_allreduce(comm, op, dtype, a, shape, ndim, dims, ndims, out, workspace, workspace_bytes, stream, 1);
}
extern "C" int dx_reduce_allreduce_begin(dx_comm *comm, int op, int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims,
                                         int ndims, void *out, void *workspace, size_t workspace_bytes, void *stream) {
    return reduce_allreduce(comm, op, dtype, a, shape, ndim, dims, ndims, out, workspace, workspace_bytes, stream, 0);
}

// ---- reduce without any device allocation ---------------------------------------------------------
// Some hosts that embed this library cannot obtain device memory at the moment they need a
// reduction: an executor whose whole memory budget was handed to a pre-sized pool, a plugin
// running inside another framework's allocator callback, a service that forbids cudaMalloc
// after start-up because it synchronises the device.  dx_reduce() leaves the cross-block scratch
// to the caller; this variant brings its own, a fixed array that lives in the module image.
//
// The array costs DX_REDUCE_STATIC_SCRATCH bytes on every GPU that loads the library, until the
// process exits.  Every call on a device uses the same array, so two calls that may run at the
// same time on that device (different streams, different threads) would overwrite each other's
// partials: keep such calls on one stream.  Nothing in the array has to start at zero — each
// partial slot is written by exactly one block before the combining kernel reads it — so what
// the previous call left behind is harmless and is not cleared.
constexpr size_t DX_REDUCE_STATIC_SCRATCH = size_t(1) << 20;  // 1 MiB
static __device__ __align__(256) unsigned char g_static_scratch[DX_REDUCE_STATIC_SCRATCH];

namespace {
std::mutex g_static_mu;
void *g_static_ptr[64] = {};  // per device: the array's DEVICE address (the symbol name is only a host-side handle)
}

extern "C" int dx_reduce_noalloc(int op, int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims,
                                 int ndims, void *out, void *stream) {
    if (dx_dtype_size(dtype) == 0 || dtype == DX_BOOL)
        return fail(DX_E_DTYPE, "reduce: unsupported dtype code %d", dtype);
    Plan pl;
    if (int e = make_plan(dtype, shape, ndim, dims, ndims, sm_count(), residency(op, dtype), &pl)) return e;
    if (pl.workspace > DX_REDUCE_STATIC_SCRATCH)
        return fail(DX_E_WORKSPACE,
                    "reduce (no-alloc): this shape needs %zu bytes of scratch, the built-in scratch holds %zu; "
                    "use dx_reduce with a caller-provided workspace",
                    pl.workspace, (size_t)DX_REDUCE_STATIC_SCRATCH);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return fail(DX_E_CUDA, "reduce (no-alloc): cannot identify the current device");
    void *scratch;
    {
        // First call on a device: resolve where the array lives on THAT device (it must be current).
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!g_static_ptr[dev]) {
            // The lookup below is not a stream operation and must not happen while this stream is being
            // captured into a graph: the first call on a device has to come before any capture.
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            if (cudaStreamIsCapturing(as_stream(stream), &cap) == cudaSuccess && cap != cudaStreamCaptureStatusNone)
                return fail(DX_E_ARG, "reduce (no-alloc): the first call on a device resolves the scratch address and cannot run "
                                      "inside a stream capture; call it once on this device before capturing");
            void *p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess || !p)
                return fail(DX_E_CUDA, "reduce (no-alloc): cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            g_static_ptr[dev] = p;
        }
        scratch = g_static_ptr[dev];
    }
    return dx_reduce(op, dtype, a, shape, ndim, dims, ndims, out, scratch, DX_REDUCE_STATIC_SCRATCH, stream);
}
