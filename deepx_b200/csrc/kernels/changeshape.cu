// dx_transpose / dx_concat / dx_broadcast_to / dx_indexselect / dx_repeat.
//
// All five are pure data movement, so the kernels are written over W-byte words
// (W = 16 when extents and pointers allow, else the widest power of two that
// divides every contiguous run and aligns every pointer, never below the element
// size) and are instantiated per word width, not per dtype.  Index arithmetic is
// done once per word with 32-bit multiply-shift division by launch-time constants
// carried in the kernel parameters; nothing is uploaded to or allocated on the
// device per call (the reference uploads three stride vectors per call and, for
// concat, calls malloc inside the kernel:
// executor/op-cuda/src/deepx/tensorfunc/changeshape_miaobyte.cu:52-54,127-128).
#include <algorithm>
#include <vector>

#include "common.cuh"

namespace dx {
namespace {

constexpr int CB = 256;
constexpr int CUNROLL = 4;
constexpr int MAXD = DX_MAX_DIMS;

template <int W> struct word_of;
template <> struct word_of<16> { using type = int4; };
template <> struct word_of<8> { using type = int2; };
template <> struct word_of<4> { using type = int; };
template <> struct word_of<2> { using type = short; };
template <> struct word_of<1> { using type = char; };
template <int W> using word_t = typename word_of<W>::type;

struct Dims {
    int n;
    FastDiv fd[MAXD];     // extents, outermost first
    int64_t stride[MAXD]; // source stride in BYTES for each extent
};

__device__ __forceinline__ int64_t unravel_bytes(uint32_t idx, const Dims &g) {
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

int widest_word(int es, std::initializer_list<int64_t> run_bytes, std::initializer_list<const void *> ptrs) {
    int w = 16;
    auto ok = [&](int w_) {
        for (int64_t b : run_bytes)
            if (b % w_ != 0) return false;
        for (const void *p : ptrs)
            if (!aligned_to(p, w_)) return false;
        return true;
    };
    while (w > es && !ok(w)) w >>= 1;
    return w;
}

#define DISPATCH_W(w, ...)                                 \
    switch (w) {                                           \
        case 16: { constexpr int W = 16; __VA_ARGS__; } break; \
        case 8: { constexpr int W = 8; __VA_ARGS__; } break;   \
        case 4: { constexpr int W = 4; __VA_ARGS__; } break;   \
        case 2: { constexpr int W = 2; __VA_ARGS__; } break;   \
        default: { constexpr int W = 1; __VA_ARGS__; } break;  \
    }

int grid_for(int64_t units, unsigned *grid) {
    const int64_t per = int64_t(CB) * CUNROLL;
    int64_t g = (units + per - 1) / per;
    if (units >= (1ll << 31)) return fail(DX_E_SHAPE, "changeshape: %lld words exceed the 2^31 per-launch limit", (long long)units);
    *grid = (unsigned)g;
    return DX_OK;
}

// ---- generic gather of contiguous runs ------------------------------------------------
// out word v = (row, pos): row is a row-major index over `rows` whose strides point into
// the source; pos walks a contiguous run of `run.d` words.  Serves transpose with the
// innermost axis preserved, and broadcastTo whose innermost axis is not broadcast.
struct RunGatherParams {
    Dims rows;
    FastDiv run;  // words per contiguous run
    uint32_t units;
};

template <int W>
__global__ void __launch_bounds__(CB) run_gather_kernel(const char *__restrict__ in, char *__restrict__ out, RunGatherParams p,
                                                        bool stream_src) {
    const uint32_t v0 = blockIdx.x * (CB * CUNROLL) + threadIdx.x;
    word_t<W> w[CUNROLL];
#pragma unroll
    for (int k = 0; k < CUNROLL; ++k) {
        const uint32_t v = v0 + k * CB;
        if (v < p.units) {
            const uint32_t row = fd_div(v, p.run);
            const uint32_t pos = v - row * p.run.d;
            const char *src = in + unravel_bytes(row, p.rows) + int64_t(pos) * W;
            w[k] = stream_src ? __ldcs(reinterpret_cast<const word_t<W> *>(src))
                              : *reinterpret_cast<const word_t<W> *>(src);
        }
    }
#pragma unroll
    for (int k = 0; k < CUNROLL; ++k) {
        const uint32_t v = v0 + k * CB;
        if (v < p.units) __stcs(reinterpret_cast<word_t<W> *>(out + int64_t(v) * W), w[k]);
    }
}

// ---- tiled transpose (innermost axis moves) ------------------------------------------------
// Source axis B is contiguous in the input, destination axis A is contiguous in the
// output.  A CTA moves a 64×64 patch of the (A, B) plane through shared memory so
// both sides see coalesced rows; the remaining axes are a batch index.
struct TileParams {
    Dims batch;            // strides: source bytes
    Dims batch_out;        // same extents, strides: destination bytes
    uint32_t na, nb;       // extents of A and B
    int64_t a_src_stride;  // bytes between consecutive A in the source
    int64_t b_dst_stride;  // bytes between consecutive B in the destination
    FastDiv tiles_a, tiles_b;
};

template <typename E, int TILE>
__global__ void __launch_bounds__(CB) tile_transpose_kernel(const char *__restrict__ in, char *__restrict__ out, TileParams p) {
    __shared__ E tile[TILE][TILE + 1];
    uint32_t b = blockIdx.x;
    uint32_t q = fd_div(b, p.tiles_b);
    const uint32_t tb = b - q * p.tiles_b.d;
    const uint32_t bt = fd_div(q, p.tiles_a);
    const uint32_t ta = q - bt * p.tiles_a.d;
    const char *src = in + unravel_bytes(bt, p.batch);
    char *dst = out + unravel_bytes(bt, p.batch_out);
    constexpr int NY = CB / TILE;    // tile rows covered by one pass of the CTA
    constexpr int PER = TILE / NY;   // elements per thread
    const int tx = threadIdx.x % TILE, ty = threadIdx.x / TILE;
    // load: x walks B (contiguous in the source), y walks A.  All of a thread's loads are issued
    // before the first shared-memory store, so PER independent requests per thread are in flight.
    {
        const uint32_t ib = tb * TILE + tx;
        E v[PER];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const uint32_t ia = ta * TILE + ty + i * NY;
            v[i] = (ia < p.na && ib < p.nb)
                       ? __ldcs(reinterpret_cast<const E *>(src + int64_t(ia) * p.a_src_stride + int64_t(ib) * sizeof(E)))
                       : E(0);
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) tile[ty + i * NY][tx] = v[i];
    }
    __syncthreads();
    // store: x walks A (contiguous in the destination), y walks B
    {
        const uint32_t ia = ta * TILE + tx;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const uint32_t ib = tb * TILE + ty + i * NY;
            if (ia < p.na && ib < p.nb)
                __stcs(reinterpret_cast<E *>(dst + int64_t(ib) * p.b_dst_stride + int64_t(ia) * sizeof(E)), tile[tx][ty + i * NY]);
        }
    }
}

// 2-byte elements, both moving extents even: global accesses are 4-byte words (two elements), so a
// thread has 16 × 4 bytes in flight instead of 16 × 2.  Patch = 64 (A) × 128 (B) elements.
__global__ void __launch_bounds__(CB) tile_transpose_pairs16_kernel(const char *__restrict__ in, char *__restrict__ out, TileParams p) {
    constexpr int TA = 64, TB = 128, PITCH = TB + 2;  // pitch in elements; rows stay 4-byte aligned
    __shared__ __align__(4) uint16_t tile[TA][PITCH];
    uint32_t b = blockIdx.x;
    uint32_t q = fd_div(b, p.tiles_b);
    const uint32_t tb = b - q * p.tiles_b.d;
    const uint32_t bt = fd_div(q, p.tiles_a);
    const uint32_t ta = q - bt * p.tiles_a.d;
    const char *src = in + unravel_bytes(bt, p.batch);
    char *dst = out + unravel_bytes(bt, p.batch_out);
    {   // load: 64 words across B per row, 4 rows of A per pass, 16 passes
        const int wx = threadIdx.x & 63, ty = threadIdx.x >> 6;
        const uint32_t ib = tb * TB + 2 * wx;
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t ia = ta * TA + ty + 4 * i;
            v[i] = (ia < p.na && ib < p.nb) ? __ldcs(reinterpret_cast<const uint32_t *>(src + int64_t(ia) * p.a_src_stride + int64_t(ib) * 2)) : 0u;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) *reinterpret_cast<uint32_t *>(&tile[ty + 4 * i][2 * wx]) = v[i];
    }
    __syncthreads();
    {   // store: 32 words across A per output row, 8 rows of B per pass, 16 passes
        const int wx = threadIdx.x & 31, ty = threadIdx.x >> 5;
        const uint32_t ia = ta * TA + 2 * wx;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int lb = ty + 8 * i;
            const uint32_t ib = tb * TB + lb;
            if (ia < p.na && ib < p.nb) {
                const uint32_t w = uint32_t(tile[2 * wx][lb]) | (uint32_t(tile[2 * wx + 1][lb]) << 16);
                __stcs(reinterpret_cast<uint32_t *>(dst + int64_t(ib) * p.b_dst_stride + int64_t(ia) * 2), w);
            }
        }
    }
}

// 1-byte elements, both moving extents multiples of 4: global accesses are 4-byte words (four
// elements).  Patch = 128 (A) × 128 (B) bytes, held as 128 rows of 32 words; the word column is
// rotated by the row's quad index so that both the row-wise writes (a warp writes one row) and the
// column-wise reads (lane q reads rows 4q..4q+3 of one word column) are bank-conflict free.  A
// thread turns four such words into four output words with a 4 × 4 byte transpose in registers.
__global__ void __launch_bounds__(CB) tile_transpose_quads8_kernel(const char *__restrict__ in, char *__restrict__ out, TileParams p) {
    constexpr int T = 128, NW = T / 4;
    __shared__ uint32_t tile[T][NW];
    uint32_t b = blockIdx.x;
    uint32_t q = fd_div(b, p.tiles_b);
    const uint32_t tb = b - q * p.tiles_b.d;
    const uint32_t bt = fd_div(q, p.tiles_a);
    const uint32_t ta = q - bt * p.tiles_a.d;
    const char *src = in + unravel_bytes(bt, p.batch);
    char *dst = out + unravel_bytes(bt, p.batch_out);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    {   // load: a warp reads one 128-byte row of the source per pass; 8 warps, 16 passes
        const uint32_t ib = tb * T + 4 * lane;
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t ia = ta * T + warp + 8 * i;
            v[i] = (ia < p.na && ib < p.nb) ? __ldcs(reinterpret_cast<const uint32_t *>(src + int64_t(ia) * p.a_src_stride + ib)) : 0u;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int row = warp + 8 * i;
            tile[row][(lane + (row >> 2)) & (NW - 1)] = v[i];
        }
    }
    __syncthreads();
    {   // store: lane = quad of A (output bytes 4*lane..4*lane+3), a warp covers a 128-byte output row
        const uint32_t ia = ta * T + 4 * lane;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int wb = warp + 8 * i;  // word column = four consecutive B
            const int col = (wb + lane) & (NW - 1);
            const uint32_t r0 = tile[4 * lane + 0][col], r1 = tile[4 * lane + 1][col];
            const uint32_t r2 = tile[4 * lane + 2][col], r3 = tile[4 * lane + 3][col];
            // byte j of row k → byte k of output word j
            const uint32_t lo01 = __byte_perm(r0, r1, 0x5140), hi01 = __byte_perm(r0, r1, 0x7362);
            const uint32_t lo23 = __byte_perm(r2, r3, 0x5140), hi23 = __byte_perm(r2, r3, 0x7362);
            const uint32_t o[4] = {__byte_perm(lo01, lo23, 0x5410), __byte_perm(lo01, lo23, 0x7632),
                                   __byte_perm(hi01, hi23, 0x5410), __byte_perm(hi01, hi23, 0x7632)};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t ib = tb * T + 4 * wb + j;
                if (ia < p.na && ib < p.nb) __stcs(reinterpret_cast<uint32_t *>(dst + int64_t(ib) * p.b_dst_stride + ia), o[j]);
            }
        }
    }
}

// ---- concat -----------------------------------------------------------------------------------
constexpr int CONCAT_MAX = 16;
struct ConcatParams {
    const char *src[CONCAT_MAX];
    uint32_t start[CONCAT_MAX + 1];  // first word of each input inside a group row; start[n] = group row words
    int n;
    FastDiv group_row;     // words per output row that this launch covers
    int64_t out_row_bytes; // full output row pitch
    int64_t out_col_bytes; // where this launch's inputs start inside an output row
    uint32_t units;        // outer * group_row
};

template <int W>
__global__ void __launch_bounds__(CB) concat_kernel(char *__restrict__ out, ConcatParams p) {
    const uint32_t v0 = blockIdx.x * (CB * CUNROLL) + threadIdx.x;
    word_t<W> w[CUNROLL];
    int64_t dst[CUNROLL];
#pragma unroll
    for (int k = 0; k < CUNROLL; ++k) {
        const uint32_t v = v0 + k * CB;
        if (v < p.units) {
            const uint32_t outer = fd_div(v, p.group_row);
            const uint32_t pos = v - outer * p.group_row.d;
            int j = 0;
#pragma unroll 1
            while (j + 1 < p.n && pos >= p.start[j + 1]) ++j;
            const uint32_t len = p.start[j + 1] - p.start[j];
            const char *s = p.src[j] + (int64_t(outer) * len + (pos - p.start[j])) * W;
            w[k] = __ldcs(reinterpret_cast<const word_t<W> *>(s));
            dst[k] = int64_t(outer) * p.out_row_bytes + p.out_col_bytes + int64_t(pos) * W;
        }
    }
#pragma unroll
    for (int k = 0; k < CUNROLL; ++k)
        if (v0 + k * CB < p.units) __stcs(reinterpret_cast<word_t<W> *>(out + dst[k]), w[k]);
}

// ---- broadcast with the innermost axis replicated ---------------------------------------------
// Every output word of W bytes holds W/sizeof(E) copies of ONE source element.
struct SplatParams {
    Dims rows;    // outer output axes; stride 0 where broadcast
    FastDiv run;  // words per innermost (replicated) run
    uint32_t units;
};
template <int W, typename E>
__global__ void __launch_bounds__(CB) splat_kernel(const char *__restrict__ in, char *__restrict__ out, SplatParams p) {
    const uint32_t v0 = blockIdx.x * (CB * CUNROLL) + threadIdx.x;
#pragma unroll
    for (int k = 0; k < CUNROLL; ++k) {
        const uint32_t v = v0 + k * CB;
        if (v < p.units) {
            const uint32_t row = fd_div(v, p.run);
            const E e = *reinterpret_cast<const E *>(in + unravel_bytes(row, p.rows));
            Pack<E, W / sizeof(E)> w;
#pragma unroll
            for (int i = 0; i < int(W / sizeof(E)); ++i) w.v[i] = e;
            st_stream<E, W / sizeof(E)>(reinterpret_cast<E *>(out + int64_t(v) * W), w);
        }
    }
}

// ---- indexselect -------------------------------------------------------------------------------
struct GatherParams {
    FastDiv run;      // words per gathered slice (post bytes / W)
    FastDiv nidx;     // number of indices
    int64_t axis_len; // extent of the gathered axis
    int64_t slice_bytes;
    uint32_t units;
};
template <int W, typename I>
__global__ void __launch_bounds__(CB) indexselect_kernel(const char *__restrict__ in, const I *__restrict__ idx,
                                                         char *__restrict__ out, GatherParams p, int32_t *oob) {
    const uint32_t v0 = blockIdx.x * (CB * CUNROLL) + threadIdx.x;
    word_t<W> w[CUNROLL];
#pragma unroll
    for (int k = 0; k < CUNROLL; ++k) {
        const uint32_t v = v0 + k * CB;
        if (v < p.units) {
            const uint32_t row = fd_div(v, p.run);
            const uint32_t pos = v - row * p.run.d;
            const uint32_t pre = fd_div(row, p.nidx);
            const uint32_t qi = row - pre * p.nidx.d;
            const int64_t ix = static_cast<int64_t>(idx[qi]);
            if (ix >= 0 && ix < p.axis_len) {
                const char *s = in + (int64_t(pre) * p.axis_len + ix) * p.slice_bytes + int64_t(pos) * W;
                w[k] = *reinterpret_cast<const word_t<W> *>(s);
            } else {
                w[k] = word_t<W>{};
                if (oob && pos == 0) atomicOr(oob, 1);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < CUNROLL; ++k) {
        const uint32_t v = v0 + k * CB;
        if (v < p.units) __stcs(reinterpret_cast<word_t<W> *>(out + int64_t(v) * W), w[k]);
    }
}

// Gather along the INNERMOST axis (slices of one element): a thread assembles a whole 16-byte output
// vector from VEC element reads of one source row (neighbouring threads read the same row, so the
// reads stay in L1) instead of moving one element per thread.
struct InnerGatherParams {
    FastDiv run;       // output vectors per row (indices / VEC)
    int64_t axis_len;  // elements per source row
    uint32_t units;    // output vectors
};
template <typename E, typename I>
__global__ void __launch_bounds__(CB) indexselect_inner_kernel(const E *__restrict__ in, const I *__restrict__ idx, E *__restrict__ out,
                                                               InnerGatherParams p, int32_t *oob) {
    constexpr int VEC = 16 / int(sizeof(E));
    const uint32_t v = blockIdx.x * CB + threadIdx.x;
    if (v >= p.units) return;
    const uint32_t row = fd_div(v, p.run);
    const uint32_t j0 = (v - row * p.run.d) * VEC;
    const E *src = in + int64_t(row) * p.axis_len;
    int64_t ix[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) ix[j] = static_cast<int64_t>(idx[j0 + j]);
    Pack<E, VEC> o;
    bool bad = false;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        const bool ok = ix[j] >= 0 && ix[j] < p.axis_len;
        o.v[j] = ok ? src[ok ? ix[j] : 0] : E(0);
        bad |= !ok;
    }
    if (bad && oob) atomicOr(oob, 1);
    st_stream<E, VEC>(out + int64_t(v) * VEC, o);
}

// The same gather with the source rows staged in shared memory: random element reads cost one L1
// sector access per lane from global memory (32 per warp load), but only a few bank conflicts from
// shared memory.  A CTA keeps the (validated) index list in shared memory and walks groups of R
// source rows: coalesced 16-byte loads in, picks, 16-byte stores out.
struct InnerGatherSmemParams {
    int64_t rows;   // source rows (product of the outer axes)
    int K, J, R;    // elements per source row, indices, rows staged per pass
    int row_vec;    // 1: source rows can be loaded as 16-byte vectors
};
template <typename E, typename I>
__global__ void __launch_bounds__(CB) indexselect_inner_smem_kernel(const E *__restrict__ in, const I *__restrict__ idx, E *__restrict__ out,
                                                                    InnerGatherSmemParams p, int32_t *oob) {
    constexpr int VEC = 16 / int(sizeof(E));
    extern __shared__ __align__(16) unsigned char smem_gather[];
    int32_t *sidx = reinterpret_cast<int32_t *>(smem_gather);
    E *srow = reinterpret_cast<E *>(smem_gather + ((size_t(p.J) * 4 + 15) / 16) * 16);
    bool bad = false;
    for (int j = threadIdx.x; j < p.J; j += CB) {
        const int64_t ix = static_cast<int64_t>(idx[j]);
        const bool ok = ix >= 0 && ix < p.K;
        sidx[j] = ok ? int32_t(ix) : -1;
        bad |= !ok;
    }
    if (bad && oob) atomicOr(oob, 1);
    const int jvec = p.J / VEC;
    for (int64_t r0 = int64_t(blockIdx.x) * p.R; r0 < p.rows; r0 += int64_t(gridDim.x) * p.R) {
        const int nr = int(p.rows - r0 < p.R ? p.rows - r0 : p.R);
        __syncthreads();  // the index list is complete / the previous group's picks are done
        const E *src = in + r0 * p.K;
        const int total = nr * p.K;
        if (p.row_vec) {
            for (int i = threadIdx.x; i < total / VEC; i += CB)
                reinterpret_cast<Pack<E, VEC> *>(srow)[i] = ld_stream<E, VEC>(src + int64_t(i) * VEC);
        } else {
            for (int i = threadIdx.x; i < total; i += CB) srow[i] = src[i];
        }
        __syncthreads();
        E *dst = out + r0 * p.J;
        // A thread keeps the VEC indices of ITS output column group in registers and walks the staged rows with
        // them: one shared-memory read per element (the picked value) instead of two (index and value).
        auto pick_rows = [&](int c, int lr_first, int lr_step) {
            int32_t ix[VEC];
#pragma unroll
            for (int j = 0; j < VEC; ++j) ix[j] = sidx[c * VEC + j];
            for (int lr = lr_first; lr < nr; lr += lr_step) {
                const E *row = srow + lr * p.K;
                Pack<E, VEC> o;
#pragma unroll
                for (int j = 0; j < VEC; ++j) o.v[j] = ix[j] >= 0 ? row[ix[j]] : E(0);
                st_stream<E, VEC>(dst + int64_t(lr) * p.J + c * VEC, o);
            }
        };
        if (jvec <= CB && CB % jvec == 0) {
            pick_rows(threadIdx.x % jvec, threadIdx.x / jvec, CB / jvec);  // several rows per sweep of the CTA
        } else {
            for (int c = threadIdx.x; c < jvec; c += CB) pick_rows(c, 0, 1);
        }
    }
}

// ---- repeat, per element (only for ranks whose (S, r) axis pairs exceed the kernels' axis limit) ---
struct RepeatParams {
    Dims outd;                 // output extents; stride = source bytes
    FastDiv rep[MAXD];         // repeats per axis
    uint32_t units;
};
template <typename E>
__global__ void __launch_bounds__(CB) repeat_kernel(const char *__restrict__ in, E *__restrict__ out, RepeatParams p) {
    const uint32_t v = blockIdx.x * CB + threadIdx.x;
    if (v >= p.units) return;
    uint32_t idx = v;
    int64_t off = 0;
#pragma unroll 1
    for (int i = p.outd.n - 1; i >= 0; --i) {
        uint32_t q = (i > 0) ? fd_div(idx, p.outd.fd[i]) : 0;
        uint32_t c = idx - q * p.outd.fd[i].d;
        off += int64_t(fd_div(c, p.rep[i])) * p.outd.stride[i];
        idx = q;
    }
    out[v] = *reinterpret_cast<const E *>(in + off);
}

// ---- repeat along the innermost axis (each source element r times in a row) ------------------
// One thread builds one 16-byte output vector; its source elements are neighbours of the ones the
// next threads read, so the (cached) element loads of a warp fall into a few sectors.
struct InnerRepeatParams {
    Dims rows;        // outer output axes; strides point into the source (0 for a repeat axis)
    FastDiv run;      // 16-byte vectors per output row
    FastDiv rep;      // r
    uint32_t units;   // output vectors
};
template <typename E>
__global__ void __launch_bounds__(CB) inner_repeat_kernel(const char *__restrict__ in, char *__restrict__ out, InnerRepeatParams p) {
    constexpr int VEC = 16 / int(sizeof(E));
    const uint32_t v = blockIdx.x * CB + threadIdx.x;
    if (v >= p.units) return;
    const uint32_t row = fd_div(v, p.run);
    const uint32_t e0 = (v - row * p.run.d) * VEC;
    const E *src = reinterpret_cast<const E *>(in + unravel_bytes(row, p.rows));
    Pack<E, VEC> o;
#pragma unroll
    for (int j = 0; j < VEC; ++j) o.v[j] = src[fd_div(e0 + j, p.rep)];
    st_stream<E, VEC>(reinterpret_cast<E *>(out) + int64_t(v) * VEC, o);
}

// Byte-permute selector for output word `word` (bytes 4·word .. 4·word+3 of a 16-byte output vector) when elements of
// ES bytes are each repeated R times: output byte b comes from source byte (b / (R·ES))·ES + b % ES.
template <int ES, int R> __host__ __device__ constexpr uint32_t repeat_selector(int word) {
    uint32_t sel = 0;
    for (int j = 0; j < 4; ++j) {
        const int b = 4 * word + j;
        sel |= uint32_t((b / (R * ES)) * ES + b % ES) << (4 * j);
    }
    return sel;
}

// r a power of two: the VEC / R (at least one) source elements of an output vector are one aligned
// load, expanded in registers.
// NB (1, 2, 4 or 8) naturally aligned bytes as ONE load, in the low bytes of the result.  (A struct of eight
// uint8_t copied as a struct came out as eight byte loads: the 1-byte repeat ran at 0.73 of the copy rate where the
// 2-byte one, same bytes per thread, ran at 0.95.)
template <int NB> __device__ __forceinline__ unsigned long long load_word(const void *p) {
    if constexpr (NB == 8) return *reinterpret_cast<const unsigned long long *>(p);
    else if constexpr (NB == 4) return *reinterpret_cast<const uint32_t *>(p);
    else if constexpr (NB == 2) return *reinterpret_cast<const uint16_t *>(p);
    else return *reinterpret_cast<const uint8_t *>(p);
}
template <typename E, int R>
__global__ void __launch_bounds__(CB) inner_repeat_pow2_kernel(const char *__restrict__ in, char *__restrict__ out, InnerRepeatParams p) {
    constexpr int VEC = 16 / int(sizeof(E));
    constexpr int M = (VEC / R) > 0 ? (VEC / R) : 1;
    constexpr bool SMALL = sizeof(E) <= 2;  // 1- and 2-byte elements: source bytes in one word, expanded by byte permutes
    const uint32_t v0 = blockIdx.x * (CB * CUNROLL) + threadIdx.x;
    Pack<E, M> sv[CUNROLL];
    unsigned long long raw[CUNROLL];
#pragma unroll
    for (int k = 0; k < CUNROLL; ++k) {  // every load of the thread is issued before the first store
        const uint32_t v = v0 + k * CB;
        raw[k] = 0;
        if (v < p.units) {
            const uint32_t row = fd_div(v, p.run);
            const uint32_t e0 = (v - row * p.run.d) * VEC;
            const E *src = reinterpret_cast<const E *>(in + unravel_bytes(row, p.rows)) + e0 / R;
            if constexpr (SMALL) raw[k] = load_word<int(sizeof(E)) * M>(src);
            else sv[k] = ld_cached<E, M>(src);
        }
    }
#pragma unroll
    for (int k = 0; k < CUNROLL; ++k) {
        const uint32_t v = v0 + k * CB;
        if (v < p.units) {
            Pack<E, VEC> o;
            if constexpr (SMALL) {
                // the at most 8 source bytes sit in two words and every output word is one byte permute of them (left
                // to the compiler this became an extract and an insert per byte: 0.61 of the copy rate)
                const uint32_t w0 = static_cast<uint32_t>(raw[k]), w1 = static_cast<uint32_t>(raw[k] >> 32);
                uint32_t *ow = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) ow[i] = __byte_perm(w0, w1, repeat_selector<int(sizeof(E)), R>(i));
            } else {
#pragma unroll
                for (int j = 0; j < VEC; ++j) o.v[j] = sv[k].v[(j / R) < M ? (j / R) : 0];
            }
            st_stream<E, VEC>(reinterpret_cast<E *>(out) + int64_t(v) * VEC, o);
        }
    }
}
template <typename E> void launch_inner_repeat(unsigned g, cudaStream_t st, const void *a, void *out, const InnerRepeatParams &q, int64_t r,
                                               bool src_aligned) {
    constexpr int VEC = 16 / int(sizeof(E));
    const char *in = (const char *)a;
    char *o = (char *)out;
    // the wide source load needs the source rows aligned to VEC / r elements
    if (src_aligned) {
        const unsigned g4 = (unsigned)((int64_t(q.units) + int64_t(CB) * CUNROLL - 1) / (int64_t(CB) * CUNROLL));
        switch (r) {
            case 2: inner_repeat_pow2_kernel<E, 2><<<g4, CB, 0, st>>>(in, o, q); return;
            case 4: inner_repeat_pow2_kernel<E, 4><<<g4, CB, 0, st>>>(in, o, q); return;
            case 8: inner_repeat_pow2_kernel<E, 8><<<g4, CB, 0, st>>>(in, o, q); return;
            case 16: inner_repeat_pow2_kernel<E, 16><<<g4, CB, 0, st>>>(in, o, q); return;
            default: break;
        }
    }
    (void)VEC;
    inner_repeat_kernel<E><<<g, CB, 0, st>>>(in, o, q);
}

template <int W, typename E>
void launch_splat(unsigned grid, cudaStream_t st, const void *a, void *out, const SplatParams &p) {
    if constexpr (W >= int(sizeof(E))) splat_kernel<W, E><<<grid, CB, 0, st>>>((const char *)a, (char *)out, p);
}

int check_shape(const char *what, const int64_t *shape, int ndim, int64_t *count) {
    if (ndim < 0 || ndim > MAXD) return fail(DX_E_SHAPE, "%s: rank %d outside [0, %d]", what, ndim, MAXD);
    if (ndim > 0 && !shape) return fail(DX_E_ARG, "%s: null shape", what);
    int64_t n = 1;
    for (int i = 0; i < ndim; ++i) {
        if (shape[i] < 0) return fail(DX_E_SHAPE, "%s: negative extent", what);
        n *= shape[i];
    }
    *count = n;
    return DX_OK;
}

bool overlaps(const void *a, int64_t abytes, const void *b, int64_t bbytes) {
    const char *x = (const char *)a, *y = (const char *)b;
    return x < y + bbytes && y < x + abytes;
}

}  // namespace
}  // namespace dx

using namespace dx;

// ==================================================================================================
extern "C" int dx_transpose(int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *perm, void *out,
                            void *stream) {
    cudaStream_t st = as_stream(stream);
    const int es = dx_dtype_size(dtype);
    if (es == 0) return fail(DX_E_DTYPE, "transpose: unsupported dtype code %d", dtype);
    int64_t n;
    if (int e = check_shape("transpose", shape, ndim, &n)) return e;
    if (ndim > 0 && !perm) return fail(DX_E_ARG, "transpose: null dim order");
    bool seen[MAXD] = {false};
    for (int i = 0; i < ndim; ++i) {
        if (perm[i] < 0 || perm[i] >= ndim || seen[perm[i]])
            return fail(DX_E_SHAPE, "transpose: dim order is not a permutation of 0..%d", ndim - 1);
        seen[perm[i]] = true;
    }
    if (n == 0) return DX_OK;
    if (!a || !out) return fail(DX_E_ARG, "transpose: null pointer");
    if (overlaps(a, n * es, out, n * es)) return fail(DX_E_ALIAS, "transpose: output overlaps input");

    // source strides (elements) and the output axes as (extent, source stride)
    int64_t sstride[MAXD];
    {
        int64_t s = 1;
        for (int i = ndim - 1; i >= 0; --i) { sstride[i] = s; s *= shape[i]; }
    }
    struct Ax { int64_t size, stride; };
    std::vector<Ax> ax;  // outermost first, extent-1 axes dropped, source-contiguous neighbours merged
    for (int i = 0; i < ndim; ++i) {
        const int64_t sz = shape[perm[i]], sd = sstride[perm[i]];
        if (sz == 1) continue;
        if (!ax.empty() && ax.back().stride == sd * sz) { ax.back().size *= sz; ax.back().stride = sd; }
        else ax.push_back({sz, sd});
    }
    if (ax.empty() || (ax.size() == 1)) {  // identity layout
        cudaError_t e = cudaMemcpyAsync(out, a, size_t(n) * es, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return fail(DX_E_CUDA, "transpose(copy): %s", cudaGetErrorString(e));
        return DX_OK;
    }
    for (auto &x : ax)
        if (x.size >= (1ll << 31)) return fail(DX_E_SHAPE, "transpose: merged axis too long");

    if (ax.back().stride == 1) {
        // innermost axis preserved: gather contiguous runs
        const int64_t run_bytes = ax.back().size * es;
        const int w = widest_word(es, {run_bytes}, {a, out});
        RunGatherParams p;
        p.rows.n = int(ax.size()) - 1;
        for (int i = 0; i < p.rows.n; ++i) {
            p.rows.fd[i] = make_fastdiv((uint32_t)ax[i].size);
            p.rows.stride[i] = ax[i].stride * es;
        }
        p.run = make_fastdiv((uint32_t)(run_bytes / w));
        const int64_t units = n * es / w;
        unsigned grid;
        if (int e = grid_for(units, &grid)) return e;
        p.units = (uint32_t)units;
        DISPATCH_W(w, run_gather_kernel<W><<<grid, CB, 0, st>>>((const char *)a, (char *)out, p, true));
        return check_launch("transpose(runs)");
    }

    // innermost axis moves: tile over A (output-innermost) and B (source-innermost)
    const int na_i = int(ax.size()) - 1;
    int nb_i = -1;
    for (int i = 0; i < int(ax.size()); ++i)
        if (ax[i].stride == 1) nb_i = i;
    if (nb_i < 0) return fail(DX_E_SHAPE, "transpose: internal: no unit-stride axis");
    TileParams p;
    p.na = (uint32_t)ax[na_i].size;
    p.nb = (uint32_t)ax[nb_i].size;
    p.a_src_stride = ax[na_i].stride * es;
    // destination strides of the merged output axes
    std::vector<int64_t> dstride(ax.size());
    {
        int64_t s = 1;
        for (int i = int(ax.size()) - 1; i >= 0; --i) { dstride[i] = s; s *= ax[i].size; }
    }
    p.b_dst_stride = dstride[nb_i] * es;
    p.batch.n = p.batch_out.n = 0;
    int64_t nbatch = 1;
    for (int i = 0; i < int(ax.size()); ++i) {
        if (i == na_i || i == nb_i) continue;
        p.batch.fd[p.batch.n] = p.batch_out.fd[p.batch.n] = make_fastdiv((uint32_t)ax[i].size);
        p.batch.stride[p.batch.n] = ax[i].stride * es;
        p.batch_out.stride[p.batch.n] = dstride[i] * es;
        ++p.batch.n;
        ++p.batch_out.n;
        nbatch *= ax[i].size;
    }
    // 2-byte elements with even moving extents and 4-byte aligned bases: the paired-word kernel
    const bool pairs16 = es == 2 && (p.na % 2 == 0) && (p.nb % 2 == 0) && aligned_to(a, 4) && aligned_to(out, 4);
    // 1-byte elements, moving extents and every stride a multiple of 4: the quad-word kernel
    bool quads8 = es == 1 && (p.na % 4 == 0) && (p.nb % 4 == 0) && aligned_to(a, 4) && aligned_to(out, 4) &&
                  (p.a_src_stride % 4 == 0) && (p.b_dst_stride % 4 == 0);
    for (int i = 0; i < p.batch.n; ++i) quads8 = quads8 && (p.batch.stride[i] % 4 == 0) && (p.batch_out.stride[i] % 4 == 0);
    const int tile_a = quads8 ? 128 : 64, tile_b = (pairs16 || quads8) ? 128 : 64;
    const int64_t ta = (p.na + tile_a - 1) / tile_a, tb = (p.nb + tile_b - 1) / tile_b;
    p.tiles_a = make_fastdiv((uint32_t)ta);
    p.tiles_b = make_fastdiv((uint32_t)tb);
    const int64_t ctas = ta * tb * nbatch;
    if (ctas >= (1ll << 31)) return fail(DX_E_SHAPE, "transpose: grid too large");
    if (pairs16) {
        tile_transpose_pairs16_kernel<<<(unsigned)ctas, CB, 0, st>>>((const char *)a, (char *)out, p);
        return check_launch("transpose(tiles/pairs)");
    }
    if (quads8) {
        tile_transpose_quads8_kernel<<<(unsigned)ctas, CB, 0, st>>>((const char *)a, (char *)out, p);
        return check_launch("transpose(tiles/quads)");
    }
    switch (es) {
        case 8: tile_transpose_kernel<uint64_t, 64><<<(unsigned)ctas, CB, 0, st>>>((const char *)a, (char *)out, p); break;
        case 4: tile_transpose_kernel<uint32_t, 64><<<(unsigned)ctas, CB, 0, st>>>((const char *)a, (char *)out, p); break;
        case 2: tile_transpose_kernel<uint16_t, 64><<<(unsigned)ctas, CB, 0, st>>>((const char *)a, (char *)out, p); break;
        default: tile_transpose_kernel<uint8_t, 64><<<(unsigned)ctas, CB, 0, st>>>((const char *)a, (char *)out, p); break;
    }
    return check_launch("transpose(tiles)");
}

// ==================================================================================================
extern "C" int dx_concat(int dtype, const void *const *inputs, const int64_t *axis_len, int ninputs,
                         const int64_t *out_shape, int ndim, int axis, void *out, void *stream) {
    cudaStream_t st = as_stream(stream);
    const int es = dx_dtype_size(dtype);
    if (es == 0) return fail(DX_E_DTYPE, "concat: unsupported dtype code %d", dtype);
    int64_t n;
    if (int e = check_shape("concat", out_shape, ndim, &n)) return e;
    if (ninputs < 1 || !inputs || !axis_len) return fail(DX_E_ARG, "concat: no inputs");
    if (axis < 0 || axis >= ndim) return fail(DX_E_SHAPE, "concat: axis %d out of range for rank %d", axis, ndim);
    int64_t total = 0;
    for (int i = 0; i < ninputs; ++i) {
        if (axis_len[i] < 0) return fail(DX_E_SHAPE, "concat: negative extent");
        total += axis_len[i];
    }
    if (total != out_shape[axis])
        return fail(DX_E_SHAPE, "concat: inputs cover %lld along axis %d, output has %lld", (long long)total, axis,
                    (long long)out_shape[axis]);
    if (n == 0) return DX_OK;
    if (!out) return fail(DX_E_ARG, "concat: null output");
    int64_t outer = 1, inner = 1;
    for (int i = 0; i < axis; ++i) outer *= out_shape[i];
    for (int i = axis + 1; i < ndim; ++i) inner *= out_shape[i];
    // word width: must divide every input's row and align every pointer
    int w = 16;
    auto fits = [&](int w_) {
        if (!aligned_to(out, w_)) return false;
        for (int i = 0; i < ninputs; ++i) {
            if (axis_len[i] == 0) continue;
            if ((axis_len[i] * inner * es) % w_ != 0) return false;
            if (!aligned_to(inputs[i], w_)) return false;
        }
        return true;
    };
    while (w > es && !fits(w)) w >>= 1;
    for (int i = 0; i < ninputs; ++i) {
        if (axis_len[i] == 0) continue;
        if (!inputs[i]) return fail(DX_E_ARG, "concat: inputs[%d] is null", i);
        if (overlaps(inputs[i], outer * axis_len[i] * inner * es, out, n * es))
            return fail(DX_E_ALIAS, "concat: output overlaps inputs[%d]", i);
    }
    const int64_t out_row_bytes = total * inner * es;
    int64_t col = 0;  // byte offset inside an output row
    int i = 0;
    while (i < ninputs) {
        ConcatParams p;
        p.n = 0;
        int64_t words = 0;
        const int64_t col0 = col;
        while (i < ninputs && p.n < CONCAT_MAX) {
            if (axis_len[i] > 0) {
                p.src[p.n] = (const char *)inputs[i];
                p.start[p.n] = (uint32_t)words;
                const int64_t row_words = axis_len[i] * inner * es / w;
                words += row_words;
                col += row_words * w;
                ++p.n;
            }
            ++i;
        }
        if (p.n == 0) break;
        if (words >= (1ll << 31)) return fail(DX_E_SHAPE, "concat: row too long");
        p.start[p.n] = (uint32_t)words;
        for (int k = p.n; k < CONCAT_MAX; ++k) p.src[k] = nullptr;
        p.group_row = make_fastdiv((uint32_t)words);
        p.out_row_bytes = out_row_bytes;
        p.out_col_bytes = col0;
        const int64_t units = outer * words;
        unsigned grid;
        if (int e = grid_for(units, &grid)) return e;
        p.units = (uint32_t)units;
        DISPATCH_W(w, concat_kernel<W><<<grid, CB, 0, st>>>((char *)out, p));
        if (int e = check_launch("concat")) return e;
    }
    return DX_OK;
}

// ==================================================================================================
extern "C" int dx_broadcast_to(int dtype, const void *a, const int64_t *a_shape, int a_ndim, const int64_t *out_shape,
                               int out_ndim, void *out, void *stream) {
    cudaStream_t st = as_stream(stream);
    const int es = dx_dtype_size(dtype);
    if (es == 0) return fail(DX_E_DTYPE, "broadcastTo: unsupported dtype code %d", dtype);
    int64_t na, n;
    if (int e = check_shape("broadcastTo", a_shape, a_ndim, &na)) return e;
    if (int e = check_shape("broadcastTo", out_shape, out_ndim, &n)) return e;
    if (a_ndim > out_ndim) return fail(DX_E_SHAPE, "broadcastTo: Shapes are not broadcastable for operation");
    const int lead = out_ndim - a_ndim;
    for (int i = 0; i < a_ndim; ++i)
        if (a_shape[i] != out_shape[lead + i] && a_shape[i] != 1)
            return fail(DX_E_SHAPE, "broadcastTo: Shapes are not broadcastable for operation");
    if (n == 0) return DX_OK;
    if (!a || !out) return fail(DX_E_ARG, "broadcastTo: null pointer");
    if (overlaps(a, na * es, out, n * es)) return fail(DX_E_ALIAS, "broadcastTo: output overlaps input");
    if (na == n) {
        cudaError_t e = cudaMemcpyAsync(out, a, size_t(n) * es, cudaMemcpyDeviceToDevice, st);
        if (e != cudaSuccess) return fail(DX_E_CUDA, "broadcastTo(copy): %s", cudaGetErrorString(e));
        return DX_OK;
    }
    // output axes as (extent, source stride in elements; 0 = broadcast); merge neighbours of one kind
    struct Ax { int64_t size, stride; bool bc; };
    std::vector<Ax> ax;
    {
        int64_t sstride[MAXD];
        int64_t s = 1;
        for (int i = a_ndim - 1; i >= 0; --i) { sstride[i] = s; s *= a_shape[i]; }
        for (int i = 0; i < out_ndim; ++i) {
            const int64_t sz = out_shape[i];
            if (sz == 1) continue;
            const bool bc = (i < lead) || a_shape[i - lead] == 1;
            const int64_t sd = bc ? 0 : sstride[i - lead];
            if (!ax.empty() && ax.back().bc == bc && (bc || ax.back().stride == sd * sz)) {
                ax.back().size *= sz;
                ax.back().stride = sd;
            } else ax.push_back({sz, sd, bc});
        }
    }
    for (auto &x : ax)
        if (x.size >= (1ll << 31)) return fail(DX_E_SHAPE, "broadcastTo: merged axis too long");
    const int64_t run_bytes = ax.back().size * es;
    if (!ax.back().bc) {
        const int w = widest_word(es, {run_bytes}, {a, out});
        RunGatherParams p;
        p.rows.n = int(ax.size()) - 1;
        for (int i = 0; i < p.rows.n; ++i) {
            p.rows.fd[i] = make_fastdiv((uint32_t)ax[i].size);
            p.rows.stride[i] = ax[i].stride * es;
        }
        p.run = make_fastdiv((uint32_t)(run_bytes / w));
        const int64_t units = n * es / w;
        unsigned grid;
        if (int e = grid_for(units, &grid)) return e;
        p.units = (uint32_t)units;
        // the source is re-read many times: keep it cached
        DISPATCH_W(w, run_gather_kernel<W><<<grid, CB, 0, st>>>((const char *)a, (char *)out, p, false));
        return check_launch("broadcastTo(runs)");
    }
    // innermost axis replicated
    const int w = widest_word(es, {run_bytes}, {out});
    SplatParams p;
    p.rows.n = int(ax.size()) - 1;
    for (int i = 0; i < p.rows.n; ++i) {
        p.rows.fd[i] = make_fastdiv((uint32_t)ax[i].size);
        p.rows.stride[i] = ax[i].stride * es;
    }
    p.run = make_fastdiv((uint32_t)(run_bytes / w));
    const int64_t units = n * es / w;
    unsigned grid;
    if (int e = grid_for(units, &grid)) return e;
    p.units = (uint32_t)units;
#define SPLAT(E) DISPATCH_W(w, launch_splat<W, E>(grid, st, a, out, p))
    switch (es) {
        case 8: SPLAT(uint64_t); break;
        case 4: SPLAT(uint32_t); break;
        case 2: SPLAT(uint16_t); break;
        default: SPLAT(uint8_t); break;
    }
#undef SPLAT
    return check_launch("broadcastTo(splat)");
}

// ==================================================================================================
extern "C" int dx_indexselect(int dtype, const void *a, const int64_t *a_shape, int a_ndim, int idx_dtype,
                              const void *idx, const int64_t *idx_shape, int idx_ndim, int axis, void *out,
                              int32_t *oob_flag, void *stream) {
    cudaStream_t st = as_stream(stream);
    const int es = dx_dtype_size(dtype);
    if (es == 0) return fail(DX_E_DTYPE, "indexselect: unsupported dtype code %d", dtype);
    if (idx_dtype != DX_I32 && idx_dtype != DX_I64)
        return fail(DX_E_DTYPE, "indexselect: index dtype must be int64 or int32 (dtype code %d)", idx_dtype);
    int64_t na, ni;
    if (int e = check_shape("indexselect", a_shape, a_ndim, &na)) return e;
    if (int e = check_shape("indexselect", idx_shape, idx_ndim, &ni)) return e;
    if (axis < 0) axis += a_ndim;
    if (axis < 0 || axis >= a_ndim) return fail(DX_E_SHAPE, "indexselect: Axis is out of bounds");
    int64_t pre = 1, post = 1;
    for (int i = 0; i < axis; ++i) pre *= a_shape[i];
    for (int i = axis + 1; i < a_ndim; ++i) post *= a_shape[i];
    const int64_t n = pre * ni * post;
    if (n == 0) return DX_OK;
    if (!a || !idx || !out) return fail(DX_E_ARG, "indexselect: null pointer");
    if (overlaps(a, na * es, out, n * es)) return fail(DX_E_ALIAS, "indexselect: output overlaps input");
    const int64_t slice_bytes = post * es;
    if (post == 1 && (ni * es) % 16 == 0 && aligned_to(out, 16) && ni * 4 <= 16384 && a_shape[axis] * es <= 16384 && pre >= 64) {
        // rows and index list fit in shared memory
        InnerGatherSmemParams q;
        q.rows = pre;
        q.K = (int)a_shape[axis];
        q.J = (int)ni;
        q.R = (int)std::max<int64_t>(1, std::min<int64_t>(32768 / (a_shape[axis] * es), 32));
        q.row_vec = (aligned_to(a, 16) && (a_shape[axis] * es) % 16 == 0) ? 1 : 0;
        const size_t smem = ((size_t(q.J) * 4 + 15) / 16) * 16 + size_t(q.R) * q.K * es;
        const int64_t groups = (pre + q.R - 1) / q.R;
        const unsigned g = (unsigned)std::min<int64_t>(groups, int64_t(sm_count()) * 4);
#define DX_INNER_SMEM(E)                                                                                                           \
    do {                                                                                                                           \
        if (idx_dtype == DX_I32) indexselect_inner_smem_kernel<E, int32_t><<<g, CB, smem, st>>>((const E *)a, (const int32_t *)idx, (E *)out, q, oob_flag); \
        else indexselect_inner_smem_kernel<E, int64_t><<<g, CB, smem, st>>>((const E *)a, (const int64_t *)idx, (E *)out, q, oob_flag);       \
    } while (0)
        switch (es) {
            case 8: DX_INNER_SMEM(uint64_t); break;
            case 4: DX_INNER_SMEM(uint32_t); break;
            case 2: DX_INNER_SMEM(uint16_t); break;
            default: DX_INNER_SMEM(uint8_t); break;
        }
#undef DX_INNER_SMEM
        return check_launch("indexselect(inner, staged)");
    }
    if (post == 1 && (ni * es) % 16 == 0 && aligned_to(out, 16) && n * es / 16 < (1ll << 31) && pre < (1ll << 31)) {
        InnerGatherParams q;
        q.run = make_fastdiv((uint32_t)(ni * es / 16));
        q.axis_len = a_shape[axis];
        q.units = (uint32_t)(n * es / 16);
        const unsigned g = (unsigned)((int64_t(q.units) + CB - 1) / CB);
#define DX_INNER_GATHER(E)                                                                                                        \
    do {                                                                                                                          \
        if (idx_dtype == DX_I32) indexselect_inner_kernel<E, int32_t><<<g, CB, 0, st>>>((const E *)a, (const int32_t *)idx, (E *)out, q, oob_flag); \
        else indexselect_inner_kernel<E, int64_t><<<g, CB, 0, st>>>((const E *)a, (const int64_t *)idx, (E *)out, q, oob_flag);       \
    } while (0)
        switch (es) {
            case 8: DX_INNER_GATHER(uint64_t); break;
            case 4: DX_INNER_GATHER(uint32_t); break;
            case 2: DX_INNER_GATHER(uint16_t); break;
            default: DX_INNER_GATHER(uint8_t); break;
        }
#undef DX_INNER_GATHER
        return check_launch("indexselect(inner)");
    }
    const int w = widest_word(es, {slice_bytes}, {a, out});
    if (ni >= (1ll << 31) || slice_bytes / w >= (1ll << 31)) return fail(DX_E_SHAPE, "indexselect: extent too large");
    GatherParams p;
    p.run = make_fastdiv((uint32_t)(slice_bytes / w));
    p.nidx = make_fastdiv((uint32_t)ni);
    p.axis_len = a_shape[axis];
    p.slice_bytes = slice_bytes;
    const int64_t units = n * es / w;
    unsigned grid;
    if (int e = grid_for(units, &grid)) return e;
    p.units = (uint32_t)units;
    if (idx_dtype == DX_I32) {
        DISPATCH_W(w, indexselect_kernel<W, int32_t><<<grid, CB, 0, st>>>((const char *)a, (const int32_t *)idx, (char *)out, p, oob_flag));
    } else {
        DISPATCH_W(w, indexselect_kernel<W, int64_t><<<grid, CB, 0, st>>>((const char *)a, (const int64_t *)idx, (char *)out, p, oob_flag));
    }
    return check_launch("indexselect");
}

// ==================================================================================================
extern "C" int dx_repeat(int dtype, const void *a, const int64_t *a_shape, int ndim, const int64_t *repeats, void *out,
                         void *stream) {
    cudaStream_t st = as_stream(stream);
    const int es = dx_dtype_size(dtype);
    if (es == 0) return fail(DX_E_DTYPE, "repeat: unsupported dtype code %d", dtype);
    int64_t na;
    if (int e = check_shape("repeat", a_shape, ndim, &na)) return e;
    if (ndim > 0 && !repeats) return fail(DX_E_ARG, "repeat: null repeats");
    RepeatParams p;
    p.outd.n = ndim;
    int64_t n = 1, s = 1;
    for (int i = ndim - 1; i >= 0; --i) {
        if (repeats[i] < 1) return fail(DX_E_SHAPE, "repeat: repeats must be >= 1");
        const int64_t o = a_shape[i] * repeats[i];
        if (o >= (1ll << 31) || repeats[i] >= (1ll << 31)) return fail(DX_E_SHAPE, "repeat: extent too large");
        p.outd.fd[i] = make_fastdiv((uint32_t)std::max<int64_t>(o, 1));
        p.rep[i] = make_fastdiv((uint32_t)repeats[i]);
        p.outd.stride[i] = s * es;
        s *= a_shape[i];
        n *= o;
    }
    if (n == 0) return DX_OK;
    if (!a || !out) return fail(DX_E_ARG, "repeat: null pointer");
    if (n >= (1ll << 31)) return fail(DX_E_SHAPE, "repeat: output too large");
    if (overlaps(a, na * es, out, n * es)) return fail(DX_E_ALIAS, "repeat: output overlaps input");
    // innermost axis repeated a few times: the splat kernel's words would be r elements wide, too narrow
    if (ndim >= 1 && repeats[ndim - 1] > 1 && repeats[ndim - 1] <= 64 && aligned_to(out, 16) &&
        (a_shape[ndim - 1] * repeats[ndim - 1] * es) % 16 == 0 && n * es / 16 < (1ll << 31)) {
        InnerRepeatParams q;
        q.rows.n = 0;
        int64_t sstride = a_shape[ndim - 1];  // source stride, in elements, of the axis being added
        bool fits = true;
        std::vector<std::pair<int64_t, int64_t>> axes;  // (extent, source byte stride), innermost first
        for (int i = ndim - 2; i >= 0; --i) {
            if (repeats[i] > 1) axes.push_back({repeats[i], 0});
            axes.push_back({a_shape[i], sstride * es});
            sstride *= a_shape[i];
        }
        if (int(axes.size()) > MAXD) fits = false;
        if (fits) {
            for (auto it = axes.rbegin(); it != axes.rend(); ++it) {  // outermost first
                q.rows.fd[q.rows.n] = make_fastdiv((uint32_t)it->first);
                q.rows.stride[q.rows.n] = it->second;
                ++q.rows.n;
            }
            q.run = make_fastdiv((uint32_t)(a_shape[ndim - 1] * repeats[ndim - 1] * es / 16));
            q.rep = make_fastdiv((uint32_t)repeats[ndim - 1]);
            q.units = (uint32_t)(n * es / 16);
            const unsigned g = (unsigned)((int64_t(q.units) + CB - 1) / CB);
            // every source row starts on a 16-byte boundary (so any VEC / r element load inside it is aligned)
            const bool src_aligned = aligned_to(a, 16) && (a_shape[ndim - 1] * es) % 16 == 0;
            const int64_t r = repeats[ndim - 1];
            switch (es) {
                case 8: launch_inner_repeat<uint64_t>(g, st, a, out, q, r, src_aligned); break;
                case 4: launch_inner_repeat<uint32_t>(g, st, a, out, q, r, src_aligned); break;
                case 2: launch_inner_repeat<uint16_t>(g, st, a, out, q, r, src_aligned); break;
                default: launch_inner_repeat<uint8_t>(g, st, a, out, q, r, src_aligned); break;
            }
            return check_launch("repeat(inner)");
        }
    }
    // Each axis of extent S repeated r times is the pair of axes (S, r) with source strides
    // (stride, 0): the repeat is a broadcast of [S0,1,S1,1,…] to [S0,r0,S1,r1,…], which the word-wide
    // run / splat kernels move at memory speed.  Only when that needs more axes than the kernels
    // carry does the per-element kernel below run.
    {
        std::vector<int64_t> src_shape, dst_shape;
        for (int i = 0; i < ndim; ++i) {
            src_shape.push_back(a_shape[i]);
            dst_shape.push_back(a_shape[i]);
            if (repeats[i] > 1) {
                src_shape.push_back(1);
                dst_shape.push_back(repeats[i]);
            }
        }
        if (int(dst_shape.size()) <= MAXD)
            return dx_broadcast_to(dtype, a, src_shape.data(), int(src_shape.size()), dst_shape.data(), int(dst_shape.size()), out, stream);
    }
    p.units = (uint32_t)n;
    const unsigned grid = (unsigned)((n + CB - 1) / CB);
    switch (es) {
        case 8: repeat_kernel<uint64_t><<<grid, CB, 0, st>>>((const char *)a, (uint64_t *)out, p); break;
        case 4: repeat_kernel<uint32_t><<<grid, CB, 0, st>>>((const char *)a, (uint32_t *)out, p); break;
        case 2: repeat_kernel<uint16_t><<<grid, CB, 0, st>>>((const char *)a, (uint16_t *)out, p); break;
        default: repeat_kernel<uint8_t><<<grid, CB, 0, st>>>((const char *)a, (uint8_t *)out, p); break;
    }
    return check_launch("repeat");
}
