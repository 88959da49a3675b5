// Streaming elementwise kernel templates.
//
// One CTA handles one tile of BLOCK*UNROLL*VEC elements.  Inside a tile the
// vectors are interleaved across threads (thread t takes vectors t, t+BLOCK,
// ...), so each warp-level load/store covers 32 consecutive 16-byte vectors
// (512 contiguous bytes), and every thread has UNROLL independent 16-byte loads
// per input in flight before the first use.  Full tiles run without bounds
// checks; the last, partial tile falls back to guarded scalar accesses.  Each
// thread reads all its inputs before it writes, and only writes indices it has
// read, so an output that aliases an input at the same base pointer is safe.
#pragma once
#include "common.cuh"

namespace dx {

constexpr int EW_BLOCK = 256;
constexpr int EW_UNROLL = 4;

// Whether a functor offers `pair(a0, a1, c0, c1)`, two elements per call (packed arithmetic inside).
template <typename F, typename = void> struct functor_has_pair : std::false_type {};
template <typename F> struct functor_has_pair<F, std::void_t<decltype(F::has_pair)>> : std::integral_constant<bool, F::has_pair> {};
// ... and a cheap test on a whole input vector (`vector_is_plain`) after which `pair_plain` may replace `pair`.
template <typename F, typename = void> struct functor_has_vector_check : std::false_type {};
template <typename F> struct functor_has_vector_check<F, std::void_t<decltype(F::has_vector_check)>> : std::integral_constant<bool, F::has_vector_check> {};

template <int VEC, typename TA, typename TC, typename F>
__global__ void __launch_bounds__(EW_BLOCK) ew1_kernel(const TA *a, TC *c, int64_t n, F f) {
    griddep_wait_cta();
    constexpr int64_t TILE = int64_t(EW_BLOCK) * EW_UNROLL * VEC;
    const int64_t base = int64_t(blockIdx.x) * TILE;
    if (base + TILE <= n) {
        Pack<TA, VEC> va[EW_UNROLL];
#pragma unroll
        for (int u = 0; u < EW_UNROLL; ++u)
            va[u] = ld_stream<TA, VEC>(a + base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC);
#pragma unroll
        for (int u = 0; u < EW_UNROLL; ++u) {
            Pack<TC, VEC> vc;
            if constexpr (functor_has_pair<F>::value && functor_has_vector_check<F>::value && VEC % 2 == 0) {
                if (F::template vector_is_plain<VEC>(va[u])) {
#pragma unroll
                    for (int i = 0; i < VEC; i += 2) f.pair_plain(va[u].v[i], va[u].v[i + 1], vc.v[i], vc.v[i + 1]);
                } else {
#pragma unroll
                    for (int i = 0; i < VEC; i += 2) f.pair(va[u].v[i], va[u].v[i + 1], vc.v[i], vc.v[i + 1]);
                }
            } else if constexpr (functor_has_pair<F>::value && VEC % 2 == 0) {
#pragma unroll
                for (int i = 0; i < VEC; i += 2) f.pair(va[u].v[i], va[u].v[i + 1], vc.v[i], vc.v[i + 1]);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) vc.v[i] = f(va[u].v[i]);
            }
            st_stream<TC, VEC>(c + base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC, vc);
        }
    } else {
        for (int64_t i = base + threadIdx.x; i < n; i += EW_BLOCK) c[i] = f(a[i]);
    }
}

template <int VEC, typename TA, typename TB, typename TC, typename F>
__global__ void __launch_bounds__(EW_BLOCK)
    ew2_kernel(const TA *a, const TB *b, TC *c, int64_t n, F f) {
    griddep_wait_cta();
    constexpr int64_t TILE = int64_t(EW_BLOCK) * EW_UNROLL * VEC;
    const int64_t base = int64_t(blockIdx.x) * TILE;
    if (base + TILE <= n) {
        Pack<TA, VEC> va[EW_UNROLL];
        Pack<TB, VEC> vb[EW_UNROLL];
#pragma unroll
        for (int u = 0; u < EW_UNROLL; ++u)
            va[u] = ld_stream<TA, VEC>(a + base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC);
#pragma unroll
        for (int u = 0; u < EW_UNROLL; ++u)
            vb[u] = ld_stream<TB, VEC>(b + base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC);
#pragma unroll
        for (int u = 0; u < EW_UNROLL; ++u) {
            Pack<TC, VEC> vc;
            if constexpr (functor_has_pair<F>::value && VEC % 2 == 0) {
#pragma unroll
                for (int i = 0; i < VEC; i += 2) f.pair(va[u].v[i], va[u].v[i + 1], vb[u].v[i], vb[u].v[i + 1], vc.v[i], vc.v[i + 1]);
            } else {
#pragma unroll
                for (int i = 0; i < VEC; ++i) vc.v[i] = f(va[u].v[i], vb[u].v[i]);
            }
            st_stream<TC, VEC>(c + base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC, vc);
        }
    } else {
        for (int64_t i = base + threadIdx.x; i < n; i += EW_BLOCK) c[i] = f(a[i], b[i]);
    }
}

// Output-only (fill).
template <int VEC, typename TC>
__global__ void __launch_bounds__(EW_BLOCK) ew0_kernel(TC *__restrict__ c, int64_t n, TC value) {
    constexpr int64_t TILE = int64_t(EW_BLOCK) * EW_UNROLL * VEC;
    const int64_t base = int64_t(blockIdx.x) * TILE;
    if (base + TILE <= n) {
        Pack<TC, VEC> vc;
#pragma unroll
        for (int i = 0; i < VEC; ++i) vc.v[i] = value;
#pragma unroll
        for (int u = 0; u < EW_UNROLL; ++u)
            st_stream<TC, VEC>(c + base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC, vc);
    } else {
        for (int64_t i = base + threadIdx.x; i < n; i += EW_BLOCK) c[i] = value;
    }
}

template <typename... Ts> constexpr size_t max_sizeof() {
    size_t m = 0;
    ((m = sizeof(Ts) > m ? sizeof(Ts) : m), ...);
    return m;
}

inline int ew_grid(int64_t n, int vec, int64_t *grid) {
    const int64_t tile = int64_t(EW_BLOCK) * EW_UNROLL * vec;
    *grid = (n + tile - 1) / tile;
    if (*grid > 0x7fffffffLL) return fail(DX_E_SHAPE, "element count %lld too large for one launch", (long long)n);
    return DX_OK;
}

// Vector width: 16 bytes for the widest operand; drops to scalar if any pointer
// is not aligned for that.
template <typename TA, typename TC, typename F>
int launch_ew1(const TA *a, TC *c, int64_t n, F f, cudaStream_t st, const char *what) {
    if (n == 0) return DX_OK;
    if (n < 0 || !a || !c) return fail(DX_E_ARG, "%s: bad pointer or count", what);
    constexpr int VEC = 16 / max_sizeof<TA, TC>();
    int64_t grid;
    if (aligned_to(a, sizeof(TA) * VEC) && aligned_to(c, sizeof(TC) * VEC)) {
        if (int e = ew_grid(n, VEC, &grid)) return e;
        launch_pdl(ew1_kernel<VEC, TA, TC, F>, dim3((unsigned)grid), dim3(EW_BLOCK), 0, st, a, c, n, f);
    } else {
        if (int e = ew_grid(n, 1, &grid)) return e;
        launch_pdl(ew1_kernel<1, TA, TC, F>, dim3((unsigned)grid), dim3(EW_BLOCK), 0, st, a, c, n, f);
    }
    return check_launch(what);
}

template <typename TA, typename TB, typename TC, typename F>
int launch_ew2(const TA *a, const TB *b, TC *c, int64_t n, F f, cudaStream_t st, const char *what) {
    if (n == 0) return DX_OK;
    if (n < 0 || !a || !b || !c) return fail(DX_E_ARG, "%s: bad pointer or count", what);
    constexpr int VEC = 16 / max_sizeof<TA, TB, TC>();
    int64_t grid;
    if (aligned_to(a, sizeof(TA) * VEC) && aligned_to(b, sizeof(TB) * VEC) && aligned_to(c, sizeof(TC) * VEC)) {
        if (int e = ew_grid(n, VEC, &grid)) return e;
        launch_pdl(ew2_kernel<VEC, TA, TB, TC, F>, dim3((unsigned)grid), dim3(EW_BLOCK), 0, st, a, b, c, n, f);
    } else {
        if (int e = ew_grid(n, 1, &grid)) return e;
        launch_pdl(ew2_kernel<1, TA, TB, TC, F>, dim3((unsigned)grid), dim3(EW_BLOCK), 0, st, a, b, c, n, f);
    }
    return check_launch(what);
}

template <typename TC> int launch_ew0(TC *c, int64_t n, TC value, cudaStream_t st, const char *what) {
    if (n == 0) return DX_OK;
    if (n < 0 || !c) return fail(DX_E_ARG, "%s: bad pointer or count", what);
    constexpr int VEC = 16 / sizeof(TC);
    int64_t grid;
    if (aligned_to(c, 16)) {
        if (int e = ew_grid(n, VEC, &grid)) return e;
        ew0_kernel<VEC, TC><<<(unsigned)grid, EW_BLOCK, 0, st>>>(c, n, value);
    } else {
        if (int e = ew_grid(n, 1, &grid)) return e;
        ew0_kernel<1, TC><<<(unsigned)grid, EW_BLOCK, 0, st>>>(c, n, value);
    }
    return check_launch(what);
}

// Runtime dtype → compile-time type.  `CASE` bodies see `T`.
#define DX_DISPATCH_CASE(code, ...)                   \
    case code: {                                      \
        using T = typename dtype_of<code>::type;      \
        __VA_ARGS__;                                  \
    } break;

#define DX_DISPATCH_NUMERIC(dtype, what, ...)                                     \
    switch (dtype) {                                                              \
        DX_DISPATCH_CASE(DX_F64, __VA_ARGS__)                                     \
        DX_DISPATCH_CASE(DX_F32, __VA_ARGS__)                                     \
        DX_DISPATCH_CASE(DX_F16, __VA_ARGS__)                                     \
        DX_DISPATCH_CASE(DX_BF16, __VA_ARGS__)                                    \
        DX_DISPATCH_CASE(DX_I64, __VA_ARGS__)                                     \
        DX_DISPATCH_CASE(DX_I32, __VA_ARGS__)                                     \
        DX_DISPATCH_CASE(DX_I16, __VA_ARGS__)                                     \
        DX_DISPATCH_CASE(DX_I8, __VA_ARGS__)                                      \
        default:                                                                  \
            return fail(DX_E_DTYPE, "%s: unsupported dtype code %d", what, dtype); \
    }

#define DX_DISPATCH_FLOAT(dtype, what, ...)                                       \
    switch (dtype) {                                                              \
        DX_DISPATCH_CASE(DX_F64, __VA_ARGS__)                                     \
        DX_DISPATCH_CASE(DX_F32, __VA_ARGS__)                                     \
        DX_DISPATCH_CASE(DX_F16, __VA_ARGS__)                                     \
        DX_DISPATCH_CASE(DX_BF16, __VA_ARGS__)                                    \
        default:                                                                  \
            return fail(DX_E_DTYPE, "%s: unsupported dtype code %d", what, dtype); \
    }

}  // namespace dx
