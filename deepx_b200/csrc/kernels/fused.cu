// Row-fused kernels for the two op chains the front end builds out of single deepxIR ops:
//
//   RMSNorm  (front/py/deepx/nn/modules/norm/t5layernorm.py:19-23): powscalar(x,2) | mul(x,x) →
//            sum(last axis, keepdims) → divscalar(H) → addscalar(eps) → sqrt → rdivscalar(1) →
//            broadcastTo → mul(x, ·) [→ broadcastTo(weight) → mul(weight, ·)]
//   softmax  (front/py/deepx/nn/functional/normalization.py:4-18): reducemax(last axis, keepdims) →
//            broadcastTo → sub → exp → sum(last axis, keepdims) → broadcastTo → div
//
// As separate ops the RMSNorm chain moves about 7 tensor-sized streams through HBM and softmax 9;
// fused, each row is read once, kept in registers, and written once.  Every step applies the
// same functor (and, for 16-bit floats, the same rounding to the tensor's dtype) as the
// single-op kernels, so the only difference from running the chain is the order of the
// floating-point additions inside the row sum.
//
// Layout: a row is shared by a TEAM of threads (one warp, or a whole CTA of 256 / 1024 threads),
// each holding V 16-byte vectors of the row.  Rows that do not fit (or are not 16-byte aligned)
// take a CTA-per-row kernel that walks the row from global memory (second and third pass hit L2).
#include "common.cuh"
#include "ew_ops.cuh"

namespace dx {
namespace {

constexpr int ROW_CTA = 256;

struct SumOp {
    template <typename C> __device__ __forceinline__ C operator()(C a, C b) const { return a + b; }
};
struct MaxOp {
    template <typename C> __device__ __forceinline__ C operator()(C a, C b) const { return a > b ? a : b; }
};

// All threads of the team end with the same value: the butterfly adds the same pairs in every
// lane, and the cross-warp step walks the warp partials in one fixed order.
template <int TEAM, typename C, typename F> __device__ __forceinline__ C team_reduce(C v, F f, C *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
    if constexpr (TEAM > 32) {
        constexpr int W = TEAM / 32;
        __syncthreads();  // `red` may still be read from the previous reduction
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
        __syncthreads();
        C r = red[0];
#pragma unroll
        for (int w = 1; w < W; ++w) r = f(r, red[w]);
        v = r;
    }
    return v;
}

template <typename T> __device__ __forceinline__ T lowest_of() {
    if constexpr (std::is_same<T, double>::value) return -__longlong_as_double(0x7ff0000000000000LL);
    else return from_compute<T>(-__int_as_float(0x7f800000));
}

// The scalar tail of the RMSNorm chain on one row sum: divscalar, addscalar, sqrt, rdivscalar.
template <typename T> __device__ __forceinline__ T rms_scale(compute_t<T> sumsq, T divisor, T eps, T one) {
    const T s = from_compute<T>(sumsq);
    const T m = ScalarFn<DX_DIVS, T>{divisor}(s);
    const T e = ScalarFn<DX_ADDS, T>{eps}(m);
    const T q = UnaryFn<DX_SQRT, T>()(e);
    return ScalarFn<DX_RDIVS, T>{one}(q);
}

template <typename T, int TEAM, int V>
__global__ void __launch_bounds__(TEAM > ROW_CTA ? TEAM : ROW_CTA)
    rmsnorm_rows_kernel(const T *x, const T *w, T *out, int64_t rows, int cols, T divisor, T eps, T one) {
    constexpr int N = 16 / sizeof(T);
    constexpr int CTA = TEAM > ROW_CTA ? TEAM : ROW_CTA;
    constexpr int RPC = CTA / TEAM;
    using C = compute_t<T>;
    __shared__ C red[32];
    const int t = threadIdx.x % TEAM;
    const int64_t row = int64_t(blockIdx.x) * RPC + threadIdx.x / TEAM;
    const bool live = row < rows;
    const int nvec = cols / N;
    const T *xr = x + row * cols;
    Pack<T, N> xv[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
        const int i = t + v * TEAM;
        if (live && i < nvec) xv[v] = ld_stream<T, N>(xr + int64_t(i) * N);
        else {
#pragma unroll
            for (int k = 0; k < N; ++k) xv[v].v[k] = from_compute<T>(C(0));
        }
    }
    C acc = C(0);
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
        for (int k = 0; k < N; ++k) acc += to_compute(BinaryFn<DX_MUL, T>()(xv[v].v[k], xv[v].v[k]));
    acc = team_reduce<TEAM>(acc, SumOp(), red);
    const T r = rms_scale<T>(acc, divisor, eps, one);
    T *orow = out + row * cols;
#pragma unroll
    for (int v = 0; v < V; ++v) {
        const int i = t + v * TEAM;
        if (live && i < nvec) {
            Pack<T, N> o;
#pragma unroll
            for (int k = 0; k < N; ++k) o.v[k] = BinaryFn<DX_MUL, T>()(xv[v].v[k], r);
            if (w != nullptr) {
                const Pack<T, N> wv = ld_cached<T, N>(w + int64_t(i) * N);
#pragma unroll
                for (int k = 0; k < N; ++k) o.v[k] = BinaryFn<DX_MUL, T>()(wv.v[k], o.v[k]);
            }
            st_stream<T, N>(orow + int64_t(i) * N, o);
        }
    }
}

template <typename T, int TEAM, int V>
__global__ void __launch_bounds__(TEAM > ROW_CTA ? TEAM : ROW_CTA)
    softmax_rows_kernel(const T *x, T *out, int64_t rows, int cols) {
    constexpr int N = 16 / sizeof(T);
    constexpr int CTA = TEAM > ROW_CTA ? TEAM : ROW_CTA;
    constexpr int RPC = CTA / TEAM;
    using C = compute_t<T>;
    __shared__ C red[32];
    const int t = threadIdx.x % TEAM;
    const int64_t row = int64_t(blockIdx.x) * RPC + threadIdx.x / TEAM;
    const bool live = row < rows;
    const int nvec = cols / N;
    const T *xr = x + row * cols;
    const T low = lowest_of<T>();
    Pack<T, N> xv[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
        const int i = t + v * TEAM;
        if (live && i < nvec) xv[v] = ld_stream<T, N>(xr + int64_t(i) * N);
        else {
#pragma unroll
            for (int k = 0; k < N; ++k) xv[v].v[k] = low;  // exp(-inf - max) adds 0 to the row sum
        }
    }
    C mx = to_compute(low);
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
        for (int k = 0; k < N; ++k) mx = MaxOp()(mx, to_compute(xv[v].v[k]));
    mx = team_reduce<TEAM>(mx, MaxOp(), red);
    const T m = from_compute<T>(mx);
    C acc = C(0);
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
        for (int k = 0; k < N; ++k) {
            const T e = UnaryFn<DX_EXP, T>()(BinaryFn<DX_SUB, T>()(xv[v].v[k], m));
            xv[v].v[k] = e;
            acc += to_compute(e);
        }
    acc = team_reduce<TEAM>(acc, SumOp(), red);
    const T s = from_compute<T>(acc);
    T *orow = out + row * cols;
#pragma unroll
    for (int v = 0; v < V; ++v) {
        const int i = t + v * TEAM;
        if (live && i < nvec) {
            Pack<T, N> o;
#pragma unroll
            for (int k = 0; k < N; ++k) o.v[k] = BinaryFn<DX_DIV, T>()(xv[v].v[k], s);
            st_stream<T, N>(orow + int64_t(i) * N, o);
        }
    }
}

// CTA-per-row forms for any row length and alignment.
template <typename T>
__global__ void __launch_bounds__(ROW_CTA)
    rmsnorm_long_kernel(const T *x, const T *w, T *out, int cols, T divisor, T eps, T one) {
    using C = compute_t<T>;
    __shared__ C red[32];
    const T *xr = x + int64_t(blockIdx.x) * cols;
    T *orow = out + int64_t(blockIdx.x) * cols;
    C acc = C(0);
    for (int i = threadIdx.x; i < cols; i += ROW_CTA) acc += to_compute(BinaryFn<DX_MUL, T>()(xr[i], xr[i]));
    acc = team_reduce<ROW_CTA>(acc, SumOp(), red);
    const T r = rms_scale<T>(acc, divisor, eps, one);
    for (int i = threadIdx.x; i < cols; i += ROW_CTA) {
        T o = BinaryFn<DX_MUL, T>()(xr[i], r);
        if (w != nullptr) o = BinaryFn<DX_MUL, T>()(w[i], o);
        orow[i] = o;
    }
}

template <typename T>
__global__ void __launch_bounds__(ROW_CTA) softmax_long_kernel(const T *x, T *out, int cols) {
    using C = compute_t<T>;
    __shared__ C red[32];
    const T *xr = x + int64_t(blockIdx.x) * cols;
    T *orow = out + int64_t(blockIdx.x) * cols;
    C mx = to_compute(lowest_of<T>());
    for (int i = threadIdx.x; i < cols; i += ROW_CTA) mx = MaxOp()(mx, to_compute(xr[i]));
    mx = team_reduce<ROW_CTA>(mx, MaxOp(), red);
    const T m = from_compute<T>(mx);
    C acc = C(0);
    for (int i = threadIdx.x; i < cols; i += ROW_CTA)
        acc += to_compute(UnaryFn<DX_EXP, T>()(BinaryFn<DX_SUB, T>()(xr[i], m)));
    acc = team_reduce<ROW_CTA>(acc, SumOp(), red);  // every read of x is done before any write: out may alias x
    const T s = from_compute<T>(acc);
    for (int i = threadIdx.x; i < cols; i += ROW_CTA)
        orow[i] = BinaryFn<DX_DIV, T>()(UnaryFn<DX_EXP, T>()(BinaryFn<DX_SUB, T>()(xr[i], m)), s);
}

// TEAM / V for a row of `nvec` 16-byte vectors; false when the row does not fit in registers.
struct RowPlan {
    int team, v;
};
bool plan_row(int64_t nvec, RowPlan *p) {
    for (int team : {32, 256, 1024}) {
        const int64_t need = (nvec + team - 1) / team;
        if (need <= 8) {
            p->team = team;
            p->v = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
            return true;
        }
    }
    return false;
}

template <typename T, int TEAM, int V>
void launch_rms(const T *x, const T *w, T *out, int64_t rows, int cols, T d, T e, T one, cudaStream_t st) {
    constexpr int CTA = TEAM > ROW_CTA ? TEAM : ROW_CTA;
    constexpr int RPC = CTA / TEAM;
    rmsnorm_rows_kernel<T, TEAM, V><<<unsigned((rows + RPC - 1) / RPC), CTA, 0, st>>>(x, w, out, rows, cols, d, e, one);
}
template <typename T, int TEAM, int V> void launch_sm(const T *x, T *out, int64_t rows, int cols, cudaStream_t st) {
    constexpr int CTA = TEAM > ROW_CTA ? TEAM : ROW_CTA;
    constexpr int RPC = CTA / TEAM;
    softmax_rows_kernel<T, TEAM, V><<<unsigned((rows + RPC - 1) / RPC), CTA, 0, st>>>(x, out, rows, cols);
}

#define DX_ROW_DISPATCH(CALL)                                                          \
    switch (plan.team * 16 + plan.v) {                                                 \
        case 32 * 16 + 1: CALL(32, 1); break;                                          \
        case 32 * 16 + 2: CALL(32, 2); break;                                          \
        case 32 * 16 + 4: CALL(32, 4); break;                                          \
        case 32 * 16 + 8: CALL(32, 8); break;                                          \
        case 256 * 16 + 1: CALL(256, 1); break;                                        \
        case 256 * 16 + 2: CALL(256, 2); break;                                        \
        case 256 * 16 + 4: CALL(256, 4); break;                                        \
        case 256 * 16 + 8: CALL(256, 8); break;                                        \
        case 1024 * 16 + 1: CALL(1024, 1); break;                                      \
        case 1024 * 16 + 2: CALL(1024, 2); break;                                      \
        case 1024 * 16 + 4: CALL(1024, 4); break;                                      \
        default: CALL(1024, 8); break;                                                 \
    }

template <typename T>
int rmsnorm_t(const void *x_, const void *w_, void *out_, int64_t rows, int64_t cols, double divisor, double eps, cudaStream_t st) {
    const T *x = static_cast<const T *>(x_), *w = static_cast<const T *>(w_);
    T *out = static_cast<T *>(out_);
    const T d = scalar_as<T>(divisor, 0), e = scalar_as<T>(eps, 0), one = scalar_as<T>(1.0, 0);
    constexpr int N = 16 / sizeof(T);
    RowPlan plan;
    const bool vec = cols % N == 0 && aligned_to(x, 16) && aligned_to(out, 16) && (w == nullptr || aligned_to(w, 16));
    if (vec && plan_row(cols / N, &plan)) {
#define DX_CALL(TEAM, V) launch_rms<T, TEAM, V>(x, w, out, rows, int(cols), d, e, one, st)
        DX_ROW_DISPATCH(DX_CALL)
#undef DX_CALL
    } else {
        rmsnorm_long_kernel<T><<<unsigned(rows), ROW_CTA, 0, st>>>(x, w, out, int(cols), d, e, one);
    }
    return check_launch("rmsnorm");
}

template <typename T> int softmax_t(const void *x_, void *out_, int64_t rows, int64_t cols, cudaStream_t st) {
    const T *x = static_cast<const T *>(x_);
    T *out = static_cast<T *>(out_);
    constexpr int N = 16 / sizeof(T);
    RowPlan plan;
    const bool vec = cols % N == 0 && aligned_to(x, 16) && aligned_to(out, 16);
    if (vec && plan_row(cols / N, &plan)) {
#define DX_CALL(TEAM, V) launch_sm<T, TEAM, V>(x, out, rows, int(cols), st)
        DX_ROW_DISPATCH(DX_CALL)
#undef DX_CALL
    } else {
        softmax_long_kernel<T><<<unsigned(rows), ROW_CTA, 0, st>>>(x, out, int(cols));
    }
    return check_launch("softmax");
}

int check_rows(const char *what, int64_t rows, int64_t cols) {
    if (rows < 0 || cols <= 0) return fail(DX_E_SHAPE, "%s: rows %lld, cols %lld", what, (long long)rows, (long long)cols);
    if (cols > INT32_MAX / 2) return fail(DX_E_SHAPE, "%s: a row of %lld elements exceeds the 2^30 limit", what, (long long)cols);
    if ((rows + 7) / 8 > INT32_MAX || rows > INT32_MAX) return fail(DX_E_SHAPE, "%s: %lld rows exceed the grid limit", what, (long long)rows);
    return DX_OK;
}

}  // namespace
}  // namespace dx

extern "C" int dx_rmsnorm(int dtype, const void *x, const void *weight, void *out, int64_t rows, int64_t cols,
                          double divisor, double eps, void *stream) {
    using namespace dx;
    if (int e = check_rows("rmsnorm", rows, cols)) return e;
    if (rows == 0) return DX_OK;
    if (!x || !out) return fail(DX_E_ARG, "rmsnorm: null tensor pointer");
    cudaStream_t st = as_stream(stream);
    switch (dtype) {
        case DX_F64: return rmsnorm_t<double>(x, weight, out, rows, cols, divisor, eps, st);
        case DX_F32: return rmsnorm_t<float>(x, weight, out, rows, cols, divisor, eps, st);
        case DX_F16: return rmsnorm_t<f16>(x, weight, out, rows, cols, divisor, eps, st);
        case DX_BF16: return rmsnorm_t<bf16>(x, weight, out, rows, cols, divisor, eps, st);
        default: return fail(DX_E_DTYPE, "rmsnorm: unsupported dtype code %d (float dtypes only)", dtype);
    }
}

extern "C" int dx_softmax(int dtype, const void *x, void *out, int64_t rows, int64_t cols, void *stream) {
    using namespace dx;
    if (int e = check_rows("softmax", rows, cols)) return e;
    if (rows == 0) return DX_OK;
    if (!x || !out) return fail(DX_E_ARG, "softmax: null tensor pointer");
    cudaStream_t st = as_stream(stream);
    switch (dtype) {
        case DX_F64: return softmax_t<double>(x, out, rows, cols, st);
        case DX_F32: return softmax_t<float>(x, out, rows, cols, st);
        case DX_F16: return softmax_t<f16>(x, out, rows, cols, st);
        case DX_BF16: return softmax_t<bf16>(x, out, rows, cols, st);
        default: return fail(DX_E_DTYPE, "softmax: unsupported dtype code %d (float dtypes only)", dtype);
    }
}
