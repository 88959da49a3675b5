// Harness around the REFERENCE's own CUDA kernels — TEST INFRASTRUCTURE, NOT PRODUCT.
//
// Built only where the reference tree is present (oracle/Makefile, target ref_cuda): the
// reference's executor/op-cuda/src/deepx/tensorfunc/*.cu files are compiled where they lie (for
// sm_100, as its CMakeLists.txt:41 does for sm_75) and linked with this file into
// oracle/_ref/libdeepx_ref_cuda.so.  Two uses:
//   * pin the CPU oracle's elementwise / compare / switch / cast / sum arithmetic to code the
//     reference itself holds (the GPU parity tests compare this library with oracle.cpp);
//   * time the reference's kernels as they are today beside ours.
// Every entry point calls the reference's launch_*<T> host wrapper with the caller's device
// pointers, the way its dispatchers do (elementwise_miaobyte_basic.hpp, reduce_miaobyte.hpp:17-29,
// changeshape_miaobyte.hpp, matmul_cublas.hpp:16-80), and returns 0 or -1 with a message.
//
// Left out on purpose, by reading the source: launch_concat (its kernel calls cudaMalloc per
// thread, changeshape_miaobyte.cu:127-128), reducemax / reducemin / prod (non-atomic
// read-modify-write of the output, reduce_miaobyte.cu:230-256,339-365), sum on 64-bit and 8/16-bit
// integers (a CAS loop followed by a plain store, cuda_atomic.cuh:39-49), sin / cos / tan (no
// grid-stride loop: elements beyond the capped grid are never written).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "deepx/shape_changeshape.hpp"
#include "deepx/shape_reduce.hpp"
#include "deepx/tensor.hpp"
#include "deepx/tensorfunc/changeshape_miaobyte.cuh"
#include "deepx/tensorfunc/elementwise_miaobyte_basic.cuh"
#include "deepx/tensorfunc/elementwise_miaobyte_compare.cuh"
#include "deepx/tensorfunc/elementwise_miaobyte_sqrt.cuh"
#include "deepx/tensorfunc/init_miaobyte.cuh"
#include "deepx/tensorfunc/matmul_cublas.hpp"
#include "deepx/tensorfunc/reduce_miaobyte.cuh"

#include "ref_shape_standin.hpp"

using namespace deepx;
using namespace deepx::tensorfunc;

namespace {
thread_local std::string g_err;

// dtype and op codes: those of include/dx_kernels.h, so one test table drives both libraries
enum { F64 = 0, F32 = 1, F16 = 2, BF16 = 3, I64 = 4, I32 = 5, I16 = 6, I8 = 7, BOOL = 8 };
enum { ADD = 0, SUB = 1, MUL = 2, DIV = 3, MAX = 4, MIN = 5, POW = 6 };
enum { ADDS = 0, SUBS = 1, RSUBS = 2, MULS = 3, DIVS = 4, RDIVS = 5, MAXS = 6, MINS = 7, POWS = 8, RPOWS = 9 };
enum { SQRT = 0, LOG = 1, EXP = 2, INVERT = 6 };
enum { EQ = 0, NE = 1, LT = 2, GT = 3 };

template <typename F> int guarded(F &&f) {
    try {
        f();
        const cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) {
            g_err = std::string("CUDA error after the reference kernel: ") + cudaGetErrorString(e);
            return -1;
        }
        return 0;
    } catch (const std::exception &e) {
        g_err = e.what();
        return -1;
    }
}
[[noreturn]] void unsupported(const char *what) { throw std::invalid_argument(std::string("ref_cuda: unsupported ") + what); }

template <typename T> T scalar_of(double f, int64_t i) {
    if constexpr (std::is_integral_v<T>) return T(i);
    else if constexpr (std::is_same_v<T, half>) return __float2half(float(f));
    else if constexpr (std::is_same_v<T, nv_bfloat16>) return __float2bfloat16(float(f));
    else return T(f);
}

template <typename T> void binary_t(int op, const void *a, const void *b, void *c, int n) {
    const T *A = (const T *)a, *B = (const T *)b;
    T *C = (T *)c;
    switch (op) {
        case ADD: launch_add<T>(A, B, C, n); return;
        case SUB: launch_sub<T>(A, B, C, n); return;
        case MUL: launch_mul<T>(A, B, C, n); return;
        case DIV: launch_div<T>(A, B, C, n); return;
        case MAX: launch_max<T>(A, B, C, n); return;
        case MIN: launch_min<T>(A, B, C, n); return;
        case POW:
            if constexpr (std::is_same_v<T, double> || std::is_same_v<T, float>) { launch_pow<T>(A, B, C, n); return; }
        default: unsupported("binary op for this dtype");
    }
}
template <typename T> void scalar_t(int op, const void *a, double f, int64_t i, void *c, int n) {
    const T *A = (const T *)a;
    T *C = (T *)c;
    const T s = scalar_of<T>(f, i);
    switch (op) {
        case ADDS: launch_addscalar<T>(A, s, C, n); return;
        case SUBS: launch_subscalar<T>(A, s, C, n); return;
        case RSUBS: launch_rsubscalar<T>(s, A, C, n); return;
        case MULS: launch_mulscalar<T>(A, s, C, n); return;
        case DIVS: launch_divscalar<T>(A, s, C, n); return;
        case RDIVS: launch_rdivscalar<T>(s, A, C, n); return;
        case MAXS: launch_maxscalar<T>(A, s, C, n); return;
        case MINS: launch_minscalar<T>(A, s, C, n); return;
        case POWS:
            if constexpr (std::is_same_v<T, double> || std::is_same_v<T, float>) { launch_powscalar<T>(A, s, C, n); return; }
        case RPOWS:
            if constexpr (std::is_same_v<T, double> || std::is_same_v<T, float>) { launch_rpowscalar<T>(s, A, C, n); return; }
        default: unsupported("scalar op for this dtype");
    }
}
template <typename T> void unary_t(int op, const void *a, void *c, int n) {
    const T *A = (const T *)a;
    T *C = (T *)c;
    if constexpr (std::is_integral_v<T>) {
        if (op == INVERT) { launch_invert<T>(A, C, n); return; }
    } else {
        switch (op) {
            case SQRT: launch_sqrt<T>(A, C, n); return;
            case LOG: launch_log<T>(A, C, n); return;
            case EXP: launch_exp<T>(A, C, n); return;
            default: break;
        }
    }
    unsupported("unary op for this dtype");
}
template <typename T> void compare_t(int op, const void *a, const void *b, float eps, void *m, int n) {
    const T *A = (const T *)a, *B = (const T *)b;
    bool *M = (bool *)m;
    switch (op) {
        case EQ: launch_equal<T, bool>(A, B, eps, M, n); return;
        case NE: launch_notequal<T, bool>(A, B, eps, M, n); return;
        case LT: launch_less<T, bool>(A, B, M, n); return;
        case GT: launch_greater<T, bool>(A, B, M, n); return;
        default: unsupported("compare op");
    }
}
template <typename T> void compare_scalar_t(int op, const void *a, double f, int64_t i, float eps, void *m, int n) {
    const T *A = (const T *)a;
    bool *M = (bool *)m;
    const T s = scalar_of<T>(f, i);
    switch (op) {
        case EQ: launch_equalscalar<T, bool>(A, s, eps, M, n); return;
        case NE: launch_notequalscalar<T, bool>(A, s, eps, M, n); return;
        case LT: launch_lessscalar<T, bool>(A, s, M, n); return;
        case GT: launch_greaterscalar<T, bool>(A, s, M, n); return;
        default: unsupported("compare op");
    }
}
template <typename T> void switch_t(const void *const *srcs, int k, int cases_dtype, const void *cases, void *c, int n) {
    if (cases_dtype == BOOL) launch_switch<T, bool>((const T **)srcs, k, (const bool *)cases, (T *)c, n);
    else if (cases_dtype == I32) launch_switch<T, int32_t>((const T **)srcs, k, (const int32_t *)cases, (T *)c, n);
    else unsupported("cases dtype");
}

#define BY_DTYPE(dtype, FN, ...)                                   \
    switch (dtype) {                                               \
        case F64: FN<double>(__VA_ARGS__); break;                  \
        case F32: FN<float>(__VA_ARGS__); break;                   \
        case F16: FN<half>(__VA_ARGS__); break;                    \
        case BF16: FN<nv_bfloat16>(__VA_ARGS__); break;            \
        case I64: FN<int64_t>(__VA_ARGS__); break;                 \
        case I32: FN<int32_t>(__VA_ARGS__); break;                 \
        case I16: FN<int16_t>(__VA_ARGS__); break;                 \
        case I8: FN<int8_t>(__VA_ARGS__); break;                   \
        default: unsupported("dtype");                             \
    }

template <typename S> void cast_from(const void *a, int dst, void *c, int n) {
    const S *A = (const S *)a;
#define TO(D) if constexpr (!std::is_same_v<S, D>) { launch_todtype<S, D>(A, (D *)c, n); return; } else unsupported("cast to the same dtype");
    switch (dst) {
        case F64: TO(double)
        case F32: TO(float)
        case F16: TO(half)
        case BF16: TO(nv_bfloat16)
        case I64: TO(int64_t)
        case I32: TO(int32_t)
        case I16: TO(int16_t)
        case I8: TO(int8_t)
        default: unsupported("dtype");
    }
#undef TO
}

std::vector<int> as_int(const int64_t *v, int n) {
    std::vector<int> out(n);
    for (int i = 0; i < n; ++i) {
        if (v[i] < 0 || v[i] > INT32_MAX) throw std::invalid_argument("ref_cuda: extent outside the reference's int range");
        out[i] = int(v[i]);
    }
    return out;
}
int checked_len(const Shape &s) {
    int64_t n = 1;
    for (int d : s.shape) n *= d;
    if (n > INT32_MAX) throw std::invalid_argument("ref_cuda: more than INT_MAX elements");
    return int(n);
}
template <typename T> Tensor<T> borrow(const void *data, const std::vector<int> &shape) {
    Tensor<T> t{shape};
    t.data = (T *)data;
    t.deleter = nullptr;
    t.newer = nullptr;
    t.copyer = nullptr;
    t.saver = nullptr;
    t.loader = nullptr;
    return t;
}

template <typename T> void sum_t(const void *a, const Shape &in, const std::vector<int> &dims, bool keepdims, void *out) {
    // sumDispatcher<miaobyte,T>::sum, reduce_miaobyte.hpp:17-29
    const std::vector<int> cd = checkedDims(in.shape, dims);
    const std::vector<int> rd = reducedDim(in.shape, cd);
    const Shape os(reducedShape(in.shape, cd, keepdims));
    launch_constant<T>((T *)out, T(0), checked_len(os));
    launch_sum<T>((const T *)a, in.strides.data(), in.dim(), checked_len(in), rd.data(), keepdims, (T *)out, os.strides.data(), os.dim());
}
template <typename T> void transpose_t(const void *a, const Shape &in, const std::vector<int> &order, void *out) {
    // transposeDispatcher<miaobyte,T>, changeshape_miaobyte.hpp
    const Shape os(transposeShape(in.shape, order));
    launch_transpose<T>((const T *)a, in.strides.data(), (T *)out, os.strides.data(), in.dim(), checked_len(in), order.data());
}
template <typename T> void broadcast_t(const void *a, const Shape &in, const std::vector<int> &to, void *out) {
    const Shape os(to);
    const std::vector<BroadcastMap> bm = broadcastMap(in.shape, to);
    launch_broadcastTo<T>((const T *)a, in.strides.data(), in.dim(), bm.data(), (T *)out, os.strides.data(), os.dim(), checked_len(os));
}
template <typename T> void indexselect_t(const void *a, const Shape &in, int idx_dtype, const void *idx, const Shape &is, int axis, void *out) {
    const Shape os(indexselectShape(in.shape, is.shape, axis));
    if (idx_dtype == I32)
        launch_indexselect<T, int32_t>((const T *)a, in.strides.data(), in.dim(), (const int32_t *)idx, is.strides.data(), is.dim(), axis, (T *)out,
                                       os.strides.data(), os.dim(), checked_len(os));
    else if (idx_dtype == I64)
        launch_indexselect<T, int64_t>((const T *)a, in.strides.data(), in.dim(), (const int64_t *)idx, is.strides.data(), is.dim(), axis, (T *)out,
                                       os.strides.data(), os.dim(), checked_len(os));
    else unsupported("index dtype");
}
}  // namespace

extern "C" {

const char *refcu_last_error(void) { return g_err.c_str(); }

int refcu_binary(int op, int dtype, const void *a, const void *b, void *c, int n) {
    return guarded([&] { BY_DTYPE(dtype, binary_t, op, a, b, c, n) });
}
int refcu_scalar(int op, int dtype, const void *a, double fscalar, int64_t iscalar, void *c, int n) {
    return guarded([&] { BY_DTYPE(dtype, scalar_t, op, a, fscalar, iscalar, c, n) });
}
int refcu_unary(int op, int dtype, const void *a, void *c, int n) {
    return guarded([&] { BY_DTYPE(dtype, unary_t, op, a, c, n) });
}
int refcu_compare(int op, int dtype, const void *a, const void *b, float epsilon, void *mask, int n) {
    return guarded([&] { BY_DTYPE(dtype, compare_t, op, a, b, epsilon, mask, n) });
}
int refcu_compare_scalar(int op, int dtype, const void *a, double fscalar, int64_t iscalar, float epsilon, void *mask, int n) {
    return guarded([&] { BY_DTYPE(dtype, compare_scalar_t, op, a, fscalar, iscalar, epsilon, mask, n) });
}
int refcu_switch(int dtype, const void *const *srcs, int k, int cases_dtype, const void *cases, void *c, int n) {
    return guarded([&] { BY_DTYPE(dtype, switch_t, srcs, k, cases_dtype, cases, c, n) });
}
int refcu_cast(int src_dtype, const void *a, int dst_dtype, void *c, int n) {
    return guarded([&] { BY_DTYPE(src_dtype, cast_from, a, dst_dtype, c, n) });
}
// float32 / float64 / int32 only (see the header comment).  Refused: every axis reduced without keepdims — the
// kernel then fills no output index and reads an uninitialised one (reduce_miaobyte.cu:33-46).
int refcu_sum(int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims, int ndims, int keepdims, void *out) {
    return guarded([&] {
        const Shape in(as_int(shape, ndim));
        const std::vector<int> d(dims, dims + ndims);
        if (!keepdims && (ndims == 0 || ndims == ndim)) unsupported("full reduction without keepdims (undefined in the reference's kernel)");
        if (dtype == F32) sum_t<float>(a, in, d, keepdims != 0, out);
        else if (dtype == F64) sum_t<double>(a, in, d, keepdims != 0, out);
        else if (dtype == I32) sum_t<int32_t>(a, in, d, keepdims != 0, out);
        else unsupported("sum dtype");
    });
}
int refcu_transpose(int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *order, void *out) {
    return guarded([&] {
        const Shape in(as_int(shape, ndim));
        const std::vector<int> o(order, order + ndim);
        BY_DTYPE(dtype, transpose_t, a, in, o, out)
    });
}
int refcu_broadcast_to(int dtype, const void *a, const int64_t *shape, int ndim, const int64_t *to, int to_ndim, void *out) {
    return guarded([&] {
        const Shape in(as_int(shape, ndim));
        const std::vector<int> t = as_int(to, to_ndim);
        BY_DTYPE(dtype, broadcast_t, a, in, t, out)
    });
}
int refcu_indexselect(int dtype, const void *a, const int64_t *shape, int ndim, int idx_dtype, const void *idx, const int64_t *idx_shape, int idx_ndim,
                      int axis, void *out) {
    return guarded([&] {
        const Shape in(as_int(shape, ndim)), is(as_int(idx_shape, idx_ndim));
        BY_DTYPE(dtype, indexselect_t, a, in, idx_dtype, idx, is, axis, out)
    });
}
// matmulDispatcher<cublas,float|double>, matmul_cublas.hpp:16-145 (the double form passes A before B,
// i.e. computes the column-major product: kept as the reference has it)
int refcu_matmul(int dtype, const void *a, const void *b, void *c, const int64_t *a_shape, const int64_t *b_shape, int ndim) {
    return guarded([&] {
        const std::vector<int> as = as_int(a_shape, ndim), bs = as_int(b_shape, ndim);
        std::vector<int> cs = as;
        cs[ndim - 1] = bs[ndim - 1];
        if (dtype == F32) {
            auto A = borrow<float>(a, as), B = borrow<float>(b, bs), C = borrow<float>(c, cs);
            matmul<cublas, float>(A, B, C);
        } else if (dtype == F64) {
            auto A = borrow<double>(a, as), B = borrow<double>(b, bs), C = borrow<double>(c, cs);
            matmul<cublas, double>(A, B, C);
        } else unsupported("matmul dtype");
    });
}

}
