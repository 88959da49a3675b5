// dx_ew_binary / dx_ew_scalar: C = A ∘ B and C = A ∘ s.
#include "ew_launch.cuh"
#include "ew_ops.cuh"

using namespace dx;

template <int OP> static int binary_all(int dtype, const void *a, const void *b, void *c, int64_t n, cudaStream_t st) {
    DX_DISPATCH_NUMERIC(dtype, "ew_binary",
                        return launch_ew2((const T *)a, (const T *)b, (T *)c, n, BinaryFn<OP, T>(), st, "ew_binary"))
    return DX_OK;
}
template <int OP> static int binary_fp(int dtype, const void *a, const void *b, void *c, int64_t n, cudaStream_t st) {
    switch (dtype) {
        DX_DISPATCH_CASE(DX_F64, return launch_ew2((const T *)a, (const T *)b, (T *)c, n, BinaryFn<OP, T>(), st, "ew_binary"))
        DX_DISPATCH_CASE(DX_F32, return launch_ew2((const T *)a, (const T *)b, (T *)c, n, BinaryFn<OP, T>(), st, "ew_binary"))
        default:
            return fail(DX_E_DTYPE, "pow: only float64/float32 are supported (dtype code %d)", dtype);
    }
    return DX_OK;
}

extern "C" int dx_ew_binary(int op, int dtype, const void *a, const void *b, void *c, int64_t n, void *stream) {
    cudaStream_t st = as_stream(stream);
    switch (op) {
        case DX_ADD: return binary_all<DX_ADD>(dtype, a, b, c, n, st);
        case DX_SUB: return binary_all<DX_SUB>(dtype, a, b, c, n, st);
        case DX_MUL: return binary_all<DX_MUL>(dtype, a, b, c, n, st);
        case DX_DIV: return binary_all<DX_DIV>(dtype, a, b, c, n, st);
        case DX_MAX: return binary_all<DX_MAX>(dtype, a, b, c, n, st);
        case DX_MIN: return binary_all<DX_MIN>(dtype, a, b, c, n, st);
        case DX_POW: return binary_fp<DX_POW>(dtype, a, b, c, n, st);
        default: return fail(DX_E_ARG, "ew_binary: unknown op code %d", op);
    }
}

template <int OP>
static int scalar_all(int dtype, const void *a, double fs, int64_t is, void *c, int64_t n, cudaStream_t st) {
    DX_DISPATCH_NUMERIC(dtype, "ew_scalar",
                        return launch_ew1((const T *)a, (T *)c, n, ScalarFn<OP, T>{scalar_as<T>(fs, is)}, st, "ew_scalar"))
    return DX_OK;
}
template <int OP>
static int scalar_fp(int dtype, const void *a, double fs, int64_t is, void *c, int64_t n, cudaStream_t st) {
    switch (dtype) {
        DX_DISPATCH_CASE(DX_F64, return launch_ew1((const T *)a, (T *)c, n, ScalarFn<OP, T>{scalar_as<T>(fs, is)}, st, "ew_scalar"))
        DX_DISPATCH_CASE(DX_F32, return launch_ew1((const T *)a, (T *)c, n, ScalarFn<OP, T>{scalar_as<T>(fs, is)}, st, "ew_scalar"))
        default:
            return fail(DX_E_DTYPE, "powscalar: only float64/float32 are supported (dtype code %d)", dtype);
    }
    return DX_OK;
}

template <int K> static int pow_small(int dtype, const void *a, void *c, int64_t n, cudaStream_t st) {
    if (dtype == DX_F64) return launch_ew1((const double *)a, (double *)c, n, PowSmallFn<K, double>(), st, "ew_scalar");
    return launch_ew1((const float *)a, (float *)c, n, PowSmallFn<K, float>(), st, "ew_scalar");
}

extern "C" int dx_ew_scalar(int op, int dtype, const void *a, double fs, int64_t is, void *c, int64_t n,
                            void *stream) {
    cudaStream_t st = as_stream(stream);
    if (op == DX_POWS && (dtype == DX_F32 || dtype == DX_F64)) {
        if (fs == 2.0) return pow_small<2>(dtype, a, c, n, st);
        if (fs == 1.0) return pow_small<1>(dtype, a, c, n, st);
        if (fs == 3.0) return pow_small<3>(dtype, a, c, n, st);
        if (fs == -1.0) return pow_small<-1>(dtype, a, c, n, st);
    }
    if (op == DX_DIVS && (dtype == DX_I8 || dtype == DX_I16)) {
        const int64_t d = dtype == DX_I8 ? int64_t(int8_t(is)) : int64_t(int16_t(is));  // the scalar as the element type holds it
        const uint64_t mag = uint64_t(d < 0 ? -d : d);
        if (mag >= 2) {
            const uint32_t magic = uint32_t((uint64_t(1) << 32) / mag + 1);
            if (dtype == DX_I8) return launch_ew1((const int8_t *)a, (int8_t *)c, n, DivConstFn<int8_t>{magic, d < 0}, st, "ew_scalar");
            return launch_ew1((const int16_t *)a, (int16_t *)c, n, DivConstFn<int16_t>{magic, d < 0}, st, "ew_scalar");
        }
    }
    switch (op) {
        case DX_ADDS: return scalar_all<DX_ADDS>(dtype, a, fs, is, c, n, st);
        case DX_SUBS: return scalar_all<DX_SUBS>(dtype, a, fs, is, c, n, st);
        case DX_RSUBS: return scalar_all<DX_RSUBS>(dtype, a, fs, is, c, n, st);
        case DX_MULS: return scalar_all<DX_MULS>(dtype, a, fs, is, c, n, st);
        case DX_DIVS: return scalar_all<DX_DIVS>(dtype, a, fs, is, c, n, st);
        case DX_RDIVS: return scalar_all<DX_RDIVS>(dtype, a, fs, is, c, n, st);
        case DX_MAXS: return scalar_all<DX_MAXS>(dtype, a, fs, is, c, n, st);
        case DX_MINS: return scalar_all<DX_MINS>(dtype, a, fs, is, c, n, st);
        case DX_POWS: return scalar_fp<DX_POWS>(dtype, a, fs, is, c, n, st);
        case DX_RPOWS: return scalar_fp<DX_RPOWS>(dtype, a, fs, is, c, n, st);
        default: return fail(DX_E_ARG, "ew_scalar: unknown op code %d", op);
    }
}
