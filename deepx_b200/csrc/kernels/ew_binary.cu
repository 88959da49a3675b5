// dx_ew_binary / dx_ew_scalar: C = A ∘ B and C = A ∘ s.
#include <cmath>

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

// int8 ∘ scalar through a table: an int8 has 256 values, so division by a scalar (either way round) is one
// shared-memory byte load per element from a table the host fills with the exact truncated quotients, instead
// of unpacking, dividing and packing sixteen elements of every 16-byte vector.
struct Int8Table {
    int8_t t[256];
};
__global__ void __launch_bounds__(EW_BLOCK) i8_table_kernel(const int8_t *a, int8_t *c, int64_t n, const __grid_constant__ Int8Table tab) {
    __shared__ int8_t sm[256];
    sm[threadIdx.x] = tab.t[threadIdx.x];
    static_assert(EW_BLOCK == 256, "one table entry per thread");
    __syncthreads();
    constexpr int VEC = 16;
    constexpr int64_t TILE = int64_t(EW_BLOCK) * EW_UNROLL * VEC;
    const int64_t base = int64_t(blockIdx.x) * TILE;
    if (base + TILE <= n) {
        Pack<int8_t, VEC> va[EW_UNROLL];
#pragma unroll
        for (int u = 0; u < EW_UNROLL; ++u) va[u] = ld_stream<int8_t, VEC>(a + base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC);
#pragma unroll
        for (int u = 0; u < EW_UNROLL; ++u) {
            Pack<int8_t, VEC> vc;
#pragma unroll
            for (int i = 0; i < VEC; ++i) vc.v[i] = sm[static_cast<uint8_t>(va[u].v[i])];
            st_stream<int8_t, VEC>(c + base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC, vc);
        }
    } else {
        for (int64_t i = base + threadIdx.x; i < n; i += EW_BLOCK) c[i] = sm[static_cast<uint8_t>(a[i])];
    }
}
// Division of every int8 value by d (reversed: of s by every int8 value); a zero divisor has no defined result in
// the reference (elementwise_miaobyte.hpp:267, :307 divide without a check) and yields 0 here.
static int launch_i8_division_table(const void *a, void *c, int64_t n, int scalar, bool reversed, cudaStream_t st) {
    Int8Table tab;
    for (int v = -128; v < 128; ++v) {
        const int num = reversed ? scalar : v, den = reversed ? v : scalar;
        tab.t[static_cast<uint8_t>(static_cast<int8_t>(v))] = den == 0 ? int8_t(0) : static_cast<int8_t>(num / den);  // -128 / -1 wraps like the kernels
    }
    int64_t grid;
    if (int e = ew_grid(n, 16, &grid)) return e;
    i8_table_kernel<<<(unsigned)grid, EW_BLOCK, 0, st>>>((const int8_t *)a, (int8_t *)c, n, tab);
    return check_launch("ew_scalar");
}

extern "C" int dx_ew_scalar(int op, int dtype, const void *a, double fs, int64_t is, void *c, int64_t n,
                            void *stream) {
    cudaStream_t st = as_stream(stream);
    if (dtype == DX_I8 && (op == DX_DIVS || op == DX_RDIVS) && n > 0 && a && c && aligned_to(a, 16) && aligned_to(c, 16) &&
        int8_t(is) != 0)
        return launch_i8_division_table(a, c, n, int(int8_t(is)), op == DX_RDIVS, st);
    if (op == DX_POWS && (dtype == DX_F32 || dtype == DX_F64)) {
        if (fs == 2.0) return pow_small<2>(dtype, a, c, n, st);
        if (fs == 1.0) return pow_small<1>(dtype, a, c, n, st);
        if (fs == 3.0) return pow_small<3>(dtype, a, c, n, st);
        if (fs == -1.0) return pow_small<-1>(dtype, a, c, n, st);
    }
    if (op == DX_RPOWS && dtype == DX_F32) {
        // constant base: log2 of it once, in double, as a sum of two floats (positive normal bases; others take the general path)
        const float base = static_cast<float>(fs);
        if (base >= 1.17549435e-38f && base <= 3.40282347e+38f) {
            const double l = std::log2(static_cast<double>(base));
            const float l_hi = static_cast<float>(l);
            return launch_ew1((const float *)a, (float *)c, n, RPowConstFn{base, l_hi, static_cast<float>(l - static_cast<double>(l_hi))}, st, "ew_scalar");
        }
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
