// dx_ew_unary, dx_ew_compare(_scalar), dx_switch, dx_cast, dx_fill.
#include "ew_launch.cuh"
#include "ew_ops.cuh"

using namespace dx;

template <int OP> static int unary_fp(int dtype, const void *a, void *c, int64_t n, cudaStream_t st) {
    DX_DISPATCH_FLOAT(dtype, "ew_unary", return launch_ew1((const T *)a, (T *)c, n, UnaryFn<OP, T>(), st, "ew_unary"))
    return DX_OK;
}

extern "C" int dx_ew_unary(int op, int dtype, const void *a, void *c, int64_t n, void *stream) {
    cudaStream_t st = as_stream(stream);
    switch (op) {
        case DX_SQRT: return unary_fp<DX_SQRT>(dtype, a, c, n, st);
        case DX_LOG: return unary_fp<DX_LOG>(dtype, a, c, n, st);
        case DX_EXP: return unary_fp<DX_EXP>(dtype, a, c, n, st);
        case DX_SIN: return unary_fp<DX_SIN>(dtype, a, c, n, st);
        case DX_COS: return unary_fp<DX_COS>(dtype, a, c, n, st);
        case DX_TAN: return unary_fp<DX_TAN>(dtype, a, c, n, st);
        case DX_INVERT:
            switch (dtype) {
                DX_DISPATCH_CASE(DX_I64, return launch_ew1((const T *)a, (T *)c, n, UnaryFn<DX_INVERT, T>(), st, "invert"))
                DX_DISPATCH_CASE(DX_I32, return launch_ew1((const T *)a, (T *)c, n, UnaryFn<DX_INVERT, T>(), st, "invert"))
                DX_DISPATCH_CASE(DX_I16, return launch_ew1((const T *)a, (T *)c, n, UnaryFn<DX_INVERT, T>(), st, "invert"))
                DX_DISPATCH_CASE(DX_I8, return launch_ew1((const T *)a, (T *)c, n, UnaryFn<DX_INVERT, T>(), st, "invert"))
                DX_DISPATCH_CASE(DX_BOOL, return launch_ew1((const T *)a, (T *)c, n, UnaryFn<DX_INVERT, T>(), st, "invert"))
                default:
                    return fail(DX_E_DTYPE, "invert: integer or bool dtype required (dtype code %d)", dtype);
            }
            return DX_OK;
        default: return fail(DX_E_ARG, "ew_unary: unknown op code %d", op);
    }
}

template <int OP>
static int compare_all(int dtype, const void *a, const void *b, float eps, void *m, int64_t n, cudaStream_t st) {
    DX_DISPATCH_NUMERIC(dtype, "ew_compare",
                        return launch_ew2((const T *)a, (const T *)b, (uint8_t *)m, n, CompareFn<OP, T>{eps}, st, "ew_compare"))
    return DX_OK;
}
extern "C" int dx_ew_compare(int op, int dtype, const void *a, const void *b, float eps, void *mask, int64_t n,
                             void *stream) {
    cudaStream_t st = as_stream(stream);
    switch (op) {
        case DX_EQ: return compare_all<DX_EQ>(dtype, a, b, eps, mask, n, st);
        case DX_NE: return compare_all<DX_NE>(dtype, a, b, eps, mask, n, st);
        case DX_LT: return compare_all<DX_LT>(dtype, a, b, 0.f, mask, n, st);
        case DX_GT: return compare_all<DX_GT>(dtype, a, b, 0.f, mask, n, st);
        default: return fail(DX_E_ARG, "ew_compare: unknown op code %d", op);
    }
}

template <int OP>
static int compare_scalar_all(int dtype, const void *a, double fs, int64_t is, float eps, void *m, int64_t n,
                              cudaStream_t st) {
    DX_DISPATCH_NUMERIC(dtype, "ew_compare_scalar",
                        return launch_ew1((const T *)a, (uint8_t *)m, n,
                                          CompareScalarFn<OP, T>{scalar_as<T>(fs, is), eps}, st, "ew_compare_scalar"))
    return DX_OK;
}
extern "C" int dx_ew_compare_scalar(int op, int dtype, const void *a, double fs, int64_t is, float eps, void *mask,
                                    int64_t n, void *stream) {
    cudaStream_t st = as_stream(stream);
    switch (op) {
        case DX_EQ: return compare_scalar_all<DX_EQ>(dtype, a, fs, is, eps, mask, n, st);
        case DX_NE: return compare_scalar_all<DX_NE>(dtype, a, fs, is, eps, mask, n, st);
        case DX_LT: return compare_scalar_all<DX_LT>(dtype, a, fs, is, 0.f, mask, n, st);
        case DX_GT: return compare_scalar_all<DX_GT>(dtype, a, fs, is, 0.f, mask, n, st);
        default: return fail(DX_E_ARG, "ew_compare_scalar: unknown op code %d", op);
    }
}

// ---- switch -----------------------------------------------------------------------
// The pointer table travels in the kernel parameters.  Data movement only, so the
// kernel is instantiated per element size, not per dtype.
template <typename E> struct SwitchTable {
    const E *t[DX_SWITCH_MAX];
};

// NT > 0: exactly NT sources, all read as vectors up front (every load of a thread is in flight
// before the first select); NT == 0: any number of sources, each element fetched from the source
// its case names.  Both read each source sector once when the cases are mixed.
template <int VEC, typename E, typename CT, int NT, int EW_UNROLL = dx::EW_UNROLL>
__global__ void __launch_bounds__(EW_BLOCK)
    switch_kernel(SwitchTable<E> tab, int ntensors, const CT *cases, E *c, int64_t n) {
    constexpr int64_t TILE = int64_t(EW_BLOCK) * EW_UNROLL * VEC;
    const int64_t base = int64_t(blockIdx.x) * TILE;
    auto pick = [&](int64_t i, CT k) -> E {
        int w = static_cast<int>(k);
        if constexpr (sizeof(CT) == 1) w = (k != 0);
        return (w >= 0 && w < ntensors) ? tab.t[w][i] : E(0);
    };
    if (base + TILE <= n) {
        if constexpr (NT > 0) {
            Pack<CT, VEC> k[EW_UNROLL];
            Pack<E, VEC> x[EW_UNROLL][NT];
#pragma unroll
            for (int u = 0; u < EW_UNROLL; ++u) {
                const int64_t i0 = base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC;
                k[u] = ld_stream<CT, VEC>(cases + i0);
#pragma unroll
                for (int t = 0; t < NT; ++t) x[u][t] = ld_stream<E, VEC>(tab.t[t] + i0);
            }
#pragma unroll
            for (int u = 0; u < EW_UNROLL; ++u) {
                const int64_t i0 = base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC;
                Pack<E, VEC> r;
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    int w = static_cast<int>(k[u].v[j]);
                    if constexpr (sizeof(CT) == 1) w = (k[u].v[j] != 0);
                    E v = E(0);  // a case outside [0, NT) selects nothing
#pragma unroll
                    for (int t = 0; t < NT; ++t) v = (w == t) ? x[u][t].v[j] : v;
                    r.v[j] = v;
                }
                st_stream<E, VEC>(c + i0, r);
            }
        } else {
#pragma unroll
            for (int u = 0; u < EW_UNROLL; ++u) {
                const int64_t i0 = base + (int64_t(u) * EW_BLOCK + threadIdx.x) * VEC;
                Pack<CT, VEC> k = ld_stream<CT, VEC>(cases + i0);
                Pack<E, VEC> r;
#pragma unroll
                for (int j = 0; j < VEC; ++j) r.v[j] = pick(i0 + j, k.v[j]);
                st_stream<E, VEC>(c + i0, r);
            }
        }
    } else {
        for (int64_t i = base + threadIdx.x; i < n; i += EW_BLOCK) c[i] = pick(i, cases[i]);
    }
}

template <typename E, typename CT>
static int launch_switch(const void *const *tensors, int ntensors, const void *cases, void *c, int64_t n,
                         cudaStream_t st) {
    SwitchTable<E> tab;
    bool al = aligned_to(c, 16);
    for (int i = 0; i < DX_SWITCH_MAX; ++i) {
        tab.t[i] = i < ntensors ? (const E *)tensors[i] : nullptr;
        if (i < ntensors) {
            if (!tensors[i]) return fail(DX_E_ARG, "switch: tensors[%d] is null", i);
            al = al && aligned_to(tensors[i], 16);
        }
    }
    constexpr int VEC = 16 / (sizeof(E) > sizeof(CT) ? sizeof(E) : sizeof(CT));
    al = al && aligned_to(cases, sizeof(CT) * VEC);
    int64_t grid;
    if (al && sizeof(E) < sizeof(CT) && ntensors == 2) {
        // narrow elements under wide cases: a thread's vector is only VEC = 16 / sizeof(CT) elements, so it takes
        // twice as many vectors to keep as many bytes in flight as the other streaming kernels
        constexpr int U = 2 * dx::EW_UNROLL;
        grid = (n + int64_t(EW_BLOCK) * U * VEC - 1) / (int64_t(EW_BLOCK) * U * VEC);
        if (grid > 0x7fffffffLL) return fail(DX_E_SHAPE, "switch: element count %lld too large for one launch", (long long)n);
        switch_kernel<VEC, E, CT, 2, U><<<(unsigned)grid, EW_BLOCK, 0, st>>>(tab, ntensors, (const CT *)cases, (E *)c, n);
    } else if (al) {
        if (int e = ew_grid(n, VEC, &grid)) return e;
        const unsigned g = (unsigned)grid;
        switch (ntensors) {
            case 1: switch_kernel<VEC, E, CT, 1><<<g, EW_BLOCK, 0, st>>>(tab, ntensors, (const CT *)cases, (E *)c, n); break;
            case 2: switch_kernel<VEC, E, CT, 2><<<g, EW_BLOCK, 0, st>>>(tab, ntensors, (const CT *)cases, (E *)c, n); break;
            case 3: switch_kernel<VEC, E, CT, 3><<<g, EW_BLOCK, 0, st>>>(tab, ntensors, (const CT *)cases, (E *)c, n); break;
            default: switch_kernel<VEC, E, CT, 0><<<g, EW_BLOCK, 0, st>>>(tab, ntensors, (const CT *)cases, (E *)c, n); break;
        }
    } else {
        if (int e = ew_grid(n, 1, &grid)) return e;
        switch_kernel<1, E, CT, 0><<<(unsigned)grid, EW_BLOCK, 0, st>>>(tab, ntensors, (const CT *)cases, (E *)c, n);
    }
    return check_launch("switch");
}

extern "C" int dx_switch(int dtype, const void *const *tensors, int ntensors, int cases_dtype, const void *cases,
                         void *c, int64_t n, void *stream) {
    cudaStream_t st = as_stream(stream);
    if (n == 0) return DX_OK;
    if (!tensors || !cases || !c || n < 0) return fail(DX_E_ARG, "switch: bad pointer or count");
    if (ntensors < 1 || ntensors > DX_SWITCH_MAX)
        return fail(DX_E_ARG, "switch: ntensors %d outside [1, %d]", ntensors, DX_SWITCH_MAX);
    if (cases_dtype == DX_BOOL && ntensors != 2)
        return fail(DX_E_ARG, "switch: For bool cases, tensors size must be 2");
    if (cases_dtype != DX_BOOL && cases_dtype != DX_I32)
        return fail(DX_E_DTYPE, "switch: cases must be bool or int32 (dtype code %d)", cases_dtype);
    const int es = dx_dtype_size(dtype);
#define SW(E)                                                                                           \
    return cases_dtype == DX_BOOL ? launch_switch<E, uint8_t>(tensors, ntensors, cases, c, n, st)         \
                                  : launch_switch<E, int32_t>(tensors, ntensors, cases, c, n, st)
    switch (es) {
        case 8: SW(uint64_t);
        case 4: SW(uint32_t);
        case 2: SW(uint16_t);
        case 1: SW(uint8_t);
        default: return fail(DX_E_DTYPE, "switch: unsupported dtype code %d", dtype);
    }
#undef SW
}

// ---- fill ---------------------------------------------------------------------------
extern "C" int dx_fill(int dtype, void *c, double fs, int64_t is, int64_t n, void *stream) {
    cudaStream_t st = as_stream(stream);
    if (dtype == DX_BOOL) return launch_ew0((uint8_t *)c, n, (uint8_t)((is != 0) || (fs != 0.0)), st, "fill");
    DX_DISPATCH_NUMERIC(dtype, "fill", return launch_ew0((T *)c, n, scalar_as<T>(fs, is), st, "fill"))
    return DX_OK;
}
