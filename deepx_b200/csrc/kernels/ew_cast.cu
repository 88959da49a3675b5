// dx_cast: todtype between any two tensor dtypes.
#include "ew_launch.cuh"
#include "ew_ops.cuh"

using namespace dx;

template <typename S> static int cast_from(const S *a, int dst, void *c, int64_t n, cudaStream_t st) {
    switch (dst) {
        case DX_F64: return launch_ew1(a, (double *)c, n, CastFn<S, double>(), st, "cast");
        case DX_F32: return launch_ew1(a, (float *)c, n, CastFn<S, float>(), st, "cast");
        case DX_F16: return launch_ew1(a, (f16 *)c, n, CastFn<S, f16>(), st, "cast");
        case DX_BF16: return launch_ew1(a, (bf16 *)c, n, CastFn<S, bf16>(), st, "cast");
        case DX_I64: return launch_ew1(a, (int64_t *)c, n, CastFn<S, int64_t>(), st, "cast");
        case DX_I32: return launch_ew1(a, (int32_t *)c, n, CastFn<S, int32_t>(), st, "cast");
        case DX_I16: return launch_ew1(a, (int16_t *)c, n, CastFn<S, int16_t>(), st, "cast");
        case DX_I8: return launch_ew1(a, (int8_t *)c, n, CastFn<S, int8_t>(), st, "cast");
        case DX_BOOL: return launch_ew1(a, (uint8_t *)c, n, CastFn<S, uint8_t>(), st, "cast");
        default: return fail(DX_E_DTYPE, "cast: unsupported destination dtype code %d", dst);
    }
}

extern "C" int dx_cast(int src, const void *a, int dst, void *c, int64_t n, void *stream) {
    cudaStream_t st = as_stream(stream);
    switch (src) {
        case DX_F64: return cast_from((const double *)a, dst, c, n, st);
        case DX_F32: return cast_from((const float *)a, dst, c, n, st);
        case DX_F16: return cast_from((const f16 *)a, dst, c, n, st);
        case DX_BF16: return cast_from((const bf16 *)a, dst, c, n, st);
        case DX_I64: return cast_from((const int64_t *)a, dst, c, n, st);
        case DX_I32: return cast_from((const int32_t *)a, dst, c, n, st);
        case DX_I16: return cast_from((const int16_t *)a, dst, c, n, st);
        case DX_I8: return cast_from((const int8_t *)a, dst, c, n, st);
        case DX_BOOL: return cast_from((const uint8_t *)a, dst, c, n, st);
        default: return fail(DX_E_DTYPE, "cast: unsupported source dtype code %d", src);
    }
}
