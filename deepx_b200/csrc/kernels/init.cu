// dx_arange / dx_uniform / dx_normal / dx_dropout: tensor initialisers.
//
// arange follows the reference kernel exactly: the value is formed in fp32 as
// start + step * float(i) and then cast to the tensor dtype
// (executor/op-cuda/src/deepx/tensorfunc/init_miaobyte.cu:77-95).
// The random fills are counter-based: element i of a tensor filled with `seed` is a pure
// function of (seed, i), so the result does not depend on the launch geometry or the GPU
// count.  (The reference seeds cuRAND XORWOW per threadIdx.x, :104-119, and its CPU executor
// uses std::default_random_engine, so no two of its executors agree on these values either.)
#include "ew_launch.cuh"

namespace dx {
namespace {

__device__ __forceinline__ uint32_t mix32(uint64_t x) {  // splitmix64 finaliser, high word
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    x ^= x >> 31;
    return static_cast<uint32_t>(x >> 32);
}
__device__ __forceinline__ float u01(uint64_t seed, uint64_t i, uint32_t lane) {
    // (0, 1]: 24 random bits, never zero so log() below is finite
    const uint32_t r = mix32(seed * 0xD1342543DE82EF95ull + i * 2 + lane);
    return (float(r >> 8) + 1.0f) * (1.0f / 16777216.0f);
}

template <typename T> __device__ __forceinline__ T from_f32(float v) {
    if constexpr (std::is_same<T, f16>::value) return __float2half_rn(v);
    else if constexpr (std::is_same<T, bf16>::value) return __float2bfloat16_rn(v);
    else return static_cast<T>(v);
}

enum InitKind { K_ARANGE, K_UNIFORM, K_NORMAL, K_DROPOUT };

template <int KIND, typename T>
__global__ void __launch_bounds__(256) init_kernel(T *out, int64_t n, float p0, float p1, uint64_t seed) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        if constexpr (KIND == K_ARANGE) out[i] = from_f32<T>(p0 + p1 * static_cast<float>(i));
        else if constexpr (KIND == K_UNIFORM) out[i] = from_f32<T>(p0 + (p1 - p0) * (1.0f - u01(seed, i, 0)));  // [low, high)
        else if constexpr (KIND == K_NORMAL) {
            const float r = sqrtf(-2.0f * logf(u01(seed, i, 0)));
            out[i] = from_f32<T>(p0 + p1 * r * cospif(2.0f * u01(seed, i, 1)));
        } else {
            if (u01(seed, i, 0) <= p0) out[i] = from_f32<T>(0.0f);  // dropped with probability p
        }
    }
}

template <int KIND> int launch_init(int dtype, void *out, int64_t n, float p0, float p1, uint64_t seed, cudaStream_t st,
                                    const char *what) {
    if (n == 0) return DX_OK;
    if (n < 0 || !out) return fail(DX_E_ARG, "%s: bad pointer or count", what);
    const unsigned grid = (unsigned)std::min<int64_t>((n + 255) / 256, int64_t(sm_count()) * 16);
    DX_DISPATCH_NUMERIC(dtype, what, init_kernel<KIND, T><<<grid, 256, 0, st>>>((T *)out, n, p0, p1, seed))
    return check_launch(what);
}

}  // namespace
}  // namespace dx

using namespace dx;

extern "C" int dx_arange(int dtype, void *out, double start, double step, int64_t n, void *stream) {
    return launch_init<K_ARANGE>(dtype, out, n, float(start), float(step), 0, as_stream(stream), "arange");
}
extern "C" int dx_uniform(int dtype, void *out, double low, double high, uint64_t seed, int64_t n, void *stream) {
    return launch_init<K_UNIFORM>(dtype, out, n, float(low), float(high), seed, as_stream(stream), "uniform");
}
extern "C" int dx_normal(int dtype, void *out, double mean, double stddev, uint64_t seed, int64_t n, void *stream) {
    return launch_init<K_NORMAL>(dtype, out, n, float(mean), float(stddev), seed, as_stream(stream), "normal");
}
extern "C" int dx_dropout(int dtype, void *inout, double p, uint64_t seed, int64_t n, void *stream) {
    return launch_init<K_DROPOUT>(dtype, inout, n, float(p), 0.f, seed, as_stream(stream), "dropout");
}
