// Shared device/host helpers for the sm_100a tensor-function kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <type_traits>

#include "dx_kernels.h"

namespace dx {

// ---- error reporting ---------------------------------------------------------
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);
int check_launch(const char *what);  // cudaGetLastError → DX_E_CUDA

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// ---- programmatic dependent launch -----------------------------------------------
// A kernel launched through launch_pdl may be scheduled while the kernel before it on the stream drains: its CTAs
// become resident and run up to griddep_wait(), which returns once the earlier kernel has completed and its writes
// are visible.  Every kernel launched this way calls griddep_wait() before its first access to global memory, so
// the order of the stream is kept exactly; what is saved is the launch latency at every kernel boundary.  Without
// the launch attribute the instruction returns at once.  DX_PDL=0 launches everything the ordinary way.
bool pdl_enabled();
#ifdef __CUDACC__
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// The whole CTA behind one waiting thread: warps parked in griddepcontrol.wait were measured to slow down the CTAs of
// the earlier kernel that are still running (a GEMM whose last wave fills a quarter of the SMs: 194 -> 233 µs with
// every thread of the early-resident CTAs waiting, 199 µs with one), warps parked at a CTA barrier do not.
__device__ __forceinline__ void griddep_wait_cta() {
    if (threadIdx.x == 0) griddep_wait();
    __syncthreads();
}
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);  // an error stays for check_launch to find
}
#endif

// ---- dtype ↔ C++ type ----------------------------------------------------------
using f16 = __half;
using bf16 = __nv_bfloat16;

template <int D> struct dtype_of;
template <> struct dtype_of<DX_F64> { using type = double; };
template <> struct dtype_of<DX_F32> { using type = float; };
template <> struct dtype_of<DX_F16> { using type = f16; };
template <> struct dtype_of<DX_BF16> { using type = bf16; };
template <> struct dtype_of<DX_I64> { using type = int64_t; };
template <> struct dtype_of<DX_I32> { using type = int32_t; };
template <> struct dtype_of<DX_I16> { using type = int16_t; };
template <> struct dtype_of<DX_I8> { using type = int8_t; };
template <> struct dtype_of<DX_BOOL> { using type = uint8_t; };

// Arithmetic happens in `compute_t<T>`: fp32 for the 16-bit floats (one rounding
// on the way out), the type itself otherwise.
template <typename T> struct compute { using type = T; };
template <> struct compute<f16> { using type = float; };
template <> struct compute<bf16> { using type = float; };
template <typename T> using compute_t = typename compute<T>::type;

template <typename T> __host__ __device__ __forceinline__ compute_t<T> to_compute(T v) { return v; }
template <> __host__ __device__ __forceinline__ float to_compute<f16>(f16 v) { return __half2float(v); }
template <> __host__ __device__ __forceinline__ float to_compute<bf16>(bf16 v) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(static_cast<unsigned int>(__bfloat16_as_ushort(v)) << 16);  // a bf16 is the float's upper half
#else
    return __bfloat162float(v);
#endif
}

template <typename T> __host__ __device__ __forceinline__ T from_compute(compute_t<T> v) { return v; }
template <> __host__ __device__ __forceinline__ f16 from_compute<f16>(float v) { return __float2half_rn(v); }
template <> __host__ __device__ __forceinline__ bf16 from_compute<bf16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> constexpr bool is_float_v =
    std::is_same<T, double>::value || std::is_same<T, float>::value || std::is_same<T, f16>::value ||
    std::is_same<T, bf16>::value;

// Scalar argument of the C ABI (double for floats, int64 for ints) → T.
template <typename T> inline T scalar_as(double fs, int64_t is) {
    if constexpr (std::is_same<T, double>::value) return fs;
    else if constexpr (std::is_same<T, float>::value) return static_cast<float>(fs);
    else if constexpr (std::is_same<T, f16>::value) return __float2half_rn(static_cast<float>(fs));
    else if constexpr (std::is_same<T, bf16>::value) return __float2bfloat16_rn(static_cast<float>(fs));
    else return static_cast<T>(is);
}

// ---- 128-bit packs ---------------------------------------------------------------
template <typename T, int N> struct alignas(sizeof(T) * N) Pack {
    T v[N];
};

// Streaming (evict-first) loads/stores: every tensor here is touched once.
template <typename T, int N> __device__ __forceinline__ Pack<T, N> ld_stream(const T *p) {
    constexpr int B = sizeof(T) * N;
    Pack<T, N> r;
    if constexpr (B == 16) {
        int4 t = __ldcs(reinterpret_cast<const int4 *>(p));
        r = *reinterpret_cast<Pack<T, N> *>(&t);
    } else if constexpr (B == 8) {
        int2 t = __ldcs(reinterpret_cast<const int2 *>(p));
        r = *reinterpret_cast<Pack<T, N> *>(&t);
    } else if constexpr (B == 4) {
        int t = __ldcs(reinterpret_cast<const int *>(p));
        r = *reinterpret_cast<Pack<T, N> *>(&t);
    } else if constexpr (B == 2) {
        short t = __ldcs(reinterpret_cast<const short *>(p));
        r = *reinterpret_cast<Pack<T, N> *>(&t);
    } else {
        static_assert(B == 1, "pack size");
        char t = __ldcs(reinterpret_cast<const char *>(p));
        r = *reinterpret_cast<Pack<T, N> *>(&t);
    }
    return r;
}
template <typename T, int N> __device__ __forceinline__ void st_stream(T *p, const Pack<T, N> &r) {
    constexpr int B = sizeof(T) * N;
    if constexpr (B == 16) __stcs(reinterpret_cast<int4 *>(p), *reinterpret_cast<const int4 *>(&r));
    else if constexpr (B == 8) __stcs(reinterpret_cast<int2 *>(p), *reinterpret_cast<const int2 *>(&r));
    else if constexpr (B == 4) __stcs(reinterpret_cast<int *>(p), *reinterpret_cast<const int *>(&r));
    else if constexpr (B == 2) __stcs(reinterpret_cast<short *>(p), *reinterpret_cast<const short *>(&r));
    else {
        static_assert(B == 1, "pack size");
        __stcs(reinterpret_cast<char *>(p), *reinterpret_cast<const char *>(&r));
    }
}
// Cached load for data that is re-read (broadcast sources, gather tables).
// (Read as ONE word of the pack's size: a pack of 1-byte elements copied as a struct came out as byte loads.)
template <typename T, int N> __device__ __forceinline__ Pack<T, N> ld_cached(const T *p) {
    constexpr int B = sizeof(T) * N;
    Pack<T, N> r;
    if constexpr (B == 16) {
        const int4 t = *reinterpret_cast<const int4 *>(p);
        r = *reinterpret_cast<const Pack<T, N> *>(&t);
    } else if constexpr (B == 8) {
        const int2 t = *reinterpret_cast<const int2 *>(p);
        r = *reinterpret_cast<const Pack<T, N> *>(&t);
    } else if constexpr (B == 4) {
        const int t = *reinterpret_cast<const int *>(p);
        r = *reinterpret_cast<const Pack<T, N> *>(&t);
    } else if constexpr (B == 2) {
        const short t = *reinterpret_cast<const short *>(p);
        r = *reinterpret_cast<const Pack<T, N> *>(&t);
    } else {
        r = *reinterpret_cast<const Pack<T, N> *>(p);
    }
    return r;
}

// Makes `dev` the current device for a scope and puts the caller's device back afterwards.
struct DeviceGuard {
    int prev = -1;
    bool changed = false;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) changed = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (changed) cudaSetDevice(prev);
    }
};

inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---- 32-bit fast division by a runtime constant (Granlund–Montgomery) -------------
struct FastDiv {
    uint32_t d, m, s;  // n / d == (umulhi(n, m) + n) >> s   for n < 2^31
};
inline FastDiv make_fastdiv(uint32_t d) {
    FastDiv f;
    f.d = d;
    if (d == 1) {
        f.m = 0;
        f.s = 0;
        return f;
    }
    uint32_t s = 0;
    while ((1ull << s) < d) ++s;
    uint64_t m = ((1ull << 32) * ((1ull << s) - d)) / d + 1;
    f.m = static_cast<uint32_t>(m);
    f.s = s;
    return f;
}
__device__ __forceinline__ uint32_t fd_div(uint32_t n, const FastDiv &f) {
    return (__umulhi(n, f.m) + n) >> f.s;
}

// ---- launch geometry ------------------------------------------------------------
int sm_count();

}  // namespace dx
