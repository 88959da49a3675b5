// Accumulation types and combine rules shared by the reduction kernels and the cross-GPU combine.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace dx {

// ---- accumulation types and combine rules ----------------------------------------
template <typename T> struct acc_of { using type = T; };
template <> struct acc_of<f16> { using type = float; };
template <> struct acc_of<bf16> { using type = float; };
template <> struct acc_of<int16_t> { using type = int32_t; };
template <> struct acc_of<int8_t> { using type = int32_t; };
template <typename T> using acc_t = typename acc_of<T>::type;

template <typename T> __host__ __device__ __forceinline__ acc_t<T> widen(T v) {
    if constexpr (std::is_same<T, f16>::value) return __half2float(v);
    else if constexpr (std::is_same<T, bf16>::value) {
#ifdef __CUDA_ARCH__
        // a bf16 is the upper half of the float: one shift, where the conversion instruction is slower
        return __uint_as_float(static_cast<unsigned int>(__bfloat16_as_ushort(v)) << 16);
#else
        return __bfloat162float(v);
#endif
    } else return static_cast<acc_t<T>>(v);
}
template <typename T> __host__ __device__ __forceinline__ T narrow(acc_t<T> v) {
    if constexpr (std::is_same<T, f16>::value) return __float2half_rn(v);
    else if constexpr (std::is_same<T, bf16>::value) return __float2bfloat16_rn(v);
    else return static_cast<T>(v);  // int16/int8: keeps the low bits = wraparound sum
}

template <typename T> __host__ __device__ __forceinline__ T lowest_of() {
    if constexpr (std::is_same<T, f16>::value) return __ushort_as_half((unsigned short)0xFBFF);       // -65504
    else if constexpr (std::is_same<T, bf16>::value) return __ushort_as_bfloat16((unsigned short)0xFF7F);  // -3.39e38
    else if constexpr (std::is_same<T, float>::value) return -3.402823466e+38f;
    else if constexpr (std::is_same<T, double>::value) return -1.7976931348623157e+308;
    else if constexpr (std::is_same<T, int64_t>::value) return (int64_t)0x8000000000000000ull;
    else if constexpr (std::is_same<T, int32_t>::value) return (int32_t)0x80000000u;
    else if constexpr (std::is_same<T, int16_t>::value) return (int16_t)-32768;
    else return (int8_t)-128;
}
template <typename T> __host__ __device__ __forceinline__ T highest_of() {
    if constexpr (std::is_same<T, f16>::value) return __ushort_as_half((unsigned short)0x7BFF);
    else if constexpr (std::is_same<T, bf16>::value) return __ushort_as_bfloat16((unsigned short)0x7F7F);
    else if constexpr (std::is_same<T, float>::value) return 3.402823466e+38f;
    else if constexpr (std::is_same<T, double>::value) return 1.7976931348623157e+308;
    else if constexpr (std::is_same<T, int64_t>::value) return (int64_t)0x7fffffffffffffffll;
    else if constexpr (std::is_same<T, int32_t>::value) return (int32_t)0x7fffffff;
    else if constexpr (std::is_same<T, int16_t>::value) return (int16_t)32767;
    else return (int8_t)127;
}

// Identity = the value the reference pre-fills the output with
// (reduce_miaobyte.hpp:22 sum 0, :36 prod 1, :49 max lowest(), :63 min max()).
template <int OP, typename T> __host__ __device__ __forceinline__ acc_t<T> identity() {
    if constexpr (OP == DX_SUM) return acc_t<T>(0);
    else if constexpr (OP == DX_PROD) return acc_t<T>(1);
    else if constexpr (OP == DX_RMAX) return widen<T>(lowest_of<T>());
    else return widen<T>(highest_of<T>());
}

template <int OP, typename A> __device__ __forceinline__ A combine(A a, A b) {
    if constexpr (OP == DX_SUM) {
        if constexpr (std::is_integral<A>::value) {
            using U = typename std::make_unsigned<A>::type;
            return static_cast<A>(static_cast<U>(a) + static_cast<U>(b));
        } else return a + b;
    } else if constexpr (OP == DX_PROD) {
        if constexpr (std::is_integral<A>::value) {
            using U = typename std::make_unsigned<A>::type;
            return static_cast<A>(static_cast<U>(a) * static_cast<U>(b));
        } else return a * b;
    } else if constexpr (OP == DX_RMAX) return (a < b) ? b : a;  // std::max
    else return (b < a) ? b : a;                                 // std::min
}

}  // namespace dx
