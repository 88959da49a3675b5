// Elementwise functors.  The arithmetic restates the scalar lambdas of the CPU
// executor (executor/op-ompsimd/src/deepx/tensorfunc/elementwise_miaobyte.hpp);
// 16-bit floats are widened to fp32, computed, and rounded once (RNE).
#pragma once
#include "common.cuh"

namespace dx {

// ---- binary -------------------------------------------------------------------
// |v| < 2^22 as a float, and the truncation of a small quotient, on the ordinary ALU / FMA pipes.
__device__ __forceinline__ float small_int_to_float(int v) { return __int_as_float(0x4B400000 + v) - 12582912.0f; }
__device__ __forceinline__ int trunc_pushed(float q, float push) {
    const float half = __int_as_float((__float_as_int(q) & 0x80000000) | 0x3F000000);  // copysign(0.5, q)
    const float u = __fmaf_rn(q, push, -half);
    return __float_as_int(__fadd_rn(u, 12582912.0f)) - 0x4B400000;
}

// Two fp32 values in one 64-bit register and the packed fp32 instructions of sm_100 (one instruction, two
// results): the routines below are bound by how many instructions a warp can issue, not by the FMA pipe.
struct F2 { unsigned long long v; };
__device__ __forceinline__ F2 f2_pack(float lo, float hi) { F2 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r.v) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void f2_unpack(F2 a, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(a.v)); }
__device__ __forceinline__ F2 f2_splat(float c) { return f2_pack(c, c); }
__device__ __forceinline__ F2 f2_fma(F2 a, F2 b, F2 c) { F2 r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r.v) : "l"(a.v), "l"(b.v), "l"(c.v)); return r; }
__device__ __forceinline__ F2 f2_mul(F2 a, F2 b) { F2 r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v)); return r; }
__device__ __forceinline__ F2 f2_add(F2 a, F2 b) { F2 r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r.v) : "l"(a.v), "l"(b.v)); return r; }

__device__ __forceinline__ float ex2_approx(float t) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
    return r;
}

// powf for two (x, y) pairs at once, within 3e-6 relative of the correctly rounded result (the bound every float32
// pow test here uses is 1e-5): x^y = 2^(y·log2 x) with log2 x carried as a sum of two floats.
//   x = m·2^e, m in [sqrt(1/2), sqrt(2)), by integer arithmetic on the bits; f = m − 1 is exact.
//   log2 m = f/ln2 + f²·Q(f): Q a degree-8 polynomial (weighted minimax fit, 1.1e-9 absolute on log2 m); the
//   leading term with 1/ln2 split in two floats and the product's rounding error recovered by an FMA.
//   L = e + log2 m as hi + lo by two error-free additions; t = y·L as hi + lo the same way.
//   2^t_hi by the hardware approximation (2^-22 relative), times 1 + ln2·t_lo.
// The library routine costs 60–80 issue slots per element and held pow at 0.53–0.75 of the copy bandwidth; this is
// about 36 floating-point operations, issued as packed instructions two elements at a time.  An element whose x is
// not a positive normal number (zero, negative, subnormal, inf, NaN), whose y is not finite, or whose result would
// leave [2^-125, 2^125] goes to powf on its own, so a result never depends on which element shares the pair.
constexpr float POW_Q0 = -7.213471532e-01f, POW_Q1 = 4.808981419e-01f, POW_Q2 = -3.607088029e-01f, POW_Q3 = 2.885792851e-01f,
                POW_Q4 = -2.393930554e-01f, POW_Q5 = 2.042880207e-01f, POW_Q6 = -1.923508048e-01f, POW_Q7 = 1.883963346e-01f,
                POW_Q8 = -1.097617820e-01f;
constexpr float POW_INVLN2_HI = 1.4426950216293335f, POW_INVLN2_LO = 1.925963033500011e-08f, POW_LN2 = 0.693147182f;

// the rare elements the fast path hands back: one copy of the library routine, not one per call site
static __device__ __noinline__ float powf_library(float x, float y) { return powf(x, y); }

__device__ __forceinline__ void pow_f32_x2(float x0, float x1, float y0, float y1, float &r0, float &r1) {
    const uint32_t b0 = __float_as_uint(x0), b1 = __float_as_uint(x1);
    const uint32_t e0 = (b0 - 0x3f3504f3u) & 0xff800000u, e1 = (b1 - 0x3f3504f3u) & 0xff800000u;
    const F2 one = f2_splat(-1.0f);
    const F2 f = f2_add(f2_pack(__uint_as_float(b0 - e0), __uint_as_float(b1 - e1)), one);
    const F2 e = f2_add(f2_pack(__int_as_float(0x4B400000 + (static_cast<int>(e0) >> 23)), __int_as_float(0x4B400000 + (static_cast<int>(e1) >> 23))),
                        f2_splat(-12582912.0f));
    F2 q = f2_fma(f2_splat(POW_Q8), f, f2_splat(POW_Q7));
    q = f2_fma(q, f, f2_splat(POW_Q6));
    q = f2_fma(q, f, f2_splat(POW_Q5));
    q = f2_fma(q, f, f2_splat(POW_Q4));
    q = f2_fma(q, f, f2_splat(POW_Q3));
    q = f2_fma(q, f, f2_splat(POW_Q2));
    q = f2_fma(q, f, f2_splat(POW_Q1));
    q = f2_fma(q, f, f2_splat(POW_Q0));
    const F2 neg1 = f2_splat(-1.0f);
    const F2 ff = f2_mul(f, f);
    const F2 chi = f2_splat(POW_INVLN2_HI);
    const F2 p_hi = f2_mul(f, chi);
    F2 p_lo = f2_fma(f, chi, f2_mul(p_hi, neg1));
    p_lo = f2_fma(f, f2_splat(POW_INVLN2_LO), p_lo);
    const F2 u = f2_fma(ff, q, p_lo);
    const F2 s1 = f2_add(p_hi, u);                                  // |p_hi| >= |u|: the two sums below lose nothing
    const F2 c1 = f2_add(f2_fma(s1, neg1, p_hi), u);
    const F2 s = f2_add(e, s1);                                     // e is 0 or |e| >= 1 > |s1|
    const F2 c2 = f2_add(f2_fma(s, neg1, e), s1);
    const F2 l = f2_add(c1, c2);
    const F2 y = f2_pack(y0, y1);
    const F2 t_hi = f2_mul(y, s);
    F2 t_lo = f2_fma(y, s, f2_mul(t_hi, neg1));
    t_lo = f2_fma(y, l, t_lo);
    float th0, th1;
    f2_unpack(t_hi, th0, th1);
    const F2 p = f2_pack(ex2_approx(th0), ex2_approx(th1));
    const F2 r = f2_fma(p, f2_mul(t_lo, f2_splat(POW_LN2)), p);
    f2_unpack(r, r0, r1);
    // positive normal x (biased exponent 1..254, sign clear) and a moderate, non-NaN y·log2 x
    if (!(b0 - 0x00800000u < 0x7f000000u && fabsf(th0) < 125.0f)) r0 = powf_library(x0, y0);
    if (!(b1 - 0x00800000u < 0x7f000000u && fabsf(th1) < 125.0f)) r1 = powf_library(x1, y1);
}

// pow(s, a) for a constant positive base: log2 s is computed once on the host in double precision and handed over as
// hi + lo; per element that leaves the product, the hardware 2^t and one correction.
struct RPowConstFn {
    float s, l_hi, l_lo;
    static constexpr bool has_pair = true;
    __device__ __forceinline__ void pair(float a0, float a1, float &c0, float &c1) const {
        const F2 y = f2_pack(a0, a1), lh = f2_splat(l_hi);
        const F2 t_hi = f2_mul(y, lh);
        F2 t_lo = f2_fma(y, lh, f2_mul(t_hi, f2_splat(-1.0f)));
        t_lo = f2_fma(y, f2_splat(l_lo), t_lo);
        float th0, th1;
        f2_unpack(t_hi, th0, th1);
        const F2 p = f2_pack(ex2_approx(th0), ex2_approx(th1));
        const F2 r = f2_fma(p, f2_mul(t_lo, f2_splat(POW_LN2)), p);
        f2_unpack(r, c0, c1);
        if (!(fabsf(th0) < 125.0f)) c0 = powf_library(s, a0);
        if (!(fabsf(th1) < 125.0f)) c1 = powf_library(s, a1);
    }
    __device__ __forceinline__ float operator()(float a) const {
        float c, unused;
        pair(a, a, c, unused);
        return c;
    }
};

template <int OP, typename T> struct BinaryFn {
    __device__ __forceinline__ T operator()(T a, T b) const {
        using C = compute_t<T>;
        C x = to_compute(a), y = to_compute(b), r;
        if constexpr (OP == DX_ADD) {
            if constexpr (std::is_integral<T>::value && std::is_signed<T>::value) {
                using U = typename std::make_unsigned<T>::type;  // wraparound, not UB
                r = static_cast<T>(static_cast<U>(x) + static_cast<U>(y));
            } else r = x + y;  // elementwise_miaobyte.hpp:123
        } else if constexpr (OP == DX_SUB) {
            if constexpr (std::is_integral<T>::value && std::is_signed<T>::value) {
                using U = typename std::make_unsigned<T>::type;
                r = static_cast<T>(static_cast<U>(x) - static_cast<U>(y));
            } else r = x - y;  // :164
        } else if constexpr (OP == DX_MUL) {
            if constexpr (std::is_integral<T>::value && std::is_signed<T>::value) {
                using U = typename std::make_unsigned<T>::type;
                r = static_cast<T>(static_cast<U>(static_cast<U>(x) * static_cast<U>(y)));
            } else r = x * y;  // :226
        } else if constexpr (OP == DX_DIV) {
            if constexpr (std::is_integral<T>::value && sizeof(T) <= 2) {
                // 8- and 16-bit integers: quotient in fp32, truncated — with none of the int<->float conversion
                // instructions, which share the quarter-rate unit with the reciprocal and were what bounded this op.
                //  * int -> float: the bits of 1.5·2^23 plus v are the float 1.5·2^23 + v; subtract 1.5·2^23.
                //  * quotient q: 16-bit: IEEE division (an exact integer quotient is exact, any other is at least
                //    1/|b| from an integer); 8-bit: numerator × approximate reciprocal (off by <= 2 ulp).
                //  * truncation: q is pushed away from zero by a factor 1 + p (p = 2^-17 / 2^-12: more than q's
                //    error, yet (|q| + 1)·p < 1/|b|, so it never reaches the next integer), half is taken off, and
                //    adding 1.5·2^23 rounds to the nearest integer, which is now the truncated quotient.
                // Checked for every int8 pair and a spread of int16 divisors on the CPU (the same arithmetic in
                // numpy) and on the GPU against the integer division.
                const float fx = small_int_to_float(static_cast<int>(x)), fy = small_int_to_float(static_cast<int>(y));
                if constexpr (sizeof(T) == 1) r = static_cast<C>(trunc_pushed(__fdividef(fx, fy), 1.000244140625f));
                else r = static_cast<C>(trunc_pushed(__fdiv_rn(fx, fy), 1.00000762939453125f));
            } else r = x / y;  // :267 (integer: truncating; divisor 0 is undefined in the reference)
        } else if constexpr (OP == DX_MAX) {
            r = (x < y) ? y : x;  // std::max, :614
        } else if constexpr (OP == DX_MIN) {
            r = (y < x) ? y : x;  // std::min, :698
        } else {
            static_assert(OP == DX_POW, "binary op");
            if constexpr (std::is_same<C, double>::value) r = pow(x, y);  // std::pow, :441
            else {
                float unused;
                pow_f32_x2(x, x, y, y, r, unused);  // the arithmetic of the paired path: the same bits wherever an element sits
            }
        }
        return from_compute<T>(r);
    }
    // Two elements per call on the packed instructions (the streaming kernel uses it when present).
    static constexpr bool has_pair = OP == DX_POW && std::is_same<T, float>::value;
    __device__ __forceinline__ void pair(T a0, T a1, T b0, T b1, T &c0, T &c1) const {
        if constexpr (has_pair) pow_f32_x2(a0, a1, b0, b1, c0, c1);
        else {
            c0 = (*this)(a0, b0);
            c1 = (*this)(a1, b1);
        }
    }
};

// ---- tensor ∘ scalar -------------------------------------------------------------
template <int OP, typename T> struct ScalarFn {
    T s;
    __device__ __forceinline__ T operator()(T a) const {
        if constexpr (OP == DX_ADDS) return BinaryFn<DX_ADD, T>()(a, s);
        else if constexpr (OP == DX_SUBS) return BinaryFn<DX_SUB, T>()(a, s);
        else if constexpr (OP == DX_RSUBS) return BinaryFn<DX_SUB, T>()(s, a);  // :204
        else if constexpr (OP == DX_MULS) return BinaryFn<DX_MUL, T>()(a, s);
        else if constexpr (OP == DX_DIVS) return BinaryFn<DX_DIV, T>()(a, s);
        else if constexpr (OP == DX_RDIVS) return BinaryFn<DX_DIV, T>()(s, a);  // :307
        else if constexpr (OP == DX_MAXS) return BinaryFn<DX_MAX, T>()(a, s);
        else if constexpr (OP == DX_MINS) return BinaryFn<DX_MIN, T>()(a, s);
        else if constexpr (OP == DX_POWS) return BinaryFn<DX_POW, T>()(a, s);  // :462
        else {
            static_assert(OP == DX_RPOWS, "scalar op");
            return BinaryFn<DX_POW, T>()(s, a);  // :482
        }
    }
    static constexpr bool has_pair = (OP == DX_POWS || OP == DX_RPOWS) && std::is_same<T, float>::value;
    __device__ __forceinline__ void pair(T a0, T a1, T &c0, T &c1) const {
        if constexpr (has_pair && OP == DX_POWS) pow_f32_x2(a0, a1, s, s, c0, c1);
        else if constexpr (has_pair) pow_f32_x2(s, s, a0, a1, c0, c1);
        else {
            c0 = (*this)(a0);
            c1 = (*this)(a1);
        }
    }
};

// pow(a, k) for the exponents models use all the time (x.pow(2) in every norm layer): plain
// multiplications stream at memory speed where powf's ~40 instructions per element do not, and
// x*x is the correctly rounded square.  K = 1, 2, 3 or -1 (reciprocal, IEEE division).
template <int K, typename T> struct PowSmallFn {
    __device__ __forceinline__ T operator()(T a) const {
        if constexpr (K == 1) return a;
        else if constexpr (K == 2) return a * a;
        else if constexpr (K == 3) return a * a * a;
        else {
            static_assert(K == -1, "exponent");
            return T(1) / a;
        }
    }
};

// int8 / int16 divided by a constant d, |d| >= 2: |a| * (floor(2^32/|d|) + 1) >> 32 is the exact
// truncated quotient for |a| < 2^16 (the error term is below 2^-16 <= 1/|d|), one multiply-high
// instead of a division per element.
template <typename T> struct DivConstFn {
    uint32_t magic;
    int negative;  // divisor < 0
    __device__ __forceinline__ T operator()(T a) const {
        const int x = a;
        const uint32_t q = __umulhi(static_cast<uint32_t>(x < 0 ? -x : x), magic);
        const int r = ((x < 0) != (negative != 0)) ? -static_cast<int>(q) : static_cast<int>(q);
        return static_cast<T>(r);
    }
};

// ---- unary ---------------------------------------------------------------------
// sin / cos for arguments that came from a 16-bit float, in fp32 to about 1.8 ulp (every finite f16 argument
// then rounds to the same f16 as the C library's sinf / cosf; checked on the CPU).  The library routine costs
// about 30 instructions per element, two of them int<->float conversions on the quarter-rate unit, which
// held these ops at 0.62–0.73 of the copy bandwidth (4 bytes of traffic per element).  Here: quadrant n =
// nearest integer to x·2/π by adding 1.5·2^23 (its low mantissa bits are n), three-constant Cody–Waite
// reduction with FMAs, one short polynomial each for sin and cos on [−π/4, π/4] (Cephes single-precision
// coefficients), select and sign by n.  Beyond 1e5 (CHECK: bfloat16 only; float16 ends at 65504, and its
// infinities and NaNs come out as NaN by themselves) the library's full reduction is used.
template <int WANT_COS, bool CHECK> __device__ __forceinline__ float trig_of_16bit(float x) {
    if (CHECK && !(fabsf(x) < 100000.0f)) return WANT_COS ? cosf(x) : sinf(x);
    const float j = __fmaf_rn(x, 0.636619747f, 12582912.0f);
    const int n = __float_as_int(j) + WANT_COS;
    const float jf = j - 12582912.0f;
    float r = __fmaf_rn(jf, -1.57079601e+00f, x);
    r = __fmaf_rn(jf, -3.13916473e-07f, r);
    r = __fmaf_rn(jf, -5.39030253e-15f, r);
    const float r2 = r * r;
    float ps = __fmaf_rn(r2, -1.9515295891e-4f, 8.3321608736e-3f);
    ps = __fmaf_rn(ps, r2, -1.6666654611e-1f);
    const float s = r * __fmaf_rn(r2, ps, 1.0f);  // as a product, so that sin(-0) is -0
    float pc = __fmaf_rn(r2, 2.443315711809948e-5f, -1.388731625493765e-3f);
    pc = __fmaf_rn(pc, r2, 4.166664568298827e-2f);
    pc = __fmaf_rn(pc, r2, -0.5f);
    const float c = __fmaf_rn(pc, r2, 1.0f);
    const float v = (n & 1) ? c : s;
    return (n & 2) ? -v : v;
}

// trig_of_16bit for two arguments at once: the same operations in the same order (same bits), the floating-point
// ones as packed instructions.
template <int WANT_COS, bool CHECK> __device__ __forceinline__ void trig_of_16bit_x2(float x0, float x1, float &y0, float &y1) {
    if (CHECK && (!(fabsf(x0) < 100000.0f) || !(fabsf(x1) < 100000.0f))) {
        y0 = trig_of_16bit<WANT_COS, CHECK>(x0);
        y1 = trig_of_16bit<WANT_COS, CHECK>(x1);
        return;
    }
    const F2 x = f2_pack(x0, x1);
    const F2 j = f2_fma(x, f2_splat(0.636619747f), f2_splat(12582912.0f));
    float j0, j1;
    f2_unpack(j, j0, j1);
    const int n0 = __float_as_int(j0) + WANT_COS, n1 = __float_as_int(j1) + WANT_COS;
    const F2 jf = f2_add(j, f2_splat(-12582912.0f));
    F2 r = f2_fma(jf, f2_splat(-1.57079601e+00f), x);
    r = f2_fma(jf, f2_splat(-3.13916473e-07f), r);
    r = f2_fma(jf, f2_splat(-5.39030253e-15f), r);
    const F2 r2 = f2_mul(r, r);
    F2 ps = f2_fma(r2, f2_splat(-1.9515295891e-4f), f2_splat(8.3321608736e-3f));
    ps = f2_fma(ps, r2, f2_splat(-1.6666654611e-1f));
    const F2 s = f2_mul(r, f2_fma(r2, ps, f2_splat(1.0f)));
    F2 pc = f2_fma(r2, f2_splat(2.443315711809948e-5f), f2_splat(-1.388731625493765e-3f));
    pc = f2_fma(pc, r2, f2_splat(4.166664568298827e-2f));
    pc = f2_fma(pc, r2, f2_splat(-0.5f));
    const F2 c = f2_fma(pc, r2, f2_splat(1.0f));
    float s0, s1, c0, c1;
    f2_unpack(s, s0, s1);
    f2_unpack(c, c0, c1);
    const float v0 = (n0 & 1) ? c0 : s0, v1 = (n1 & 1) ? c1 : s1;
    y0 = (n0 & 2) ? -v0 : v0;
    y1 = (n1 & 2) ? -v1 : v1;
}

// log for arguments that came from a 16-bit float, two at once on the packed instructions, to 0.71 ulp of fp32
// (checked for every positive f16 and bf16 argument on the CPU): x = m·2^e with m in [sqrt(1/2), sqrt(2)) by
// integer arithmetic on the bits, e to float through the magic number, log(m) by the Cephes single-precision
// polynomial in m − 1, and e·ln2 added in two parts.  Zero, negative, subnormal, infinite and NaN arguments
// go to the library routine.
__device__ __forceinline__ void log_of_16bit_x2(float x0, float x1, float &y0, float &y1) {
    const uint32_t b0 = __float_as_uint(x0), b1 = __float_as_uint(x1);
    if (b0 - 0x00800000u >= 0x7f000000u || b1 - 0x00800000u >= 0x7f000000u) {
        y0 = logf(x0);
        y1 = logf(x1);
        return;
    }
    const uint32_t e0 = (b0 - 0x3f3504f3u) & 0xff800000u, e1 = (b1 - 0x3f3504f3u) & 0xff800000u;
    const F2 m = f2_pack(__uint_as_float(b0 - e0), __uint_as_float(b1 - e1));
    const F2 e = f2_add(f2_pack(__int_as_float(0x4B400000 + (static_cast<int>(e0) >> 23)), __int_as_float(0x4B400000 + (static_cast<int>(e1) >> 23))),
                        f2_splat(-12582912.0f));
    const F2 f = f2_add(m, f2_splat(-1.0f));
    const F2 z = f2_mul(f, f);
    F2 y = f2_fma(f2_splat(7.0376836292e-2f), f, f2_splat(-1.1514610310e-1f));
    y = f2_fma(y, f, f2_splat(1.1676998740e-1f));
    y = f2_fma(y, f, f2_splat(-1.2420140846e-1f));
    y = f2_fma(y, f, f2_splat(1.4249322787e-1f));
    y = f2_fma(y, f, f2_splat(-1.6668057665e-1f));
    y = f2_fma(y, f, f2_splat(2.0000714765e-1f));
    y = f2_fma(y, f, f2_splat(-2.4999993993e-1f));
    y = f2_fma(y, f, f2_splat(3.3333331174e-1f));
    y = f2_mul(f2_mul(y, f), z);
    y = f2_fma(e, f2_splat(-2.12194440e-4f), y);
    y = f2_fma(z, f2_splat(-0.5f), y);
    const F2 r = f2_fma(e, f2_splat(0.693359375f), f2_add(f, y));
    f2_unpack(r, y0, y1);
}

template <int OP, typename T> struct UnaryFn {
    __device__ __forceinline__ T operator()(T a) const {
        if constexpr (OP == DX_INVERT) {
            if constexpr (std::is_same<T, uint8_t>::value) return static_cast<uint8_t>(!a);  // bool, :353
            else return static_cast<T>(~a);                                                  // :332
        } else {
            using C = compute_t<T>;
            C x = to_compute(a), r;
            if constexpr (std::is_same<C, double>::value) {
                if constexpr (OP == DX_SQRT) r = sqrt(x);
                else if constexpr (OP == DX_LOG) r = log(x);
                else if constexpr (OP == DX_EXP) r = exp(x);
                else if constexpr (OP == DX_SIN) r = sin(x);
                else if constexpr (OP == DX_COS) r = cos(x);
                else r = tan(x);
            } else {
                if constexpr (OP == DX_SQRT) r = sqrtf(x);  // IEEE (-prec-sqrt=true)
                else if constexpr (OP == DX_LOG) {
                    if constexpr (std::is_same<T, f16>::value || std::is_same<T, bf16>::value) {
                        float unused;
                        log_of_16bit_x2(x, x, r, unused);  // the same arithmetic as the paired path: same bits wherever an element sits
                    } else r = logf(x);
                }
                else if constexpr (OP == DX_EXP) r = expf(x);
                else if constexpr (OP == DX_SIN) {
                    if constexpr (std::is_same<T, f16>::value || std::is_same<T, bf16>::value) r = trig_of_16bit<0, std::is_same<T, bf16>::value>(x);
                    else r = sinf(x);
                } else if constexpr (OP == DX_COS) {
                    if constexpr (std::is_same<T, f16>::value || std::is_same<T, bf16>::value) r = trig_of_16bit<1, std::is_same<T, bf16>::value>(x);
                    else r = cosf(x);
                }
                else r = tanf(x);
            }
            return from_compute<T>(r);
        }
    }
    // Two elements at once, for the ops that have a packed routine (the streaming kernel uses it when present).
    static constexpr bool has_pair = (OP == DX_SIN || OP == DX_COS || OP == DX_LOG) && (std::is_same<T, f16>::value || std::is_same<T, bf16>::value);
    __device__ __forceinline__ void pair(T a0, T a1, T &c0, T &c1) const { pair_impl<true>(a0, a1, c0, c1); }
    // For a whole vector whose `vector_is_plain` check passed: the same results without the per-pair range check.
    __device__ __forceinline__ void pair_plain(T a0, T a1, T &c0, T &c1) const { pair_impl<false>(a0, a1, c0, c1); }
    // bfloat16 sin / cos: true when no element of the vector reaches 65536 in magnitude (nor is inf / NaN), decided
    // on the raw bit patterns two at a time (adding 0x8000 − 0x4780 to each 15-bit magnitude carries into bit 15
    // exactly when it is too large).  One test and one branch per vector instead of one per pair.
    static constexpr bool has_vector_check = (OP == DX_SIN || OP == DX_COS) && std::is_same<T, bf16>::value;
    template <int VEC> __device__ __forceinline__ static bool vector_is_plain(const Pack<T, VEC> &v) {
        static_assert(VEC % 2 == 0, "whole 32-bit words");
        const uint32_t *w = reinterpret_cast<const uint32_t *>(&v);
        uint32_t o = 0;
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) o |= (w[i] & 0x7fff7fffu) + 0x38803880u;  // bit 15 of a half: |pattern| >= 0x4780 (65536.0)
        return (o & 0x80008000u) == 0;
    }

private:
    template <bool CHECKED> __device__ __forceinline__ void pair_impl(T a0, T a1, T &c0, T &c1) const {
        if constexpr (has_pair) {
            float y0, y1;
            if constexpr (OP == DX_LOG) log_of_16bit_x2(to_compute(a0), to_compute(a1), y0, y1);
            else trig_of_16bit_x2<OP == DX_COS ? 1 : 0, CHECKED && std::is_same<T, bf16>::value>(to_compute(a0), to_compute(a1), y0, y1);
            c0 = from_compute<T>(y0);
            c1 = from_compute<T>(y1);
        } else {
            c0 = (*this)(a0);
            c1 = (*this)(a1);
        }
    }

public:
};

// ---- compare → 0/1 byte ------------------------------------------------------------
// EQ/NE with epsilon follow elementwise_miaobyte.hpp:778-845: `std::abs(a-b) <= epsilon`
// evaluated in the promoted type of (T, float).
template <typename T> __device__ __forceinline__ bool within_eps(T a, T b, float eps) {
    if constexpr (std::is_same<T, double>::value) return fabs(a - b) <= static_cast<double>(eps);
    else if constexpr (is_float_v<T>) return fabsf(to_compute(a) - to_compute(b)) <= eps;
    else if constexpr (std::is_same<T, int64_t>::value) {
        int64_t d = a - b;
        return static_cast<float>(d < 0 ? -d : d) <= eps;
    } else {
        int d = static_cast<int>(a) - static_cast<int>(b);
        return static_cast<float>(d < 0 ? -d : d) <= eps;
    }
}

template <int OP, typename T> struct CompareFn {
    float eps;
    __device__ __forceinline__ uint8_t operator()(T a, T b) const {
        using C = compute_t<T>;
        if constexpr (OP == DX_EQ) {
            if (eps == 0.f) return to_compute(a) == to_compute(b);
            return within_eps<T>(a, b, eps);
        } else if constexpr (OP == DX_NE) {
            if (eps == 0.f) return to_compute(a) != to_compute(b);
            return !within_eps<T>(a, b, eps);
        } else if constexpr (OP == DX_LT) {
            return C(to_compute(a)) < C(to_compute(b));  // :900
        } else {
            static_assert(OP == DX_GT, "compare op");
            return C(to_compute(a)) > C(to_compute(b));  // :944
        }
    }
};

template <int OP, typename T> struct CompareScalarFn {
    T s;
    float eps;
    __device__ __forceinline__ uint8_t operator()(T a) const { return CompareFn<OP, T>{eps}(a, s); }
};

// ---- cast (static_cast semantics, elementwise_miaobyte.hpp:103-112) ------------------
template <typename S, typename D> struct CastFn {
    __device__ __forceinline__ D operator()(S a) const {
        if constexpr (std::is_same<S, D>::value) return a;
        else if constexpr (std::is_same<D, uint8_t>::value) {  // bool
            if constexpr (is_float_v<S>) return to_compute(a) != compute_t<S>(0);
            else return a != 0;
        } else if constexpr (is_float_v<D>) {
            if constexpr (std::is_same<D, double>::value) return static_cast<double>(to_compute(a));
            else if constexpr (std::is_same<D, float>::value) return static_cast<float>(to_compute(a));
            else if constexpr (std::is_same<S, double>::value) {
                // double → f16/bf16 in one rounding
                if constexpr (std::is_same<D, f16>::value) return __double2half(a);
                else return __double2bfloat16(a);
            } else if constexpr (std::is_same<S, int64_t>::value) {
                if constexpr (std::is_same<D, f16>::value) return __ll2half_rn(a);
                else return __ll2bfloat16_rn(a);
            } else if constexpr (std::is_same<S, int32_t>::value) {
                if constexpr (std::is_same<D, f16>::value) return __int2half_rn(a);
                else return __int2bfloat16_rn(a);
            } else return from_compute<D>(static_cast<float>(to_compute(a)));
        } else {
            // → integer: truncation toward zero; out-of-range is undefined in C++ (saturates here)
            if constexpr (is_float_v<S>) return static_cast<D>(to_compute(a));
            else return static_cast<D>(a);
        }
    }
};

}  // namespace dx
