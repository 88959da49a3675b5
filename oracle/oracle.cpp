// CPU oracle for the deepxIR tensor functions — TEST INFRASTRUCTURE, NOT PRODUCT.
//
// A plain C++17/OpenMP restatement of what the reference CPU executor
// (executor/op-ompsimd) computes for each op on the hot path.  Only tests/,
// __graft_entry__.smoke() and the cpu_baseline / --impl reference legs of bench.py
// may load this library, and only as the checker or as the timed CPU baseline.
// The GPU product never calls into it.
//
// What is restated, and from where (paths inside the reference project):
//   elementwise  executor/op-ompsimd/src/deepx/tensorfunc/elementwise_miaobyte.hpp
//                (the scalar lambdas; Highway lanes are IEEE-exact for + - * / sqrt
//                max min, so the scalar form defines the result).  The reference's
//                range driver (executor/deepxcore/src/deepx/shape_range.cpp:116-135)
//                hands the lambdas an absolute end where they expect a length and so
//                runs past the buffer; this file restates the math, not that driver.
//   reduce       executor/op-ompsimd/src/deepx/tensorfunc/reduce_miaobyte.hpp
//                + executor/deepxcore/src/deepx/shape_reduce.cpp
//   changeshape  executor/op-ompsimd/src/deepx/tensorfunc/changeshape_miaobyte.hpp
//                + executor/deepxcore/src/deepx/shape_changeshape.cpp
//   matmul       executor/op-ompsimd/src/deepx/tensorfunc/matmul_cblas.hpp:14-59
//                (row-major batched C = A·B; OpenBLAS there, a blocked fp32 loop here)
// float16 / bfloat16 do not exist in op-ompsimd; for them the rule is: widen to
// fp32, apply the fp32 op, round to nearest even once.
//
// Op and dtype codes are the ones of include/dx_kernels.h so a test can drive both
// sides with the same arguments.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <type_traits>
#include <vector>

#include "../include/dx_kernels.h"

namespace {

// ---- 16-bit floats -----------------------------------------------------------------
struct bf16_t { uint16_t bits; };
struct f16_t { uint16_t bits; };

inline float bf16_to_f32(bf16_t v) {
    uint32_t u = uint32_t(v.bits) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline bf16_t f32_to_bf16(float f) {  // round to nearest even; NaN stays NaN
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return bf16_t{uint16_t((u >> 16) | 0x40)};
    u += 0x7fffu + ((u >> 16) & 1u);
    return bf16_t{uint16_t(u >> 16)};
}
inline float f16_to_f32(f16_t v) {
    _Float16 h;
    std::memcpy(&h, &v.bits, 2);
    return static_cast<float>(h);
}
inline f16_t f32_to_f16(float f) {
    _Float16 h = static_cast<_Float16>(f);  // IEEE round to nearest even
    f16_t r;
    std::memcpy(&r.bits, &h, 2);
    return r;
}

template <typename T> struct compute { using type = T; };
template <> struct compute<bf16_t> { using type = float; };
template <> struct compute<f16_t> { using type = float; };
template <typename T> using compute_t = typename compute<T>::type;

template <typename T> inline compute_t<T> up(T v) { return v; }
template <> inline float up<bf16_t>(bf16_t v) { return bf16_to_f32(v); }
template <> inline float up<f16_t>(f16_t v) { return f16_to_f32(v); }
template <typename T> inline T down(compute_t<T> v) { return v; }
template <> inline bf16_t down<bf16_t>(float v) { return f32_to_bf16(v); }
template <> inline f16_t down<f16_t>(float v) { return f32_to_f16(v); }

template <typename T> constexpr bool is_fp = std::is_floating_point<compute_t<T>>::value;

template <typename T> inline T scalar_as(double fs, int64_t is) {
    if constexpr (std::is_same<T, double>::value) return fs;
    else if constexpr (std::is_same<T, float>::value) return static_cast<float>(fs);
    else if constexpr (std::is_same<T, bf16_t>::value) return f32_to_bf16(static_cast<float>(fs));
    else if constexpr (std::is_same<T, f16_t>::value) return f32_to_f16(static_cast<float>(fs));
    else return static_cast<T>(is);
}

#define ORC_NUMERIC(dtype, ...)                                                          \
    switch (dtype) {                                                                     \
        case DX_F64: { using T = double; __VA_ARGS__; } break;                           \
        case DX_F32: { using T = float; __VA_ARGS__; } break;                            \
        case DX_F16: { using T = f16_t; __VA_ARGS__; } break;                            \
        case DX_BF16: { using T = bf16_t; __VA_ARGS__; } break;                          \
        case DX_I64: { using T = int64_t; __VA_ARGS__; } break;                          \
        case DX_I32: { using T = int32_t; __VA_ARGS__; } break;                          \
        case DX_I16: { using T = int16_t; __VA_ARGS__; } break;                          \
        case DX_I8: { using T = int8_t; __VA_ARGS__; } break;                            \
        default: return DX_E_DTYPE;                                                      \
    }

// ---- elementwise ---------------------------------------------------------------------
// Wrapping integer arithmetic is spelled through the unsigned type so that the
// oracle itself has no undefined behaviour; the value is what two's-complement
// hardware gives for the reference's `a + b`.
template <typename T> inline T binary(int op, T a, T b) {
    using C = compute_t<T>;
    C x = up(a), y = up(b), r{};
    switch (op) {
        case DX_ADD:  // elementwise_miaobyte.hpp:123-124  c = a + b
            if constexpr (std::is_integral<C>::value) r = C(std::make_unsigned_t<C>(x) + std::make_unsigned_t<C>(y));
            else r = x + y;
            break;
        case DX_SUB:  // :164-165  c = a - b
            if constexpr (std::is_integral<C>::value) r = C(std::make_unsigned_t<C>(x) - std::make_unsigned_t<C>(y));
            else r = x - y;
            break;
        case DX_MUL:  // :226-227  c = a * b
            if constexpr (std::is_integral<C>::value) {
                using U = std::conditional_t<(sizeof(C) < 4), uint32_t, std::make_unsigned_t<C>>;
                r = C(U(x) * U(y));
            } else r = x * y;
            break;
        case DX_DIV:  // :267-268  c = a / b
            r = x / y;
            break;
        case DX_MAX:  // :614  std::max(a, b)
            r = std::max(x, y);
            break;
        case DX_MIN:  // :698  std::min(a, b)
            r = std::min(x, y);
            break;
        case DX_POW:  // :441  std::pow(a, b)
            if constexpr (is_fp<T>) r = std::pow(x, y);
            break;
    }
    return down<T>(r);
}

template <typename T> int ew_binary(int op, const T *a, const T *b, T *c, int64_t n) {
    if (op == DX_POW && !(std::is_same<T, double>::value || std::is_same<T, float>::value)) return DX_E_DTYPE;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) c[i] = binary<T>(op, a[i], b[i]);
    return DX_OK;
}

template <typename T> int ew_scalar(int op, const T *a, T s, T *c, int64_t n) {
    int bop;
    bool rev = false;
    switch (op) {
        case DX_ADDS: bop = DX_ADD; break;
        case DX_SUBS: bop = DX_SUB; break;
        case DX_RSUBS: bop = DX_SUB; rev = true; break;  // :204-205  c = b - a
        case DX_MULS: bop = DX_MUL; break;
        case DX_DIVS: bop = DX_DIV; break;
        case DX_RDIVS: bop = DX_DIV; rev = true; break;  // :307-308  c = b / a
        case DX_MAXS: bop = DX_MAX; break;               // :656
        case DX_MINS: bop = DX_MIN; break;               // :740
        case DX_POWS: bop = DX_POW; break;               // :462  pow(a, value)
        case DX_RPOWS: bop = DX_POW; rev = true; break;  // :482  pow(value, a)
        default: return DX_E_ARG;
    }
    if (bop == DX_POW && !(std::is_same<T, double>::value || std::is_same<T, float>::value)) return DX_E_DTYPE;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) c[i] = rev ? binary<T>(bop, s, a[i]) : binary<T>(bop, a[i], s);
    return DX_OK;
}

template <typename T> int ew_unary(int op, const T *a, T *c, int64_t n) {
    if constexpr (!is_fp<T>) return DX_E_DTYPE;
    else {
        using C = compute_t<T>;
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < n; ++i) {
            C x = up(a[i]), r{};
            switch (op) {
                case DX_SQRT: r = std::sqrt(x); break;  // :379
                case DX_LOG: r = std::log(x); break;    // :501
                case DX_EXP: r = std::exp(x); break;    // :520
                case DX_SIN: r = std::sin(x); break;
                case DX_COS: r = std::cos(x); break;
                case DX_TAN: r = std::tan(x); break;
            }
            c[i] = down<T>(r);
        }
        return DX_OK;
    }
}

template <typename T> inline bool compare(int op, T a, T b, float eps) {
    using C = compute_t<T>;
    C x = up(a), y = up(b);
    switch (op) {
        case DX_EQ:  // :778-785  eps == 0 ? a == b : |a - b| <= eps
            if (eps == 0) return x == y;
            if constexpr (std::is_integral<C>::value) {
                using W = std::conditional_t<(sizeof(C) < 8), int, int64_t>;
                return static_cast<float>(std::abs(W(x) - W(y))) <= eps;  // usual arithmetic conversions: int vs float → float
            } else return std::abs(x - y) <= eps;
        case DX_NE:  // :832-845  eps == 0 ? a != b : |a - b| > eps
            if (eps == 0) return x != y;
            if constexpr (std::is_integral<C>::value) {
                using W = std::conditional_t<(sizeof(C) < 8), int, int64_t>;
                return static_cast<float>(std::abs(W(x) - W(y))) > eps;
            } else return std::abs(x - y) > eps;
        case DX_LT: return x < y;  // :900
        case DX_GT: return x > y;  // :944
    }
    return false;
}

template <typename T> int ew_compare(int op, const T *a, const T *b, float eps, uint8_t *m, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) m[i] = compare<T>(op, a[i], b[i], eps);
    return DX_OK;
}
template <typename T> int ew_compare_scalar(int op, const T *a, T s, float eps, uint8_t *m, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) m[i] = compare<T>(op, a[i], s, eps);
    return DX_OK;
}

// static_cast between element types (elementwise_miaobyte.hpp:103-112)
template <typename S, typename D> int cast(const S *a, D *c, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        if constexpr (std::is_same<S, D>::value) c[i] = a[i];
        else if constexpr (std::is_same<D, bf16_t>::value || std::is_same<D, f16_t>::value) {
            // one rounding from the source value: go through double for 64-bit sources
            if constexpr (sizeof(compute_t<S>) == 8) {
                // double → float → 16-bit would round twice.  Truncate the magnitude to
                // float and keep a sticky low bit (round-to-odd); the final RNE is then exact.
                const double d = static_cast<double>(up(a[i]));
                float f = static_cast<float>(d);
                if (std::isfinite(f) && static_cast<double>(f) != d) {
                    uint32_t u;
                    std::memcpy(&u, &f, 4);
                    if (std::fabs(static_cast<double>(f)) > std::fabs(d)) u -= 1;
                    u |= 1u;
                    std::memcpy(&f, &u, 4);
                }
                c[i] = down<D>(f);
            } else c[i] = down<D>(static_cast<float>(up(a[i])));
        } else c[i] = static_cast<D>(up(a[i]));
    }
    return DX_OK;
}

template <typename S> int cast_from(const S *a, int dst, void *c, int64_t n) {
    switch (dst) {
        case DX_F64: return cast(a, (double *)c, n);
        case DX_F32: return cast(a, (float *)c, n);
        case DX_F16: return cast(a, (f16_t *)c, n);
        case DX_BF16: return cast(a, (bf16_t *)c, n);
        case DX_I64: return cast(a, (int64_t *)c, n);
        case DX_I32: return cast(a, (int32_t *)c, n);
        case DX_I16: return cast(a, (int16_t *)c, n);
        case DX_I8: return cast(a, (int8_t *)c, n);
        default: return DX_E_DTYPE;
    }
}

// ---- shape helpers (executor/deepxcore/src/deepx/shape.cpp:21-32,73-91) ----------------
std::vector<int64_t> strides_of(const int64_t *shape, int ndim) {
    std::vector<int64_t> s(ndim);
    int64_t acc = 1;
    for (int i = ndim - 1; i >= 0; --i) { s[i] = acc; acc *= shape[i]; }
    return s;
}
int64_t count_of(const int64_t *shape, int ndim) {
    int64_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= shape[i];
    return n;
}
// Shape::linearto
inline void linearto(int64_t idx, const std::vector<int64_t> &strides, int64_t *indices) {
    for (size_t i = 0; i < strides.size(); ++i) { indices[i] = idx / strides[i]; idx %= strides[i]; }
}

// ---- reduce (reduce_miaobyte.hpp) ---------------------------------------------------------
template <typename T> struct racc { using type = compute_t<T>; };
template <typename T> using racc_t = typename racc<T>::type;

template <typename T> T lowest_of() {
    if constexpr (std::is_same<T, bf16_t>::value) return bf16_t{0xFF7F};
    else if constexpr (std::is_same<T, f16_t>::value) return f16_t{0xFBFF};
    else return std::numeric_limits<T>::lowest();
}
template <typename T> T highest_of() {
    if constexpr (std::is_same<T, bf16_t>::value) return bf16_t{0x7F7F};
    else if constexpr (std::is_same<T, f16_t>::value) return f16_t{0x7BFF};
    else return std::numeric_limits<T>::max();
}

template <typename T>
int reduce(int op, const T *a, const int64_t *shape, int ndim, const int32_t *dims, int ndims, T *out) {
    using A = racc_t<T>;
    std::vector<int> reduced(ndim, 0);  // reducedDim(), shape_reduce.cpp:77-85
    for (int i = 0; i < ndims; ++i) {
        if (dims[i] < 0 || dims[i] >= ndim) return DX_E_SHAPE;
        reduced[dims[i]] = 1;
    }
    const auto istr = strides_of(shape, ndim);
    std::vector<int64_t> oshape;
    for (int i = 0; i < ndim; ++i)
        if (!reduced[i]) oshape.push_back(shape[i]);
    const auto ostr = strides_of(oshape.data(), (int)oshape.size());
    const int64_t nout = count_of(oshape.data(), (int)oshape.size());
    const int64_t nin = count_of(shape, ndim);
    // pre-fill: sum 0 (:22), prod 1 (:104), max lowest() (:192), min max() (:275)
    A init;
    switch (op) {
        case DX_SUM: init = A(0); break;
        case DX_PROD: init = A(1); break;
        case DX_RMAX: init = up(lowest_of<T>()); break;
        case DX_RMIN: init = up(highest_of<T>()); break;
        default: return DX_E_ARG;
    }
    // Per output element, walk its reduced sub-space in row-major input order and
    // fold — the order a single-threaded run of the reference's rangeParallel visits.
    std::vector<int64_t> rshape, rstr;
    for (int i = 0; i < ndim; ++i)
        if (reduced[i]) { rshape.push_back(shape[i]); rstr.push_back(istr[i]); }
    const int64_t nred = nout ? nin / std::max<int64_t>(nout, 1) : 0;
    const auto rlin = strides_of(rshape.data(), (int)rshape.size());
    std::vector<int64_t> kstr;
    for (int i = 0; i < ndim; ++i)
        if (!reduced[i]) kstr.push_back(istr[i]);
#pragma omp parallel for schedule(static) if (nout > 1)
    for (int64_t o = 0; o < nout; ++o) {
        int64_t base = 0, rem = o;
        for (size_t k = 0; k < ostr.size(); ++k) { base += (rem / ostr[k]) * kstr[k]; rem %= ostr[k]; }
        A acc = init;
        for (int64_t r = 0; r < nred; ++r) {
            int64_t off = base, rr = r;
            for (size_t k = 0; k < rlin.size(); ++k) { off += (rr / rlin[k]) * rstr[k]; rr %= rlin[k]; }
            const A v = up(a[off]);
            switch (op) {
                case DX_SUM:
                    if constexpr (std::is_integral<A>::value) acc = A(std::make_unsigned_t<A>(acc) + std::make_unsigned_t<A>(v));
                    else acc += v;  // :41 result += tensor
                    break;
                case DX_PROD:
                    if constexpr (std::is_integral<A>::value) {
                        using U = std::conditional_t<(sizeof(A) < 4), uint32_t, std::make_unsigned_t<A>>;
                        acc = A(U(acc) * U(v));
                    } else acc *= v;  // :122
                    break;
                case DX_RMAX: acc = std::max(acc, v); break;  // :209
                case DX_RMIN: acc = std::min(acc, v); break;  // :292
            }
        }
        out[o] = down<T>(acc);
    }
    return DX_OK;
}

// Global float sum of a large flat array, split over threads (used by the timed CPU
// baseline where one output would otherwise run on one core).
template <typename T> int reduce_all_parallel(int op, const T *a, int64_t n, T *out) {
    using A = racc_t<T>;
    if (op != DX_SUM && op != DX_RMAX && op != DX_RMIN) return DX_E_ARG;
    A total = (op == DX_SUM) ? A(0) : (op == DX_RMAX ? up(lowest_of<T>()) : up(highest_of<T>()));
    if (op == DX_SUM) {
        if constexpr (std::is_floating_point<A>::value) {
#pragma omp parallel for reduction(+ : total) schedule(static)
            for (int64_t i = 0; i < n; ++i) total += up(a[i]);
        } else {
            std::make_unsigned_t<A> t = 0;
#pragma omp parallel for reduction(+ : t) schedule(static)
            for (int64_t i = 0; i < n; ++i) t += std::make_unsigned_t<A>(up(a[i]));
            total = A(t);
        }
    } else if (op == DX_RMAX) {
#pragma omp parallel for reduction(max : total) schedule(static)
        for (int64_t i = 0; i < n; ++i) total = std::max(total, up(a[i]));
    } else {
#pragma omp parallel for reduction(min : total) schedule(static)
        for (int64_t i = 0; i < n; ++i) total = std::min(total, up(a[i]));
    }
    out[0] = down<T>(total);
    return DX_OK;
}

// ---- changeshape (changeshape_miaobyte.hpp), on raw element bytes ----------------------------
template <typename E>
int transpose(const E *a, const int64_t *shape, int ndim, const int32_t *perm, E *out) {
    // :48-66  for each output index: input_index[dim_order[i]] = output_index[i]
    std::vector<int64_t> oshape(ndim);
    for (int i = 0; i < ndim; ++i) oshape[i] = shape[perm[i]];  // transposeShape, shape_changeshape.cpp:17-29
    const auto istr = strides_of(shape, ndim);
    const auto ostr = strides_of(oshape.data(), ndim);
    const int64_t n = count_of(shape, ndim);
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < n; ++o) {
        int64_t oi[DX_MAX_DIMS];
        linearto(o, ostr, oi);
        int64_t in = 0;
        for (int i = 0; i < ndim; ++i) in += oi[i] * istr[perm[i]];
        out[o] = a[in];
    }
    return DX_OK;
}

template <typename E>
int concat(const E *const *inputs, const int64_t *axis_len, int ninputs, const int64_t *oshape, int ndim, int axis,
           E *out) {
    // :72-99  walk the output up to and including `axis`; find the owning input by
    // subtracting extents; copy strides[axis] contiguous elements.
    int64_t outer = 1, inner = 1, total = 0;
    for (int i = 0; i < axis; ++i) outer *= oshape[i];
    for (int i = axis + 1; i < ndim; ++i) inner *= oshape[i];
    for (int i = 0; i < ninputs; ++i) total += axis_len[i];
    if (total != oshape[axis]) return DX_E_SHAPE;  // checkShapeConcat, shape_changeshape.hpp:38-63
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t p = 0; p < outer; ++p)
        for (int64_t x = 0; x < total; ++x) {
            int64_t xi = x;
            int t = 0;
            while (t < ninputs && xi >= axis_len[t]) { xi -= axis_len[t]; ++t; }
            const E *src = inputs[t] + (p * axis_len[t] + xi) * inner;
            std::copy(src, src + inner, out + (p * total + x) * inner);
        }
    return DX_OK;
}

template <typename E>
int broadcast_to(const E *a, const int64_t *ashape, int andim, const int64_t *oshape, int ondim, E *out) {
    // broadcastMap (shape_changeshape.cpp:81-105) + fromBroadcastIndices (changeshape_miaobyte.hpp:101-119)
    if (andim > ondim) return DX_E_SHAPE;
    const int lead = ondim - andim;
    for (int i = 0; i < andim; ++i)
        if (ashape[i] != oshape[lead + i] && ashape[i] != 1) return DX_E_SHAPE;
    const auto astr = strides_of(ashape, andim);
    const auto ostr = strides_of(oshape, ondim);
    const int64_t n = count_of(oshape, ondim);
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < n; ++o) {
        int64_t oi[DX_MAX_DIMS];
        linearto(o, ostr, oi);
        int64_t in = 0;
        for (int i = lead; i < ondim; ++i)
            if (ashape[i - lead] != 1) in += oi[i] * astr[i - lead];  // xTox keeps the index, xTo1 → 0, nullTo1 dropped
        out[o] = a[in];
    }
    return DX_OK;
}

template <typename E, typename I>
int indexselect(const E *a, const int64_t *ashape, int andim, const I *idx, const int64_t *ishape, int indim, int axis,
                E *out) {
    // :144-177 with indexselectShape (shape_changeshape.cpp:122-141):
    // out[pre.., idx_dims.., post..] = a[pre.., idx[idx_dims], post..]
    if (axis < 0) axis += andim;
    if (axis < 0 || axis >= andim) return DX_E_SHAPE;
    int64_t pre = 1, post = 1;
    for (int i = 0; i < axis; ++i) pre *= ashape[i];
    for (int i = axis + 1; i < andim; ++i) post *= ashape[i];
    const int64_t ni = count_of(ishape, indim), alen = ashape[axis];
#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t p = 0; p < pre; ++p)
        for (int64_t q = 0; q < ni; ++q) {
            const int64_t ix = static_cast<int64_t>(idx[q]);
            E *dst = out + (p * ni + q) * post;
            if (ix < 0 || ix >= alen) std::fill(dst, dst + post, E(0));  // undefined in the reference; zeros here and in the GPU path
            else std::copy(a + (p * alen + ix) * post, a + (p * alen + ix + 1) * post, dst);
        }
    return DX_OK;
}

template <typename E>
int repeat(const E *a, const int64_t *ashape, int ndim, const int64_t *repeats, E *out) {
    // :184-199  src_index[i] = out_index[i] / repeats[i]
    std::vector<int64_t> oshape(ndim);
    for (int i = 0; i < ndim; ++i) oshape[i] = ashape[i] * repeats[i];  // repeatShape, shape_changeshape.cpp:144-156
    const auto astr = strides_of(ashape, ndim);
    const auto ostr = strides_of(oshape.data(), ndim);
    const int64_t n = count_of(oshape.data(), ndim);
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < n; ++o) {
        int64_t oi[DX_MAX_DIMS];
        linearto(o, ostr, oi);
        int64_t in = 0;
        for (int i = 0; i < ndim; ++i) in += (oi[i] / repeats[i]) * astr[i];
        out[o] = a[in];
    }
    return DX_OK;
}

#define ORC_BY_SIZE(es, ...)                                         \
    switch (es) {                                                    \
        case 8: { using E = uint64_t; __VA_ARGS__; } break;          \
        case 4: { using E = uint32_t; __VA_ARGS__; } break;          \
        case 2: { using E = uint16_t; __VA_ARGS__; } break;          \
        case 1: { using E = uint8_t; __VA_ARGS__; } break;           \
        default: return DX_E_DTYPE;                                  \
    }

int esize(int dtype) {
    switch (dtype) {
        case DX_F64: case DX_I64: return 8;
        case DX_F32: case DX_I32: return 4;
        case DX_F16: case DX_BF16: case DX_I16: return 2;
        case DX_I8: case DX_BOOL: return 1;
        default: return 0;
    }
}

// ---- matmul: batched row-major C = A·B (matmul_cblas.hpp:30-58) -----------------------------
// Accumulates in the compute type (fp32 for f32/f16/bf16, fp64 for f64), k innermost,
// i-k-j loop order over cache blocks so the timed baseline is not a strawman.
template <typename T> int matmul(const T *A, const T *B, T *C, int64_t batch, int64_t M, int64_t N, int64_t K) {
    using Cc = compute_t<T>;
    constexpr int64_t BI = 64, BK = 256;
#pragma omp parallel
    {
        std::vector<Cc> acc(BI * N);
#pragma omp for schedule(dynamic) collapse(2)
        for (int64_t b = 0; b < batch; ++b)
            for (int64_t i0 = 0; i0 < M; i0 += BI) {
                const int64_t i1 = std::min(M, i0 + BI);
                std::fill(acc.begin(), acc.end(), Cc(0));
                for (int64_t k0 = 0; k0 < K; k0 += BK) {
                    const int64_t k1 = std::min(K, k0 + BK);
                    for (int64_t i = i0; i < i1; ++i) {
                        Cc *row = acc.data() + (i - i0) * N;
                        for (int64_t k = k0; k < k1; ++k) {
                            const Cc av = up(A[(b * M + i) * K + k]);
                            const T *brow = B + (b * K + k) * N;
                            for (int64_t j = 0; j < N; ++j) row[j] += av * up(brow[j]);
                        }
                    }
                }
                for (int64_t i = i0; i < i1; ++i)
                    for (int64_t j = 0; j < N; ++j) C[(b * M + i) * N + j] = down<T>(acc[(i - i0) * N + j]);
            }
    }
    return DX_OK;
}

}  // namespace

extern "C" {

int orc_ew_binary(int op, int dtype, const void *a, const void *b, void *c, int64_t n) {
    if (op < 0 || op >= DX_BINARY_COUNT) return DX_E_ARG;
    ORC_NUMERIC(dtype, return ew_binary<T>(op, (const T *)a, (const T *)b, (T *)c, n))
    return DX_OK;
}
int orc_ew_scalar(int op, int dtype, const void *a, double fs, int64_t is, void *c, int64_t n) {
    ORC_NUMERIC(dtype, return ew_scalar<T>(op, (const T *)a, scalar_as<T>(fs, is), (T *)c, n))
    return DX_OK;
}
int orc_ew_unary(int op, int dtype, const void *a, void *c, int64_t n) {
    if (op == DX_INVERT) {  // elementwise_miaobyte.hpp:332 (~a), :353 (!a for bool)
        switch (dtype) {
            case DX_I64: for (int64_t i = 0; i < n; ++i) ((int64_t *)c)[i] = ~((const int64_t *)a)[i]; return DX_OK;
            case DX_I32: for (int64_t i = 0; i < n; ++i) ((int32_t *)c)[i] = ~((const int32_t *)a)[i]; return DX_OK;
            case DX_I16: for (int64_t i = 0; i < n; ++i) ((int16_t *)c)[i] = int16_t(~((const int16_t *)a)[i]); return DX_OK;
            case DX_I8: for (int64_t i = 0; i < n; ++i) ((int8_t *)c)[i] = int8_t(~((const int8_t *)a)[i]); return DX_OK;
            case DX_BOOL: for (int64_t i = 0; i < n; ++i) ((uint8_t *)c)[i] = !((const uint8_t *)a)[i]; return DX_OK;
            default: return DX_E_DTYPE;
        }
    }
    if (op < 0 || op >= DX_INVERT) return DX_E_ARG;
    ORC_NUMERIC(dtype, return ew_unary<T>(op, (const T *)a, (T *)c, n))
    return DX_OK;
}
int orc_ew_compare(int op, int dtype, const void *a, const void *b, float eps, void *mask, int64_t n) {
    if (op < 0 || op >= DX_COMPARE_COUNT) return DX_E_ARG;
    ORC_NUMERIC(dtype, return ew_compare<T>(op, (const T *)a, (const T *)b, eps, (uint8_t *)mask, n))
    return DX_OK;
}
int orc_ew_compare_scalar(int op, int dtype, const void *a, double fs, int64_t is, float eps, void *mask, int64_t n) {
    if (op < 0 || op >= DX_COMPARE_COUNT) return DX_E_ARG;
    ORC_NUMERIC(dtype, return ew_compare_scalar<T>(op, (const T *)a, scalar_as<T>(fs, is), eps, (uint8_t *)mask, n))
    return DX_OK;
}
int orc_switch(int dtype, const void *const *tensors, int ntensors, int cases_dtype, const void *cases, void *c,
               int64_t n) {
    // elementwise_miaobyte.hpp:988-989 (int cases) and :1018 (bool cases, exactly two tensors)
    const int es = esize(dtype);
    if (cases_dtype == DX_BOOL && ntensors != 2) return DX_E_ARG;
    if (cases_dtype != DX_BOOL && cases_dtype != DX_I32) return DX_E_DTYPE;
    ORC_BY_SIZE(es, {
        for (int64_t i = 0; i < n; ++i) {
            int w = cases_dtype == DX_BOOL ? (((const uint8_t *)cases)[i] ? 1 : 0) : ((const int32_t *)cases)[i];
            ((E *)c)[i] = (w >= 0 && w < ntensors) ? ((const E *)tensors[w])[i] : E(0);
        }
        return DX_OK;
    })
    return DX_OK;
}
int orc_cast(int src, const void *a, int dst, void *c, int64_t n) {
    if (dst == DX_BOOL || src == DX_BOOL) return DX_E_DTYPE;  // op-ompsimd has no bool todtype
    ORC_NUMERIC(src, return cast_from<T>((const T *)a, dst, c, n))
    return DX_OK;
}
int orc_reduce(int op, int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *dims, int ndims,
               void *out) {
    ORC_NUMERIC(dtype, return reduce<T>(op, (const T *)a, shape, ndim, dims, ndims, (T *)out))
    return DX_OK;
}
int orc_reduce_all_parallel(int op, int dtype, const void *a, int64_t n, void *out) {
    ORC_NUMERIC(dtype, return reduce_all_parallel<T>(op, (const T *)a, n, (T *)out))
    return DX_OK;
}
int orc_transpose(int dtype, const void *a, const int64_t *shape, int ndim, const int32_t *perm, void *out) {
    ORC_BY_SIZE(esize(dtype), return transpose<E>((const E *)a, shape, ndim, perm, (E *)out))
    return DX_OK;
}
int orc_concat(int dtype, const void *const *inputs, const int64_t *axis_len, int ninputs, const int64_t *out_shape,
               int ndim, int axis, void *out) {
    ORC_BY_SIZE(esize(dtype), return concat<E>((const E *const *)inputs, axis_len, ninputs, out_shape, ndim, axis, (E *)out))
    return DX_OK;
}
int orc_broadcast_to(int dtype, const void *a, const int64_t *a_shape, int a_ndim, const int64_t *out_shape, int out_ndim,
                     void *out) {
    ORC_BY_SIZE(esize(dtype), return broadcast_to<E>((const E *)a, a_shape, a_ndim, out_shape, out_ndim, (E *)out))
    return DX_OK;
}
int orc_indexselect(int dtype, const void *a, const int64_t *a_shape, int a_ndim, int idx_dtype, const void *idx,
                    const int64_t *idx_shape, int idx_ndim, int axis, void *out) {
    if (idx_dtype == DX_I32) {
        ORC_BY_SIZE(esize(dtype), return indexselect<E, int32_t>((const E *)a, a_shape, a_ndim, (const int32_t *)idx, idx_shape, idx_ndim, axis, (E *)out))
    } else if (idx_dtype == DX_I64) {
        ORC_BY_SIZE(esize(dtype), return indexselect<E, int64_t>((const E *)a, a_shape, a_ndim, (const int64_t *)idx, idx_shape, idx_ndim, axis, (E *)out))
    } else return DX_E_DTYPE;
    return DX_OK;
}
int orc_repeat(int dtype, const void *a, const int64_t *a_shape, int ndim, const int64_t *repeats, void *out) {
    ORC_BY_SIZE(esize(dtype), return repeat<E>((const E *)a, a_shape, ndim, repeats, (E *)out))
    return DX_OK;
}
int orc_matmul(int dtype, const void *A, const void *B, void *C, int64_t batch, int64_t M, int64_t N, int64_t K) {
    switch (dtype) {
        case DX_F64: return matmul<double>((const double *)A, (const double *)B, (double *)C, batch, M, N, K);
        case DX_F32: return matmul<float>((const float *)A, (const float *)B, (float *)C, batch, M, N, K);
        case DX_F16: return matmul<f16_t>((const f16_t *)A, (const f16_t *)B, (f16_t *)C, batch, M, N, K);
        case DX_BF16: return matmul<bf16_t>((const bf16_t *)A, (const bf16_t *)B, (bf16_t *)C, batch, M, N, K);
        default: return DX_E_DTYPE;
    }
}
int orc_num_threads(void);
}

#ifdef _OPENMP
#include <omp.h>
extern "C" int orc_num_threads(void) { return omp_get_max_threads(); }
#else
extern "C" int orc_num_threads(void) { return 1; }
#endif
