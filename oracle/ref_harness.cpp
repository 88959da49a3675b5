// Harness around the REFERENCE's own sources — TEST INFRASTRUCTURE, NOT PRODUCT.
//
// Built only where the reference tree is present (see oracle/Makefile): the reference's
// deepxcore translation units (tf.cpp, tffactory.cpp, shape_changeshape.cpp,
// shape_reduce.cpp, shape_matmul.cpp, shape_range.cpp, stdutil/*.cpp) and the CPU
// executor's changeshape header are compiled where they lie and linked with this file
// into oracle/_ref/libdeepx_ref.so.  It is used to (a) validate the oracle restatement
// and the product's IR parser / registry / shape algebra against the reference's real
// code, and (b) generate the fixtures under tests/golden/.
//
// The reference's shape.cpp needs yaml-cpp, which is not installed; the non-YAML members
// of deepx::Shape are therefore defined here, following shape.cpp:11-91.  Everything else
// in this library is the reference's code.
#include <cstring>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "deepx/dtype.hpp"
#include "deepx/shape.hpp"
#include "deepx/shape_changeshape.hpp"
#include "deepx/shape_matmul.hpp"
#include "deepx/shape_reduce.hpp"
#include "deepx/tensor.hpp"
#include "deepx/tf/tf.hpp"
#include "deepx/tf/tffactory.hpp"
#include "deepx/tensorfunc/changeshape_miaobyte.hpp"

#include "ref_shape_standin.hpp"

using namespace deepx;

namespace {
int put(const std::string &s, char *out, int cap) {
    if ((int)s.size() + 1 > cap) return -1;
    std::memcpy(out, s.c_str(), s.size() + 1);
    return (int)s.size();
}
int put_vec(const std::vector<int> &v, int *out, int cap) {
    if ((int)v.size() > cap) return -1;
    for (size_t i = 0; i < v.size(); ++i) out[i] = v[i];
    return (int)v.size();
}
template <typename T> Tensor<T> borrow(const void *data, const int *shape, int ndim) {
    Tensor<T> t{std::vector<int>(shape, shape + ndim)};
    t.data = (T *)data;
    t.deleter = nullptr;
    t.newer = nullptr;
    t.copyer = nullptr;
    t.saver = nullptr;
    t.loader = nullptr;
    return t;
}
}  // namespace

extern "C" {

// IR text → what the reference's parser understood, in one line:
// "<name>|<arg0 dtype>:<arg0 text>,...|<ret0 dtype>:<ret0 text>,...|author=<a> id=<id> repeat=<n>"
int ref_parse_ir(const char *ir, char *out, int cap) {
    try {
        tf::TF t;
        t.metadata.id = 0;
        t.parse(ir);
        std::ostringstream ss;
        ss << t.name << "|";
        for (size_t i = 0; i < t.args.size(); ++i) ss << (i ? "," : "") << t.args[i].to_string();
        ss << "|";
        for (size_t i = 0; i < t.returns.size(); ++i) ss << (i ? "," : "") << t.returns[i].to_string();
        ss << "|author=" << t.metadata.author << " id=" << t.metadata.id << " repeat=" << t.metadata.benchmark.repeat;
        return put(ss.str(), out, cap);
    } catch (const std::exception &e) {
        return put(std::string("!") + e.what(), out, cap);
    }
}

int ref_dtype_roundtrip(const char *text, char *out, int cap) { return put(dtype_str(dtype(text)), out, cap); }
unsigned ref_dtype_value(const char *text) { return dtype(text).value; }
int ref_precision_bits(const char *prec) { return precision_bits(precision(prec)); }

// A registry holding plain TFs built from IR-style signature lines; get returns the
// index (registration order) of the entry the reference's matching rule picks, -1 for none.
struct RefFactory {
    tf::TfFactory f;
    std::vector<std::shared_ptr<tf::TF>> all;
};
void *ref_factory_new() { return new RefFactory(); }
void ref_factory_free(void *h) { delete (RefFactory *)h; }
int ref_factory_add(void *h, const char *signature_ir) {
    auto *rf = (RefFactory *)h;
    auto t = std::make_shared<tf::TF>();
    t->parse(signature_ir);
    t->tftype = std::to_string(rf->all.size());
    rf->all.push_back(t);
    rf->f.add_tf(t);
    return (int)rf->all.size() - 1;
}
int ref_factory_get(void *h, const char *ir) {
    auto *rf = (RefFactory *)h;
    tf::TF q;
    q.parse(ir);
    auto got = rf->f.get_tf(q);
    if (!got) return -1;
    return std::stoi(got->tftype);
}

// ---- shape algebra --------------------------------------------------------------------
int ref_transpose_shape(const int *shape, int ndim, const int *order, int *out, int cap) {
    try {
        return put_vec(transposeShape(std::vector<int>(shape, shape + ndim), std::vector<int>(order, order + ndim)), out, cap);
    } catch (...) { return -2; }
}
int ref_broadcast_shape(const int *a, int na, const int *b, int nb, int *out, int cap) {
    return put_vec(broadcastShape(std::vector<int>(a, a + na), std::vector<int>(b, b + nb)), out, cap);
}
int ref_indexselect_shape(const int *a, int na, const int *idx, int ni, int axis, int *out, int cap) {
    return put_vec(indexselectShape(std::vector<int>(a, a + na), std::vector<int>(idx, idx + ni), axis), out, cap);
}
int ref_reduced_shape(const int *shape, int ndim, const int *dims, int ndims, int keepdims, int *out, int cap) {
    try {
        std::vector<int> s(shape, shape + ndim);
        auto checked = checkedDims(s, std::vector<int>(dims, dims + ndims));
        return put_vec(reducedShape(s, checked, keepdims != 0), out, cap);
    } catch (...) { return -2; }
}
int ref_checked_dims(const int *shape, int ndim, const int *dims, int ndims, int *out, int cap) {
    try {
        return put_vec(checkedDims(std::vector<int>(shape, shape + ndim), std::vector<int>(dims, dims + ndims)), out, cap);
    } catch (...) { return -2; }
}
int ref_repeat_shape(const int *shape, int ndim, const int *rep, int *out, int cap) {
    try {
        return put_vec(repeatShape(std::vector<int>(shape, shape + ndim), std::vector<int>(rep, rep + ndim)), out, cap);
    } catch (...) { return -2; }
}
int ref_matmul_shape(const int *a, int na, const int *b, int nb, int *out, int cap) {
    try {
        return put_vec(matmul_shape(Shape(std::vector<int>(a, a + na)), Shape(std::vector<int>(b, b + nb))).shape, out, cap);
    } catch (...) { return -2; }
}

// ---- the CPU executor's changeshape tensor functions, on 1/2/4/8-byte elements --------------
#define BY_SIZE(es, ...)                                   \
    switch (es) {                                          \
        case 8: { using E = int64_t; __VA_ARGS__; } break; \
        case 4: { using E = int32_t; __VA_ARGS__; } break; \
        case 2: { using E = int16_t; __VA_ARGS__; } break; \
        case 1: { using E = int8_t; __VA_ARGS__; } break;  \
        default: return -1;                                \
    }

int ref_transpose(int es, const void *a, const int *shape, int ndim, const int *order, void *out) {
    try {
        std::vector<int> ord(order, order + ndim);
        auto oshape = transposeShape(std::vector<int>(shape, shape + ndim), ord);
        BY_SIZE(es, {
            auto A = borrow<E>(a, shape, ndim);
            auto C = borrow<E>(out, oshape.data(), ndim);
            tensorfunc::transpose<tensorfunc::miaobyte, E>(A, ord, C);
        })
        return 0;
    } catch (...) { return -2; }
}
int ref_concat(int es, const void *const *inputs, const int *const *shapes, int ninputs, int ndim, int axis, void *out) {
    try {
        BY_SIZE(es, {
            std::vector<Tensor<E>> hold;
            hold.reserve(ninputs);
            std::vector<Tensor<E> *> ptrs;
            for (int i = 0; i < ninputs; ++i) hold.push_back(borrow<E>(inputs[i], shapes[i], ndim));
            for (auto &t : hold) ptrs.push_back(&t);
            Shape os = concatShape(ptrs, axis);
            auto C = borrow<E>(out, os.shape.data(), ndim);
            tensorfunc::concat<tensorfunc::miaobyte, E>(ptrs, axis, C);
            for (auto &t : hold) t.data = nullptr;
            C.data = nullptr;
        })
        return 0;
    } catch (...) { return -2; }
}
int ref_broadcast_to(int es, const void *a, const int *ashape, int andim, const int *oshape, int ondim, void *out) {
    try {
        std::vector<int> ns(oshape, oshape + ondim);
        BY_SIZE(es, {
            auto A = borrow<E>(a, ashape, andim);
            auto B = borrow<E>(out, oshape, ondim);
            tensorfunc::broadcastTo<tensorfunc::miaobyte, E>(A, ns, B);
        })
        return 0;
    } catch (...) { return -2; }
}
int ref_indexselect(int es, const void *a, const int *ashape, int andim, int idx_es, const void *idx, const int *ishape,
                    int indim, int axis, void *out) {
    try {
        auto oshape = indexselectShape(std::vector<int>(ashape, ashape + andim), std::vector<int>(ishape, ishape + indim),
                                       axis < 0 ? axis + andim : axis);
        BY_SIZE(es, {
            auto A = borrow<E>(a, ashape, andim);
            auto B = borrow<E>(out, oshape.data(), (int)oshape.size());
            if (idx_es == 4) {
                auto I = borrow<int32_t>(idx, ishape, indim);
                tensorfunc::indexselect<tensorfunc::miaobyte, E, int32_t>(A, I, axis, B);
            } else {
                auto I = borrow<int64_t>(idx, ishape, indim);
                tensorfunc::indexselect<tensorfunc::miaobyte, E, int64_t>(A, I, axis, B);
            }
        })
        return 0;
    } catch (...) { return -2; }
}
int ref_repeat(int es, const void *a, const int *ashape, int ndim, const int *rep, void *out) {
    try {
        std::vector<int> r(rep, rep + ndim);
        auto oshape = repeatShape(std::vector<int>(ashape, ashape + ndim), r);
        BY_SIZE(es, {
            auto A = borrow<E>(a, ashape, ndim);
            auto B = borrow<E>(out, oshape.data(), ndim);
            tensorfunc::repeat<tensorfunc::miaobyte, E>(A, r, B);
        })
        return 0;
    } catch (...) { return -2; }
}
}
