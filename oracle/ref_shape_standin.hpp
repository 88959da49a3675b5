// The non-YAML members of the reference's deepx::Shape — TEST INFRASTRUCTURE, NOT PRODUCT.
//
// The reference defines them in executor/deepxcore/src/deepx/shape.cpp:11-91, a file that also
// needs yaml-cpp (not installed here), so the harnesses around the reference's own sources define
// them from this header instead.  Include it in exactly one translation unit per library.
#pragma once
#include <stdexcept>
#include <string>
#include <vector>

#include "deepx/dtype.hpp"
#include "deepx/shape.hpp"

namespace deepx {
// ---- deepx::Shape, the members shape.cpp defines without YAML (shape.cpp:11-91) ----------
Shape::Shape(const int *shape, int dim) { setshape(shape, dim); }
int Shape::dim() const { return shape.size(); }
int64_t Shape::bytes() const { return size * (precision_bits(dtype) / 8); }
void Shape::setshape(const int *shape, int dim) {
    this->shape.assign(shape, shape + dim);
    strides.resize(dim);
    strides[dim - 1] = 1;
    for (int i = dim - 2; i >= 0; --i) strides[i] = strides[i + 1] * shape[i + 1];
    size = strides[0] * shape[0];
}
Shape::Shape(const std::vector<int> &shape) { setshape(shape.data(), shape.size()); }
Shape::Shape(const std::initializer_list<int> &shape) { setshape(shape.begin(), shape.size()); }
int Shape::operator[](int index) const { return shape[index < 0 ? index + (int)shape.size() : index]; }
int &Shape::operator[](int index) { return shape[index < 0 ? index + (int)shape.size() : index]; }
void Shape::print() const {}
int Shape::linearat(const std::vector<int> &indices) const {
    int idx = 0;
    size_t stride_i = 0, indices_i = 0;
    if (indices.size() > shape.size()) indices_i = indices.size() - shape.size();
    for (; stride_i < strides.size() && stride_i < indices.size();) idx += indices[indices_i++] * strides[stride_i++];
    return idx;
}
std::vector<int> Shape::linearto(int idx_linear) const {
    std::vector<int> indices(dim(), 0);
    for (int i = 0; i < dim(); i++) {
        indices[i] = idx_linear / strides[i];
        idx_linear %= strides[i];
    }
    return indices;
}
std::string Shape::toYaml() const { return ""; }
void Shape::fromYaml(const std::string &) { throw std::runtime_error("yaml-cpp not available"); }
void Shape::saveShape(const std::string &) const {}
std::pair<std::string, Shape> Shape::loadShape(const std::string &) { throw std::runtime_error("yaml-cpp not available"); }
}  // namespace deepx
