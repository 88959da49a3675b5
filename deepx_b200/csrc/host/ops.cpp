// deepxIR ops: one TF subclass per op family, and the registration table.
//
// Names, authors, argument order, dtype masks and error strings follow
// executor/op-cuda/src/client/tfs.cpp and executor/op-cuda/src/deepx/tf/*.hpp; the bodies
// are new: tensors are type-erased, so an op validates names/dtypes/shapes and makes ONE call
// into the kernel C ABI with the tensor's dtype code instead of a 9-way switch over C++ types.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <unistd.h>

#include <cctype>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>

#include "core.hpp"

namespace dxh {
namespace {

void dx_check(int rc) {
    if (rc == DX_OK) return;
    if (rc == DX_E_SHAPE) throw TensorShapeError(dx_last_error());
    throw std::runtime_error(dx_last_error());
}

// A scalar as the reference narrows it: text → std::stof → T (tf.hpp:119-123).
struct Scalar { double f; int64_t i; };
Scalar scalar_for(const TF &tf, int idx, const Mem &mem) {
    const float v = tf.var_f32(idx, mem);
    return Scalar{double(v), int64_t(v)};
}

std::string type_mismatch(std::initializer_list<uint16_t> ps) {
    std::string s = "Type mismatch: ";
    bool first = true;
    for (auto p : ps) {
        if (!first) s += " != ";
        s += precision_str(p);
        first = false;
    }
    return s;
}

// ---- operands of an op that works row by row (shard.hpp) ------------------------------------------------------
// With a single rank, or when nothing is partitioned, this is the whole tensors and the checks the reference makes.
// Otherwise every operand is taken by this rank's rows: a partitioned tensor as it is, a replicated one of the same
// global shape through the rows [row0, row0 + rows) of its full copy.  A replicated OUTPUT computed that way is
// completed by finish(): an all-gather of the row blocks over the communicator.
struct Rowwise {
    Mem &mem;
    bool by_rows = false;
    int64_t n = 0;           // elements this rank computes
    int64_t rows = 0;        // local rows (by_rows)
    TensorPtr gather;        // replicated output to complete
    std::vector<void *> ptr; // inputs in order, then the output
    std::vector<int64_t> local_shape;  // of the output, as computed here

    Rowwise(Mem &m, const std::vector<TensorPtr> &inputs, const TensorPtr &out) : mem(m) {
        std::vector<Layout> in;
        for (const auto &t : inputs) in.push_back(t->layout());
        const RowwisePlan plan = plan_rowwise(in, out->layout());
        if (!plan.error.empty()) throw std::invalid_argument(plan.error);
        by_rows = plan.by_rows;
        if (!by_rows) {
            for (const auto &t : inputs) ptr.push_back(t->data);
            ptr.push_back(out->data);
            n = out->shape.size;
            local_shape = out->shape.shape;
            return;
        }
        const std::vector<int64_t> g = out->global_shape();
        const RowBlock b = row_block(g[0], mem.shard.rank, mem.shard.world);
        auto rows_of = [&](const TensorPtr &t) -> void * {
            if (t->partitioned()) {
                if (t->row0 != b.row0 || t->shape.shape[0] != b.rows) throw std::runtime_error("tensors are partitioned differently");
                return t->data;
            }
            return static_cast<char *>(t->data) + b.row0 * t->row_bytes();
        };
        for (const auto &t : inputs) ptr.push_back(rows_of(t));
        ptr.push_back(rows_of(out));
        rows = b.rows;
        local_shape = g;
        local_shape[0] = b.rows;
        n = 1;
        for (auto d : local_shape) n *= d;
        if (plan.gather_output) gather = out;
    }
    void finish() {
        if (!gather) return;
        if (mem.capturing && !mem.shard.comm) return;
        dx_check(dx_comm_allgather_rows(mem.shard.comm, gather->data, gather->shape.shape[0], gather->row_bytes(), mem.stream()));
    }
};

// Ops that have no row-wise form: refuse partitioned operands with a reply that says what to do.
void refuse_partitioned(const std::string &op, std::initializer_list<TensorPtr> ts) {
    for (const auto &t : ts)
        if (t && t->partitioned())
            throw std::runtime_error(op + ": this form of the op does not work on row-partitioned tensors (a tensor of " +
                                     std::to_string(t->global_rows) + " rows is split over the GPUs); keep its operands below the partition threshold");
}

#define DX_TF_BOILERPLATE(Class)                                              \
    std::shared_ptr<TF> clone() const override { return std::make_shared<Class>(*this); } \
    std::string math_formula() const override { return formula; }

// ---- elementwise -----------------------------------------------------------------------------
struct BinaryTF : TF {  // add sub mul div max min pow  (tf/elementwise_basic.hpp:365-430 pattern)
    int op;
    std::string formula;
    BinaryTF(const char *nm, const char *author, int op_, const char *formula_, std::vector<Param> a, std::vector<Param> r)
        : op(op_), formula(formula_) { name = nm; metadata.author = author; tftype = "elementwise"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(BinaryTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({args[0].textvalue, args[1].textvalue, returns[0].textvalue}, mem, error)) return 1;
        auto A = mem.get_tensor(args[0].textvalue), B = mem.get_tensor(args[1].textvalue), C = mem.get_tensor(returns[0].textvalue);
        if (A->shape.dtype != B->shape.dtype || A->shape.dtype != C->shape.dtype) {
            error = type_mismatch({A->shape.dtype, B->shape.dtype, C->shape.dtype});
            return 1;
        }
        Rowwise rw(mem, {A, B}, C);
        dx_check(dx_ew_binary(op, A->dx(), rw.ptr[0], rw.ptr[1], rw.ptr[2], rw.n, mem.stream()));
        rw.finish();
        return 0;
    }
};

struct ScalarTF : TF {  // addscalar … rpowscalar; `reversed` ops take (scalar, tensor)
    int op;
    bool reversed;
    std::string formula;
    ScalarTF(const char *nm, int op_, bool rev, const char *formula_, std::vector<Param> a, std::vector<Param> r)
        : op(op_), reversed(rev), formula(formula_) { name = nm; metadata.author = "miaobyte"; tftype = "elementwise"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(ScalarTF)
    int run(Mem &mem, std::string &error) override {
        const int ti = reversed ? 1 : 0, si = reversed ? 0 : 1;
        if (!check_tensors({args[ti].textvalue, returns[0].textvalue}, mem, error)) return 1;
        auto A = mem.get_tensor(args[ti].textvalue), C = mem.get_tensor(returns[0].textvalue);
        if (A->shape.dtype != C->shape.dtype) { error = type_mismatch({A->shape.dtype, C->shape.dtype}); return 1; }
        Rowwise rw(mem, {A}, C);
        const Scalar s = scalar_for(*this, si, mem);
        dx_check(dx_ew_scalar(op, A->dx(), rw.ptr[0], s.f, s.i, rw.ptr[1], rw.n, mem.stream()));
        rw.finish();
        return 0;
    }
};

struct UnaryTF : TF {  // sqrt log exp sin cos tan invert
    int op;
    std::string formula;
    UnaryTF(const char *nm, int op_, const char *formula_, std::vector<Param> a, std::vector<Param> r)
        : op(op_), formula(formula_) { name = nm; metadata.author = "miaobyte"; tftype = "elementwise"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(UnaryTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({args[0].textvalue, returns[0].textvalue}, mem, error)) return 1;
        auto A = mem.get_tensor(args[0].textvalue), C = mem.get_tensor(returns[0].textvalue);
        if (A->shape.dtype != C->shape.dtype) { error = type_mismatch({A->shape.dtype, C->shape.dtype}); return 1; }
        Rowwise rw(mem, {A}, C);
        dx_check(dx_ew_unary(op, A->dx(), rw.ptr[0], rw.ptr[1], rw.n, mem.stream()));
        rw.finish();
        return 0;
    }
};

struct CompareTF : TF {  // equal notequal (with epsilon) less greater
    int op;
    bool has_eps;
    std::string formula;
    CompareTF(const char *nm, int op_, bool eps, const char *formula_, std::vector<Param> a, std::vector<Param> r)
        : op(op_), has_eps(eps), formula(formula_) { name = nm; metadata.author = "miaobyte"; tftype = "elementwise"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(CompareTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({args[0].textvalue, args[1].textvalue, returns[0].textvalue}, mem, error)) return 1;
        auto A = mem.get_tensor(args[0].textvalue), B = mem.get_tensor(args[1].textvalue), M = mem.get_tensor(returns[0].textvalue);
        const float eps = (has_eps && args.size() > 2) ? var_f32(2, mem) : 0.f;
        if (A->shape.dtype != B->shape.dtype || M->shape.dtype != P_BOOL) {
            error = type_mismatch({A->shape.dtype, B->shape.dtype}) + " or " + type_mismatch({A->shape.dtype, M->shape.dtype});
            return 1;
        }
        Rowwise rw(mem, {A, B}, M);
        dx_check(dx_ew_compare(op, A->dx(), rw.ptr[0], rw.ptr[1], eps, rw.ptr[2], rw.n, mem.stream()));
        rw.finish();
        return 0;
    }
};

struct CompareScalarTF : TF {
    int op;
    bool has_eps;
    std::string formula;
    CompareScalarTF(const char *nm, int op_, bool eps, const char *formula_, std::vector<Param> a, std::vector<Param> r)
        : op(op_), has_eps(eps), formula(formula_) { name = nm; metadata.author = "miaobyte"; tftype = "elementwise"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(CompareScalarTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({args[0].textvalue, returns[0].textvalue}, mem, error)) return 1;
        auto A = mem.get_tensor(args[0].textvalue), M = mem.get_tensor(returns[0].textvalue);
        const float eps = (has_eps && args.size() > 2) ? var_f32(2, mem) : 0.f;
        if (M->shape.dtype != P_BOOL) { error = type_mismatch({A->shape.dtype, M->shape.dtype}); return 1; }
        Rowwise rw(mem, {A}, M);
        const Scalar s = scalar_for(*this, 1, mem);
        dx_check(dx_ew_compare_scalar(op, A->dx(), rw.ptr[0], s.f, s.i, eps, rw.ptr[1], rw.n, mem.stream()));
        rw.finish();
        return 0;
    }
};

struct SwitchTF : TF {  // tf/elementwise_compare.hpp:813-939
    std::string formula = "C=switch(tensors,cases)";
    SwitchTF(std::vector<Param> a, std::vector<Param> r) { name = "switch"; metadata.author = "miaobyte"; tftype = "elementwise"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(SwitchTF)
    int run(Mem &mem, std::string &error) override {
        auto C = mem.get_tensor(returns[0].textvalue);
        auto cases = mem.get_tensor(args[1].textvalue);
        std::vector<TensorPtr> sources;
        for (const auto &n : vector_text(0)) {
            if (!mem.exists_tensor(n)) { std::cerr << "tensor not found: " << n << std::endl; continue; }  // gettensors, mem.hpp:134-151
            auto t = mem.get_tensor(n);
            if (t->shape.dtype != C->shape.dtype) { error = type_mismatch({t->shape.dtype, C->shape.dtype}); return 1; }
            if (!mem.shard.active() && t->shape.size != C->shape.size) throw std::invalid_argument("shape mismatch");
            sources.push_back(t);
        }
        if (cases->shape.dtype == P_BOOL && sources.size() != 2) throw std::invalid_argument("For bool cases, tensors size must be 2");
        std::vector<const void *> ptrs;
        const void *cases_ptr;
        void *out_ptr;
        int64_t count;
        if (!mem.shard.active()) {  // the reference compares element counts only for the sources, shapes for the cases
            if (cases->shape.shape != C->shape.shape) throw std::invalid_argument("shape mismatch");
            for (const auto &t : sources) ptrs.push_back(t->data);
            cases_ptr = cases->data;
            out_ptr = C->data;
            count = C->shape.size;
            dx_check(dx_switch(C->dx(), ptrs.data(), int(ptrs.size()), cases->dx(), cases_ptr, out_ptr, count, mem.stream()));
            return 0;
        }
        std::vector<TensorPtr> inputs = sources;
        inputs.push_back(cases);
        Rowwise rw(mem, inputs, C);
        for (size_t i = 0; i < sources.size(); ++i) ptrs.push_back(rw.ptr[i]);
        dx_check(dx_switch(C->dx(), ptrs.data(), int(ptrs.size()), cases->dx(), rw.ptr[sources.size()], rw.ptr.back(), rw.n, mem.stream()));
        rw.finish();
        return 0;
    }
};

struct TodtypeTF : TF {  // tf/elementwise_basic.hpp:13-362
    std::string formula = "T3(dtypeA)->T1(dtypeB)";
    TodtypeTF(std::vector<Param> a, std::vector<Param> r) { name = "todtype"; tftype = "elementwise"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(TodtypeTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({args[0].textvalue, returns[0].textvalue}, mem, error)) return 1;
        auto A = mem.get_tensor(args[0].textvalue), C = mem.get_tensor(returns[0].textvalue);
        if (!A->partitioned() && !C->partitioned()) {
            if (A->shape.size != C->shape.size) {
                error = "Shape mismatch: " + std::to_string(A->shape.size) + " != " + std::to_string(C->shape.size);
                return 1;
            }
            dx_check(dx_cast(A->dx(), A->data, C->dx(), C->data, A->shape.size, mem.stream()));
            return 0;
        }
        Rowwise rw(mem, {A}, C);  // a cast changes the bytes per element: one side can be partitioned and the other not
        dx_check(dx_cast(A->dx(), rw.ptr[0], C->dx(), rw.ptr[1], rw.n, mem.stream()));
        rw.finish();
        return 0;
    }
};

// ---- reduce (tf/reduce.hpp) -------------------------------------------------------------------------
struct ReduceTF : TF {
    int op;
    std::string formula;
    ReduceTF(const char *nm, int op_, const char *formula_, std::vector<Param> a, std::vector<Param> r)
        : op(op_), formula(formula_) { name = nm; metadata.author = "miaobyte"; tftype = "reduce"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(ReduceTF)
    int run(Mem &mem, std::string &error) override {
        auto A = mem.get_tensor(args[0].textvalue);
        const std::vector<int> dims = vector_int(1);
        const bool keepdims = var_bool(2);
        auto B = mem.get_tensor(returns[0].textvalue);
        if (A->shape.dtype != B->shape.dtype) { error = type_mismatch({A->shape.dtype, B->shape.dtype}); return 1; }
        const std::vector<int64_t> ag = A->global_shape();
        const std::vector<int> cd = checked_dims(ag, dims);
        const ReducePlan plan = plan_reduce(A->layout(), cd, keepdims, B->layout(), dx_comm_max_bytes());
        if (plan.kind == ReducePlan::REFUSE) throw TensorShapeError(name + ": " + plan.error);
        if (A->data == B->data && A->shape.size != B->shape.size) {
            error = name + ": output tensor is the input tensor";
            return 1;
        }
        const int nd = A->shape.dim();
        const int64_t *shp = A->shape.shape.data();  // the local rows of a partitioned input
        const size_t need = dx_reduce_workspace_bytes(op, A->dx(), shp, nd, cd.data(), int(cd.size()));
        void *ws = need ? mem.scratch(need) : nullptr;
        void *st = mem.stream();
        dx_comm *comm = mem.shard.comm;
        switch (plan.kind) {
            case ReducePlan::WHOLE:
            case ReducePlan::ROWS:  // the output's rows follow the input's partition: nothing to exchange
                dx_check(dx_reduce(op, A->dx(), A->data, shp, nd, cd.data(), int(cd.size()), B->data, ws, need, st));
                break;
            case ReducePlan::ROWS_GATHER: {  // replicated output: this rank's rows of it, then the other ranks' blocks
                void *mine = static_cast<char *>(B->data) + A->row0 * B->row_bytes();
                dx_check(dx_reduce(op, A->dx(), A->data, shp, nd, cd.data(), int(cd.size()), mine, ws, need, st));
                dx_check(dx_comm_allgather_rows(comm, B->data, B->shape.shape[0], B->row_bytes(), st));
                break;
            }
            case ReducePlan::COMBINE_DEFERRED:
                // reduce + publish in one go; the wait for the peers and the combine run when B is next needed
                dx_check(dx_reduce_allreduce_begin(comm, op, A->dx(), A->data, shp, nd, cd.data(), int(cd.size()), B->data, ws, need, st));
                break;
            case ReducePlan::COMBINE_ROUNDS:
                dx_check(dx_reduce(op, A->dx(), A->data, shp, nd, cd.data(), int(cd.size()), B->data, ws, need, st));
                dx_check(dx_comm_allreduce(comm, op, A->dx(), B->data, B->shape.size, st));
                break;
            case ReducePlan::COMBINE_SCATTER: {
                // the result is itself partitioned: combine the whole partial in a temporary, keep this rank's rows
                if (mem.capturing) throw std::runtime_error("a reduction into a row-partitioned output needs a temporary, which a captured program cannot hold");
                int64_t total = 1;
                for (auto v : plan.out_global) total *= v;
                const size_t es = size_t(precision_bits(A->shape.dtype) / 8);
                void *tmp = dx_pool_alloc(mem.pool(), std::max<size_t>(size_t(total) * es, 1));
                if (!tmp) throw std::runtime_error(dx_last_error());
                int rc = dx_reduce(op, A->dx(), A->data, shp, nd, cd.data(), int(cd.size()), tmp, ws, need, st);
                if (rc == DX_OK) rc = dx_comm_allreduce(comm, op, A->dx(), tmp, total, st);
                if (rc == DX_OK && B->shape.bytes() > 0)
                    cudaMemcpyAsync(B->data, static_cast<char *>(tmp) + B->row0 * B->row_bytes(), size_t(B->shape.bytes()), cudaMemcpyDeviceToDevice,
                                    static_cast<cudaStream_t>(st));
                dx_pool_free(mem.pool(), tmp);  // reuse is ordered behind the copy on the one compute stream
                dx_check(rc);
                break;
            }
            default: break;
        }
        return 0;
    }
};

// ---- changeshape (tf/changeshape.hpp) -----------------------------------------------------------------
// An op whose output names its input would race in place in the reference; here it is staged
// through a pool temporary so the result is defined.
struct Staged {
    Mem &mem;
    TensorPtr out;
    void *tmp = nullptr;
    Staged(Mem &m, TensorPtr o, bool aliased) : mem(m), out(std::move(o)) {
        if (aliased && mem.capturing) throw std::runtime_error("an op whose output is also its input needs a temporary, which a captured program cannot hold");
        if (aliased) {
            tmp = dx_pool_alloc(mem.pool(), size_t(std::max<int64_t>(out->shape.bytes(), 1)));
            if (!tmp) throw std::runtime_error(dx_last_error());
        }
    }
    void *dst() const { return tmp ? tmp : out->data; }
    void commit() {
        if (!tmp) return;
        cudaMemcpyAsync(out->data, tmp, size_t(out->shape.bytes()), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(mem.stream()));
    }
    ~Staged() { if (tmp) dx_pool_free(mem.pool(), tmp); }  // reuse is ordered behind the copy on the one compute stream
};

struct ReshapeTF : TF {  // :17-83; tensorfunc changeshape_miaobyte.hpp:17-42
    std::string formula = "T1.reshape(shape)->T2";
    ReshapeTF(std::vector<Param> a, std::vector<Param> r) { name = "reshape"; metadata.author = "miaobyte"; tftype = "changeshape"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(ReshapeTF)
    int run(Mem &mem, std::string &error) override {
        auto A = mem.get_tensor(args[0].textvalue);
        std::vector<int64_t> ns = vector_i64(1);
        auto B = mem.get_tensor(returns[0].textvalue);
        if (A->shape.dtype != B->shape.dtype) { error = type_mismatch({A->shape.dtype, B->shape.dtype}); return 1; }
        if (A->partitioned() || B->partitioned()) {
            // the rows stay where they are only if the new shape keeps the leading axis
            if (!A->partitioned() || !B->partitioned() || A->global_rows != B->global_rows || ns.empty() || ns[0] != A->global_rows)
                throw std::runtime_error("reshape: a row-partitioned tensor can only be reshaped to a shape with the same leading axis (" +
                                         std::to_string(A->partitioned() ? A->global_rows : B->global_rows) + " rows)");
            ns[0] = A->shape.shape[0];  // the local rows
        }
        int64_t prod = 1;
        for (auto v : ns) prod *= v;
        if (A->shape.size != prod) throw std::invalid_argument("Shape size mismatch");
        const uint16_t dt = B->shape.dtype;
        if (A->data != B->data) {
            if (B->shape.size != prod) throw std::invalid_argument("Shape size mismatch");
            cudaMemcpyAsync(B->data, A->data, size_t(A->shape.bytes()), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(mem.stream()));
        }
        B->shape.set(ns);  // the only op that rewrites a tensor's shape metadata
        B->shape.dtype = dt;
        return 0;
    }
};

struct TransposeTF : TF {  // :85-152
    std::string formula = "T2 = T1.transpose(dimorder=[1,0])";
    TransposeTF(std::vector<Param> a, std::vector<Param> r) { name = "transpose"; metadata.author = "miaobyte"; tftype = "changeshape"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(TransposeTF)
    int run(Mem &mem, std::string &error) override {
        auto A = mem.get_tensor(args[0].textvalue);
        const std::vector<int> order = vector_int(1);
        auto C = mem.get_tensor(returns[0].textvalue);
        if (A->shape.dtype != C->shape.dtype) { error = type_mismatch({A->shape.dtype, C->shape.dtype}); return 1; }
        if (int(order.size()) != A->shape.dim()) throw std::invalid_argument("dimOrder size does not match the number of dimensions in the TensorCPU.");
        if (A->partitioned() || C->partitioned()) {
            if (!(A->partitioned() && C->partitioned() && A->global_rows == C->global_rows && order[0] == 0)) refuse_partitioned("transpose (an order that moves axis 0)", {A, C});
        }
        if (C->shape.size != A->shape.size) throw std::runtime_error("transpose error!shape");
        Staged st(mem, C, A->data == C->data);
        dx_check(dx_transpose(A->dx(), A->data, A->shape.shape.data(), A->shape.dim(), order.data(), st.dst(), mem.stream()));
        st.commit();
        return 0;
    }
};

struct ConcatTF : TF {  // :154-287
    std::string formula = "Tresult = concat([T1, T2...], axis=3)";
    ConcatTF(std::vector<Param> a, std::vector<Param> r) { name = "concat"; metadata.author = "miaobyte"; tftype = "changeshape"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(ConcatTF)
    int run(Mem &mem, std::string &error) override {
        const std::vector<std::string> names = vector_text(0);
        if (!check_tensors(names, mem, error)) return 1;
        if (!check_tensors({returns[0].textvalue}, mem, error)) return 1;
        auto C = mem.get_tensor(returns[0].textvalue);
        int axis = var_int(1, mem);
        const int nd = C->shape.dim();
        if (axis < 0) axis += nd;
        if (axis < 0 || axis >= nd) throw TensorShapeError("concat axis out of range");
        std::vector<const void *> ptrs;
        std::vector<int64_t> lens;
        bool aliased = false;
        int64_t total = 0;
        for (const auto &n : names) {
            auto t = mem.get_tensor(n);
            if (t->partitioned() != C->partitioned() || (C->partitioned() && (axis == 0 || t->global_rows != C->global_rows)))
                refuse_partitioned("concat (along axis 0, or of tensors that are not all partitioned alike)", {t->partitioned() ? t : C});
            if (t->shape.dtype != C->shape.dtype) { error = type_mismatch({t->shape.dtype, C->shape.dtype}); return 1; }
            if (t->shape.dim() != nd) throw TensorShapeError("All input tensors must have the same dimension size for concat");
            for (int j = 0; j < nd; ++j)
                if (j != axis && t->shape.shape[j] != C->shape.shape[j])
                    throw TensorShapeError("All input tensors must have the same dimension size for concat");
            total += t->shape.shape[axis];
            ptrs.push_back(t->data);
            lens.push_back(t->shape.shape[axis]);
            aliased = aliased || t->data == C->data;
        }
        if (total != C->shape.shape[axis])
            throw TensorShapeError("Output tensor shape size must match the sum of input tensor shape sizes for concat");
        Staged st(mem, C, aliased);
        dx_check(dx_concat(C->dx(), ptrs.data(), lens.data(), int(ptrs.size()), C->shape.shape.data(), nd, axis, st.dst(), mem.stream()));
        st.commit();
        return 0;
    }
};

struct BroadcastToTF : TF {  // :289-353
    std::string formula = "T2 = T1.broadcastTo(new_shape=[4,3,2])";
    BroadcastToTF(std::vector<Param> a, std::vector<Param> r) { name = "broadcastTo"; metadata.author = "miaobyte"; tftype = "changeshape"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(BroadcastToTF)
    int run(Mem &mem, std::string &error) override {
        auto A = mem.get_tensor(args[0].textvalue);
        std::vector<int64_t> ns = vector_i64(1);
        auto B = mem.get_tensor(returns[0].textvalue);
        if (A->shape.dtype != B->shape.dtype) { error = type_mismatch({A->shape.dtype, B->shape.dtype}); return 1; }
        if (A->partitioned() || B->partitioned()) {
            // rows of the output come from the same rows of a partitioned source, or from a source that has no axis 0 of its own
            const bool source_ok = A->partitioned() ? (A->shape.dim() == int(ns.size()) && !ns.empty() && A->global_rows == ns[0])
                                                    : (A->shape.dim() < int(ns.size()) || (A->shape.dim() > 0 && A->shape.shape[0] == 1));
            if (!B->partitioned() || ns.empty() || B->global_rows != ns[0] || !source_ok) refuse_partitioned("broadcastTo (source and output rows do not line up)", {A, B});
            ns[0] = B->shape.shape[0];
        }
        const auto bs = broadcast_shape(A->shape.shape, ns);
        if (bs.empty() || bs != ns || B->shape.shape != ns) throw TensorShapeError("Broadcast shape mismatch");
        Staged st(mem, B, A->data == B->data);
        dx_check(dx_broadcast_to(A->dx(), A->data, A->shape.shape.data(), A->shape.dim(), ns.data(), int(ns.size()), st.dst(), mem.stream()));
        st.commit();
        return 0;
    }
};

struct IndexSelectTF : TF {  // :355-499
    std::string formula = "T2 = T1.indexselect(index=T3, axis=3)";
    IndexSelectTF(std::vector<Param> a, std::vector<Param> r) { name = "indexselect"; metadata.author = "miaobyte"; tftype = "changeshape"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(IndexSelectTF)
    int run(Mem &mem, std::string &error) override {
        auto A = mem.get_tensor(args[0].textvalue), I = mem.get_tensor(args[1].textvalue), B = mem.get_tensor(returns[0].textvalue);
        const int axis_in = var_int(2, mem);
        if (A->shape.dtype != B->shape.dtype) {
            error = "output_type " + precision_str(B->shape.dtype) + " or input_type " + precision_str(A->shape.dtype) + " must be the same";
            return 1;
        }
        if (I->shape.dtype != P_I64 && I->shape.dtype != P_I32) {
            error = "index_type " + precision_str(I->shape.dtype) + " only support " + precision_str(P_I64) + " or " + precision_str(P_I32);
            return 1;
        }
        const int axis = axis_in < 0 ? axis_in + A->shape.dim() : axis_in;
        if (axis < 0 || axis >= A->shape.dim()) throw std::invalid_argument("Axis is out of bounds");
        if (A->partitioned() || I->partitioned() || B->partitioned()) {
            // rows of a replicated table picked by a partitioned index, or positions along an inner axis of a partitioned table
            const bool by_index_rows = axis == 0 && !A->partitioned() && I->partitioned() && B->partitioned() && I->global_rows == B->global_rows;
            const bool by_table_rows = axis > 0 && A->partitioned() && !I->partitioned() && B->partitioned() && A->global_rows == B->global_rows;
            if (!by_index_rows && !by_table_rows) refuse_partitioned("indexselect (operands whose rows do not line up)", {A, I, B});
        }
        if (indexselect_shape(A->shape.shape, I->shape.shape, axis) != B->shape.shape) throw TensorShapeError("Indexselect shape mismatch");
        Staged st(mem, B, A->data == B->data);
        dx_check(dx_indexselect(A->dx(), A->data, A->shape.shape.data(), A->shape.dim(), I->dx(), I->data, I->shape.shape.data(),
                                I->shape.dim(), axis, st.dst(), nullptr, mem.stream()));
        st.commit();
        return 0;
    }
};

struct RepeatTF : TF {  // :501-566
    std::string formula = "T2 = T1.repeat(repeats=[4,3,2])";
    RepeatTF(std::vector<Param> a, std::vector<Param> r) { name = "repeat"; metadata.author = "miaobyte"; tftype = "changeshape"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(RepeatTF)
    int run(Mem &mem, std::string &error) override {
        auto A = mem.get_tensor(args[0].textvalue);
        const std::vector<int64_t> r64 = vector_i64(1);
        auto B = mem.get_tensor(returns[0].textvalue);
        if (A->shape.dtype != B->shape.dtype) { error = type_mismatch({A->shape.dtype, B->shape.dtype}); return 1; }
        if (A->partitioned() || B->partitioned()) {
            if (!(A->partitioned() && B->partitioned() && !r64.empty() && r64[0] == 1 && A->global_rows == B->global_rows)) refuse_partitioned("repeat (along axis 0)", {A, B});
        }
        if (repeat_shape(A->shape.shape, r64) != B->shape.shape) throw TensorShapeError("Repeat shape mismatch");
        Staged st(mem, B, A->data == B->data);
        dx_check(dx_repeat(A->dx(), A->data, A->shape.shape.data(), A->shape.dim(), r64.data(), st.dst(), mem.stream()));
        st.commit();
        return 0;
    }
};

// ---- matmul (tf/matmul.hpp:15-76) ---------------------------------------------------------------------------
struct MatMulTF : TF {
    std::string formula = "T3=T1 @ T2";
    MatMulTF(std::vector<Param> a, std::vector<Param> r) { name = "matmul"; metadata.author = "cublas"; tftype = "matmul"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(MatMulTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({args[0].textvalue, args[1].textvalue, returns[0].textvalue}, mem, error)) return 1;
        auto A = mem.get_tensor(args[0].textvalue), B = mem.get_tensor(args[1].textvalue), C = mem.get_tensor(returns[0].textvalue);
        if (A->shape.dtype != B->shape.dtype || A->shape.dtype != C->shape.dtype) {
            error = type_mismatch({A->shape.dtype, B->shape.dtype, C->shape.dtype});
            return 1;
        }
        if (A->partitioned() || B->partitioned() || C->partitioned()) {
            // rows of A against a replicated B (2-D), or whole matrices of a batch partitioned along its leading axis
            const bool by_rows = A->shape.dim() == 2 && A->partitioned() && !B->partitioned() && C->partitioned() && A->global_rows == C->global_rows;
            const bool by_batch = A->shape.dim() > 2 && A->partitioned() && B->partitioned() && C->partitioned() && A->global_rows == B->global_rows &&
                                  A->global_rows == C->global_rows;
            if (!by_rows && !by_batch) refuse_partitioned("matmul (operands whose rows do not line up)", {A, B, C});
        }
        if (!check_matmul_shape(A->shape.shape, B->shape.shape)) throw std::invalid_argument("A.shape could matmul with B.shape");
        const int64_t m = A->shape.at(-2), k = A->shape.at(-1), n = B->shape.at(-1);
        const int64_t batch = (m * k) ? A->shape.size / (m * k) : 0;
        if (C->shape.size != batch * m * n) throw std::invalid_argument("shape mismatch");
        if (C->data == A->data || C->data == B->data) { error = "matmul: output tensor is an input tensor"; return 1; }
        // a few rows of tiles: the K range is split over independent CTA pairs through scratch memory
        // (a captured program keeps using the path it was captured with: the scratch cannot grow then)
        size_t need = dx_matmul_workspace_bytes(A->dx(), batch, m, n, k);
        void *ws = nullptr;
        if (need) {
            try {
                ws = mem.scratch(need);
            } catch (const std::exception &) {
                ws = nullptr;  // no room (or capturing): the kernels that need no scratch
                need = 0;
            }
        }
        dx_check(dx_matmul_ws(A->dx(), A->data, B->data, C->data, batch, m, n, k, ws, need, mem.stream()));
        return 0;
    }
};

// ---- tensor lifetime (tf/tensorlife.hpp) ----------------------------------------------------------------------
struct NewTensorTF : TF {
    std::string formula = "T1 = zeros(shape)";
    NewTensorTF(std::vector<Param> a, std::vector<Param> r) { name = "newtensor"; tftype = "tensorlife"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(NewTensorTF)
    int run(Mem &mem, std::string &error) override {
        const TypeDef type = returns[0].dtype;
        if ((type.category & CAT_TENSOR) == 0) { error = "newtensor: return type must include tensor category"; return 1; }
        const std::vector<int64_t> shp = vector_i64(0);
        for (int64_t d : shp)
            if (d < 0) { error = "newtensor: negative extent"; return 1; }
        switch (type.precision) {
            case P_F8E5M2: error = "newtensor: Float8E5M2 has not been implemented,if you need it, please contact the author"; return 1;
            case P_F8E4M3: error = "newtensor: Float8E4M3 has not been implemented,if you need it, please contact the author"; return 1;
            case P_F4E2M1: error = "newtensor: Float4E2M1 has not been implemented,if you need it, please contact the author"; return 1;
            case P_I4: error = "newtensor: Int4 has not been implemented,if you need it, please contact the author"; return 1;
            default: break;
        }
        if (dx_code_of(type.precision) < 0) { error = "newtensor: unsupported precision"; return 1; }
        mem.new_tensor(returns[0].textvalue, type.precision, shp);  // one allocation, no copy
        return 0;
    }
};

struct CopyTensorTF : TF {
    std::string formula = "T2.data = T1.data";
    CopyTensorTF(std::vector<Param> a, std::vector<Param> r) { name = "copytensor"; tftype = "tensorlife"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(CopyTensorTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({args[0].textvalue, returns[0].textvalue}, mem, error)) return 1;
        auto S = mem.get_tensor(args[0].textvalue), D = mem.get_tensor(returns[0].textvalue);
        if (S->shape.dtype != D->shape.dtype) { error = "copytensor: input type and return type must be the same"; return 1; }
        if (S->partitioned() || D->partitioned()) {
            Rowwise rw(mem, {S}, D);
            if (rw.ptr[0] != rw.ptr[1] && rw.n > 0)
                cudaMemcpyAsync(rw.ptr[1], rw.ptr[0], size_t(rw.n) * size_t(precision_bits(S->shape.dtype) / 8), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(mem.stream()));
            rw.finish();
            return 0;
        }
        if (D->shape.size < S->shape.size) { error = "copytensor: destination is smaller than the source"; return 1; }
        if (S->data != D->data)
            cudaMemcpyAsync(D->data, S->data, size_t(S->shape.bytes()), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(mem.stream()));
        return 0;
    }
};

struct DelTensorTF : TF {
    std::string formula = "del->T1";
    DelTensorTF(std::vector<Param> a, std::vector<Param> r) { name = "deltensor"; tftype = "tensorlife"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(DelTensorTF)
    int run(Mem &mem, std::string &) override { mem.delete_tensor(returns[0].textvalue); return 0; }
};

struct RenameTensorTF : TF {
    std::string formula = "rename(newname)->T1";
    RenameTensorTF(std::vector<Param> a, std::vector<Param> r) { name = "renametensor"; tftype = "tensorlife"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(RenameTensorTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({returns[0].textvalue}, mem, error)) return 1;
        mem.rename_tensor(returns[0].textvalue, args[0].textvalue);
        return 0;
    }
};

// ---- args (tf/arg.hpp) --------------------------------------------------------------------------------------------
struct ArgSetTF : TF {
    std::string formula = "argvalue->argname";
    ArgSetTF(std::vector<Param> a, std::vector<Param> r) { name = "argset"; tftype = "arg"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(ArgSetTF)
    int run(Mem &mem, std::string &error) override {
        if (args.size() != 1) { error = "argset(int32) must have 1 argument"; return 1; }
        const TypeDef t = returns[0].dtype;
        if ((t.category & CAT_VAR) == 0) { error = "datatype must be var"; return 1; }
        const std::string &v = args[0].textvalue;
        switch (t.precision) {
            case P_I32: mem.add_arg(returns[0].textvalue, ArgValue(atoi(v.c_str()))); break;
            case P_F32: mem.add_arg(returns[0].textvalue, ArgValue(std::stof(v))); break;
            case P_F64: mem.add_arg(returns[0].textvalue, ArgValue(std::stod(v))); break;
            default: error = "Unsupportednone dtype: " + typedef_str(args[0].dtype); return 1;
        }
        return 0;
    }
};

struct VecSetTF : TF {
    std::string formula = "[3  4  5]->shape";
    VecSetTF(std::vector<Param> a, std::vector<Param> r) { name = "vecset"; tftype = "arg"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(VecSetTF)
    int run(Mem &mem, std::string &error) override {
        const TypeDef t = returns[0].dtype;
        if ((t.category & CAT_VECTOR) == 0) { error = "datatype must be vector"; return 1; }
        const std::vector<std::string> items = vector_text(0);
        switch (t.precision) {
            case P_I32: { std::vector<int> v; for (auto &s : items) if (!s.empty()) v.push_back(std::stoi(s)); mem.add_arg(returns[0].textvalue, ArgValue(v)); break; }
            case P_F32: { std::vector<float> v; for (auto &s : items) if (!s.empty()) v.push_back(std::stof(s)); mem.add_arg(returns[0].textvalue, ArgValue(v)); break; }
            case P_F64: { std::vector<double> v; for (auto &s : items) if (!s.empty()) v.push_back(std::stod(s)); mem.add_arg(returns[0].textvalue, ArgValue(v)); break; }
            default: error = "Unsupported dtype: " + typedef_str(t); return 1;
        }
        return 0;
    }
};

// ---- init (tf/init.hpp) ---------------------------------------------------------------------------------------------
struct InitTF : TF {
    enum Kind { CONSTANT, ARANGE, UNIFORM, NORMAL, DROPOUT } kind;
    std::string formula;
    InitTF(const char *nm, Kind k, const char *formula_, std::vector<Param> a, std::vector<Param> r)
        : kind(k), formula(formula_) { name = nm; metadata.author = "miaobyte"; tftype = "init"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(InitTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({returns[0].textvalue}, mem, error)) return 1;
        auto T = mem.get_tensor(returns[0].textvalue);
        void *st = mem.stream();
        switch (kind) {
            case CONSTANT: {
                if (T->shape.dtype == P_BOOL) {
                    dx_check(dx_fill(DX_BOOL, T->data, 0.0, var_bool(0) ? 1 : 0, T->shape.size, st));
                } else {
                    const Scalar s = scalar_for(*this, 0, mem);
                    dx_check(dx_fill(T->dx(), T->data, s.f, s.i, T->shape.size, st));
                }
                break;
            }
            case ARANGE: {
                // a partitioned tensor continues the sequence where its first local element sits
                const double start = var_f32(0, mem), step = var_f32(1, mem);
                const double first = T->partitioned() && T->shape.shape[0] > 0 ? double(T->row0) * double(T->shape.size / T->shape.shape[0]) : 0.0;
                dx_check(dx_arange(T->dx(), T->data, start + step * first, step, T->shape.size, st));
                break;
            }
            case UNIFORM: refuse_partitioned(name + " (the random stream is per tensor, not per row block)", {T}); dx_check(dx_uniform(T->dx(), T->data, var_f32(0, mem), var_f32(1, mem), uint64_t(uint32_t(var_int(2, mem))), T->shape.size, st)); break;
            case NORMAL: refuse_partitioned(name + " (the random stream is per tensor, not per row block)", {T}); dx_check(dx_normal(T->dx(), T->data, var_f32(0, mem), var_f32(1, mem), uint64_t(uint32_t(var_int(2, mem))), T->shape.size, st)); break;
            case DROPOUT: refuse_partitioned(name + " (the random stream is per tensor, not per row block)", {T}); dx_check(dx_dropout(T->dx(), T->data, var_f32(0, mem), uint64_t(uint32_t(var_int(1, mem))), T->shape.size, st)); break;
        }
        return 0;
    }
};

// ---- io (tf/io.hpp) -----------------------------------------------------------------------------------------------------
std::vector<char> download(Mem &mem, const Tensor &t) {
    std::vector<char> host(size_t(std::max<int64_t>(t.shape.bytes(), 0)));
    cudaStream_t st = static_cast<cudaStream_t>(mem.stream());
    if (!host.empty()) {
        cudaError_t e = cudaMemcpyAsync(host.data(), t.data, host.size(), cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) throw std::runtime_error(std::string("device to host copy failed: ") + cudaGetErrorString(e));
    }
    return host;
}

float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FF;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) u = sign;
        else {
            int e = -1;
            uint32_t m = man;
            do { ++e; m <<= 1; } while ((m & 0x400) == 0);
            u = sign | ((127 - 15 - e) << 23) | ((m & 0x3FF) << 13);
        }
    } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
    else u = sign | ((exp - 15 + 127) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

}  // namespace

// The print format arrives in a datagram and would be handed to printf: only a format with exactly one
// numeric conversion is accepted (flags, width, precision, one of d i u x X o for integer and bool
// tensors, f F e E g G for floating ones; "%%" is literal text).  %s, %n, %c, %p, '*' widths and a second
// conversion are refused.  Whatever length modifier the caller wrote is replaced by the one that matches
// what print_element passes (long long for int64, int otherwise, double for floats), so the argument
// always has the type the conversion reads.  The reference passes the text through unchecked
// (executor/deepxcore/src/stdutil/print.hpp:13-57).
bool checked_print_format(const std::string &fmt, uint16_t dtype, std::string &out, std::string &error) {
    const bool is_float = (dtype & P_FLOAT) != 0;
    out.clear();
    int conversions = 0;
    for (size_t i = 0; i < fmt.size(); ++i) {
        if (fmt[i] != '%') { out += fmt[i]; continue; }
        if (i + 1 < fmt.size() && fmt[i + 1] == '%') { out += "%%"; ++i; continue; }
        size_t j = i + 1;
        while (j < fmt.size() && std::strchr("-+ #0", fmt[j])) ++j;
        while (j < fmt.size() && std::isdigit(static_cast<unsigned char>(fmt[j]))) ++j;
        if (j < fmt.size() && fmt[j] == '.') {
            ++j;
            while (j < fmt.size() && std::isdigit(static_cast<unsigned char>(fmt[j]))) ++j;
        }
        const size_t spec_end = j;  // flags, width, precision
        while (j < fmt.size() && std::strchr("hlLqjzt", fmt[j])) ++j;
        if (j >= fmt.size()) { error = "print: incomplete conversion in format '" + fmt + "'"; return false; }
        const char conv = fmt[j];
        const bool int_conv = std::strchr("diuxXo", conv) != nullptr, float_conv = std::strchr("fFeEgG", conv) != nullptr;
        if (!int_conv && !float_conv) { error = std::string("print: conversion '%") + conv + "' is not allowed (numeric conversions only)"; return false; }
        if (int_conv == is_float) { error = std::string("print: conversion '%") + conv + "' does not fit a " + precision_str(dtype) + " tensor"; return false; }
        if (++conversions > 1) { error = "print: the format must hold exactly one conversion"; return false; }
        if (spec_end - i > 10) { error = "print: width or precision too long"; return false; }
        out += fmt.substr(i, spec_end - i);
        if (int_conv && dtype == P_I64) out += "ll";
        out += conv;
        i = j;
    }
    if (conversions != 1) { error = "print: the format must hold exactly one conversion"; return false; }
    return true;
}

namespace {

void print_element(const char *data, int64_t i, uint16_t dtype, const std::string &fmt) {  // stdutil/print.hpp:13-57
    switch (dtype) {
        case P_BOOL: std::printf(fmt.c_str(), int(reinterpret_cast<const uint8_t *>(data)[i])); break;
        case P_I8: std::printf(fmt.c_str(), int(reinterpret_cast<const int8_t *>(data)[i])); break;
        case P_I16: std::printf(fmt.c_str(), int(reinterpret_cast<const int16_t *>(data)[i])); break;
        case P_I32: std::printf(fmt.c_str(), reinterpret_cast<const int32_t *>(data)[i]); break;
        case P_I64: std::printf(fmt.c_str(), (long long)reinterpret_cast<const int64_t *>(data)[i]); break;
        case P_F64: std::printf(fmt.c_str(), reinterpret_cast<const double *>(data)[i]); break;
        case P_F32: std::printf(fmt.c_str(), double(reinterpret_cast<const float *>(data)[i])); break;
        case P_F16: std::printf(fmt.c_str(), double(half_bits_to_float(reinterpret_cast<const uint16_t *>(data)[i]))); break;
        case P_BF16: {
            uint32_t u = uint32_t(reinterpret_cast<const uint16_t *>(data)[i]) << 16;
            float f;
            std::memcpy(&f, &u, 4);
            std::printf(fmt.c_str(), double(f));
            break;
        }
        default: break;
    }
}

struct PrintTF : TF {  // tf/io.hpp:17-99, layout of stdutil/print.hpp:84-129
    std::string formula = "print(T1)";
    PrintTF(std::vector<Param> a, std::vector<Param> r) { name = "print"; metadata.author = "miaobyte"; tftype = "io"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(PrintTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({args[0].textvalue}, mem, error)) return 1;
        auto T = mem.get_tensor(args[0].textvalue);
        std::string asked = args.size() > 1 ? args[1].textvalue : "";
        if (asked.empty()) asked = (T->shape.dtype & P_FLOAT) ? "%.4f" : "%d";
        std::string fmt;
        if (!checked_print_format(asked, T->shape.dtype, fmt, error)) return 1;
        const std::vector<char> host = download(mem, *T);
        const Shape &s = T->shape;
        if (T->partitioned())
            std::printf("rows %lld..%lld of %lld (rank %d of %d)\n", (long long)T->row0, (long long)(T->row0 + (s.dim() ? s.shape[0] : 0)),
                        (long long)T->global_rows, mem.shard.rank, mem.shard.world);
        std::printf("shape:[");
        for (int i = 0; i < s.dim(); ++i) std::printf("%s%lld", i ? ", " : "", (long long)s.shape[i]);
        std::printf("]\n");
        if (s.dim() <= 1) {
            std::printf("[");
            for (int64_t i = 0; i < s.size; ++i) { if (i) std::printf(" "); print_element(host.data(), i, s.dtype, fmt); }
            std::printf("]\n");
        } else {
            const int64_t rows = s.at(-2), cols = s.at(-1), mats = (rows * cols) ? s.size / (rows * cols) : 0;
            for (int64_t m = 0; m < mats; ++m) {
                std::printf("[");
                int64_t rem = m;
                std::vector<int64_t> idx(s.dim() - 2);
                for (int d = s.dim() - 3; d >= 0; --d) { idx[d] = rem % s.shape[d]; rem /= s.shape[d]; }
                for (size_t d = 0; d < idx.size(); ++d) std::printf("%s%lld", d ? ", " : "", (long long)idx[d]);
                std::printf("]=[\n");
                for (int64_t i = 0; i < rows; ++i) {
                    std::printf(" [");
                    for (int64_t j = 0; j < cols; ++j) { if (j) std::printf(" "); print_element(host.data(), (m * rows + i) * cols + j, s.dtype, fmt); }
                    std::printf("]%s\n", i < rows - 1 ? "," : "");
                }
                std::printf("]\n");
            }
        }
        std::fflush(stdout);
        return 0;
    }
};

std::string file_stem(const std::string &path) {  // stdutil::filename + strip extension (shape.cpp:138-141)
    const size_t slash = path.find_last_of('/');
    const std::string file = slash == std::string::npos ? path : path.substr(slash + 1);
    return file.substr(0, file.find_last_of('.'));
}

void load_data_into(Mem &mem, const std::string &path, Tensor &t) {
    std::ifstream in(path + ".data", std::ios::binary);
    if (!in.is_open()) throw std::runtime_error("Failed to open file: " + path + ".data");
    std::vector<char> host(size_t(t.shape.bytes()));
    if (t.partitioned()) in.seekg(std::streamoff(t.row0 * t.row_bytes()));  // this rank's rows of the file a single GPU would read whole
    in.read(host.data(), std::streamsize(host.size()));
    if (size_t(in.gcount()) != host.size()) throw std::runtime_error("file size mismatch: " + path + ".data");
    cudaStream_t st = static_cast<cudaStream_t>(mem.stream());
    cudaError_t e = cudaMemcpyAsync(t.data, host.data(), host.size(), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) throw std::runtime_error(std::string("host to device copy failed: ") + cudaGetErrorString(e));
}

struct SaveTF : TF {
    std::string formula = "save(T1,path)";
    SaveTF(std::vector<Param> a, std::vector<Param> r) { name = "save"; tftype = "io"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(SaveTF)
    int run(Mem &mem, std::string &error) override {
        const std::string &n = args[0].textvalue, &path = args[1].textvalue;
        if (!mem.exists_tensor(n)) { error = "save " + n + " not found"; return 1; }
        auto T = mem.get_tensor(n);
        const std::vector<char> host = download(mem, *T);
        if (mem.shard.active()) {
            // Every rank runs the same line on a file system they share: the files must come out as a single GPU would
            // write them.  Rank 0 writes the description (of the GLOBAL shape) and sets the data file's size; each rank
            // writes its own rows at their offset (a replicated tensor is written by rank 0 alone).
            Shape g = T->shape;
            if (T->partitioned()) { g.set(T->global_shape()); g.dtype = T->shape.dtype; }
            const int fd = ::open((path + ".data").c_str(), O_WRONLY | O_CREAT, 0644);
            if (fd < 0) { error = "save: cannot write " + path; return 1; }
            bool ok = true;
            if (mem.shard.rank == 0) {
                std::ofstream sf(path + ".shape", std::ios::binary);
                const std::string y = g.to_yaml();
                sf.write(y.data(), std::streamsize(y.size()));
                ok = sf.good() && ::ftruncate(fd, off_t(g.bytes())) == 0;
            }
            if (ok && (T->partitioned() || mem.shard.rank == 0)) {
                const off_t at = T->partitioned() ? off_t(T->row0 * T->row_bytes()) : 0;
                size_t done = 0;
                while (ok && done < host.size()) {
                    const ssize_t w = ::pwrite(fd, host.data() + done, host.size() - done, at + off_t(done));
                    ok = w > 0;
                    done += ok ? size_t(w) : 0;
                }
            }
            ::close(fd);
            if (!ok) { error = "save: cannot write " + path; return 1; }
            return 0;
        }
        std::ofstream sf(path + ".shape", std::ios::binary);
        const std::string y = T->shape.to_yaml();
        sf.write(y.data(), std::streamsize(y.size()));
        std::ofstream df(path + ".data", std::ios::binary);
        df.write(host.data(), std::streamsize(host.size()));
        if (!sf.good() || !df.good()) { error = "save: cannot write " + path; return 1; }
        return 0;
    }
};

struct LoadTF : TF {
    std::string formula = "load(path)";
    LoadTF(std::vector<Param> a, std::vector<Param> r) { name = "load"; tftype = "io"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(LoadTF)
    int run(Mem &mem, std::string &) override {
        const std::string &path = args[0].textvalue;
        std::ifstream sf(path + ".shape", std::ios::binary);
        if (!sf.is_open()) throw std::runtime_error("Failed to open shape file: " + path + ".shape");
        const std::string text((std::istreambuf_iterator<char>(sf)), std::istreambuf_iterator<char>());
        const Shape s = Shape::from_yaml(text);
        const std::string tname = file_stem(path);
        if (mem.exists_tensor(tname)) {
            std::cout << "warning: " << tname << " already exists,deepx will delete it,create new one" << std::endl;
            mem.delete_tensor(tname);
        }
        auto T = mem.new_tensor(tname, s.dtype, s.shape);
        load_data_into(mem, path, *T);
        return 0;
    }
};

struct LoadTensorDataTF : TF {
    std::string formula = "loadtensordata(path)->tensor";
    LoadTensorDataTF(std::vector<Param> a, std::vector<Param> r) { name = "loadtensordata"; tftype = "io"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(LoadTensorDataTF)
    int run(Mem &mem, std::string &error) override {
        const std::string &tname = returns[0].textvalue;
        if (!mem.exists_tensor(tname)) { error = "loadtensordata " + tname + " not found"; return 1; }
        load_data_into(mem, args[0].textvalue, *mem.get_tensor(tname));
        return 0;
    }
};

// ---- fused row chains (no reference counterpart: what the fusion pass rewrites an op chain into) ---------------------
// rmsnorm(x, weight, divisor, eps)->(out) and rmsnorm(x, divisor, eps)->(out) stand for the chain
// powscalar(x,2)|mul(x,x), sum(last,keepdims), divscalar, addscalar, sqrt, rdivscalar(1), broadcastTo, mul
// [, broadcastTo(weight), mul] of front/py/deepx/nn/modules/norm/t5layernorm.py:19-23; softmax(x)->(out)
// for reducemax, broadcastTo, sub, exp, sum, broadcastTo, div over the last axis of
// front/py/deepx/nn/functional/normalization.py:4-18.  Scalars take the same text → stof → dtype path.
struct RmsNormTF : TF {
    bool has_weight;
    std::string formula;
    RmsNormTF(bool weight, std::vector<Param> a, std::vector<Param> r)
        : has_weight(weight), formula(weight ? "T3=W*(T1/sqrt(sum(T1^2,-1)/divisor+eps))" : "T3=T1/sqrt(sum(T1^2,-1)/divisor+eps)") {
        name = "rmsnorm"; metadata.author = "b200"; tftype = "fused"; args = std::move(a); returns = std::move(r);
    }
    DX_TF_BOILERPLATE(RmsNormTF)
    int run(Mem &mem, std::string &error) override {
        const int di = has_weight ? 2 : 1;
        std::vector<std::string> names{args[0].textvalue, returns[0].textvalue};
        if (has_weight) names.push_back(args[1].textvalue);
        if (!check_tensors(names, mem, error)) return 1;
        auto X = mem.get_tensor(args[0].textvalue), O = mem.get_tensor(returns[0].textvalue);
        TensorPtr W = has_weight ? mem.get_tensor(args[1].textvalue) : nullptr;
        if (X->shape.dtype != O->shape.dtype || (W && W->shape.dtype != X->shape.dtype)) {
            error = W ? type_mismatch({X->shape.dtype, W->shape.dtype, O->shape.dtype}) : type_mismatch({X->shape.dtype, O->shape.dtype});
            return 1;
        }
        if (X->shape.dim() < 1 || X->shape.shape != O->shape.shape || X->global_rows != O->global_rows) throw std::invalid_argument("shape mismatch");
        if (X->shape.dim() == 1) refuse_partitioned("rmsnorm (over the partitioned axis)", {X});
        if (W) refuse_partitioned("rmsnorm (weight)", {W});
        const int64_t cols = X->shape.shape.back();
        if (W && (W->shape.size != cols || W->shape.dim() < 1 || W->shape.shape.back() != cols))
            throw TensorShapeError("rmsnorm: weight must hold one row of " + std::to_string(cols) + " elements");
        const Scalar d = scalar_for(*this, di, mem), e = scalar_for(*this, di + 1, mem);
        dx_check(dx_rmsnorm(X->dx(), X->data, W ? W->data : nullptr, O->data, cols ? X->shape.size / cols : 0, cols, d.f, e.f, mem.stream()));
        return 0;
    }
};

struct SoftmaxTF : TF {
    std::string formula = "T3=softmax(T1, axis=-1)";
    SoftmaxTF(std::vector<Param> a, std::vector<Param> r) { name = "softmax"; metadata.author = "b200"; tftype = "fused"; args = std::move(a); returns = std::move(r); }
    DX_TF_BOILERPLATE(SoftmaxTF)
    int run(Mem &mem, std::string &error) override {
        if (!check_tensors({args[0].textvalue, returns[0].textvalue}, mem, error)) return 1;
        auto X = mem.get_tensor(args[0].textvalue), O = mem.get_tensor(returns[0].textvalue);
        if (X->shape.dtype != O->shape.dtype) { error = type_mismatch({X->shape.dtype, O->shape.dtype}); return 1; }
        if (X->shape.dim() < 1 || X->shape.shape != O->shape.shape || X->global_rows != O->global_rows) throw std::invalid_argument("shape mismatch");
        if (X->shape.dim() == 1) refuse_partitioned("softmax (over the partitioned axis)", {X});
        const int64_t cols = X->shape.shape.back();
        dx_check(dx_softmax(X->dx(), X->data, O->data, cols ? X->shape.size / cols : 0, cols, mem.stream()));
        return 0;
    }
};

// ---- registration helpers ---------------------------------------------------------------------------------------------------
Param T(const char *n, uint16_t p = P_ANY) { return Param(n, CAT_TENSOR, p); }
Param V(const char *n, uint16_t p = P_ANY) { return Param(n, CAT_VAR, p); }
Param Vec(const char *n, uint16_t p = P_ANY) { return Param(n, CAT_VECTOR, p); }
Param L(const char *n, uint16_t p = P_ANY) { return Param(n, CAT_LISTTENSOR, p); }
using PV = std::vector<Param>;

}  // namespace

// The op table of executor/op-cuda/src/client/tfs.cpp:20-646, in its order.
int register_all(TfFactory &f) {
    const uint16_t INTS_BOOL = P_I64 | P_I32 | P_I16 | P_I8 | P_BOOL;
    const uint16_t F4 = P_F64 | P_F32 | P_F16 | P_BF16, F2 = P_F64 | P_F32;
    // lifecycle (:20-81)
    f.add_tf(std::make_shared<ArgSetTF>(PV{V("value")}, PV{V("name")}));
    f.add_tf(std::make_shared<VecSetTF>(PV{Vec("value")}, PV{Vec("name")}));
    f.add_tf(std::make_shared<NewTensorTF>(PV{Vec("shape", P_I32)}, PV{T("tensor1")}));
    f.add_tf(std::make_shared<NewTensorTF>(PV{V("shape", P_STRING)}, PV{T("tensor1")}));
    f.add_tf(std::make_shared<CopyTensorTF>(PV{T("src")}, PV{T("dst")}));
    f.add_tf(std::make_shared<DelTensorTF>(PV{}, PV{T("t")}));
    f.add_tf(std::make_shared<RenameTensorTF>(PV{V("new_name", P_STRING)}, PV{T("t")}));
    // init (:83-134)
    f.add_tf(std::make_shared<InitTF>("constant", InitTF::CONSTANT, "constant(value)->T1", PV{V("value")}, PV{T("t")}));
    f.add_tf(std::make_shared<InitTF>("dropout", InitTF::DROPOUT, "dropout(p,seed)->A", PV{V("p", P_F32), V("seed", P_I32)}, PV{T("A")}));
    f.add_tf(std::make_shared<InitTF>("arange", InitTF::ARANGE, "arange(start,step)->T1", PV{V("start"), V("step")}, PV{T("t")}));
    f.add_tf(std::make_shared<InitTF>("uniform", InitTF::UNIFORM, "uniform(low,high,seed)->T1", PV{V("low"), V("high"), V("seed", P_I32)}, PV{T("t")}));
    f.add_tf(std::make_shared<InitTF>("normal", InitTF::NORMAL, "normal(mean,stddev,seed)->T1", PV{V("mean"), V("stddev"), V("seed", P_I32)}, PV{T("t")}));
    // io (:136-173)
    f.add_tf(std::make_shared<PrintTF>(PV{T("t")}, PV{}));
    f.add_tf(std::make_shared<PrintTF>(PV{T("t"), V("format", P_STRING)}, PV{}));
    f.add_tf(std::make_shared<SaveTF>(PV{T("t"), V("path", P_STRING)}, PV{}));
    f.add_tf(std::make_shared<LoadTF>(PV{V("path", P_STRING)}, PV{}));
    f.add_tf(std::make_shared<LoadTensorDataTF>(PV{V("path", P_STRING)}, PV{T("t")}));
    // elementwise (:175-506)
    f.add_tf(std::make_shared<TodtypeTF>(PV{T("a")}, PV{T("b")}));
    f.add_tf(std::make_shared<BinaryTF>("add", "miaobyte", DX_ADD, "T3=T1+T2", PV{T("a"), T("b")}, PV{T("c")}));
    f.add_tf(std::make_shared<BinaryTF>("add", "cublas", DX_ADD, "T3=T1+T2", PV{T("a"), T("b")}, PV{T("c")}));
    f.add_tf(std::make_shared<ScalarTF>("addscalar", DX_ADDS, false, "T3=T1+scalar", PV{T("A"), V("b")}, PV{T("C")}));
    f.add_tf(std::make_shared<BinaryTF>("sub", "miaobyte", DX_SUB, "T3=T1-T2", PV{T("A"), T("B")}, PV{T("C")}));
    f.add_tf(std::make_shared<ScalarTF>("subscalar", DX_SUBS, false, "T3=T1-scalar", PV{T("A"), V("b")}, PV{T("C")}));
    f.add_tf(std::make_shared<ScalarTF>("rsubscalar", DX_RSUBS, true, "T3=scalar-T1", PV{V("scalar"), T("A")}, PV{T("C")}));
    f.add_tf(std::make_shared<BinaryTF>("mul", "miaobyte", DX_MUL, "T3=T1*T2", PV{T("A"), T("B")}, PV{T("C")}));
    f.add_tf(std::make_shared<ScalarTF>("mulscalar", DX_MULS, false, "T3=T1*scalar", PV{T("A"), V("b")}, PV{T("C")}));
    f.add_tf(std::make_shared<BinaryTF>("div", "miaobyte", DX_DIV, "T3=T1/T2", PV{T("A"), T("B")}, PV{T("C")}));
    f.add_tf(std::make_shared<ScalarTF>("divscalar", DX_DIVS, false, "T3=T1/scalar", PV{T("A"), V("scalar")}, PV{T("C")}));
    f.add_tf(std::make_shared<ScalarTF>("rdivscalar", DX_RDIVS, true, "T3=scalar/T1", PV{V("scalar"), T("A")}, PV{T("C")}));
    f.add_tf(std::make_shared<UnaryTF>("invert", DX_INVERT, "T3=~T1", PV{T("A", INTS_BOOL)}, PV{T("C", INTS_BOOL)}));
    f.add_tf(std::make_shared<UnaryTF>("sqrt", DX_SQRT, "T3=sqrt(T1)", PV{T("A", F4)}, PV{T("C", F4)}));
    f.add_tf(std::make_shared<BinaryTF>("pow", "miaobyte", DX_POW, "T3=pow(T1, T2)", PV{T("A", F2), T("B", F2)}, PV{T("C", F2)}));
    f.add_tf(std::make_shared<ScalarTF>("powscalar", DX_POWS, false, "T3=pow(T1, scalar)", PV{T("A", F2), V("scalar", P_F64 | P_I32)}, PV{T("C", F2)}));
    f.add_tf(std::make_shared<ScalarTF>("rpowscalar", DX_RPOWS, true, "T3=pow(scalar, T1)", PV{V("scalar", P_F32 | P_I32), T("A", F2)}, PV{T("C", F2)}));
    f.add_tf(std::make_shared<UnaryTF>("log", DX_LOG, "T3=log(T1)", PV{T("A", F4)}, PV{T("C", F4)}));
    f.add_tf(std::make_shared<UnaryTF>("exp", DX_EXP, "T3=exp(T1)", PV{T("A", F4)}, PV{T("C", F4)}));
    f.add_tf(std::make_shared<UnaryTF>("sin", DX_SIN, "T3=sin(T1)", PV{T("A", F4)}, PV{T("C", F4)}));
    f.add_tf(std::make_shared<UnaryTF>("cos", DX_COS, "T3=cos(T1)", PV{T("A", F4)}, PV{T("C", F4)}));
    f.add_tf(std::make_shared<UnaryTF>("tan", DX_TAN, "T3=tan(T1)", PV{T("A", F2)}, PV{T("C", F2)}));
    f.add_tf(std::make_shared<BinaryTF>("max", "miaobyte", DX_MAX, "T3=max(T1, T2)", PV{T("A"), T("B")}, PV{T("C")}));
    f.add_tf(std::make_shared<ScalarTF>("maxscalar", DX_MAXS, false, "T3=max(T1, scalar)", PV{T("A"), V("scalar")}, PV{T("C")}));
    f.add_tf(std::make_shared<BinaryTF>("min", "miaobyte", DX_MIN, "T3=min(T1, T2)", PV{T("A"), T("B")}, PV{T("C")}));
    f.add_tf(std::make_shared<ScalarTF>("minscalar", DX_MINS, false, "T3=min(T1, scalar)", PV{T("A"), V("scalar")}, PV{T("C")}));
    f.add_tf(std::make_shared<CompareTF>("equal", DX_EQ, true, "equal(T1,T2)->mask", PV{T("A"), T("B"), V("epsilon", P_F32)}, PV{T("mask", P_BOOL)}));
    f.add_tf(std::make_shared<CompareScalarTF>("equalscalar", DX_EQ, true, "equalscalar(T1,scalar)->mask", PV{T("A"), V("scalar"), V("epsilon", P_F32)}, PV{T("mask", P_BOOL)}));
    f.add_tf(std::make_shared<CompareTF>("notequal", DX_NE, true, "notequal(T1,T2)->mask", PV{T("A"), T("B"), V("epsilon", P_F32)}, PV{T("mask", P_BOOL)}));
    f.add_tf(std::make_shared<CompareScalarTF>("notequalscalar", DX_NE, true, "notequalscalar(T1,scalar)->mask", PV{T("A"), V("scalar"), V("epsilon", P_F32)}, PV{T("mask", P_BOOL)}));
    f.add_tf(std::make_shared<CompareTF>("less", DX_LT, false, "mask=less(T1,T2)", PV{T("A"), T("B")}, PV{T("mask", P_BOOL)}));
    f.add_tf(std::make_shared<CompareScalarTF>("lessscalar", DX_LT, false, "mask=less(T1,scalar)", PV{T("A"), V("scalar")}, PV{T("mask", P_BOOL)}));
    f.add_tf(std::make_shared<CompareTF>("greater", DX_GT, false, "mask=greater(T1,T2)", PV{T("A"), T("B")}, PV{T("mask", P_BOOL)}));
    f.add_tf(std::make_shared<CompareScalarTF>("greaterscalar", DX_GT, false, "mask=greater(T1,scalar)", PV{T("A"), V("scalar")}, PV{T("mask", P_BOOL)}));
    f.add_tf(std::make_shared<SwitchTF>(PV{L("tensors"), T("cases", P_I32 | P_BOOL)}, PV{T("result")}));
    // matmul (:508-519)
    f.add_tf(std::make_shared<MatMulTF>(PV{T("A"), T("B")}, PV{T("C")}));
    // changeshape (:521-585)
    f.add_tf(std::make_shared<ReshapeTF>(PV{T("A"), Vec("shape", P_I32)}, PV{T("B")}));
    f.add_tf(std::make_shared<TransposeTF>(PV{T("A"), Vec("dim_order", P_I32)}, PV{T("C")}));
    f.add_tf(std::make_shared<ConcatTF>(PV{L("tensors"), V("dim", P_I32)}, PV{T("result")}));
    f.add_tf(std::make_shared<BroadcastToTF>(PV{T("A"), Vec("new_shape", P_I32)}, PV{T("B")}));
    f.add_tf(std::make_shared<IndexSelectTF>(PV{T("A"), T("indices", P_I64 | P_I32), V("axis", P_I32)}, PV{T("B")}));
    f.add_tf(std::make_shared<RepeatTF>(PV{T("A"), Vec("repeats", P_I32)}, PV{T("B")}));
    // reduce (:587-634)
    f.add_tf(std::make_shared<ReduceTF>("sum", DX_SUM, "B = sum(A, axis=[1 2], keepdims=false)", PV{T("A"), Vec("dims", P_I32), V("keepdims", P_BOOL)}, PV{T("B")}));
    f.add_tf(std::make_shared<ReduceTF>("prod", DX_PROD, "B = prod(A, axis=[1 2], keepdims=false)", PV{T("A"), Vec("dims", P_I32), V("keepdims", P_BOOL)}, PV{T("B")}));
    f.add_tf(std::make_shared<ReduceTF>("reducemax", DX_RMAX, "B = reducemax(A, axis=[1 2], keepdims=false)", PV{T("A"), Vec("dims", P_I32), V("keepdims", P_BOOL)}, PV{T("B")}));
    f.add_tf(std::make_shared<ReduceTF>("reducemin", DX_RMIN, "B = reducemin(A, axis=[1 2], keepdims=false)", PV{T("A"), Vec("dims", P_I32), V("keepdims", P_BOOL)}, PV{T("B")}));
    return 0;
}

// Ops beyond the reference's table: the single-kernel forms of the RMSNorm and softmax chains.
int register_fused(TfFactory &f) {
    const uint16_t F4 = P_F64 | P_F32 | P_F16 | P_BF16;
    f.add_tf(std::make_shared<RmsNormTF>(true, PV{T("x", F4), T("weight", F4), V("divisor"), V("eps")}, PV{T("out", F4)}));
    f.add_tf(std::make_shared<RmsNormTF>(false, PV{T("x", F4), V("divisor"), V("eps")}, PV{T("out", F4)}));
    f.add_tf(std::make_shared<SoftmaxTF>(PV{T("x", F4)}, PV{T("out", F4)}));
    return 0;
}

}  // namespace dxh
