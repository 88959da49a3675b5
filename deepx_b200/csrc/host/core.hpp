// deepxIR host core: dtype codec, shape descriptor, IR parser, op registry, tensor store.
//
// Behaviour follows the reference's executor/deepxcore (file:line cited at each piece) so
// that IR text produced by the existing front ends parses, matches and replies the same way;
// the representation is new: 64-bit shapes, type-erased tensors that carry a dtype code for
// the kernel C ABI, pool-backed storage.
#pragma once
#include <chrono>
#include <cstdint>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <variant>
#include <vector>

#include "dx_kernels.h"
#include "shard.hpp"

namespace dxh {

// ---- dtype (executor/deepxcore/src/deepx/dtype.hpp) -----------------------------------------
// Bit values are the reference's (dtype.hpp:36-43, :120-146): they define signature matching.
enum Category : uint8_t { CAT_UNKNOWN = 0, CAT_VAR = 1, CAT_VECTOR = 2, CAT_TENSOR = 4, CAT_LISTTENSOR = 8 };
enum Precision : uint16_t {
    P_F64 = 1 << 0, P_F32 = 1 << 1, P_F16 = 1 << 2, P_BF16 = 1 << 3, P_F8E5M2 = 1 << 4, P_F8E4M3 = 1 << 5, P_F4E2M1 = 1 << 6,
    P_I64 = 1 << 8, P_I32 = 1 << 9, P_I16 = 1 << 10, P_I8 = 1 << 11, P_I4 = 1 << 12,
    P_BOOL = 1 << 13, P_STRING = 1 << 15,
    P_ANY = 0xFFFF,
    P_FLOAT = P_F64 | P_F32 | P_F16 | P_BF16 | P_F8E5M2 | P_F8E4M3 | P_F4E2M1,
    P_FLOAT8 = P_F8E5M2 | P_F8E4M3,
    P_INT = P_I64 | P_I32 | P_I16 | P_I8 | P_I4,
};

struct TypeDef {
    uint8_t category = CAT_UNKNOWN;
    uint16_t precision = P_ANY;
    // `this` is the caller's type, `registered` the op's: every bit the caller sets must be allowed
    // (TypeDef::match, dtype.hpp:232-247).
    bool match(const TypeDef &registered) const {
        return (category & registered.category) == category && (precision & registered.precision) == precision;
    }
    uint32_t value() const { return uint32_t(category) | (uint32_t(precision) << 8); }
};

uint8_t category_of(const std::string &text);          // base_category, dtype.hpp:87-118
std::string category_str(uint8_t c);                   // base_category_str, dtype.hpp:60-84
uint16_t precision_of(const std::string &text);        // precision, dtype.hpp:321-365
std::string precision_str(uint16_t p);                 // dtype.hpp:266-311
TypeDef typedef_of(const std::string &text);           // dtype, dtype.hpp:368-384
std::string typedef_str(const TypeDef &t);             // dtype_str, dtype.hpp:314-318
int precision_bits(uint16_t p);                        // dtype.hpp:161-199
int dx_code_of(uint16_t precision);                    // Precision → dx_dtype code, -1 if no kernel dtype
uint16_t precision_of_dx(int code);

// ---- errors (executor/deepxcore/src/stdutil/error.hpp) -----------------------------------------
struct NotImplementError : std::logic_error {
    explicit NotImplementError(const std::string &m) : std::logic_error("Not implement: " + m) {}
};
struct TensorShapeError : std::logic_error {
    explicit TensorShapeError(const std::string &op) : std::logic_error("Tensor shape error for operation: " + op) {}
};

bool is_float_text(const std::string &s);    // std::stof succeeds (stdutil/num.cpp:24-31)
bool is_integer_text(const std::string &s);  // std::stoi succeeds (:16-23)

// ---- shape (executor/deepxcore/src/deepx/shape.hpp:44-85, shape.cpp:21-32) ----------------------
struct Shape {
    uint16_t dtype = P_ANY;
    std::vector<int64_t> shape, strides;
    int64_t size = 0;
    Shape() = default;
    explicit Shape(const std::vector<int64_t> &s) { set(s); }
    void set(const std::vector<int64_t> &s);
    int dim() const { return int(shape.size()); }
    int64_t at(int i) const { return shape[i < 0 ? i + int(shape.size()) : i]; }
    int64_t bytes() const { return size * (precision_bits(dtype) / 8); }
    std::string to_yaml() const;               // the 5-key document of shape.cpp:93-102
    static Shape from_yaml(const std::string &text);  // shape.cpp:103-121 (block or flow sequences)
};

// shape algebra (shape_changeshape.cpp, shape_reduce.cpp, shape_matmul.cpp)
std::vector<int64_t> transpose_shape(const std::vector<int64_t> &shape, const std::vector<int> &order);
std::vector<int64_t> broadcast_shape(const std::vector<int64_t> &a, const std::vector<int64_t> &b);
std::vector<int64_t> indexselect_shape(const std::vector<int64_t> &in, const std::vector<int64_t> &idx, int axis);
std::vector<int64_t> repeat_shape(const std::vector<int64_t> &src, const std::vector<int64_t> &repeats);
std::vector<int> checked_dims(const std::vector<int64_t> &shape, const std::vector<int> &dims);
std::vector<int64_t> reduced_shape(const std::vector<int64_t> &shape, const std::vector<int> &checked, bool keepdims);
std::vector<int64_t> matmul_shape(const std::vector<int64_t> &a, const std::vector<int64_t> &b);
bool check_matmul_shape(const std::vector<int64_t> &a, const std::vector<int64_t> &b);

// ---- tensors and the store (tensor.hpp:17-171, mem/mem.hpp:15-175, op-cuda mem_cuda.hpp) ------------
struct Tensor {
    Shape shape;              // what `data` holds: the LOCAL rows of a row-partitioned tensor
    void *data = nullptr;
    dx_pool *pool = nullptr;  // owner of `data`
    int device = 0;
    // Row partitioning over the ranks of a multi-GPU executor (shard.hpp): global_rows >= 0 means this rank
    // holds rows [row0, row0 + shape[0]) of a tensor whose leading axis has global_rows indices.
    int64_t global_rows = -1, row0 = 0;
    // Set while an asynchronous upload into this tensor is in flight on the copy stream: the compute stream waits
    // for it before the first op that names the tensor (dx_exec_upload_async).
    void *ready_event = nullptr;
    bool upload_in_flight = false;
    bool partitioned() const { return global_rows >= 0; }
    std::vector<int64_t> global_shape() const {
        std::vector<int64_t> g = shape.shape;
        if (partitioned() && !g.empty()) g[0] = global_rows;
        return g;
    }
    Layout layout() const { return Layout{partitioned(), global_shape(), precision_bits(shape.dtype) / 8}; }
    int64_t row_bytes() const { return shape.dim() == 0 || shape.shape[0] == 0 ? 0 : shape.bytes() / shape.shape[0]; }
    Tensor() = default;
    Tensor(const Tensor &) = delete;
    Tensor &operator=(const Tensor &) = delete;
    ~Tensor();
    int dx() const { return dx_code_of(shape.dtype); }
};
using TensorPtr = std::shared_ptr<Tensor>;
using ArgValue = std::variant<int, float, double, std::string, std::vector<int>, std::vector<float>, std::vector<double>,
                              std::vector<std::string>>;

class Mem {
  public:
    Mem(int device, size_t pool_limit_bytes);
    ~Mem();
    // tensors
    TensorPtr new_tensor(const std::string &name, uint16_t precision, const std::vector<int64_t> &shape);  // throws on exhaustion
    void add_tensor(const std::string &name, TensorPtr t);   // "tensor already exists" is logged and ignored, mem.hpp:80-87
    bool exists_tensor(const std::string &name) const { return tensors_.count(name) != 0; }
    TensorPtr get_tensor(const std::string &name) const;     // throws runtime_error("tensor not found: …"), mem.hpp:121-124
    void delete_tensor(const std::string &name) { tensors_.erase(name); }
    void rename_tensor(const std::string &old_name, const std::string &new_name);
    // args / vectors
    void add_arg(const std::string &name, ArgValue v) { args_[name] = std::move(v); }
    bool exists_arg(const std::string &name) const { return args_.count(name) != 0; }
    const ArgValue *get_arg(const std::string &name) const;
    void delete_arg(const std::string &name) { args_.erase(name); }
    void clear() { tensors_.clear(); args_.clear(); }
    // device side
    dx_pool *pool() const { return pool_; }
    int device() const { return device_; }
    void *stream() const { return stream_; }
    void *copy_stream();  // created on first use: host-to-device copies that overlap with compute
    // Host bytes into a tensor without waiting: the copy is ordered behind everything already submitted to the compute
    // stream, and ops that name the tensor afterwards are ordered behind the copy (wait_ready).
    void upload_async(Tensor &t, const void *host, size_t bytes);
    void wait_ready(Tensor &t);
    int uploads_in_flight = 0;  // tensors whose asynchronous upload no op has waited for yet
    void *scratch(size_t bytes);  // grow-only workspace for reductions, from the pool
    // While a program is being captured into a CUDA graph nothing may be allocated: the graph keeps
    // the pointers it saw.  `capturing` makes scratch growth and staging temporaries throw instead;
    // `scratch_generation` changes whenever the workspace moves, which invalidates earlier captures.
    bool capturing = false;
    uint64_t scratch_generation() const { return scratch_generation_; }
    size_t tensor_count() const { return tensors_.size(); }
    std::vector<std::string> tensor_names() const;
    // One of several ranks (shard.hpp).  new_tensor partitions large tensors by rows when shard.active().
    ShardCtx shard;
    // A cross-rank reduction may leave its combine for later (dx_comm_allreduce_finish): flush_comm completes it
    // on the compute stream; comm_pending_in says whether the outstanding exchange writes into [p, p + bytes).
    void flush_comm();
    bool comm_pending_in(const void *p, size_t bytes) const;

  private:
    int device_;
    dx_pool *pool_ = nullptr;
    void *stream_ = nullptr;
    void *copy_stream_ = nullptr;
    void *order_event_ = nullptr;
    void *scratch_ = nullptr;
    size_t scratch_bytes_ = 0;
    uint64_t scratch_generation_ = 0;
    std::unordered_map<std::string, TensorPtr> tensors_;
    std::unordered_map<std::string, ArgValue> args_;
};

// ---- IR (executor/deepxcore/src/deepx/tf/tf.hpp:25-231, tf.cpp) -----------------------------------------
struct Param {
    TypeDef dtype;
    std::string textvalue;
    Param() = default;
    Param(std::string text, uint8_t cat, uint16_t prec) : textvalue(std::move(text)) { dtype.category = cat; dtype.precision = prec; }
    void parse(const std::string &text);                 // Param::parse, tf.cpp:12-39
    std::string to_string() const { return typedef_str(dtype) + ":" + textvalue; }
};

struct Metadata {
    std::string author;
    int id = 0;
    std::chrono::system_clock::time_point created_at{}, sent_at{}, recv_at{};
    int benchmark_repeat = 0;
    void parse(const std::string &meta);                 // TFMetadata::parse, tf.cpp:92-122
};

class TF {
  public:
    std::string name, tftype;
    std::vector<Param> args, returns;
    Metadata metadata;
    TF() = default;
    explicit TF(const std::string &text) { parse(text); }
    virtual ~TF() = default;
    void parse(const std::string &text);                 // TF::parse, tf.cpp:299-316; throws runtime_error("Invalid IR format: missing arrow")
    std::string to_string() const;                       // TF::to_string(false), tf.cpp:331-372
    virtual int run(Mem &mem, std::string &error) { throw NotImplementError(name); }   // tf.hpp:72
    virtual std::string math_formula() const { return ""; }
    virtual std::shared_ptr<TF> clone() const { return std::make_shared<TF>(*this); }

    // getvar<T> (tf.hpp:84-127): bool by "true"/"false" (any case); a numeric text goes through
    // std::stof for EVERY arithmetic T; otherwise the text names a stored arg.
    bool var_bool(int idx, bool from_args = true) const;
    float var_f32(int idx, const Mem &mem, bool from_args = true) const;   // the float every numeric scalar passes through
    int var_int(int idx, const Mem &mem, bool from_args = true) const { return int(var_f32(idx, mem, from_args)); }
    // getvector<T> (tf.hpp:129-158): strip [], split on single spaces
    std::vector<std::string> vector_text(int idx, bool from_args = true) const;
    std::vector<int> vector_int(int idx, bool from_args = true) const;       // axes, orders: must fit an int
    std::vector<int64_t> vector_i64(int idx, bool from_args = true) const;   // extents, repeats: 64-bit, read exactly
    bool check_tensors(const std::vector<std::string> &names, const Mem &mem, std::string &error) const;  // tf.hpp:160-171

  protected:
    const Param &param(int idx, bool from_args) const;
};

struct OpResp {  // tf.hpp:183-231
    int id = 0;
    std::string result, message;
    std::chrono::system_clock::time_point recv_at{}, start_at{}, finish_at{};
    std::string to_string() const;
    void finish(const std::string &msg) { result = "ok"; finish_at = std::chrono::system_clock::now(); message = msg; }
    void error(const std::string &msg) { result = "error"; finish_at = std::chrono::system_clock::now(); message = msg; }
};

// ---- registry (executor/deepxcore/src/deepx/tf/tffactory.hpp, tffactory.cpp) ------------------------------
class TfFactory {
  public:
    void add_tf(std::shared_ptr<TF> tf);
    // name → author (unknown author falls back to the first one registered for that name,
    // tffactory.cpp:25-37) → first registration whose signature admits the call (:39-65);
    // returns a clone carrying the call's metadata, or nullptr.  `why` gets the diagnostic.
    std::shared_ptr<TF> get_tf(const TF &call, std::string *why = nullptr) const;
    std::string print_markdown(const std::string &executor_name) const;   // tffactory.cpp:85-119
    size_t size() const { return count_; }

  private:
    struct Author { std::string name; std::vector<std::shared_ptr<TF>> tfs; };
    struct Family { std::vector<Author> authors; };
    std::unordered_map<std::string, Family> families_;
    std::vector<std::string> order_;  // op names in registration order
    size_t count_ = 0;
};

// print's format argument, checked and normalised (ops.cpp); false + `error` when it is refused
bool checked_print_format(const std::string &fmt, uint16_t dtype, std::string &out, std::string &error);

int register_all(TfFactory &factory);   // the op table of executor/op-cuda/src/client/tfs.cpp
int register_fused(TfFactory &factory); // rmsnorm / softmax: the single-kernel forms of the front end's op chains

// What the fusion pass (fusion.hpp) has done so far.
struct FusionStats {
    uint64_t programs = 0;        // programs seen by the pass
    uint64_t rmsnorm_groups = 0;  // chains rewritten
    uint64_t softmax_groups = 0;
    uint64_t lines_absorbed = 0;  // IR lines that no longer run (chain steps, temp newtensor/deltensor)
};

struct CompiledProgram {
    struct Ref {
        std::string name;
        void *data;
        uint16_t precision;
        std::vector<int64_t> shape;
    };
    void *graph = nullptr;  // cudaGraph_t
    void *exec = nullptr;   // cudaGraphExec_t
    std::vector<Ref> refs;
    uint64_t scratch_generation = 0;
    size_t lines = 0, ops = 0, nodes = 0, fused_groups = 0;
    CompiledProgram() = default;
    CompiledProgram(const CompiledProgram &) = delete;
    CompiledProgram &operator=(const CompiledProgram &) = delete;
    ~CompiledProgram();
};

// ---- executor: one IR line in, one reply out (executor/op-cuda/src/client/main.cpp:47-102) --------------------
class Executor {
  public:
    Executor(int device, size_t pool_limit_bytes);
    OpResp run(const TF &call);              // never throws: every failure becomes an "error" reply
    OpResp run_line(const std::string &ir);  // parse + run
    // Several IR lines handed over together (one per text line): one reply per non-empty line, in
    // order.  With `fuse` on, RMSNorm / softmax op chains whose temporaries live and die inside the
    // program run as one kernel; the replies of the lines that no longer run say "ok".
    std::vector<OpResp> run_program(const std::string &text);
    const FusionStats &fusion_stats() const { return fusion_; }
    // A program whose kernels are captured once into a CUDA graph and then replayed with one launch
    // call: for sequences of small ops the host cost per IR line (parse, dispatch, launch) is what
    // limits throughput, and a replay has none of it.  The program may only compute: tensor lifetime,
    // io and arg ops, timed lines and ops that need a temporary are refused (chains that the fusion
    // pass absorbs, temporaries included, are fine).  compile() runs the program once (that run's
    // results stand) and captures a second pass; replay() first checks that every tensor the program
    // names still exists with the same storage, dtype and shape.
    std::shared_ptr<CompiledProgram> compile(const std::string &text, std::string *error);
    int replay(CompiledProgram &program, std::string *error);
    bool fuse = true;
    // Makes this executor rank `rank` of `world` (one process per GPU, the same IR lines to every rank); `comm`
    // must be connected and outlive the executor.  Tensors created afterwards are partitioned by rows when
    // they hold at least `min_bytes`; existing tensors stay as they are.
    void set_shard(int rank, int world, size_t min_bytes, dx_comm *comm);
    Mem &mem() { return mem_; }
    const TfFactory &factory() const { return factory_; }
    uint64_t ops_run() const { return ops_run_; }
    bool ir_log = false;

  private:
    Mem mem_;
    TfFactory factory_;
    std::mutex mu_;
    uint64_t ops_run_ = 0;
    FusionStats fusion_;
};

}  // namespace dxh
