// C ABI of the executor (include/dx_executor.h).
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <sstream>
#include <unordered_map>

#include "core.hpp"
#include "fusion.hpp"
#include "dx_executor.h"

using namespace dxh;

struct dx_exec {
    Executor ex;
    dx_exec(int device, size_t limit) : ex(device, limit) {}
};

struct dx_program {
    dx_exec *owner;
    std::shared_ptr<CompiledProgram> prog;
};

namespace {
thread_local std::string g_err;
int put(const std::string &s, char *out, size_t cap) {
    if (!out || s.size() + 1 > cap) return -1;
    std::memcpy(out, s.c_str(), s.size() + 1);
    return int(s.size());
}
struct ProbeTF : TF {
    int index = -1;
    std::shared_ptr<TF> clone() const override { return std::make_shared<ProbeTF>(*this); }
};
struct Registry {
    TfFactory f;
    int n = 0;
};
}  // namespace

extern "C" {

dx_exec *dx_exec_create(int device, size_t pool_limit_bytes) {
    try {
        return new dx_exec(device, pool_limit_bytes);
    } catch (const std::exception &e) {
        g_err = e.what();
        return nullptr;
    }
}
void dx_exec_destroy(dx_exec *e) { delete e; }
const char *dx_exec_last_error(void) { return g_err.c_str(); }

int dx_exec_run(dx_exec *e, const char *ir_line, char *reply, size_t cap) {
    if (!e || !ir_line) { g_err = "null executor or IR line"; return -1; }
    const OpResp r = e->ex.run_line(ir_line);
    if (put(r.to_string(), reply, cap) < 0) { g_err = "reply buffer too small"; return -1; }
    return r.result == "ok" ? 0 : 1;
}

int dx_exec_run_program(dx_exec *e, const char *program, char *replies, size_t cap) {
    if (!e || !program) { g_err = "null executor or program"; return -1; }
    const std::vector<OpResp> rs = e->ex.run_program(program);
    std::string all;
    int errors = 0;
    for (size_t i = 0; i < rs.size(); ++i) {
        if (i) all += "\n";
        all += rs[i].to_string();
        errors += rs[i].result == "ok" ? 0 : 1;
    }
    if (put(all, replies, cap) < 0) { g_err = "reply buffer too small"; return -1; }
    return errors;
}
void dx_exec_set_fusion(dx_exec *e, int on) { if (e) e->ex.fuse = on != 0; }
void dx_exec_fusion_stats(dx_exec *e, uint64_t stats[4]) {
    if (!e || !stats) return;
    const FusionStats &f = e->ex.fusion_stats();
    stats[0] = f.programs; stats[1] = f.rmsnorm_groups; stats[2] = f.softmax_groups; stats[3] = f.lines_absorbed;
}

dx_program *dx_exec_compile(dx_exec *e, const char *program) {
    if (!e || !program) { g_err = "null executor or program"; return nullptr; }
    std::string why;
    auto cp = e->ex.compile(program, &why);
    if (!cp) { g_err = "compile: " + why; return nullptr; }
    return new dx_program{e, cp};
}
int dx_program_run(dx_program *p) {
    if (!p) { g_err = "null program"; return 1; }
    std::string why;
    const int rc = p->owner->ex.replay(*p->prog, &why);
    if (rc != 0) g_err = why;
    return rc;
}
void dx_program_info(dx_program *p, size_t info[4]) {
    if (!p || !info) return;
    info[0] = p->prog->lines; info[1] = p->prog->ops; info[2] = p->prog->nodes; info[3] = p->prog->fused_groups;
}
void dx_program_free(dx_program *p) { delete p; }

int dx_exec_bind_tensor(dx_exec *e, const char *name, int dtype, const int64_t *shape, int ndim, void *device_ptr) {
    if (!e || !name || !*name || (ndim > 0 && !shape) || ndim < 0 || ndim > DX_MAX_DIMS) { g_err = "bind: bad argument"; return -1; }
    const uint16_t prec = precision_of_dx(dtype);
    if (dx_code_of(prec) < 0) { g_err = "bind: unsupported dtype code"; return -1; }
    if (e->ex.mem().exists_tensor(name)) { g_err = std::string("bind: tensor already exists: ") + name; return -1; }
    auto t = std::make_shared<Tensor>();
    std::vector<int64_t> shp(shape, shape + ndim);
    for (auto d : shp)
        if (d < 0) { g_err = "bind: negative extent"; return -1; }
    t->shape.set(shp);
    t->shape.dtype = prec;
    t->data = device_ptr;
    t->pool = nullptr;  // not ours: never freed here
    t->device = e->ex.mem().device();
    if (t->shape.size > 0 && !device_ptr) { g_err = "bind: null pointer"; return -1; }
    e->ex.mem().add_tensor(name, t);
    return 0;
}

int dx_exec_tensor_info(dx_exec *e, const char *name, int *dtype, int64_t *shape, int cap) {
    if (!e || !name || !e->ex.mem().exists_tensor(name)) return -1;
    auto t = e->ex.mem().get_tensor(name);
    if (dtype) *dtype = t->dx();
    for (int i = 0; i < t->shape.dim() && i < cap; ++i) shape[i] = t->shape.shape[i];
    return t->shape.dim();
}

void *dx_exec_tensor_ptr(dx_exec *e, const char *name) {
    if (!e || !name || !e->ex.mem().exists_tensor(name)) return nullptr;
    auto t = e->ex.mem().get_tensor(name);
    if (t->upload_in_flight) {
        e->ex.mem().wait_ready(*t);
        --e->ex.mem().uploads_in_flight;
    }
    try {  // the caller is about to look at the memory: a combine still owed to this tensor runs first
        if (e->ex.mem().comm_pending_in(t->data, size_t(std::max<int64_t>(t->shape.bytes(), 0)))) e->ex.mem().flush_comm();
    } catch (const std::exception &ex) {
        g_err = ex.what();
        return nullptr;
    }
    return t->data;
}

int dx_exec_set_shard(dx_exec *e, int rank, int world, size_t min_bytes, dx_comm *comm) {
    if (!e) { g_err = "null executor"; return -1; }
    try {
        e->ex.set_shard(rank, world, min_bytes, comm);
        return 0;
    } catch (const std::exception &ex) {
        g_err = ex.what();
        return -1;
    }
}

int dx_exec_tensor_shard(dx_exec *e, const char *name, int64_t *row0, int64_t *rows, int64_t *global_rows) {
    if (!e || !name || !e->ex.mem().exists_tensor(name)) return -1;
    auto t = e->ex.mem().get_tensor(name);
    if (row0) *row0 = t->row0;
    if (rows) *rows = t->shape.dim() ? t->shape.shape[0] : 0;
    if (global_rows) *global_rows = t->partitioned() ? t->global_rows : (t->shape.dim() ? t->shape.shape[0] : 0);
    return t->partitioned() ? 1 : 0;
}

static int copy(dx_exec *e, const char *name, void *host, size_t bytes, bool up) {
    if (!e || !name || !e->ex.mem().exists_tensor(name)) { g_err = std::string("tensor not found: ") + (name ? name : ""); return -1; }
    auto t = e->ex.mem().get_tensor(name);
    if (size_t(t->shape.bytes()) != bytes) {
        g_err = "size mismatch: tensor holds " + std::to_string(t->shape.bytes()) + " bytes, caller gave " + std::to_string(bytes);
        return -2;
    }
    if (bytes == 0) return 0;
    cudaSetDevice(e->ex.mem().device());
    try {
        if (e->ex.mem().comm_pending_in(t->data, bytes)) e->ex.mem().flush_comm();  // a combine still owed to this tensor
    } catch (const std::exception &ex) {
        g_err = ex.what();
        return -4;
    }
    if (t->upload_in_flight) {  // an asynchronous upload into this tensor comes first
        e->ex.mem().wait_ready(*t);
        --e->ex.mem().uploads_in_flight;
    }
    cudaStream_t st = static_cast<cudaStream_t>(e->ex.mem().stream());
    cudaError_t err = up ? cudaMemcpyAsync(t->data, host, bytes, cudaMemcpyHostToDevice, st)
                         : cudaMemcpyAsync(host, t->data, bytes, cudaMemcpyDeviceToHost, st);
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    if (err != cudaSuccess) { g_err = cudaGetErrorString(err); return -4; }
    return 0;
}
int dx_exec_upload(dx_exec *e, const char *name, const void *host, size_t bytes) { return copy(e, name, const_cast<void *>(host), bytes, true); }

int dx_exec_upload_async(dx_exec *e, const char *name, const void *host, size_t bytes) {
    if (!e || !name || !e->ex.mem().exists_tensor(name)) { g_err = std::string("tensor not found: ") + (name ? name : ""); return -1; }
    auto t = e->ex.mem().get_tensor(name);
    if (size_t(t->shape.bytes()) != bytes) {
        g_err = "size mismatch: tensor holds " + std::to_string(t->shape.bytes()) + " bytes, caller gave " + std::to_string(bytes);
        return -2;
    }
    if (bytes == 0) return 0;
    cudaSetDevice(e->ex.mem().device());
    try {
        Mem &m = e->ex.mem();
        if (m.comm_pending_in(t->data, bytes)) m.flush_comm();
        if (!t->upload_in_flight) ++m.uploads_in_flight;
        m.upload_async(*t, host, bytes);
    } catch (const std::exception &ex) {
        g_err = ex.what();
        return -4;
    }
    return 0;
}
int dx_exec_download(dx_exec *e, const char *name, void *host, size_t bytes) { return copy(e, name, host, bytes, false); }

int dx_exec_sync(dx_exec *e) {
    if (!e) return -1;
    cudaSetDevice(e->ex.mem().device());
    try {
        e->ex.mem().flush_comm();
    } catch (const std::exception &ex) {
        g_err = ex.what();
        return -4;
    }
    cudaError_t err = cudaStreamSynchronize(static_cast<cudaStream_t>(e->ex.mem().stream()));
    if (err == cudaSuccess && e->ex.mem().uploads_in_flight > 0) err = cudaStreamSynchronize(static_cast<cudaStream_t>(e->ex.mem().copy_stream()));
    if (err != cudaSuccess) { g_err = cudaGetErrorString(err); return -4; }
    return 0;
}
void *dx_exec_stream(dx_exec *e) { return e ? e->ex.mem().stream() : nullptr; }

size_t dx_exec_op_table(dx_exec *e, char *out, size_t cap) {
    if (!e) return 0;
    const std::string s = e->ex.factory().print_markdown("op-b200");
    if (out && cap > 0) {
        const size_t n = std::min(cap - 1, s.size());
        std::memcpy(out, s.data(), n);
        out[n] = 0;
    }
    return s.size() + 1;
}

void dx_exec_stats(dx_exec *e, size_t stats[5]) {
    if (!e || !stats) return;
    dx_pool_stats(e->ex.mem().pool(), stats);
    stats[4] = size_t(e->ex.ops_run());
}

int dx_ir_parse(const char *ir_line, char *out, size_t cap) {
    try {
        TF t;
        t.parse(ir_line ? ir_line : "");
        std::string s = t.name + "|";
        for (size_t i = 0; i < t.args.size(); ++i) s += (i ? "," : "") + t.args[i].to_string();
        s += "|";
        for (size_t i = 0; i < t.returns.size(); ++i) s += (i ? "," : "") + t.returns[i].to_string();
        s += "|author=" + t.metadata.author + " id=" + std::to_string(t.metadata.id) + " repeat=" + std::to_string(t.metadata.benchmark_repeat);
        return put(s, out, cap);
    } catch (const std::exception &e) {
        return put(std::string("!") + e.what(), out, cap);
    }
}
int dx_ir_vector_i64(const char *ir_line, int arg_index, int64_t *out, int cap) {
    try {
        TF t;
        t.parse(ir_line ? ir_line : "");
        const std::vector<int64_t> v = t.vector_i64(arg_index);
        if (int(v.size()) > cap) { g_err = "output array too small"; return -1; }
        for (size_t i = 0; i < v.size(); ++i) out[i] = v[i];
        return int(v.size());
    } catch (const std::exception &e) {
        g_err = e.what();
        return -1;
    }
}
int dx_ir_check_print_format(const char *format, int dtype, char *out, size_t cap) {
    std::string fixed, why;
    if (!checked_print_format(format ? format : "", precision_of_dx(dtype), fixed, why)) {
        g_err = why;
        return 1;
    }
    return put(fixed, out, cap) < 0 ? -1 : 0;
}
int dx_ir_dtype_roundtrip(const char *text, char *out, size_t cap) { return put(typedef_str(typedef_of(text ? text : "")), out, cap); }

int dx_ir_plan_fusion(const char *program, const char *existing, char *out, size_t cap) {
    try {
        std::vector<TF> prog;
        std::istringstream ps(program ? program : "");
        std::string line;
        while (std::getline(ps, line))
            if (line.find_first_not_of(" \t\r") != std::string::npos) prog.emplace_back(line);
        std::unordered_map<std::string, std::pair<uint16_t, std::vector<int64_t>>> known;
        std::istringstream es(existing ? existing : "");
        while (std::getline(es, line)) {
            std::istringstream ls(line);
            std::string name, dtype;
            if (!(ls >> name >> dtype)) continue;
            std::vector<int64_t> shape;
            int64_t d;
            while (ls >> d) shape.push_back(d);
            known[name] = {precision_of(dtype), shape};
        }
        FusionStats st;
        const auto plan = plan_fusion(prog, [&](const std::string &n, uint16_t &p, std::vector<int64_t> &s) {
            auto it = known.find(n);
            if (it == known.end()) return false;
            p = it->second.first;
            s = it->second.second;
            return true;
        }, &st);
        std::string text;
        for (size_t i = 0; i < plan.size(); ++i) {
            if (plan[i].kind == PlanItem::RUN) text += "run\n";
            else if (plan[i].kind == PlanItem::ABSORBED) text += "absorbed " + std::to_string(plan[i].group) + "\n";
            else text += "fused " + std::to_string(plan[i].group) + " " + plan[i].fused.to_string() + "\n";
        }
        if (put(text, out, cap) < 0) return -1;
        return int(st.rmsnorm_groups + st.softmax_groups);
    } catch (const std::exception &ex) {
        g_err = ex.what();
        return -1;
    }
}

// The partition decisions for a program, with tensors that are records only (no device).  Lines are classified by
// the same plan_rowwise / plan_reduce / should_partition the ops use; ops without a row-wise form are reported as
// the executor would treat them when an operand is partitioned.
int dx_ir_shard_plan(const char *program, int world, size_t min_bytes, char *out, size_t cap) {
    try {
        ShardCtx ctx;
        ctx.world = world;
        ctx.min_bytes = min_bytes;
        std::unordered_map<std::string, Layout> known;
        std::istringstream ps(program ? program : "");
        std::string line, text;
        int lines = 0;
        auto names_of = [](const Param &q) {
            std::vector<std::string> v;
            std::string names = q.textvalue;
            for (char &c : names) if (c == '[' || c == ']') c = ' ';
            std::istringstream ns(names);
            std::string nm;
            while (ns >> nm) v.push_back(nm);
            return v;
        };
        while (std::getline(ps, line)) {
            if (line.find_first_not_of(" \t\r") == std::string::npos) continue;
            TF t(line);
            std::string verdict;
            auto layout_of = [&](const std::string &n) -> const Layout & {
                auto it = known.find(n);
                if (it == known.end()) throw std::runtime_error("tensor not found: " + n);
                return it->second;
            };
            static const char *rowwise_ops[] = {"add", "sub", "mul", "div", "max", "min", "pow", "addscalar", "subscalar", "rsubscalar", "mulscalar",
                                                "divscalar", "rdivscalar", "maxscalar", "minscalar", "powscalar", "rpowscalar", "sqrt", "log", "exp",
                                                "sin", "cos", "tan", "invert", "equal", "notequal", "less", "greater", "equalscalar", "notequalscalar",
                                                "lessscalar", "greaterscalar", "switch", "todtype", "copytensor"};
            bool is_rowwise = false;
            for (const char *o : rowwise_ops) is_rowwise = is_rowwise || t.name == o;
            if (t.name == "newtensor") {
                Layout l;
                l.global = t.vector_i64(0);
                l.elem_bytes = precision_bits(t.returns[0].dtype.precision) / 8;
                l.partitioned = should_partition(l.global, l.elem_bytes, ctx);
                known[t.returns[0].textvalue] = l;
                verdict = "newtensor " + t.returns[0].textvalue + (l.partitioned ? ": partitioned " + std::to_string(l.global[0]) + " rows" : ": whole");
            } else if (t.name == "deltensor") {
                known.erase(t.returns[0].textvalue);
                verdict = "whole";
            } else if (is_rowwise) {
                std::vector<Layout> in;
                for (const auto &q : t.args)
                    if (q.dtype.category & (CAT_TENSOR | CAT_LISTTENSOR))
                        for (const auto &n : names_of(q))
                            if (known.count(n)) in.push_back(known[n]);
                const RowwisePlan p = plan_rowwise(in, layout_of(t.returns[0].textvalue));
                verdict = !p.error.empty() ? "refuse: " + p.error : (!p.by_rows ? "whole" : (p.gather_output ? "rows+allgather" : "rows"));
            } else if (t.name == "sum" || t.name == "prod" || t.name == "reducemax" || t.name == "reducemin") {
                const Layout &a = layout_of(t.args[0].textvalue);
                const ReducePlan p = plan_reduce(a, checked_dims(a.global, t.vector_int(1)), t.var_bool(2), layout_of(t.returns[0].textvalue), dx_comm_max_bytes());
                verdict = p.kind == ReducePlan::REFUSE ? "refuse: " + p.error : reduce_plan_name(p.kind);
            } else {
                bool any = false;
                for (const auto &q : t.args)
                    if (q.dtype.category & (CAT_TENSOR | CAT_LISTTENSOR))
                        for (const auto &n : names_of(q)) any = any || (known.count(n) && known[n].partitioned);
                for (const auto &q : t.returns)
                    for (const auto &n : names_of(q)) any = any || (known.count(n) && known[n].partitioned);
                verdict = any ? "rows-if-aligned" : "whole";
            }
            if (lines++) text += "\n";
            text += verdict;
        }
        if (put(text, out, cap) < 0) { g_err = "output buffer too small"; return -1; }
        return lines;
    } catch (const std::exception &ex) {
        g_err = ex.what();
        return -1;
    }
}

void *dx_registry_new(int with_builtin_ops) {
    auto *r = new Registry();
    if (with_builtin_ops) {
        register_all(r->f);
        r->n = int(r->f.size());
    }
    return r;
}
void dx_registry_free(void *r) { delete static_cast<Registry *>(r); }
int dx_registry_add(void *rv, const char *signature_ir) {
    auto *r = static_cast<Registry *>(rv);
    try {
        auto t = std::make_shared<ProbeTF>();
        t->parse(signature_ir);
        t->index = r->n++;
        r->f.add_tf(t);
        return t->index;
    } catch (...) { return -1; }
}
int dx_registry_get(void *rv, const char *call_ir) {
    auto *r = static_cast<Registry *>(rv);
    try {
        TF q;
        q.parse(call_ir);
        auto got = r->f.get_tf(q);
        if (!got) return -1;
        if (auto p = dynamic_cast<ProbeTF *>(got.get())) return p->index;
        return -2;  // a built-in op matched
    } catch (...) { return -1; }
}
int dx_registry_size(void *rv) { return int(static_cast<Registry *>(rv)->f.size()); }
}
