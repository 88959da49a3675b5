// The fusion pass: see fusion.hpp for what it does and when it applies.
//
// Matching is by name flow.  Starting from the op that ends a chain (the last `mul` of RMSNorm,
// the `div` of softmax) each operand is traced to the line that last wrote it, and that line must
// be the expected op with the expected parameters.  A chain is only rewritten when
//   * every intermediate tensor is mentioned by nothing in the program except the chain itself,
//     one newtensor line before it and one deltensor line after it (so dropping it is invisible),
//     and did not exist before the program;
//   * no other line writes, deletes or re-creates an input between the chain's first read of it
//     and the chain's last line (the fused op reads its inputs where the last line stood);
//   * dtypes and shapes, known from the store or from the program's own newtensor / reshape
//     lines, are those the single ops would have accepted, with the reduction over the last axis.
#include "fusion.hpp"

#include <algorithm>
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <set>
#include <unordered_map>

namespace dxh {
namespace {

// DEEPX_FUSE_DEBUG=1 prints why a candidate chain was left alone.
bool debug_on() {
    static const bool on = [] { const char *e = std::getenv("DEEPX_FUSE_DEBUG"); return e && e[0] == '1'; }();
    return on;
}
bool no(int line, const char *why, const std::string &name = std::string()) {
    if (debug_on())
        std::fprintf(stderr, "fusion: candidate ending at line %d left alone: %s%s%s\n", line, why, name.empty() ? "" : ": ", name.c_str());
    return false;
}

struct Info {
    bool known = false;
    uint16_t prec = 0;
    std::vector<int64_t> shape;
};

bool numeric(const std::string &s, float *out) {
    if (s.empty()) return false;
    char *end = nullptr;
    const float v = std::strtof(s.c_str(), &end);
    if (end == s.c_str() || *end != 0) return false;
    *out = v;
    return true;
}

bool is_lifetime_op(const TF &t) { return t.name == "newtensor" || t.name == "deltensor" || t.name == "renametensor"; }
bool is_op(const TF &t, const char *name, size_t nargs) { return t.name == name && t.args.size() == nargs && t.returns.size() == 1; }

struct Group {
    std::vector<int> chain;  // every op line of the chain, the last one included
    int last = -1;
    std::set<std::string> temps;
    std::vector<std::pair<std::string, int>> inputs;  // name, line of the chain's first read
    TF fused;
    bool rmsnorm = true;
};

struct Pass {
    const std::vector<TF> &prog;
    const TensorLookup &lookup;
    std::unordered_map<std::string, std::vector<int>> mentions;  // name → lines naming it, ascending
    std::vector<char> taken;

    Pass(const std::vector<TF> &p, const TensorLookup &m) : prog(p), lookup(m), taken(p.size(), 0) {
        for (int i = 0; i < int(prog.size()); ++i) {
            // A var / vector parameter is a number, a shape or the name of a stored arg, never a tensor
            // (tensor names are often numerals too: the front end numbers its tensors); the one
            // exception is the new name renametensor carries as a var<string>.
            const bool rename = prog[i].name == "renametensor";
            auto note = [&](const Param &q) {
                const uint8_t cat = q.dtype.category;
                if (!rename && cat != CAT_UNKNOWN && (cat & (CAT_TENSOR | CAT_LISTTENSOR)) == 0) return;
                std::string text = q.textvalue;
                if (!text.empty() && text.front() == '[') {
                    text = text.substr(1, text.size() - (text.back() == ']' ? 2 : 1));
                    size_t pos = 0;
                    while (pos <= text.size()) {
                        const size_t sp = text.find(' ', pos);
                        const std::string item = text.substr(pos, sp == std::string::npos ? std::string::npos : sp - pos);
                        if (!item.empty()) add(item, i);
                        if (sp == std::string::npos) break;
                        pos = sp + 1;
                    }
                } else if (!text.empty()) add(text, i);
            };
            for (const auto &q : prog[i].args) note(q);
            for (const auto &q : prog[i].returns) note(q);
        }
    }
    void add(const std::string &name, int line) {
        auto &v = mentions[name];
        if (v.empty() || v.back() != line) v.push_back(line);
    }

    // dtype and shape of `name` as line `at` sees it
    Info info_at(const std::string &name, int at) const {
        std::vector<int64_t> reshaped;
        bool has_reshape = false;
        auto it = mentions.find(name);
        if (it != mentions.end()) {
            for (auto j = it->second.rbegin(); j != it->second.rend(); ++j) {
                if (*j >= at) continue;
                const TF &t = prog[*j];
                const bool ret0 = !t.returns.empty() && t.returns[0].textvalue == name;
                if (t.name == "renametensor") return Info{};
                if (t.name == "deltensor" && ret0) return Info{};
                try {
                    if (t.name == "newtensor" && ret0) {
                        Info r;
                        r.known = dx_code_of(t.returns[0].dtype.precision) >= 0;
                        r.prec = t.returns[0].dtype.precision;
                        if (has_reshape) r.shape = reshaped;
                        else for (int64_t v : t.vector_i64(0)) r.shape.push_back(v);
                        return r;
                    }
                    if (t.name == "reshape" && ret0 && !has_reshape && t.args.size() == 2) {
                        for (int64_t v : t.vector_i64(1)) reshaped.push_back(v);
                        has_reshape = true;
                    }
                } catch (const std::exception &) {
                    return Info{};
                }
            }
        }
        Info r;
        if (!lookup(name, r.prec, r.shape)) return Info{};
        r.known = true;
        if (has_reshape) r.shape = reshaped;
        return r;
    }

    // the line that last wrote `name` before line `before` (lifetime ops do not write data)
    int producer(const std::string &name, int before) const {
        auto it = mentions.find(name);
        if (it == mentions.end()) return -1;
        for (auto j = it->second.rbegin(); j != it->second.rend(); ++j) {
            if (*j >= before) continue;
            const TF &t = prog[*j];
            bool writes = false;
            for (const auto &r : t.returns) writes |= (r.textvalue == name);
            if (!writes) continue;
            if (is_lifetime_op(t) || taken[*j]) return -1;
            return *j;
        }
        return -1;
    }

    static bool last_axis_keepdims(const TF &t, int rank) {
        try {
            const std::vector<int> dims = t.vector_int(1);
            if (dims.size() != 1) return false;
            const int d = dims[0] < 0 ? dims[0] + rank : dims[0];
            return d == rank - 1 && t.var_bool(2);
        } catch (const std::exception &) {
            return false;
        }
    }
    static bool shape_arg_is(const TF &t, const std::vector<int64_t> &want) {
        try {
            const std::vector<int64_t> s = t.vector_i64(1);
            if (s.size() != want.size()) return false;
            for (size_t i = 0; i < s.size(); ++i)
                if (s[i] != want[i]) return false;
            return true;
        } catch (const std::exception &) {
            return false;
        }
    }

    // x * 1/sqrt(sum(x^2)/c + eps): the part of the RMSNorm chain that ends in mul(x, rb) at `mul_line`
    bool match_inv_rms(int mul_line, const std::string &x, const std::string &rb, Group &g, std::string *divisor, std::string *eps) const {
        const int lb = producer(rb, mul_line);
        if (lb < 0 || !is_op(prog[lb], "broadcastTo", 2)) return false;
        const std::string r = prog[lb].args[0].textvalue;
        const int lr = producer(r, lb);
        float one = 0.f;
        if (lr < 0 || !is_op(prog[lr], "rdivscalar", 2) || !numeric(prog[lr].args[0].textvalue, &one) || one != 1.f) return false;
        const std::string q = prog[lr].args[1].textvalue;
        const int lq = producer(q, lr);
        if (lq < 0 || !is_op(prog[lq], "sqrt", 1)) return false;
        const std::string e = prog[lq].args[0].textvalue;
        const int le = producer(e, lq);
        float tmp = 0.f;
        if (le < 0 || !is_op(prog[le], "addscalar", 2) || !numeric(prog[le].args[1].textvalue, &tmp)) return false;
        const std::string m = prog[le].args[0].textvalue;
        const int lm = producer(m, le);
        if (lm < 0 || !is_op(prog[lm], "divscalar", 2) || !numeric(prog[lm].args[1].textvalue, &tmp)) return false;
        const std::string s = prog[lm].args[0].textvalue;
        const int ls = producer(s, lm);
        if (ls < 0 || !is_op(prog[ls], "sum", 3)) return false;
        const std::string sq = prog[ls].args[0].textvalue;
        const int lsq = producer(sq, ls);
        if (lsq < 0) return false;
        const TF &tsq = prog[lsq];
        float two = 0.f;
        const bool by_pow = is_op(tsq, "powscalar", 2) && numeric(tsq.args[1].textvalue, &two) && two == 2.f;
        const bool by_mul = is_op(tsq, "mul", 2) && tsq.args[0].textvalue == tsq.args[1].textvalue;
        if (!by_pow && !by_mul) return false;
        // The squared tensor is x itself, or the same-dtype copy the front end makes with x.float()
        // (todtype(x)->x'), which holds the same values.
        const std::string xs = tsq.args[0].textvalue;
        int first_read = lsq;
        if (xs != x) {
            const int lc = producer(xs, lsq);
            if (lc < 0 || !is_op(prog[lc], "todtype", 1) || prog[lc].args[0].textvalue != x) return false;
            const Info A = info_at(x, lc), B = info_at(xs, lc + 1);
            if (!A.known || !B.known || A.prec != B.prec || A.shape != B.shape) return false;
            first_read = lc;
        }
        const Info X = info_at(x, first_read);
        if (!X.known || X.shape.empty()) return false;
        if (!last_axis_keepdims(prog[ls], int(X.shape.size())) || !shape_arg_is(prog[lb], X.shape)) return false;
        std::vector<int64_t> small = X.shape;
        small.back() = 1;
        const std::pair<std::string, int> smalls[] = {{s, ls}, {m, lm}, {e, le}, {q, lq}, {r, lr}};
        for (const auto &p : smalls)
            if (!has(p.first, p.second + 1, X.prec, small)) return false;
        if (!has(sq, lsq + 1, X.prec, X.shape) || !has(rb, lb + 1, X.prec, X.shape)) return false;
        for (int l : {lsq, ls, lm, le, lq, lr, lb, mul_line}) g.chain.push_back(l);
        for (const auto &n : {sq, s, m, e, q, r, rb}) g.temps.insert(n);
        g.inputs.push_back({x, first_read});
        *divisor = prog[lm].args[1].textvalue;
        *eps = prog[le].args[1].textvalue;
        return true;
    }
    bool has(const std::string &name, int at, uint16_t prec, const std::vector<int64_t> &shape) const {
        const Info i = info_at(name, at);
        return i.known && i.prec == prec && i.shape == shape;
    }

    bool try_rmsnorm(int k, bool weighted, Group &out) const {
        const TF &t = prog[k];
        if (!is_op(t, "mul", 2)) return false;
        const std::string dst = t.returns[0].textvalue;
        for (int order = 0; weighted && order < 2; ++order) {  // mul(wb, y) or mul(y, wb)
            const std::string wb = t.args[order].textvalue, y = t.args[1 - order].textvalue;
            const int lwb = producer(wb, k), ly = producer(y, k);
            if (lwb < 0 || ly < 0 || !is_op(prog[lwb], "broadcastTo", 2) || !is_op(prog[ly], "mul", 2)) continue;
            for (int o2 = 0; o2 < 2; ++o2) {
                Group g;
                std::string divisor, eps;
                const std::string x = prog[ly].args[o2].textvalue, rb = prog[ly].args[1 - o2].textvalue;
                if (!match_inv_rms(ly, x, rb, g, &divisor, &eps)) continue;
                const Info X = info_at(x, k);
                const std::string w = prog[lwb].args[0].textvalue;
                const Info W = info_at(w, lwb);
                if (!X.known || !W.known || W.prec != X.prec || W.shape.empty() || W.shape.back() != X.shape.back()) continue;
                int64_t wn = 1;
                for (auto v : W.shape) wn *= v;
                if (wn != X.shape.back() || !shape_arg_is(prog[lwb], X.shape)) continue;
                if (!has(wb, lwb + 1, X.prec, X.shape) || !has(y, ly + 1, X.prec, X.shape) || !has(dst, k, X.prec, X.shape)) continue;
                g.chain.push_back(lwb);
                g.chain.push_back(k);
                g.temps.insert(wb);
                g.temps.insert(y);
                g.inputs.push_back({w, lwb});
                g.last = k;
                g.fused = t;
                g.fused.name = "rmsnorm";
                g.fused.args = {Param(x, CAT_TENSOR, X.prec), Param(w, CAT_TENSOR, X.prec), Param(divisor, CAT_VAR, P_F32), Param(eps, CAT_VAR, P_F32)};
                out = std::move(g);
                return true;
            }
        }
        for (int order = 0; !weighted && order < 2; ++order) {  // no weight: the chain ends at mul(x, rb)
            Group g;
            std::string divisor, eps;
            const std::string x = t.args[order].textvalue, rb = t.args[1 - order].textvalue;
            if (!match_inv_rms(k, x, rb, g, &divisor, &eps)) continue;
            const Info X = info_at(x, k);
            if (!X.known || !has(dst, k, X.prec, X.shape)) continue;
            g.last = k;
            g.fused = t;
            g.fused.name = "rmsnorm";
            g.fused.args = {Param(x, CAT_TENSOR, X.prec), Param(divisor, CAT_VAR, P_F32), Param(eps, CAT_VAR, P_F32)};
            out = std::move(g);
            return true;
        }
        return false;
    }

    bool try_softmax(int k, Group &out) const {
        const TF &t = prog[k];
        if (!is_op(t, "div", 2)) return false;
        const std::string e2 = t.args[0].textvalue, sb = t.args[1].textvalue, dst = t.returns[0].textvalue;
        const int lsb = producer(sb, k), le2 = producer(e2, k);
        if (lsb < 0 || le2 < 0 || !is_op(prog[lsb], "broadcastTo", 2) || !is_op(prog[le2], "exp", 1)) return false;
        const std::string s = prog[lsb].args[0].textvalue;
        const int ls = producer(s, lsb);
        if (ls < 0 || !is_op(prog[ls], "sum", 3)) return false;
        const std::string e1 = prog[ls].args[0].textvalue;
        const int le1 = producer(e1, ls);
        if (le1 < 0 || !is_op(prog[le1], "exp", 1)) return false;
        const std::string d = prog[le1].args[0].textvalue;
        if (prog[le2].args[0].textvalue != d) return false;
        const int ld = producer(d, std::min(le1, le2));
        if (ld < 0 || ld != producer(d, std::max(le1, le2)) || !is_op(prog[ld], "sub", 2)) return false;
        const std::string x = prog[ld].args[0].textvalue, mb = prog[ld].args[1].textvalue;
        const int lmb = producer(mb, ld);
        if (lmb < 0 || !is_op(prog[lmb], "broadcastTo", 2)) return false;
        const std::string m = prog[lmb].args[0].textvalue;
        const int lm = producer(m, lmb);
        if (lm < 0 || !is_op(prog[lm], "reducemax", 3) || prog[lm].args[0].textvalue != x) return false;
        const Info X = info_at(x, lm);
        if (!X.known || X.shape.empty()) return false;
        const int rank = int(X.shape.size());
        if (!last_axis_keepdims(prog[lm], rank) || !last_axis_keepdims(prog[ls], rank)) return false;
        if (!shape_arg_is(prog[lmb], X.shape) || !shape_arg_is(prog[lsb], X.shape)) return false;
        std::vector<int64_t> small = X.shape;
        small.back() = 1;
        if (!has(m, lm + 1, X.prec, small) || !has(s, ls + 1, X.prec, small)) return false;
        const std::pair<std::string, int> fulls[] = {{mb, lmb}, {d, ld}, {e1, le1}, {e2, le2}, {sb, lsb}};
        for (const auto &p : fulls)
            if (!has(p.first, p.second + 1, X.prec, X.shape)) return false;
        if (!has(dst, k, X.prec, X.shape)) return false;
        Group g;
        g.rmsnorm = false;
        for (int l : {lm, lmb, ld, le1, le2, ls, lsb, k}) g.chain.push_back(l);
        for (const auto &n : {m, mb, d, e1, e2, s, sb}) g.temps.insert(n);
        g.inputs.push_back({x, lm});
        g.last = k;
        g.fused = t;
        g.fused.name = "softmax";
        g.fused.args = {Param(x, CAT_TENSOR, X.prec)};
        out = std::move(g);
        return true;
    }

    // The checks that make dropping the chain invisible; on success `extra` gets the temps'
    // newtensor / deltensor lines.
    bool removable(Group &g, std::vector<int> &extra) const {
        std::sort(g.chain.begin(), g.chain.end());
        g.chain.erase(std::unique(g.chain.begin(), g.chain.end()), g.chain.end());
        const std::string dst = prog[g.last].returns[0].textvalue;
        const Info D = info_at(dst, g.last);
        if (!D.known || dx_code_of(D.prec) < 0 || dx_code_of(D.prec) > DX_BF16) return no(g.last, "output dtype unknown or not a float dtype");
        if (g.temps.count(dst)) return no(g.last, "the output is also an intermediate");
        for (const auto &in : g.inputs)
            if (g.temps.count(in.first)) return no(g.last, "an input is also an intermediate");
        for (int l : g.chain)
            if (taken[l] || prog[l].metadata.benchmark_repeat > 0) return no(g.last, "a chain line is shared with another group or is being timed");
        auto in_chain = [&](int l) { return std::binary_search(g.chain.begin(), g.chain.end(), l); };
        for (const auto &name : g.temps) {
            uint16_t prec;
            std::vector<int64_t> shape;
            if (lookup(name, prec, shape)) return no(g.last, "an intermediate existed before the program", name);
            int created = -1, deleted = -1, first = INT_MAX, last = -1;
            for (int l : mentions.at(name)) {
                if (in_chain(l)) {
                    first = std::min(first, l);
                    last = std::max(last, l);
                    continue;
                }
                const TF &t = prog[l];
                const bool ret_only = t.returns.size() == 1 && t.returns[0].textvalue == name;
                if (t.name == "newtensor" && ret_only && created < 0 && !taken[l]) created = l;
                else if (t.name == "deltensor" && ret_only && t.args.empty() && deleted < 0 && !taken[l]) deleted = l;
                else return no(g.last, "an intermediate is named by a line outside the chain", name);
            }
            if (created < 0 || deleted < 0 || created > first || deleted < last)
                return no(g.last, "an intermediate is not created and deleted inside the program", name);
            extra.push_back(created);
            extra.push_back(deleted);
        }
        for (const auto &in : g.inputs) {
            auto it = mentions.find(in.first);
            if (it == mentions.end()) continue;
            for (int l : it->second) {
                if (l <= in.second || l >= g.last || in_chain(l)) continue;
                for (const auto &r : prog[l].returns)
                    if (r.textvalue == in.first) return no(g.last, "an input is rewritten or deleted under the chain");
                if (prog[l].name == "renametensor") return no(g.last, "an input is renamed under the chain");
            }
        }
        return true;
    }
};

}  // namespace

std::vector<PlanItem> plan_fusion(const std::vector<TF> &program, const Mem &mem, FusionStats *stats) {
    return plan_fusion(program, [&mem](const std::string &name, uint16_t &prec, std::vector<int64_t> &shape) {
        if (!mem.exists_tensor(name)) return false;
        const TensorPtr t = mem.get_tensor(name);
        prec = t->shape.dtype;
        shape = t->shape.shape;
        return true;
    }, stats);
}

std::vector<PlanItem> plan_fusion(const std::vector<TF> &program, const TensorLookup &lookup, FusionStats *stats) {
    std::vector<PlanItem> plan(program.size());
    if (stats) ++stats->programs;
    if (program.size() < 8) return plan;  // the shortest chain has eight ops
    Pass pass(program, lookup);
    int groups = 0;
    // sweep 0: chains that end in the weight multiply, and softmax; sweep 1: RMSNorm without a weight
    // (tried second, or it would claim the front part of a weighted chain)
    for (int sweep = 0; sweep < 2; ++sweep) {
        for (int k = 0; k < int(program.size()); ++k) {
            if (pass.taken[k]) continue;
            Group g;
            const bool hit = sweep == 0 ? (pass.try_rmsnorm(k, true, g) || pass.try_softmax(k, g)) : pass.try_rmsnorm(k, false, g);
            if (!hit) continue;
            std::vector<int> extra;
            if (!pass.removable(g, extra)) continue;
            for (int l : g.chain) {
                pass.taken[l] = 1;
                plan[l].kind = PlanItem::ABSORBED;
                plan[l].group = groups;
            }
            for (int l : extra) {
                pass.taken[l] = 1;
                plan[l].kind = PlanItem::ABSORBED;
                plan[l].group = groups;
            }
            plan[g.last].kind = PlanItem::FUSED;
            plan[g.last].fused = g.fused;
            if (stats) {
                ++(g.rmsnorm ? stats->rmsnorm_groups : stats->softmax_groups);
                stats->lines_absorbed += g.chain.size() + extra.size() - 1;
            }
            ++groups;
        }
    }
    return plan;
}

}  // namespace dxh
