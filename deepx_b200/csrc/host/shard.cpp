// Row partitioning: the host-side decisions (shard.hpp says what they are for).
#include "shard.hpp"

#include "core.hpp"

namespace dxh {

RowBlock row_block(int64_t global_rows, int rank, int world) {
    RowBlock b;
    dx_shard_rows(global_rows, rank, world, &b.row0, &b.rows);
    return b;
}

bool should_partition(const std::vector<int64_t> &shape, int elem_bytes, const ShardCtx &ctx) {
    if (!ctx.active() || shape.empty() || shape[0] < ctx.world) return false;
    unsigned __int128 bytes = unsigned(elem_bytes > 0 ? elem_bytes : 1);
    for (int64_t d : shape) {
        if (d <= 0) return false;  // empty tensors are not worth splitting
        bytes *= static_cast<unsigned __int128>(d);
    }
    return bytes >= ctx.min_bytes;
}

static std::string shape_text(const std::vector<int64_t> &s) {
    std::string t = "[";
    for (size_t i = 0; i < s.size(); ++i) t += (i ? "," : "") + std::to_string(s[i]);
    return t + "]";
}

RowwisePlan plan_rowwise(const std::vector<Layout> &inputs, const Layout &output) {
    RowwisePlan p;
    bool any = output.partitioned;
    for (const auto &l : inputs) any = any || l.partitioned;
    for (const auto &l : inputs)
        if (l.global != output.global) {
            p.error = "shape mismatch: " + shape_text(l.global) + " vs " + shape_text(output.global);
            return p;
        }
    if (!any) return p;  // the single-GPU path on whole tensors
    if (output.global.empty()) {
        p.error = "a tensor without axes cannot be row-partitioned";
        return p;
    }
    p.by_rows = true;
    p.gather_output = !output.partitioned;
    return p;
}

ReducePlan plan_reduce(const Layout &in, const std::vector<int> &cd, bool keepdims, const Layout &out, size_t slot_bytes) {
    ReducePlan p;
    p.out_global = reduced_shape(in.global, cd, keepdims);
    int64_t n_out = 1, n_have = 1;
    for (auto v : p.out_global) n_out *= v;
    for (auto v : out.global) n_have *= v;
    if (n_out != n_have) {
        p.kind = ReducePlan::REFUSE;
        p.error = "output has " + std::to_string(n_have) + " elements, expected " + std::to_string(n_out);
        return p;
    }
    bool crosses = false;
    for (int d : cd) crosses = crosses || d == 0;
    if (!in.partitioned) {
        if (out.partitioned) {
            p.kind = ReducePlan::REFUSE;
            p.error = "the output is row-partitioned but the input is not; allocate the input above the partition threshold or the output below it";
            return p;
        }
        p.kind = ReducePlan::WHOLE;
        return p;
    }
    if (!crosses) {
        // the kept axis 0 leads the output: its rows follow the input's partition
        if (out.partitioned) {
            if (out.global.empty() || out.global[0] != in.global[0]) {
                p.kind = ReducePlan::REFUSE;
                p.error = "the output's leading axis must be the input's (" + std::to_string(in.global[0]) + " rows) to share its partition";
                return p;
            }
            p.kind = ReducePlan::ROWS;
        } else {
            if (out.global.empty() || out.global[0] != in.global[0]) {
                p.kind = ReducePlan::REFUSE;
                p.error = "the output's leading axis must be the input's (" + std::to_string(in.global[0]) + " rows)";
                return p;
            }
            p.kind = ReducePlan::ROWS_GATHER;
        }
        return p;
    }
    if (out.partitioned) p.kind = ReducePlan::COMBINE_SCATTER;
    else if (size_t(n_out) * size_t(out.elem_bytes) <= slot_bytes) p.kind = ReducePlan::COMBINE_DEFERRED;
    else p.kind = ReducePlan::COMBINE_ROUNDS;
    return p;
}

const char *reduce_plan_name(ReducePlan::Kind k) {
    switch (k) {
        case ReducePlan::WHOLE: return "whole";
        case ReducePlan::ROWS: return "rows";
        case ReducePlan::ROWS_GATHER: return "rows+allgather";
        case ReducePlan::COMBINE_DEFERRED: return "allreduce(deferred)";
        case ReducePlan::COMBINE_ROUNDS: return "allreduce(rounds)";
        case ReducePlan::COMBINE_SCATTER: return "allreduce(rounds)+keep-own-rows";
        default: return "refuse";
    }
}

}  // namespace dxh
