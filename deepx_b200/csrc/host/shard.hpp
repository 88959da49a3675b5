// Row partitioning of the executor's tensors over several GPUs: the host-side decisions.
//
// The reference executor is single-GPU (one Mem, one device: executor/op-cuda/src/client/main.cpp:22-105;
// the heap-tensor record has a single `device` field, executor/heapmem-cuda/README.md:19,29).  Here an
// executor can be ONE OF `world` ranks, one process per GPU, all of which receive the same IR lines:
//   * a tensor of at least `min_bytes` whose leading axis has at least `world` indices is ROW-PARTITIONED:
//     each rank holds a contiguous block of leading-axis rows (dx_shard_rows) in its own pool; smaller
//     tensors are REPLICATED (every rank holds all of it and computes the same values);
//   * ops that work row by row (elementwise, compare, switch, cast, reductions that keep axis 0, the fused
//     row chains, transposes/concats/gathers that leave axis 0 alone, batched or row-split matmul) run on
//     the local rows with no communication; a replicated operand of the same global shape is used through
//     its local rows, a replicated OUTPUT is computed by rows and then all-gathered;
//   * a reduction that removes axis 0 reduces the local rows and combines the per-rank partials over
//     NVLink peer memory (dx_comm): deferred when the result fits a mailbox slot, in rounds otherwise;
//   * anything else on a partitioned tensor is refused with an error reply that says so.
// Everything in this file is pure host logic (no CUDA calls) so that it can be tested without a GPU; ops.cpp
// executes the plans.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

struct dx_comm;

namespace dxh {

struct ShardCtx {
    int rank = 0, world = 1;
    size_t min_bytes = size_t(1) << 20;  // DEEPX_SHARD_MIN_BYTES / dx_exec_set_shard
    dx_comm *comm = nullptr;             // not owned; connected before any partitioned op runs
    bool active() const { return world > 1; }
};

struct RowBlock {
    int64_t row0 = 0, rows = 0;
};
RowBlock row_block(int64_t global_rows, int rank, int world);  // == dx_shard_rows

// Whether newtensor partitions a tensor of this shape.
bool should_partition(const std::vector<int64_t> &shape, int elem_bytes, const ShardCtx &ctx);

// A tensor as the planner sees it: its GLOBAL shape and whether it is partitioned.
struct Layout {
    bool partitioned = false;
    std::vector<int64_t> global;
    int elem_bytes = 4;
};

// Ops that work row by row on operands of one global shape.
struct RowwisePlan {
    bool by_rows = false;        // run on this rank's rows (else: on the whole, replicated tensors)
    bool gather_output = false;  // the output is replicated but was computed by rows: all-gather its row blocks
    std::string error;           // non-empty: refuse
};
RowwisePlan plan_rowwise(const std::vector<Layout> &inputs, const Layout &output);

struct ReducePlan {
    enum Kind {
        WHOLE,             // nothing partitioned: the single-GPU path
        ROWS,              // axis 0 kept, output partitioned like the input: local reduction only
        ROWS_GATHER,       // axis 0 kept, output replicated: local reduction into its row block, then all-gather
        COMBINE_DEFERRED,  // axis 0 reduced, result fits a mailbox slot: reduce + publish, combine deferred
        COMBINE_ROUNDS,    // axis 0 reduced, larger replicated result: local reduction, all-reduce in rounds
        COMBINE_SCATTER,   // axis 0 reduced, PARTITIONED result: all-reduce of the whole partial in a temporary, keep own rows
        REFUSE
    } kind = WHOLE;
    std::vector<int64_t> out_global;  // the reduced shape of the global input
    std::string error;
};
ReducePlan plan_reduce(const Layout &in, const std::vector<int> &checked_dims, bool keepdims, const Layout &out, size_t slot_bytes);

const char *reduce_plan_name(ReducePlan::Kind k);

}  // namespace dxh
