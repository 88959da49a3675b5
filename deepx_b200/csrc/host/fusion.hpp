// IR-level fusion: rewrite a multi-line deepxIR program so that the op chains the front end emits
// for RMSNorm and softmax run as one kernel each.
//
// The reference executes one IR line per kernel launch; a norm layer written with its single ops
// (front/py/deepx/nn/modules/norm/t5layernorm.py:19-23, nn/functional/normalization.py:4-18) therefore
// streams the activation through HBM seven to nine times and allocates a tensor per step.  A program
// (several IR lines handed over together: one UDP datagram, udpserver.cpp:49-58, or one
// Executor::run_program call) exposes the whole chain, and when every intermediate tensor is created
// and deleted inside that same program and used by nothing else, the chain is replaced by the fused
// op; the intermediates' newtensor / deltensor lines are dropped with it.  Anything that does not
// match exactly is left as it is: the pass never changes what a program computes, only how many
// launches it takes.
#pragma once
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "core.hpp"

namespace dxh {

struct PlanItem {
    enum Kind { RUN, ABSORBED, FUSED } kind = RUN;
    TF fused;        // kind == FUSED: the op that runs in place of the line
    int group = -1;  // index of the fused group this line belongs to (ABSORBED / FUSED)
};

// dtype (a Precision bit) and shape of a tensor that exists before the program starts; false = no such tensor
using TensorLookup = std::function<bool(const std::string &name, uint16_t &precision, std::vector<int64_t> &shape)>;

// One item per program line, in order.  The lookup (or `mem`) supplies dtype and shape of tensors that
// exist before the program starts; tensors the program creates are tracked from their newtensor lines.
std::vector<PlanItem> plan_fusion(const std::vector<TF> &program, const TensorLookup &existing, FusionStats *stats);
std::vector<PlanItem> plan_fusion(const std::vector<TF> &program, const Mem &mem, FusionStats *stats);

}  // namespace dxh
