// Reference-sweep workloads (weighted variance, Pearson, softmax backward, LARS,
// int8 quantisation): instantiations and their selection table.
#include "../../include/credit_b200.h"
#include "kernel_tables.h"
#include "row_op_kernels.cuh"

namespace credit {
namespace {

template <class Op>
const void* pick(bool aligned, bool staged) {
    if (staged)
        return aligned ? (const void*)row_op_kernel<Op, 256, true, true>
                       : (const void*)row_op_kernel<Op, 256, false, true>;
    return aligned ? (const void*)row_op_kernel<Op, 256, true, false>
                   : (const void*)row_op_kernel<Op, 256, false, false>;
}

}  // namespace

const void* row_op_kernel_for(int workload, bool aligned, bool staged) {
    switch (workload) {
        case CREDIT_WL_WEIGHTED_VAR_BACKWARD: return pick<WeightedVarOp>(aligned, staged);
        case CREDIT_WL_PEARSON_BACKWARD: return pick<PearsonOp>(aligned, staged);
        case CREDIT_WL_SOFTMAX_LOGITS_BACKWARD: return pick<SoftmaxBwdOp>(aligned, staged);
        case CREDIT_WL_LARS_MOMENTUM: return pick<LarsOp>(aligned, staged);
        case CREDIT_WL_ROWWISE_QUANT: return pick<QuantOp>(aligned, staged);
        default: return nullptr;
    }
}

}  // namespace credit
