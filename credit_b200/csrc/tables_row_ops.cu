// Reference-sweep workloads (weighted variance, Pearson, softmax backward, LARS,
// int8 quantisation): instantiations and their selection table.
#include "../../include/credit_b200.h"
#include "kernel_tables.h"
#include "row_op_kernels.cuh"

namespace credit {
namespace {

template <class Op, int THREADS>
const void* pick_threads(bool aligned, bool staged) {
    if (staged)
        return aligned ? (const void*)row_op_kernel<Op, THREADS, true, true>
                       : (const void*)row_op_kernel<Op, THREADS, false, true>;
    return aligned ? (const void*)row_op_kernel<Op, THREADS, true, false>
                   : (const void*)row_op_kernel<Op, THREADS, false, false>;
}

template <class Op>
const void* pick(int threads, bool aligned, bool staged) {
    return threads == 512 ? pick_threads<Op, 512>(aligned, staged) : pick_threads<Op, 256>(aligned, staged);
}

}  // namespace

const void* row_op_kernel_for(int workload, int threads, bool aligned, bool staged) {
    switch (workload) {
        case CREDIT_WL_WEIGHTED_VAR_BACKWARD: return pick<WeightedVarOp>(threads, aligned, staged);
        case CREDIT_WL_PEARSON_BACKWARD: return pick<PearsonOp>(threads, aligned, staged);
        case CREDIT_WL_SOFTMAX_LOGITS_BACKWARD: return pick<SoftmaxBwdOp>(threads, aligned, staged);
        case CREDIT_WL_LARS_MOMENTUM: return pick<LarsOp>(threads, aligned, staged);
        case CREDIT_WL_ROWWISE_QUANT: return pick<QuantOp>(threads, aligned, staged);
        default: return nullptr;
    }
}

}  // namespace credit
