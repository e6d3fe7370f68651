// Warp-specialised kernel instantiations: the five reference-sweep workloads.
#include "../../include/credit_b200.h"
#include "kernel_tables.h"
#include "ws_row_ops.cuh"

namespace credit {

const void* ws_row_op_kernel_for(int workload) {
    switch (workload) {
        case CREDIT_WL_WEIGHTED_VAR_BACKWARD: return (const void*)ws_row_kernel<WsWeightedVarOp>;
        case CREDIT_WL_PEARSON_BACKWARD: return (const void*)ws_row_kernel<WsPearsonOp>;
        case CREDIT_WL_SOFTMAX_LOGITS_BACKWARD: return (const void*)ws_row_kernel<WsSoftmaxBwdOp>;
        case CREDIT_WL_LARS_MOMENTUM: return (const void*)ws_row_kernel<WsLarsOp>;
        case CREDIT_WL_ROWWISE_QUANT: return (const void*)ws_row_kernel<WsQuantOp>;
        default: return nullptr;
    }
}

}  // namespace credit
