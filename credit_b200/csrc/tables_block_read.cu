// block_read baseline kernels: instantiations and their selection table.
#include <cuda_bf16.h>

#include "../../include/credit_b200.h"
#include "block_read_kernels.cuh"
#include "kernel_tables.h"

namespace credit {
namespace {

template <typename T>
const void* pick(int workload, bool aligned, bool has_stats) {
    switch (workload) {
        case CREDIT_WL_RMSNORM_FORWARD:
            return aligned ? (const void*)rmsnorm_fwd_block_read_kernel<T, 512, true>
                           : (const void*)rmsnorm_fwd_block_read_kernel<T, 512, false>;
        case CREDIT_WL_LAYERNORM_FORWARD:
            return aligned ? (const void*)layernorm_fwd_block_read_kernel<T, 512, true>
                           : (const void*)layernorm_fwd_block_read_kernel<T, 512, false>;
        case CREDIT_WL_LAYERNORM_BACKWARD:
        case CREDIT_WL_LAYERNORM_BACKWARD_STATS:
            if (has_stats)
                return aligned ? (const void*)layernorm_bwd_block_read_kernel<T, 512, true, true>
                               : (const void*)layernorm_bwd_block_read_kernel<T, 512, false, true>;
            return aligned ? (const void*)layernorm_bwd_block_read_kernel<T, 512, true, false>
                           : (const void*)layernorm_bwd_block_read_kernel<T, 512, false, false>;
        default:
            return nullptr;
    }
}

}  // namespace

const void* block_read_kernel_for(int workload, int dtype, bool aligned) {
    const bool has_stats = workload == CREDIT_WL_LAYERNORM_BACKWARD_STATS;
    return dtype == CREDIT_F32 ? pick<float>(workload, aligned, has_stats)
                               : pick<__nv_bfloat16>(workload, aligned, has_stats);
}

}  // namespace credit
