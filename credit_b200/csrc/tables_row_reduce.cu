// Streaming row reduction: kernel instantiations and their selection table.
#include "../../include/credit_b200.h"
#include "kernel_tables.h"
#include "reduce_kernels.cuh"

namespace credit {

const void* row_reduce_kernel_for(int load_path, int threads, bool aligned) {
    if (load_path == CREDIT_LOAD_TMA)
        return threads == 512 ? (const void*)row_reduce_tma_kernel<512>
                              : (const void*)row_reduce_tma_kernel<256>;
    if (!aligned) return (const void*)row_reduce_ldg_kernel<256, 1, false>;
    return threads == 512 ? (const void*)row_reduce_ldg_kernel<512, 4, true>
                          : (const void*)row_reduce_ldg_kernel<256, 8, true>;
}

}  // namespace credit
