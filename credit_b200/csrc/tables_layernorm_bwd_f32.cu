// LayerNorm backward, f32 rows: register-path kernel instantiations.
#include <cuda_bf16.h>

#include "../../include/credit_b200.h"
#include "kernel_tables.h"
#include "norm_kernels.cuh"
#include "register_row_kernels.cuh"

namespace credit {
namespace {

#define CREDIT_PICK_VPT(KERNEL, T, THREADS, FULL, ...)                     \
    switch (vpt) {                                                     \
        case 1: return (const void*)KERNEL<T, THREADS, 1, FULL __VA_ARGS__>; \
        case 2: return (const void*)KERNEL<T, THREADS, 2, FULL __VA_ARGS__>; \
        case 4: return (const void*)KERNEL<T, THREADS, 4, FULL __VA_ARGS__>; \
        case 8: return (const void*)KERNEL<T, THREADS, 8, FULL __VA_ARGS__>; \
        default: return nullptr;                                       \
    }
#define CREDIT_COMMA ,

template <typename T, bool FULL>
const void* reg_func(int threads, int vpt, bool has_stats, bool grads) {
    if (!has_stats) {
        if (threads == 512) { CREDIT_PICK_VPT(layernorm_bwd_reg_kernel, T, 512, FULL, CREDIT_COMMA false CREDIT_COMMA false) }
        CREDIT_PICK_VPT(layernorm_bwd_reg_kernel, T, 256, FULL, CREDIT_COMMA false CREDIT_COMMA false)
    }
    if (!grads) {
        if (threads == 512) { CREDIT_PICK_VPT(layernorm_bwd_reg_kernel, T, 512, FULL, CREDIT_COMMA true CREDIT_COMMA false) }
        CREDIT_PICK_VPT(layernorm_bwd_reg_kernel, T, 256, FULL, CREDIT_COMMA true CREDIT_COMMA false)
    }
    if (threads == 512) { CREDIT_PICK_VPT(layernorm_bwd_reg_kernel, T, 512, FULL, CREDIT_COMMA true CREDIT_COMMA true) }
    CREDIT_PICK_VPT(layernorm_bwd_reg_kernel, T, 256, FULL, CREDIT_COMMA true CREDIT_COMMA true)
}

}  // namespace

const void* layernorm_bwd_reg_kernel_f32(int threads, int vpt, bool full, bool has_stats,
                                             bool grads) {
    return full ? reg_func<float, true>(threads, vpt, has_stats, grads)
                : reg_func<float, false>(threads, vpt, has_stats, grads);
}

}  // namespace credit
