// LayerNorm forward: kernel instantiations and their selection table.
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

template <typename T>
const void* generic_func(int threads, bool aligned) {
    if (threads == 512)
        return aligned ? (const void*)layernorm_fwd_kernel<T, 512, true>
                       : (const void*)layernorm_fwd_kernel<T, 512, false>;
    return aligned ? (const void*)layernorm_fwd_kernel<T, 256, true>
                   : (const void*)layernorm_fwd_kernel<T, 256, false>;
}

template <typename T, bool FULL>
const void* reg_func(int threads, int vpt) {
    if (threads == 512) { CREDIT_PICK_VPT(layernorm_fwd_reg_kernel, T, 512, FULL) }
    CREDIT_PICK_VPT(layernorm_fwd_reg_kernel, T, 256, FULL)
}

template <typename T>
const void* reg_func(int threads, int vpt, bool full) {
    return full ? reg_func<T, true>(threads, vpt) : reg_func<T, false>(threads, vpt);
}

}  // namespace

const void* layernorm_fwd_kernel_for(int dtype, int threads, int vpt, bool full, bool aligned) {
    const bool f32 = dtype == CREDIT_F32;
    if (vpt > 0)
        return f32 ? reg_func<float>(threads, vpt, full) : reg_func<__nv_bfloat16>(threads, vpt, full);
    return f32 ? generic_func<float>(threads, aligned) : generic_func<__nv_bfloat16>(threads, aligned);
}

}  // namespace credit
