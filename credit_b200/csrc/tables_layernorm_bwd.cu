// LayerNorm backward: generic kernels, column-sum helpers and the selection table.
#include <cuda_bf16.h>

#include "../../include/credit_b200.h"
#include "kernel_tables.h"
#include "norm_kernels.cuh"
#include "register_row_kernels.cuh"

namespace credit {
namespace {

// Column sums dgamma/dbeta for shapes the register-path kernel cannot take (rows
// not 16-byte aligned, or slices wider than its register budget): one CTA per
// (256-column tile, row block) writes a [2][cols] partial per row block into the
// same `partials` layout, so the same finishing kernel applies.
template <typename T>
__global__ void __launch_bounds__(256)
layernorm_bwd_colsum_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                            const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                            float* __restrict__ partials, int rows, int cols, int rows_per_block) {
    const int col = blockIdx.x * 256 + threadIdx.x;
    const int block = blockIdx.y;
    const int r0 = block * rows_per_block;
    const int r1 = min(rows, r0 + rows_per_block);
    if (col >= cols) return;
    float sg = 0.0f, sb = 0.0f;
    for (int r = r0; r < r1; ++r) {
        const float m = __ldg(mean_in + r);
        const float rs = __ldg(rstd_in + r);
        const size_t idx = static_cast<size_t>(r) * cols + col;
        const float xv = RowVec<T>::to_float(x[idx]);
        const float dv = RowVec<T>::to_float(dy[idx]);
        sg = fmaf(dv, (xv - m) * rs, sg);
        sb += dv;
    }
    partials[(static_cast<size_t>(block) * 2 + 0) * cols + col] = sg;
    partials[(static_cast<size_t>(block) * 2 + 1) * cols + col] = sb;
}

// dgamma[c] = sum_k partials[k][0][c], dbeta[c] = sum_k partials[k][1][c], k in
// fixed order: deterministic, no atomics.
__global__ void __launch_bounds__(256)
layernorm_bwd_finish_kernel(const float* __restrict__ partials, float* __restrict__ dgamma,
                            float* __restrict__ dbeta, int cols, int num_partials) {
    const int col = blockIdx.x * 256 + threadIdx.x;
    if (col >= cols) return;
    float sg = 0.0f, sb = 0.0f;
    for (int k = 0; k < num_partials; ++k) {
        sg += partials[(static_cast<size_t>(k) * 2 + 0) * cols + col];
        sb += partials[(static_cast<size_t>(k) * 2 + 1) * cols + col];
    }
    dgamma[col] = sg;
    dbeta[col] = sb;
}


// dx only; statistics recomputed (has_stats=false) or given.
template <typename T>
const void* generic_func(int threads, bool aligned, bool has_stats) {
    if (has_stats) {
        if (threads == 512)
            return aligned ? (const void*)layernorm_bwd_kernel<T, 512, true, true>
                           : (const void*)layernorm_bwd_kernel<T, 512, false, true>;
        return aligned ? (const void*)layernorm_bwd_kernel<T, 256, true, true>
                       : (const void*)layernorm_bwd_kernel<T, 256, false, true>;
    }
    if (threads == 512)
        return aligned ? (const void*)layernorm_bwd_kernel<T, 512, true, false>
                       : (const void*)layernorm_bwd_kernel<T, 512, false, false>;
    return aligned ? (const void*)layernorm_bwd_kernel<T, 256, true, false>
                   : (const void*)layernorm_bwd_kernel<T, 256, false, false>;
}

}  // namespace

const void* layernorm_bwd_reg_kernel_f32(int threads, int vpt, bool full, bool has_stats, bool grads);
const void* layernorm_bwd_reg_kernel_bf16(int threads, int vpt, bool full, bool has_stats, bool grads);

const void* layernorm_bwd_kernel_for(int dtype, int threads, int vpt, bool full, bool aligned,
                                     bool has_stats, bool grads) {
    const bool f32 = dtype == CREDIT_F32;
    if (vpt > 0)
        return f32 ? layernorm_bwd_reg_kernel_f32(threads, vpt, full, has_stats, grads)
                   : layernorm_bwd_reg_kernel_bf16(threads, vpt, full, has_stats, grads);
    return f32 ? generic_func<float>(threads, aligned, has_stats)
               : generic_func<__nv_bfloat16>(threads, aligned, has_stats);
}

cudaError_t launch_layernorm_bwd_colsum(int dtype, const void* x, const void* dy, const float* mean,
                                        const float* rstd, float* partials, int rows, int cols,
                                        int num_blocks, cudaStream_t stream) {
    const int col_blocks = (cols + 255) / 256;
    const int rows_per_block = (rows + num_blocks - 1) / num_blocks;
    dim3 grid(static_cast<unsigned>(col_blocks), static_cast<unsigned>(num_blocks));
    if (dtype == CREDIT_F32)
        layernorm_bwd_colsum_kernel<float><<<grid, 256, 0, stream>>>(
            static_cast<const float*>(x), static_cast<const float*>(dy), mean, rstd, partials, rows,
            cols, rows_per_block);
    else
        layernorm_bwd_colsum_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), mean, rstd,
            partials, rows, cols, rows_per_block);
    return cudaGetLastError();
}

cudaError_t launch_layernorm_bwd_finish(const float* partials, float* dgamma, float* dbeta, int cols,
                                        int num_partials, cudaStream_t stream) {
    const int col_blocks = (cols + 255) / 256;
    layernorm_bwd_finish_kernel<<<col_blocks, 256, 0, stream>>>(partials, dgamma, dbeta, cols,
                                                               num_partials);
    return cudaGetLastError();
}

}  // namespace credit
