// Kernel selection: each function returns the __global__ entry point for a
// configuration (or nullptr if it was not instantiated). Every kernel family is
// compiled in its own translation unit so the library builds in parallel.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace credit {

// vpt > 0 selects the register-resident kernel with that many 16-byte vectors per
// thread (full: every thread of every CTA owns exactly vpt vectors, so the kernel
// carries no bounds checks); vpt == 0 the generic shared-memory kernel (aligned
// or scalar).
const void* rmsnorm_kernel_for(int dtype, int threads, int vpt, bool full, bool aligned);
const void* layernorm_fwd_kernel_for(int dtype, int threads, int vpt, bool full, bool aligned);
const void* layernorm_bwd_kernel_for(int dtype, int threads, int vpt, bool full, bool aligned,
                                     bool has_stats, bool grads);
const void* row_reduce_kernel_for(int load_path, int threads, bool aligned);
// Warp-specialised kernels (ws_row_kernels.cuh): `out_warps` output warps (16 or 8) of `vpt` 16-byte
// vectors per thread plus three service warps; arguments (NormParams, StagedArgs).
const void* ws_rmsnorm_kernel_for(int dtype, int out_warps, int vpt, bool full);
const void* ws_layernorm_fwd_kernel_for(int dtype, int out_warps, int vpt, bool full);
const void* ws_layernorm_bwd_kernel_for(int dtype, int out_warps, int vpt, bool full);
const void* ws_layernorm_bwd_dx_kernel_for(int dtype, int out_warps, int vpt, bool full, bool recompute);
// Reference-sweep workloads on the same pipeline (fp32, 8 output warps, slices of any length).
const void* ws_row_op_kernel_for(int workload);
// One CTA of 512 threads per row, nothing staged (CREDIT_VARIANT_BLOCK_READ).
const void* block_read_kernel_for(int workload, int dtype, bool aligned);
// Reference-sweep workloads (CREDIT_WL_WEIGHTED_VAR_BACKWARD ... CREDIT_WL_ROWWISE_QUANT), fp32;
// staged = false: the no-staging, one-CTA-per-row form.
const void* row_op_kernel_for(int workload, int threads, bool aligned, bool staged);

// Column sums of LayerNorm backward for shapes outside the register path, and
// the finishing reduction over per-cluster (or per-row-block) partials.
cudaError_t launch_layernorm_bwd_colsum(int dtype, const void* x, const void* dy, const float* mean,
                                        const float* rstd, float* partials, int rows, int cols,
                                        int num_blocks, cudaStream_t stream);
cudaError_t launch_layernorm_bwd_finish(const float* partials, float* dgamma, float* dbeta, int cols,
                                        int num_partials, cudaStream_t stream);

// Fused FFN (tcgen05 GEMMs). ffn_check_shape returns nullptr or the reason the
// shape is not supported.
const char* ffn_check_shape(int64_t m, int64_t d, int64_t h);
cudaError_t launch_ffn_pack_weight(const void* w, void* packed, int k, int n, cudaStream_t stream);
// Scratch after the hidden activations: partial tiles and flags of the split row-block walk.
size_t ffn_scratch_bytes(int64_t d);
cudaError_t launch_ffn_forward(const void* x, const void* w1p, const void* w2p, const float* gamma, void* y,
                               void* hidden, void* scratch, int m, int d, int h, float eps, int* status,
                               cudaStream_t stream, bool* bad_map);

}  // namespace credit
