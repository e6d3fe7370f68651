// "block_read" variants: one CTA per row, nothing staged, every pass re-reads the
// row from global memory (L2 / HBM). They are the no-DSMEM baseline the cost model
// compares the cluster kernels with, the role of the reference's block_*_read_kernel
// (src/workloads/layernorm_backward.cu:274-321), with 128-bit loads on aligned rows.
#pragma once

#include "cluster_primitives.cuh"

namespace credit {

// Sum of K per-thread values over the CTA; every thread gets the totals.
template <int K, int THREADS>
__device__ __forceinline__ void block_sum(float (&v)[K], float (*scratch)[kMaxWarpsPerCta]) {
    constexpr int kWarps = THREADS / 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = warp_sum(v[k]);
    __syncthreads();   // scratch may still be read from the previous call
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) scratch[k][warp] = v[k];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = warp_sum(lane < kWarps ? scratch[k][lane] : 0.0f);
}

// Visits the row in 16-byte vectors (aligned rows) or element by element.
template <typename T, int THREADS, bool ALIGNED, typename F>
__device__ __forceinline__ void for_each_chunk(int cols, F f) {
    constexpr int E = RowVec<T>::kElems;
    if (ALIGNED) {
        for (int v = threadIdx.x; v < cols / E; v += THREADS) f(v * E, E);
    } else {
        for (int c = threadIdx.x; c < cols; c += THREADS) f(c, 1);
    }
}

template <typename T, bool ALIGNED>
__device__ __forceinline__ void load_chunk(const T* p, float* out) {
    if (ALIGNED) {
        float tmp[RowVec<T>::kElems];
        RowVec<T>::from_global(p, tmp);
#pragma unroll
        for (int j = 0; j < RowVec<T>::kElems; ++j) out[j] = tmp[j];
    } else {
        out[0] = RowVec<T>::to_float(*p);
    }
}

template <typename T, bool ALIGNED>
__device__ __forceinline__ void store_chunk(T* p, const float* v) {
    if (ALIGNED) {
        float tmp[RowVec<T>::kElems];
#pragma unroll
        for (int j = 0; j < RowVec<T>::kElems; ++j) tmp[j] = v[j];
        RowVec<T>::to_global(p, tmp);
    } else {
        *p = RowVec<T>::from_float(v[0]);
    }
}

template <typename T, int THREADS, bool ALIGNED>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_block_read_kernel(const T* __restrict__ x, const float* __restrict__ gamma, T* __restrict__ y,
                              float eps, int rows, int cols) {
    __shared__ float scratch[1][kMaxWarpsPerCta];
    constexpr int E = ALIGNED ? RowVec<T>::kElems : 1;
    const size_t base = static_cast<size_t>(blockIdx.x) * cols;
    float part[1] = {0.0f};
    for_each_chunk<T, THREADS, ALIGNED>(cols, [&](int c, int) {
        float xv[E];
        load_chunk<T, ALIGNED>(x + base + c, xv);
#pragma unroll
        for (int j = 0; j < E; ++j) part[0] = fmaf(xv[j], xv[j], part[0]);
    });
    block_sum<1, THREADS>(part, scratch);
    const float scale = rsqrtf(part[0] / static_cast<float>(cols) + eps);
    for_each_chunk<T, THREADS, ALIGNED>(cols, [&](int c, int) {
        float xv[E];
        load_chunk<T, ALIGNED>(x + base + c, xv);
#pragma unroll
        for (int j = 0; j < E; ++j) xv[j] = xv[j] * scale * __ldg(gamma + c + j);
        store_chunk<T, ALIGNED>(y + base + c, xv);
    });
}

// mean and biased variance of a row with two passes over global memory
template <typename T, int THREADS, bool ALIGNED>
__device__ __forceinline__ void block_read_mean_var(const T* row, int cols, float (*scratch)[kMaxWarpsPerCta],
                                                    float& mean, float& var) {
    constexpr int E = ALIGNED ? RowVec<T>::kElems : 1;
    float s[1] = {0.0f};
    for_each_chunk<T, THREADS, ALIGNED>(cols, [&](int c, int) {
        float xv[E];
        load_chunk<T, ALIGNED>(row + c, xv);
#pragma unroll
        for (int j = 0; j < E; ++j) s[0] += xv[j];
    });
    block_sum<1, THREADS>(s, scratch);
    mean = s[0] / static_cast<float>(cols);
    float q[1] = {0.0f};
    for_each_chunk<T, THREADS, ALIGNED>(cols, [&](int c, int) {
        float xv[E];
        load_chunk<T, ALIGNED>(row + c, xv);
#pragma unroll
        for (int j = 0; j < E; ++j) {
            const float d = xv[j] - mean;
            q[0] = fmaf(d, d, q[0]);
        }
    });
    block_sum<1, THREADS>(q, scratch);
    var = q[0] / static_cast<float>(cols);
}

template <typename T, int THREADS, bool ALIGNED>
__global__ void __launch_bounds__(THREADS)
layernorm_fwd_block_read_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                                const float* __restrict__ beta, T* __restrict__ y,
                                float* __restrict__ mean_out, float* __restrict__ rstd_out, float eps,
                                int rows, int cols) {
    __shared__ float scratch[2][kMaxWarpsPerCta];
    constexpr int E = ALIGNED ? RowVec<T>::kElems : 1;
    const size_t base = static_cast<size_t>(blockIdx.x) * cols;
    float mean, var;
    block_read_mean_var<T, THREADS, ALIGNED>(x + base, cols, scratch, mean, var);
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
        mean_out[blockIdx.x] = mean;
        rstd_out[blockIdx.x] = rstd;
    }
    for_each_chunk<T, THREADS, ALIGNED>(cols, [&](int c, int) {
        float xv[E];
        load_chunk<T, ALIGNED>(x + base + c, xv);
#pragma unroll
        for (int j = 0; j < E; ++j)
            xv[j] = fmaf((xv[j] - mean) * rstd, __ldg(gamma + c + j), __ldg(beta + c + j));
        store_chunk<T, ALIGNED>(y + base + c, xv);
    });
}

// dx only; HAS_STATS as in the cluster kernels.
template <typename T, int THREADS, bool ALIGNED, bool HAS_STATS>
__global__ void __launch_bounds__(THREADS)
layernorm_bwd_block_read_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                const float* __restrict__ gamma, const float* __restrict__ mean_in,
                                const float* __restrict__ rstd_in, T* __restrict__ dx, float eps, int rows,
                                int cols) {
    __shared__ float scratch[2][kMaxWarpsPerCta];
    constexpr int E = ALIGNED ? RowVec<T>::kElems : 1;
    const size_t base = static_cast<size_t>(blockIdx.x) * cols;
    float mean, rstd;
    if (HAS_STATS) {
        mean = __ldg(mean_in + blockIdx.x);
        rstd = __ldg(rstd_in + blockIdx.x);
    } else {
        float var;
        block_read_mean_var<T, THREADS, ALIGNED>(x + base, cols, scratch, mean, var);
        rstd = rsqrtf(var + eps);
    }
    float part[2] = {0.0f, 0.0f};
    for_each_chunk<T, THREADS, ALIGNED>(cols, [&](int c, int) {
        float xv[E], dv[E];
        load_chunk<T, ALIGNED>(x + base + c, xv);
        load_chunk<T, ALIGNED>(dy + base + c, dv);
#pragma unroll
        for (int j = 0; j < E; ++j) {
            const float g = dv[j] * __ldg(gamma + c + j);
            part[0] += g;
            part[1] = fmaf(g, (xv[j] - mean) * rstd, part[1]);
        }
    });
    block_sum<2, THREADS>(part, scratch);
    const float mean_g = part[0] / static_cast<float>(cols);
    const float mean_gx = part[1] / static_cast<float>(cols);
    for_each_chunk<T, THREADS, ALIGNED>(cols, [&](int c, int) {
        float xv[E], dv[E];
        load_chunk<T, ALIGNED>(x + base + c, xv);
        load_chunk<T, ALIGNED>(dy + base + c, dv);
#pragma unroll
        for (int j = 0; j < E; ++j) {
            const float xhat = (xv[j] - mean) * rstd;
            const float g = dv[j] * __ldg(gamma + c + j);
            xv[j] = (g - mean_g - xhat * mean_gx) * rstd;
        }
        store_chunk<T, ALIGNED>(dx + base + c, xv);
    });
}

}  // namespace credit
