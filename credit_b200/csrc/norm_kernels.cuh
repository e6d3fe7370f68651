// Staged wide-row kernels: RMSNorm forward, LayerNorm forward, LayerNorm
// backward. One thread-block cluster owns a row at a time; CTA `rank` keeps the
// column slice [rank*slice, rank*slice+local) of that row in shared memory
// (filled by bulk-async copies behind an mbarrier, or by scalar loads when the
// row is not 16-byte aligned), per-CTA partial statistics are exchanged through
// distributed shared memory, and the outputs are produced from the staged copy,
// so every input byte crosses HBM once. A cluster walks rows
// cluster, cluster+num_clusters, ... with a ring of `stages` slices so the next
// rows are already in flight while the current one is reduced and written.
//
// The family re-designs the reference's cluster_*_staged_kernel
// (src/workloads/layernorm_backward.cu:376-438) for sm_100a.
#pragma once

#include "cluster_primitives.cuh"

namespace credit {

// Control block at the start of dynamic shared memory.
template <int K>
struct alignas(16) StagedControl {
    uint64_t full[kMaxStages];   // "slice has landed" barriers, one per ring stage
    ReduceScratch<K> red;
};

// Issues the bulk copies that bring NIN slices of `row` into ring stage `stage`.
// Called by one thread.
template <typename T, int NIN>
__device__ __forceinline__ void issue_slice_fill(const T* const (&src)[NIN], unsigned char* data,
                                                 uint64_t* full, int stage, int row,
                                                 const StagedArgs& a, const SliceGeom& g) {
    const uint32_t local_bytes = static_cast<uint32_t>(g.local) * sizeof(T);
    const uint32_t slice_bytes = static_cast<uint32_t>(a.slice_elems) * sizeof(T);
    const uint32_t bar = smem_u32(&full[stage]);
    mbar_arrive_expect_tx(bar, local_bytes * NIN);
    const size_t offset = static_cast<size_t>(row) * a.cols + g.start;
#pragma unroll
    for (int n = 0; n < NIN; ++n) {
        const uint32_t dst = smem_u32(data + (static_cast<size_t>(stage) * NIN + n) * slice_bytes);
        bulk_load_chunked(dst, src[n] + offset, local_bytes, bar);
    }
}

// Scalar fallback fill (rows that are not 16-byte aligned): all threads copy.
template <typename T, int NIN, int THREADS>
__device__ __forceinline__ void scalar_slice_fill(const T* const (&src)[NIN], unsigned char* data,
                                                  int row, const StagedArgs& a,
                                                  const SliceGeom& g) {
    const size_t offset = static_cast<size_t>(row) * a.cols + g.start;
#pragma unroll
    for (int n = 0; n < NIN; ++n) {
        T* tile = reinterpret_cast<T*>(data) + static_cast<size_t>(n) * a.slice_elems;
        for (int c = threadIdx.x; c < g.local; c += THREADS) tile[c] = src[n][offset + c];
    }
    __syncthreads();
}

template <typename T, int NIN>
__device__ __forceinline__ const T* stage_tile(const unsigned char* data, int stage, int n,
                                               int slice_elems) {
    return reinterpret_cast<const T*>(data) + (static_cast<size_t>(stage) * NIN + n) * slice_elems;
}

// Common prologue: barriers initialised, every CTA of the cluster running (a
// CTA's shared memory may only be written by peers once it has started), the
// first `stages` rows in flight.
template <typename T, int NIN, int K, bool ALIGNED>
__device__ __forceinline__ void staged_prologue(StagedControl<K>& ctl, const T* const (&src)[NIN],
                                                unsigned char* data, int cluster,
                                                const StagedArgs& a, const SliceGeom& g) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) mbar_init(smem_u32(&ctl.full[s]), 1);
        fence_mbar_init();
    }
    __syncthreads();
    cluster_sync_all();
    if (ALIGNED && threadIdx.x == 0 && g.local > 0) {
        for (int s = 0; s < a.stages; ++s) {
            const long long row = static_cast<long long>(cluster) + 1ll * s * a.num_clusters;
            if (row < a.rows) issue_slice_fill<T, NIN>(src, data, ctl.full, s, static_cast<int>(row), a, g);
        }
    }
}

// Common epilogue of one row: the stage is free again, refill it with the row
// `stages` steps ahead.
template <typename T, int NIN, int K, bool ALIGNED>
__device__ __forceinline__ void staged_release(StagedControl<K>& ctl, const T* const (&src)[NIN],
                                               unsigned char* data, int stage, int row,
                                               const StagedArgs& a, const SliceGeom& g) {
    __syncthreads();
    if (ALIGNED && threadIdx.x == 0 && g.local > 0) {
        const long long next = static_cast<long long>(row) + 1ll * a.stages * a.num_clusters;
        if (next < a.rows) {
            fence_proxy_async_smem();
            issue_slice_fill<T, NIN>(src, data, ctl.full, stage, static_cast<int>(next), a, g);
        }
    }
}

// ---------------------------------------------------------------------------
// RMSNorm forward: y = x * rsqrt(mean(x^2) + eps) * gamma
// One DSMEM stage, one partial.
// ---------------------------------------------------------------------------
template <typename T, int THREADS, bool ALIGNED>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma, T* __restrict__ y,
                   float eps, StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<StagedControl<1>*>(smem);
    unsigned char* data = smem + kControlBytes;
    constexpr int E = RowVec<T>::kElems;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const T* const src[1] = {x};

    staged_prologue<T, 1, 1, ALIGNED>(ctl, src, data, cluster, a, g);

    RingCursor cur{0, 0u};
    uint32_t red_parity = 0;
    const int nvec = g.local / E;
    const float inv_cols = 1.0f / static_cast<float>(a.cols);

    for (int row = cluster; row < a.rows; row += a.num_clusters) {
        if (ALIGNED) {
            if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[cur.stage]), cur.parity, a.status);
        } else {
            scalar_slice_fill<T, 1, THREADS>(src, data, row, a, g);
        }
        const T* tile = stage_tile<T, 1>(data, cur.stage, 0, a.slice_elems);

        float part[1] = {0.0f};
        if (ALIGNED) {
            float acc[E];
#pragma unroll
            for (int j = 0; j < E; ++j) acc[j] = 0.0f;
#pragma unroll 4
            for (int v = threadIdx.x; v < nvec; v += THREADS) {
                float xv[E];
                RowVec<T>::from_smem(tile, v, xv);
#pragma unroll
                for (int j = 0; j < E; ++j) acc[j] = fmaf(xv[j], xv[j], acc[j]);
            }
#pragma unroll
            for (int j = 0; j < E; ++j) part[0] += acc[j];
        } else {
            for (int c = threadIdx.x; c < g.local; c += THREADS) {
                const float xv = RowVec<T>::to_float(tile[c]);
                part[0] = fmaf(xv, xv, part[0]);
            }
        }
        cluster_allreduce_sum<1, THREADS>(part, ctl.red, red_parity, rank, nranks);
        red_parity ^= 1u;
        const float scale = rsqrtf(part[0] * inv_cols + eps);

        const size_t out_base = static_cast<size_t>(row) * a.cols + g.start;
        if (ALIGNED) {
#pragma unroll 4
            for (int v = threadIdx.x; v < nvec; v += THREADS) {
                float xv[E], gv[E];
                RowVec<T>::from_smem(tile, v, xv);
#pragma unroll
                for (int j = 0; j < E; j += 4) ldg_f32x4(gamma + g.start + v * E + j, gv + j);
#pragma unroll
                for (int j = 0; j < E; ++j) xv[j] = xv[j] * scale * gv[j];
                RowVec<T>::to_global(y + out_base + static_cast<size_t>(v) * E, xv);
            }
        } else {
            for (int c = threadIdx.x; c < g.local; c += THREADS) {
                const float xv = RowVec<T>::to_float(tile[c]);
                y[out_base + c] = RowVec<T>::from_float(xv * scale * gamma[g.start + c]);
            }
        }
        staged_release<T, 1, 1, ALIGNED>(ctl, src, data, cur.stage, row, a, g);
        cur.advance(a.stages);
    }
}

// ---------------------------------------------------------------------------
// Row statistics for LayerNorm from a staged slice: every CTA computes the sum
// and the sum of squared deviations about its OWN slice mean, the cluster
// exchanges (sum, M2) once, and each thread merges the P pairs with the
// parallel-variance formula. One DSMEM stage, two partials, no E[x^2]-mean^2
// cancellation. Returns mean and biased variance of the whole row.
// ---------------------------------------------------------------------------
template <typename T, int THREADS, bool ALIGNED>
__device__ __forceinline__ void staged_row_mean_var(const T* tile, const SliceGeom& g,
                                                    const StagedArgs& a, ReduceScratch<2>& red,
                                                    uint32_t parity, uint32_t rank, uint32_t nranks,
                                                    float& mean, float& var) {
    constexpr int E = RowVec<T>::kElems;
    const int nvec = g.local / E;
    float s[1] = {0.0f};
    if (ALIGNED) {
        float acc[E];
#pragma unroll
        for (int j = 0; j < E; ++j) acc[j] = 0.0f;
#pragma unroll 4
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            float xv[E];
            RowVec<T>::from_smem(tile, v, xv);
#pragma unroll
            for (int j = 0; j < E; ++j) acc[j] += xv[j];
        }
#pragma unroll
        for (int j = 0; j < E; ++j) s[0] += acc[j];
    } else {
        for (int c = threadIdx.x; c < g.local; c += THREADS) s[0] += RowVec<T>::to_float(tile[c]);
    }
    // CTA-local sum (reuses the first partial row of the same scratch).
    cta_allreduce_sum<1, THREADS>(s, reinterpret_cast<ReduceScratch<1>&>(red));
    const float local_mean = g.local > 0 ? s[0] / static_cast<float>(g.local) : 0.0f;

    float m2 = 0.0f;
    if (ALIGNED) {
        float acc[E];
#pragma unroll
        for (int j = 0; j < E; ++j) acc[j] = 0.0f;
#pragma unroll 4
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            float xv[E];
            RowVec<T>::from_smem(tile, v, xv);
#pragma unroll
            for (int j = 0; j < E; ++j) {
                const float d = xv[j] - local_mean;
                acc[j] = fmaf(d, d, acc[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < E; ++j) m2 += acc[j];
    } else {
        for (int c = threadIdx.x; c < g.local; c += THREADS) {
            const float d = RowVec<T>::to_float(tile[c]) - local_mean;
            m2 = fmaf(d, d, m2);
        }
    }
    // Exchange (slice sum, slice M2). The slice sum is already a CTA total, so
    // only thread 0 contributes it to the second reduction.
    float pair[2] = {threadIdx.x == 0 ? s[0] : 0.0f, m2};
    // cluster_allreduce_sum would add the P slots; the merge below needs them
    // one by one, so do the push by hand and read the slots back.
    {
        constexpr int kWarps = THREADS / 32;
        const int lane = threadIdx.x & 31;
        const int warp = threadIdx.x >> 5;
#pragma unroll
        for (int k = 0; k < 2; ++k) pair[k] = warp_sum(pair[k]);
        if (lane == 0) {
            red.warp_part[0][warp] = pair[0];
            red.warp_part[1][warp] = pair[1];
        }
        __syncthreads();
        if (warp == 0) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                float t = lane < kWarps ? red.warp_part[k][lane] : 0.0f;
                t = warp_sum(t);
                if (static_cast<uint32_t>(lane) < nranks) {
                    const uint32_t mine = smem_u32(&red.slot[parity][k][rank]);
                    st_cluster_f32(map_to_rank(mine, static_cast<uint32_t>(lane)), t);
                }
            }
        }
        cluster_arrive_release();
        cluster_wait_acquire();
    }
    float total = 0.0f;
    for (uint32_t r = 0; r < nranks; ++r) total += red.slot[parity][0][r];
    mean = total / static_cast<float>(a.cols);
    float m2_total = 0.0f;
    for (uint32_t r = 0; r < nranks; ++r) {
        const SliceGeom gr = slice_geometry(a.cols, a.slice_elems, r);
        if (gr.local > 0) {
            const float n = static_cast<float>(gr.local);
            const float d = red.slot[parity][0][r] / n - mean;
            m2_total += red.slot[parity][1][r] + n * d * d;
        }
    }
    var = m2_total / static_cast<float>(a.cols);
}

// ---------------------------------------------------------------------------
// LayerNorm forward: y = (x - mean) * rstd * gamma + beta; mean, rstd also
// returned (fp32). rstd = rsqrt(var + eps), var biased.
// ---------------------------------------------------------------------------
template <typename T, int THREADS, bool ALIGNED>
__global__ void __launch_bounds__(THREADS)
layernorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                     const float* __restrict__ beta, T* __restrict__ y,
                     float* __restrict__ mean_out, float* __restrict__ rstd_out, float eps,
                     StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<StagedControl<2>*>(smem);
    unsigned char* data = smem + kControlBytes;
    constexpr int E = RowVec<T>::kElems;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const T* const src[1] = {x};

    staged_prologue<T, 1, 2, ALIGNED>(ctl, src, data, cluster, a, g);

    RingCursor cur{0, 0u};
    uint32_t red_parity = 0;
    const int nvec = g.local / E;

    for (int row = cluster; row < a.rows; row += a.num_clusters) {
        if (ALIGNED) {
            if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[cur.stage]), cur.parity, a.status);
        } else {
            scalar_slice_fill<T, 1, THREADS>(src, data, row, a, g);
        }
        const T* tile = stage_tile<T, 1>(data, cur.stage, 0, a.slice_elems);

        float mean, var;
        staged_row_mean_var<T, THREADS, ALIGNED>(tile, g, a, ctl.red, red_parity, rank, nranks, mean,
                                                 var);
        red_parity ^= 1u;
        const float rstd = rsqrtf(var + eps);
        if (rank == 0 && threadIdx.x == 0) {
            mean_out[row] = mean;
            rstd_out[row] = rstd;
        }
        const float shift = -mean * rstd;

        const size_t out_base = static_cast<size_t>(row) * a.cols + g.start;
        if (ALIGNED) {
#pragma unroll 2
            for (int v = threadIdx.x; v < nvec; v += THREADS) {
                float xv[E], gv[E], bv[E];
                RowVec<T>::from_smem(tile, v, xv);
#pragma unroll
                for (int j = 0; j < E; j += 4) {
                    ldg_f32x4(gamma + g.start + v * E + j, gv + j);
                    ldg_f32x4(beta + g.start + v * E + j, bv + j);
                }
#pragma unroll
                for (int j = 0; j < E; ++j) xv[j] = fmaf(fmaf(xv[j], rstd, shift), gv[j], bv[j]);
                RowVec<T>::to_global(y + out_base + static_cast<size_t>(v) * E, xv);
            }
        } else {
            for (int c = threadIdx.x; c < g.local; c += THREADS) {
                const float xv = RowVec<T>::to_float(tile[c]);
                y[out_base + c] = RowVec<T>::from_float(
                    fmaf(fmaf(xv, rstd, shift), gamma[g.start + c], beta[g.start + c]));
            }
        }
        staged_release<T, 1, 2, ALIGNED>(ctl, src, data, cur.stage, row, a, g);
        cur.advance(a.stages);
    }
}

// ---------------------------------------------------------------------------
// LayerNorm backward, generic form (any width, any alignment): dx only.
//   xhat = (x - mean) * rstd,  g = dy * gamma
//   dx   = (g - mean_row(g) - xhat * mean_row(g * xhat)) * rstd
// HAS_STATS: mean/rstd are inputs (one DSMEM stage); otherwise they are
// recomputed from the staged x slice first (two DSMEM stages), which is the form
// of the reference kernel (src/workloads/layernorm_backward.cu:401-437) and of
// dsmem_eval/workloads.py:53-61. Both x and dy are staged, so dy is read from
// HBM once (the reference reads it twice, :418 and :434). The column sums
// dgamma/dbeta of shapes that end up here come from layernorm_bwd_colsum_kernel.
// ---------------------------------------------------------------------------
template <typename T, int THREADS, bool ALIGNED, bool HAS_STATS>
__global__ void __launch_bounds__(THREADS)
layernorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                     const float* __restrict__ gamma, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, T* __restrict__ dx, float eps,
                     StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<StagedControl<2>*>(smem);
    unsigned char* data = smem + kControlBytes;
    constexpr int E = RowVec<T>::kElems;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const T* const src[2] = {x, dy};

    staged_prologue<T, 2, 2, ALIGNED>(ctl, src, data, cluster, a, g);

    RingCursor cur{0, 0u};
    uint32_t red_parity = 0;
    const int nvec = g.local / E;
    const float inv_cols = 1.0f / static_cast<float>(a.cols);

    for (int row = cluster; row < a.rows; row += a.num_clusters) {
        float mean = 0.0f, rstd = 0.0f;
        if (HAS_STATS) {
            mean = __ldg(mean_in + row);
            rstd = __ldg(rstd_in + row);
        }
        if (ALIGNED) {
            if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[cur.stage]), cur.parity, a.status);
        } else {
            scalar_slice_fill<T, 2, THREADS>(src, data, row, a, g);
        }
        const T* xt = stage_tile<T, 2>(data, cur.stage, 0, a.slice_elems);
        const T* dyt = stage_tile<T, 2>(data, cur.stage, 1, a.slice_elems);

        if (!HAS_STATS) {
            float var;
            staged_row_mean_var<T, THREADS, ALIGNED>(xt, g, a, ctl.red, red_parity, rank, nranks, mean,
                                                     var);
            red_parity ^= 1u;
            rstd = rsqrtf(var + eps);
        }
        const float shift = -mean * rstd;

        // pass 1: row sums of g and g*xhat
        float part[2] = {0.0f, 0.0f};
        if (ALIGNED) {
            float acc0[E], acc1[E];
#pragma unroll
            for (int j = 0; j < E; ++j) { acc0[j] = 0.0f; acc1[j] = 0.0f; }
#pragma unroll 2
            for (int v = threadIdx.x; v < nvec; v += THREADS) {
                float xv[E], dv[E], gv[E];
                RowVec<T>::from_smem(xt, v, xv);
                RowVec<T>::from_smem(dyt, v, dv);
#pragma unroll
                for (int j = 0; j < E; j += 4) ldg_f32x4(gamma + g.start + v * E + j, gv + j);
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    const float xhat = fmaf(xv[j], rstd, shift);
                    const float gg = dv[j] * gv[j];
                    acc0[j] += gg;
                    acc1[j] = fmaf(gg, xhat, acc1[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < E; ++j) { part[0] += acc0[j]; part[1] += acc1[j]; }
        } else {
            for (int c = threadIdx.x; c < g.local; c += THREADS) {
                const float xhat = fmaf(RowVec<T>::to_float(xt[c]), rstd, shift);
                const float gg = RowVec<T>::to_float(dyt[c]) * gamma[g.start + c];
                part[0] += gg;
                part[1] = fmaf(gg, xhat, part[1]);
            }
        }
        cluster_allreduce_sum<2, THREADS>(part, ctl.red, red_parity, rank, nranks);
        red_parity ^= 1u;
        const float mean_g = part[0] * inv_cols;
        const float mean_gx = part[1] * inv_cols;

        // pass 2: dx from the staged slices
        const size_t out_base = static_cast<size_t>(row) * a.cols + g.start;
        if (ALIGNED) {
#pragma unroll 2
            for (int v = threadIdx.x; v < nvec; v += THREADS) {
                float xv[E], dv[E], gv[E];
                RowVec<T>::from_smem(xt, v, xv);
                RowVec<T>::from_smem(dyt, v, dv);
#pragma unroll
                for (int j = 0; j < E; j += 4) ldg_f32x4(gamma + g.start + v * E + j, gv + j);
#pragma unroll
                for (int j = 0; j < E; ++j) {
                    const float xhat = fmaf(xv[j], rstd, shift);
                    const float gg = dv[j] * gv[j];
                    xv[j] = (gg - mean_g - xhat * mean_gx) * rstd;
                }
                RowVec<T>::to_global(dx + out_base + static_cast<size_t>(v) * E, xv);
            }
        } else {
            for (int c = threadIdx.x; c < g.local; c += THREADS) {
                const float xhat = fmaf(RowVec<T>::to_float(xt[c]), rstd, shift);
                const float gg = RowVec<T>::to_float(dyt[c]) * gamma[g.start + c];
                dx[out_base + c] = RowVec<T>::from_float((gg - mean_g - xhat * mean_gx) * rstd);
            }
        }
        staged_release<T, 2, 2, ALIGNED>(ctl, src, data, cur.stage, row, a, g);
        cur.advance(a.stages);
    }
}

}  // namespace credit
