// Streaming row reduction: per-row sum, maximum and index of the first maximum
// of an fp32 matrix whose rows are far wider than on-chip memory (4 MiB per row
// in the target shape). A cluster owns a row; CTA `rank` streams its column
// slice once, keeps only (sum, max, argmax) partials, and the P partial triples
// meet in rank 0's shared memory through DSMEM. The max-type one-stage
// reduction is the shape of the reference's row-wise quantisation kernel
// (src/workloads/rowwise_quant.cu:321-363, cluster_reduce_max :209-237) with the
// index carried along.
//
// Two ways of moving the slice, same arithmetic:
//   * ring of bulk-async (TMA) chunks in shared memory behind mbarriers;
//   * unrolled 128-bit read-only loads straight into registers (also the path
//     for rows that are not 16-byte aligned, then with scalar loads).
//
// Maximum semantics are those of torch.amax / torch.argmax: ties resolve to the
// lowest column, and a NaN element wins over every number (max = NaN, argmax = the
// column of the row's first NaN). The streaming loop itself is NaN-blind (fmaxf and
// '>' skip NaNs); a NaN element always turns the row's running sum into NaN, so a CTA
// whose partial sum is NaN scans its slice once more for the first NaN before the
// partials are exchanged (rows without NaN or inf - inf never take that path).
#pragma once

#include <limits.h>

#include "cluster_primitives.cuh"

namespace credit {

struct RowBest {
    float value;
    int index;
};

// NaN ranks above every number; among equals (two NaNs included) the lower column wins.
__device__ __forceinline__ RowBest better_of(RowBest a, RowBest b) {
    const bool a_nan = a.value != a.value, b_nan = b.value != b.value;
    const bool same = (a_nan && b_nan) || b.value == a.value;
    const bool take_b = same ? b.index < a.index : (b_nan || (!a_nan && b.value > a.value));
    return take_b ? b : a;
}

// Slow path of a CTA whose partial sum came out NaN: the column of the first NaN among this
// thread's share of the slice (scalar loads from global memory), or INT_MAX.
template <int THREADS>
__device__ __noinline__ int first_nan_column(const float* __restrict__ slice, int local, int start) {
    for (int c = threadIdx.x; c < local; c += THREADS) {
        const float v = slice[c];
        if (v != v) return start + c;   // a thread visits its columns in increasing order
    }
    return INT_MAX;
}

__device__ __forceinline__ RowBest warp_best(RowBest v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        RowBest o;
        o.value = __shfl_xor_sync(0xffffffffu, v.value, offset);
        o.index = __shfl_xor_sync(0xffffffffu, v.index, offset);
        v = better_of(v, o);
    }
    return v;
}

// Folds four consecutive elements starting at column `col` into the running
// state. The common case costs four adds and three max; the index is only
// resolved when the vector beats the thread's best so far. A thread visits its
// columns in increasing order, so strict '>' keeps its first maximum.
__device__ __forceinline__ void fold4(const float4& v, int col, float4& acc, RowBest& best) {
    acc.x += v.x;
    acc.y += v.y;
    acc.z += v.z;
    acc.w += v.w;
    const float m = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
    if (m > best.value) {
        best.value = m;
        best.index = (v.x == m) ? col : (v.y == m) ? col + 1 : (v.z == m) ? col + 2 : col + 3;
    }
}

struct ReduceControl {
    uint64_t full[kMaxStages];
    float warp_sum_part[kMaxWarpsPerCta];
    float warp_max_part[kMaxWarpsPerCta];
    int warp_idx_part[kMaxWarpsPerCta];
    // rank 0 receives one triple per source rank; double-buffered by row parity
    float slot_sum[2][kMaxClusterSize];
    float slot_max[2][kMaxClusterSize];
    int slot_idx[2][kMaxClusterSize];
};

// CTA partials -> rank 0 of the cluster -> outputs. Called by all threads once
// per row, after the slice has been folded into (sum4, best).
template <int THREADS>
__device__ __forceinline__ void finish_row(ReduceControl& ctl, float total, RowBest best, int row,
                                           uint32_t parity, uint32_t rank, uint32_t nranks,
                                           const float* __restrict__ slice, const SliceGeom& g,
                                           float* __restrict__ out_sum, float* __restrict__ out_max,
                                           long long* __restrict__ out_argmax) {
    constexpr int kWarps = THREADS / 32;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    if (__syncthreads_or(total != total)) {
        const int col = first_nan_column<THREADS>(slice, g.local, g.start);
        if (col != INT_MAX) best = RowBest{__int_as_float(0x7fc00000), col};
    }
    total = warp_sum(total);
    best = warp_best(best);
    if (lane == 0) {
        ctl.warp_sum_part[warp] = total;
        ctl.warp_max_part[warp] = best.value;
        ctl.warp_idx_part[warp] = best.index;
    }
    __syncthreads();
    if (warp == 0) {
        float t = lane < kWarps ? ctl.warp_sum_part[lane] : 0.0f;
        RowBest b;
        b.value = lane < kWarps ? ctl.warp_max_part[lane] : -INFINITY;
        b.index = lane < kWarps ? ctl.warp_idx_part[lane] : INT_MAX;
        t = warp_sum(t);
        b = warp_best(b);
        if (lane == 0) {
            st_cluster_f32(map_to_rank(smem_u32(&ctl.slot_sum[parity][rank]), 0), t);
            st_cluster_f32(map_to_rank(smem_u32(&ctl.slot_max[parity][rank]), 0), b.value);
            st_cluster_u32(map_to_rank(smem_u32(&ctl.slot_idx[parity][rank]), 0),
                           static_cast<uint32_t>(b.index));
        }
    }
    cluster_arrive_release();
    cluster_wait_acquire();
    if (rank == 0 && threadIdx.x == 0) {
        float t = 0.0f;
        RowBest b{-INFINITY, INT_MAX};
        for (uint32_t r = 0; r < nranks; ++r) {
            t += ctl.slot_sum[parity][r];
            RowBest o{ctl.slot_max[parity][r], ctl.slot_idx[parity][r]};
            b = better_of(b, o);
        }
        out_sum[row] = t;
        out_max[row] = b.value;
        out_argmax[row] = b.index == INT_MAX ? 0ll : static_cast<long long>(b.index);
    }
}

// ---------------------------------------------------------------------------
// TMA ring variant. Rows must be 16-byte aligned (cols % 4 == 0).
// The ring runs across row boundaries: while a row is being finished the first
// chunks of the cluster's next row are already landing.
// ---------------------------------------------------------------------------
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
row_reduce_tma_kernel(const float* __restrict__ x, float* __restrict__ out_sum,
                      float* __restrict__ out_max, long long* __restrict__ out_argmax,
                      ReduceArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<ReduceControl*>(smem);
    unsigned char* data = smem + kControlBytes;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const int chunks_per_row = (g.local + a.chunk_elems - 1) / a.chunk_elems;
    const uint32_t chunk_bytes = static_cast<uint32_t>(a.chunk_elems) * sizeof(float);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) mbar_init(smem_u32(&ctl.full[s]), 1);
        fence_mbar_init();
    }
    __syncthreads();
    cluster_sync_all();

    // Producer state (thread 0): next (row, chunk) to request.
    int prod_row = cluster;
    int prod_chunk = 0;
    auto issue_next = [&](int stage) {
        if (chunks_per_row == 0 || prod_row >= a.rows) return;
        const int c0 = prod_chunk * a.chunk_elems;
        const int n = min(a.chunk_elems, g.local - c0);
        const uint32_t bytes = static_cast<uint32_t>(n) * sizeof(float);
        const uint32_t bar = smem_u32(&ctl.full[stage]);
        mbar_arrive_expect_tx(bar, bytes);
        bulk_load_chunked(smem_u32(data + static_cast<size_t>(stage) * chunk_bytes),
                          x + static_cast<size_t>(prod_row) * a.cols + g.start + c0, bytes, bar);
        if (++prod_chunk == chunks_per_row) {
            prod_chunk = 0;
            prod_row += a.num_clusters;
        }
    };
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) issue_next(s);
    }

    RingCursor cur{0, 0u};
    uint32_t row_parity = 0;
    for (int row = cluster; row < a.rows; row += a.num_clusters) {
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        RowBest best{-INFINITY, INT_MAX};
        for (int ch = 0; ch < chunks_per_row; ++ch) {
            mbar_wait_bounded(smem_u32(&ctl.full[cur.stage]), cur.parity, a.status);
            const float4* tile =
                reinterpret_cast<const float4*>(data + static_cast<size_t>(cur.stage) * chunk_bytes);
            const int c0 = ch * a.chunk_elems;
            const int nvec = min(a.chunk_elems, g.local - c0) >> 2;
            const int col0 = g.start + c0;
#pragma unroll 4
            for (int v = threadIdx.x; v < nvec; v += THREADS) fold4(tile[v], col0 + 4 * v, acc, best);
            __syncthreads();
            if (threadIdx.x == 0) {
                fence_proxy_async_smem();
                issue_next(cur.stage);
            }
            cur.advance(a.stages);
        }
        finish_row<THREADS>(ctl, (acc.x + acc.y) + (acc.z + acc.w), best, row, row_parity, rank,
                            nranks, x + static_cast<size_t>(row) * a.cols + g.start, g, out_sum, out_max,
                            out_argmax);
        row_parity ^= 1u;
    }
}

// ---------------------------------------------------------------------------
// Direct-load variant: UNROLL independent 128-bit loads per thread in flight.
// ALIGNED=false handles any cols / base alignment with scalar loads.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float4 ldg_stream_f32x4(const float* p) {
    float4 v;
    asm("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p));
    return v;
}

template <int THREADS, int UNROLL, bool ALIGNED>
__global__ void __launch_bounds__(THREADS)
row_reduce_ldg_kernel(const float* __restrict__ x, float* __restrict__ out_sum,
                      float* __restrict__ out_max, long long* __restrict__ out_argmax,
                      ReduceArgs a) {
    __shared__ ReduceControl ctl;
    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);

    cluster_sync_all();

    uint32_t row_parity = 0;
    for (int row = cluster; row < a.rows; row += a.num_clusters) {
        const float* src = x + static_cast<size_t>(row) * a.cols + g.start;
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        RowBest best{-INFINITY, INT_MAX};
        if (ALIGNED) {
            const int nvec = g.local >> 2;
            int v = threadIdx.x;
            for (; v + (UNROLL - 1) * THREADS < nvec; v += UNROLL * THREADS) {
                float4 buf[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) buf[u] = ldg_stream_f32x4(src + 4 * (v + u * THREADS));
#pragma unroll
                for (int u = 0; u < UNROLL; ++u)
                    fold4(buf[u], g.start + 4 * (v + u * THREADS), acc, best);
            }
            for (; v < nvec; v += THREADS) fold4(ldg_stream_f32x4(src + 4 * v), g.start + 4 * v, acc, best);
        } else {
            for (int c = threadIdx.x; c < g.local; c += THREADS) {
                const float xv = src[c];
                acc.x += xv;
                if (xv > best.value) {
                    best.value = xv;
                    best.index = g.start + c;
                }
            }
        }
        finish_row<THREADS>(ctl, (acc.x + acc.y) + (acc.z + acc.w), best, row, row_parity, rank,
                            nranks, src, g, out_sum, out_max, out_argmax);
        row_parity ^= 1u;
    }
}

}  // namespace credit
