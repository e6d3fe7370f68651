// Warp-specialised wide-row kernels: LayerNorm backward with given statistics and
// parameter gradients (dx, dgamma, dbeta).
//
// The register-resident kernels (register_row_kernels.cuh) run every warp through one
// latency chain per row: ring wait -> loads -> partial sums -> shuffle tree -> DSMEM
// exchange -> fold -> outputs, two rows deep. With the column sums in registers as well,
// that kernel sits at 128 registers and 16 warps per SM, and the chain (about 2900 cycles
// per row), not HBM, sets its pace. Here the chain is cut up and handed to specialised
// warps, and the two halves that stay in the arithmetic warps run `ahead` rows apart, so
// that no arithmetic warp waits for an exchange it has just started, or runs a shuffle
// tree at all:
//
//   producer warp (1 lane)  keeps a ring of D stages full with bulk-async (TMA) copies
//                           of the CTA's x and dy slices of the cluster's next rows;
//   output warps (16 or 8)  iteration i: pass 1 of row i (read the slice from its stage,
//                           S1 = sum g, S2 = sum g (x - mean) over the thread's own
//                           columns, leave the pair in shared memory, arrive on a
//                           CTA-local mbarrier), then pass 2 of row i - ahead (whose
//                           cluster-wide sums were published long ago: read the slice
//                           again, write dx, accumulate dgamma / dbeta in registers,
//                           free the stage);
//   collector warp          per row: waits for the output threads' pairs, adds them up
//                           and pushes the CTA's pair to every CTA of the cluster with
//                           st.async, which lands data and arrival on the receiver's
//                           mbarrier;
//   receiver warp           per row: waits for the P pairs of the cluster, adds them in
//                           rank order (every CTA gets the same bits) and publishes the
//                           row's two sums to the output warps behind one more mbarrier.
//
// A row's slice is read from shared memory twice (3 x 32 KiB of shared-memory traffic
// per 48 KiB of HBM traffic at the target shape, well inside the SM's bandwidth) instead
// of being held in registers across the exchange; that frees the registers that kept
// two rows and lets the ring run D - ahead - 1 rows ahead of the arithmetic. The service
// warps wait with the suspending mbarrier.try_wait so that they do not take issue slots
// from the output warps.
//
// Buffer depths: CTA-local partial buffers 4 >= ahead + 1 (an output warp writes row r + 4
// only after it finished pass 2 of row r + 3 - ahead, for which the collector has long read
// row r); cluster slot buffers and published totals 8 >= 2 * ahead + 2 (a peer sends row
// r + 8 only after every CTA sent row r + 7 - ahead, i.e. after every output warp of this
// CTA finished pass 2 of row r + 6 - 2 * ahead >= r). The same distances keep an mbarrier
// from being re-armed before all its waiters have seen the previous phase.
//
// Arithmetic per element is that of layernorm_bwd_reg_kernel, i.e. of the reference's
// cluster_bwd_staged_kernel (src/workloads/layernorm_backward.cu:401-437) extended to
// given statistics and parameter gradients; only the order in which a row's partial sums
// are added differs (fixed, so results are deterministic).
#pragma once

#include "cluster_primitives.cuh"
#include "norm_kernels.cuh"
#include "register_row_kernels.cuh"

namespace credit {

constexpr int kWsMaxOutputWarps = 16;
constexpr int kWsServiceWarps = 3;   // producer, collector, receiver
static_assert(kWsThreadsPerCta == (kWsMaxOutputWarps + kWsServiceWarps) * 32 &&
                  kWsThreadsPerCtaWide == (8 + kWsServiceWarps) * 32,
              "the host plans with these CTA sizes: output warps + service warps");
constexpr int kWsLocalBuffers = 4;
constexpr int kWsSlotBuffers = 8;

struct alignas(16) WsControl {
    uint64_t full[kMaxStages];                 // stage has landed (1 arrival + transaction bytes)
    uint64_t empty[kMaxStages];                // stage has been read twice by every output warp
    uint64_t local_bar[kWsLocalBuffers];       // every output warp has left its pairs of a row
    uint64_t ex_bar[kWsSlotBuffers];           // the P pairs of a row are in slot
    uint64_t ready_bar[kWsSlotBuffers];        // the row's two sums are in total
    float2 total[kWsSlotBuffers];
    float slot[kWsSlotBuffers][2 * kMaxClusterSize];   // [source rank][partial]
    float2 thread_part[kWsLocalBuffers][kWsMaxOutputWarps * 32];   // [row % 4][output thread]
};
static_assert(sizeof(WsControl) <= kWsControlBytes, "control block overflows its reservation");

// Rows between pass 1 and pass 2 of an output warp, from the ring depth the host chose.
__device__ __forceinline__ int ws_rows_ahead(int stages) { return stages >= 5 ? 2 : 1; }

// OUT_WARPS output warps: 16, or 8 with twice the row elements per thread (the per-row work of a
// warp that does not depend on its element count -- waits, row scalars, addresses -- is then paid
// by half as many warps).
template <typename T, int OUT_WARPS, int VPT, bool FULL>
__global__ void __launch_bounds__((OUT_WARPS + kWsServiceWarps) * 32, 1)
layernorm_bwd_ws_kernel(const T* __restrict__ x, const T* __restrict__ dy, const float* __restrict__ gamma,
                        const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                        T* __restrict__ dx, float* __restrict__ partials, float /*eps*/, StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<WsControl*>(smem);
    unsigned char* data = smem + kWsControlBytes;
    constexpr int E = PairVec<T>::kElems;
    constexpr int PAIRS = PairVec<T>::kPairs;
    constexpr int THREADS = OUT_WARPS * 32;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const int nvec = g.local / E;
    const T* const src[2] = {x, dy};
    const int my_rows = cluster < a.rows ? (a.rows - cluster + a.num_clusters - 1) / a.num_clusters : 0;
    const int stages = a.stages;
    const int ahead = ws_rows_ahead(stages);
    if ((FULL ? nvec != VPT * THREADS : nvec > VPT * THREADS) && threadIdx.x == 0)
        atomicOr(a.status, kStatusBadGeometry);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&ctl.full[s]), 1);
            mbar_init(smem_u32(&ctl.empty[s]), OUT_WARPS);
        }
        for (int b = 0; b < kWsLocalBuffers; ++b) mbar_init(smem_u32(&ctl.local_bar[b]), OUT_WARPS);
        for (int b = 0; b < kWsSlotBuffers; ++b) {
            mbar_init(smem_u32(&ctl.ex_bar[b]), 1);
            mbar_init(smem_u32(&ctl.ready_bar[b]), 1);
        }
        fence_mbar_init();
    }
    __syncthreads();
    cluster_sync_all();   // every CTA of the cluster runs and has its barriers before anyone sends

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;

    // ---- producer: one lane keeps the ring full
    if (warp == OUT_WARPS) {
        if (lane == 0 && g.local > 0) {
            int stage = 0;
            uint32_t parity = 1;   // parity of the phase the LAST use of the stage completed
            for (int it = 0; it < my_rows; ++it) {
                if (it >= stages) mbar_wait_parked_bounded(smem_u32(&ctl.empty[stage]), parity, a.status);
                issue_slice_fill<T, 2>(src, data, ctl.full, stage, cluster + it * a.num_clusters, a, g);
                if (++stage == stages) {
                    stage = 0;
                    parity ^= 1u;
                }
            }
        }
        return;
    }

    // ---- collector: the output threads' pairs of a row -> one pair -> every CTA of the cluster
    if (warp == OUT_WARPS + 1) {
        for (int it = 0; it < my_rows; ++it) {
            const int lb = it & (kWsLocalBuffers - 1);
            const int xb = it & (kWsSlotBuffers - 1);
            mbar_wait_parked_bounded(smem_u32(&ctl.local_bar[lb]), (static_cast<uint32_t>(it) / kWsLocalBuffers) & 1u, a.status);
            const uint32_t bar = smem_u32(&ctl.ex_bar[xb]);
            if (lane == 0) mbar_arrive_expect_tx(bar, nranks * 2u * static_cast<uint32_t>(sizeof(float)));
            const float4* parts = reinterpret_cast<const float4*>(&ctl.thread_part[lb][0]);   // two pairs each
            float2 acc0 = splat(0.0f), acc1 = splat(0.0f);
#pragma unroll
            for (int k = 0; k < THREADS / 64; ++k) {
                const float4 v = parts[lane + 32 * k];
                acc0 = __fadd2_rn(acc0, make_float2(v.x, v.y));
                acc1 = __fadd2_rn(acc1, make_float2(v.z, v.w));
            }
            const float2 mine = __fadd2_rn(acc0, acc1);
            // both sums over the warp in one tree (warp_sum_split): S1 ends in lanes 0..15, S2 in 16..31
            const float t = warp_sum_split(mine.x, mine.y);
            const float t0 = __shfl_sync(0xffffffffu, t, 0);
            const float t1 = __shfl_sync(0xffffffffu, t, 16);
            if (lane < nranks)
                st_async_f32x2(map_to_rank(smem_u32(&ctl.slot[xb][2 * rank]), lane), t0, t1, map_to_rank(bar, lane));
        }
        return;
    }

    // ---- receiver: the cluster's P pairs of a row -> the row's two sums, published to the output warps
    if (warp == OUT_WARPS + 2) {
        const uint32_t half = lane >> 4, idx = lane & 15;
        for (int it = 0; it < my_rows; ++it) {
            const int xb = it & (kWsSlotBuffers - 1);
            mbar_wait_parked_bounded(smem_u32(&ctl.ex_bar[xb]), (static_cast<uint32_t>(it) / kWsSlotBuffers) & 1u, a.status);
            float t = idx < nranks ? ctl.slot[xb][2 * idx + half] : 0.0f;
#pragma unroll
            for (int offset = 8; offset > 0; offset >>= 1) t += __shfl_xor_sync(0xffffffffu, t, offset);
            const float sum2 = __shfl_sync(0xffffffffu, t, 16);
            if (lane == 0) {
                ctl.total[xb] = make_float2(t, sum2);
                mbar_arrive(smem_u32(&ctl.ready_bar[xb]));   // release: the pair is visible to whoever sees the phase
            }
        }
        return;
    }

    // ---- output warps
    float2 gam[VPT][PAIRS], dgam[VPT][PAIRS], dbet[VPT][PAIRS];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) {
            gam[i][j] = splat(0.0f);
            dgam[i][j] = splat(0.0f);
            dbet[i][j] = splat(0.0f);
        }
        if (FULL || v < nvec) load_param_pairs<PAIRS>(gamma + g.start + v * E, gam[i]);
    }
    const float inv_cols = 1.0f / static_cast<float>(a.cols);

    // Row statistics travel through a short shift register: [0] row it + 1 (fetched one iteration
    // early), [1] row it (pass 1), [2] row it - 1, [3] row it - 2 (pass 2, by `ahead`).
    float mean_q[4] = {0.0f, 0.0f, 0.0f, 0.0f}, rstd_q[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (my_rows > 0) {
        mean_q[0] = __ldg(mean_in + cluster);
        rstd_q[0] = __ldg(rstd_in + cluster);
    }

    int stage1 = 0;               // ring stage of pass 1's row
    uint32_t parity1 = 0;
    int stage2 = 0;               // ring stage of pass 2's row

    for (int it = 0; it < my_rows + ahead; ++it) {
#pragma unroll
        for (int k = 3; k > 0; --k) {
            mean_q[k] = mean_q[k - 1];
            rstd_q[k] = rstd_q[k - 1];
        }
        if (it + 1 < my_rows) {
            const int next_row = cluster + (it + 1) * a.num_clusters;
            mean_q[0] = __ldg(mean_in + next_row);
            rstd_q[0] = __ldg(rstd_in + next_row);
        }

        // ---- pass 1 of row `it`: this thread's share of S1 = sum g and S2 = sum g * (x - mean)
        if (it < my_rows) {
            const float mean = mean_q[1];
            if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[stage1]), parity1, a.status);
            const uint4* xt = reinterpret_cast<const uint4*>(stage_tile<T, 2>(data, stage1, 0, a.slice_elems));
            const uint4* dt = reinterpret_cast<const uint4*>(stage_tile<T, 2>(data, stage1, 1, a.slice_elems));
            const float2 neg_mean = splat(-mean);
            float2 s1[2] = {splat(0.0f), splat(0.0f)}, s2[2] = {splat(0.0f), splat(0.0f)};   // two chains each
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = threadIdx.x + i * THREADS;
                if (FULL || v < nvec) {
                    float2 xv[PAIRS], dv[PAIRS];
                    PairVec<T>::unpack(xt[v], xv);
                    PairVec<T>::unpack(dt[v], dv);
#pragma unroll
                    for (int j = 0; j < PAIRS; ++j) {
                        const float2 gg = __fmul2_rn(dv[j], gam[i][j]);
                        s1[j & 1] = __fadd2_rn(s1[j & 1], gg);
                        // 16-bit rows: sum g * x here, mean * sum g comes off once per row below
                        s2[j & 1] = sizeof(T) == 2 ? __ffma2_rn(gg, xv[j], s2[j & 1])
                                                   : __ffma2_rn(gg, __fadd2_rn(xv[j], neg_mean), s2[j & 1]);
                    }
                }
            }
            const float2 s1t = __fadd2_rn(s1[0], s1[1]), s2t = __fadd2_rn(s2[0], s2[1]);
            const float t1 = s1t.x + s1t.y, t2 = s2t.x + s2t.y;
            const int lb = it & (kWsLocalBuffers - 1);
            ctl.thread_part[lb][threadIdx.x] = make_float2(t1, sizeof(T) == 2 ? fmaf(-mean, t1, t2) : t2);
            __syncwarp();   // the other lanes' stores are ordered before lane 0's release
            if (lane == 0) mbar_arrive(smem_u32(&ctl.local_bar[lb]));
            if (++stage1 == stages) {
                stage1 = 0;
                parity1 ^= 1u;
            }
        }

        // ---- pass 2 of row `it - ahead`: dx from the staged slice, column sums into registers
        if (it >= ahead) {
            const int it2 = it - ahead;
            const int row = cluster + it2 * a.num_clusters;
            const float mean = ahead == 2 ? mean_q[3] : mean_q[2];
            const float rstd = ahead == 2 ? rstd_q[3] : rstd_q[2];
            const int xb = it2 & (kWsSlotBuffers - 1);
            mbar_wait_bounded(smem_u32(&ctl.ready_bar[xb]), (static_cast<uint32_t>(it2) / kWsSlotBuffers) & 1u, a.status);
            const float2 sums = ctl.total[xb];

            const uint4* xt = reinterpret_cast<const uint4*>(stage_tile<T, 2>(data, stage2, 0, a.slice_elems));
            const uint4* dt = reinterpret_cast<const uint4*>(stage_tile<T, 2>(data, stage2, 1, a.slice_elems));
            const float2 neg_mean = splat(-mean), rstd2 = splat(rstd);
            const float2 ca = splat(-rstd * rstd * rstd * (sums.y * inv_cols));
            const float2 cb = splat(-rstd * (sums.x * inv_cols));
            // 16-bit rows work on xhat = x * rstd - mean * rstd (one fused operation; the rounding of
            // the constant is far below the output's 2^-9): dx = xhat * ca_hat + g * rstd + cb and
            // dgamma += dy * xhat, one operation less per pair than the (x - mean) form fp32 rows keep.
            const float2 shift2 = splat(-mean * rstd);
            const float2 ca_hat = splat(-rstd * rstd * (sums.y * inv_cols));
            uint4* out = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * a.cols + g.start);
#pragma unroll
            for (int i = 0; i < VPT; ++i) {
                const int v = threadIdx.x + i * THREADS;
                if (FULL || v < nvec) {
                    float2 xv[PAIRS], dv[PAIRS], o[PAIRS];
                    PairVec<T>::unpack(xt[v], xv);
                    PairVec<T>::unpack(dt[v], dv);
#pragma unroll
                    for (int j = 0; j < PAIRS; ++j) {
                        const float2 gg = __fmul2_rn(dv[j], gam[i][j]);
                        if (sizeof(T) == 2) {
                            const float2 xhat = __ffma2_rn(xv[j], rstd2, shift2);
                            o[j] = __ffma2_rn(xhat, ca_hat, __ffma2_rn(gg, rstd2, cb));
                            dgam[i][j] = __ffma2_rn(dv[j], xhat, dgam[i][j]);
                        } else {
                            const float2 c = __fadd2_rn(xv[j], neg_mean);
                            o[j] = __ffma2_rn(c, ca, __ffma2_rn(gg, rstd2, cb));
                            dgam[i][j] = __ffma2_rn(__fmul2_rn(dv[j], c), rstd2, dgam[i][j]);
                        }
                        dbet[i][j] = __fadd2_rn(dbet[i][j], dv[j]);
                    }
                    __stcs(out + v, PairVec<T>::pack(o));
                }
            }
            if (g.local > 0) {
                __syncwarp();   // every lane has read its vectors of the stage
                if (lane == 0) mbar_arrive(smem_u32(&ctl.empty[stage2]));
            }
            if (++stage2 == stages) stage2 = 0;
        }
    }

    float* out_g = partials + (static_cast<size_t>(cluster) * 2 + 0) * a.cols + g.start;
    float* out_b = partials + (static_cast<size_t>(cluster) * 2 + 1) * a.cols + g.start;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (FULL || v < nvec) {
#pragma unroll
            for (int j = 0; j < PAIRS; j += 2) {
                *reinterpret_cast<float4*>(out_g + v * E + 2 * j) =
                    make_float4(dgam[i][j].x, dgam[i][j].y, dgam[i][j + 1].x, dgam[i][j + 1].y);
                *reinterpret_cast<float4*>(out_b + v * E + 2 * j) =
                    make_float4(dbet[i][j].x, dbet[i][j].y, dbet[i][j + 1].x, dbet[i][j + 1].y);
            }
        }
    }
}

}  // namespace credit
