// Warp-specialised wide-row kernels: one pipeline for RMSNorm forward, LayerNorm forward,
// LayerNorm backward with given statistics and parameter gradients (policies below) and the
// five workloads of the reference sweep (policies in ws_row_ops.cuh).
//
// The register-resident kernels (register_row_kernels.cuh) run every warp through one
// latency chain per row: ring wait -> loads -> partial sums -> shuffle tree -> DSMEM
// exchange -> fold -> outputs, two rows deep. That chain (about 2900 cycles per row for
// LayerNorm backward at 16 warps per SM), not HBM, sets their pace. Here the chain is cut
// up and handed to specialised warps, and the two halves that stay in the arithmetic
// warps run `ahead` rows apart, so that no arithmetic warp waits for an exchange it has
// just started, or runs a shuffle tree at all:
//
//   producer warp (1 lane)  keeps a ring of D stages full with bulk-async (TMA) copies
//                           of the CTA's slices of the cluster's next rows;
//   output warps (16 or 8)  iteration i: pass 1 of row i (read the slice from its stage,
//                           the thread's share of the row's partial record -- up to 8
//                           sums, maxima or whatever the workload's `combine` folds --
//                           left in shared memory; one arrival per warp on a CTA-local
//                           mbarrier), then pass 2 of row i - ahead (whose cluster-wide
//                           record was published long ago: read the slice again, write
//                           the outputs, free the stage);
//   collector warp          per row: waits for the output threads' records, folds them
//                           and pushes the CTA's record to every CTA of the cluster with
//                           st.async, which lands data and arrival on the receiver's
//                           mbarrier; one of its lanes also loads the rows' scalars
//                           (statistics, shifts) a few rows early and publishes them;
//   receiver warp           per row: waits for the P records of the cluster, folds them
//                           in a fixed order (every CTA gets the same bits) and publishes
//                           the row's record to the output warps behind one more mbarrier.
//
// A row's slice is read from shared memory twice instead of being held in registers
// across the exchange (for LayerNorm backward 3 x 32 KiB of shared-memory traffic per
// 48 KiB of HBM traffic at the target shape, well inside the SM's bandwidth); that frees
// the registers that kept two rows and lets the ring run D - ahead - 1 rows ahead of the
// arithmetic. The service warps wait with the suspending mbarrier.try_wait so that they
// do not take issue slots from the output warps.
//
// Buffer depths: CTA-local partial buffers 4 >= ahead + 1 (an output warp writes row r + 4
// only after it finished pass 2 of row r + 3 - ahead, for which the collector has long read
// row r); cluster slot buffers and published totals 8 >= 2 * ahead + 2 (a peer sends row
// r + 8 only after every CTA sent row r + 7 - ahead, i.e. after every output warp of this
// CTA finished pass 2 of row r + 6 - 2 * ahead >= r). The same distances keep an mbarrier
// from being re-armed before all its waiters have seen the previous phase.
//
// A workload is a policy struct (RmsNormFwdOp, LayerNormFwdOp, LayerNormBwdOp below): what a
// thread keeps for the whole kernel, the per-row scalars it fetches one row early, its
// share of pass 1 and its share of pass 2. Arithmetic per element is that of the
// register-resident kernels, i.e. of the reference's cluster_bwd_staged_kernel family
// (src/workloads/layernorm_backward.cu:376-438); only the order in which a row's partial
// sums are added differs (fixed, so results are deterministic).
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
constexpr int kWsSlotBuffers = 8;

// KP floats per partial record (2, 4 or 8), L CTA-local record buffers, THREADS output threads.
template <int KP, int L, int THREADS>
struct alignas(16) WsControl {
    uint64_t full[kWsMaxStages];               // stage has landed (1 arrival + transaction bytes)
    uint64_t empty[kWsMaxStages];               // stage has been read twice by every output warp
    uint64_t local_bar[4];                     // every output warp has left its records of a row
    uint64_t ex_bar[kWsSlotBuffers];           // the P records of a row are in slot
    uint64_t ready_bar[kWsSlotBuffers];        // the row's record is in total
    uint64_t info_bar[kWsSlotBuffers];         // the row's scalars are in row_info
    float4 row_info[kWsSlotBuffers];           // per-row scalars, published kWsInfoLead rows early
    alignas(16) float total[kWsSlotBuffers][KP];
    alignas(16) float slot[kWsSlotBuffers][kMaxClusterSize][KP];   // [row % 8][source rank]
    alignas(16) float thread_part[L][THREADS][KP];                 // [row % L][output thread]
};

// Rows between pass 1 and pass 2 of an output warp, from the ring depth the host chose.
__device__ __forceinline__ int ws_rows_ahead(int stages) { return stages >= 5 ? 2 : 1; }

// Per-row scalars (given statistics, or the three samples the shift of the one-pass variance is the
// median of). The output warps never load them from global memory: the lines are cold (each is used
// during a few rows only while gigabytes stream through the L2), and a warp that waits two
// microseconds for one stalls its whole row step. One lane of the collector warp loads them
// kWsInfoLead + 1 rows ahead and publishes them in shared memory kWsInfoLead rows ahead.
struct WsRow {
    float a, b, c, d, e, f, g;
};
constexpr int kWsInfoLead = 3;   // > ahead: the output warps run at most `ahead` rows before the collector

// A partial record of KP floats to / from shared memory with the widest accesses.
template <int KP>
__device__ __forceinline__ void ws_load_record(const float* p, float (&v)[KP]) {
    if constexpr (KP == 2) {
        const float2 t = *reinterpret_cast<const float2*>(p);
        v[0] = t.x; v[1] = t.y;
    } else {
#pragma unroll
        for (int k = 0; k < KP; k += 4) {
            const float4 t = *reinterpret_cast<const float4*>(p + k);
            v[k] = t.x; v[k + 1] = t.y; v[k + 2] = t.z; v[k + 3] = t.w;
        }
    }
}
template <int KP>
__device__ __forceinline__ void ws_store_record(float* p, const float (&v)[KP]) {
    if constexpr (KP == 2) {
        *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
    } else {
#pragma unroll
        for (int k = 0; k < KP; k += 4) *reinterpret_cast<float4*>(p + k) = make_float4(v[k], v[k + 1], v[k + 2], v[k + 3]);
    }
}
// Pushes a record into the same place of CTA `peer`'s shared memory; every 8- or 16-byte message
// credits the peer's mbarrier with its bytes.
template <int KP>
__device__ __forceinline__ void ws_send_record(uint32_t local_addr, uint32_t peer, const float (&v)[KP], uint32_t local_bar) {
    const uint32_t dst = map_to_rank(local_addr, peer), bar = map_to_rank(local_bar, peer);
    if constexpr (KP == 2) {
        st_async_f32x2(dst, v[0], v[1], bar);
    } else {
#pragma unroll
        for (int k = 0; k < KP; k += 4) st_async_f32x4(dst + 4 * k, v[k], v[k + 1], v[k + 2], v[k + 3], bar);
    }
}

// ---------------------------------------------------------------------------
// the pipeline
// ---------------------------------------------------------------------------
// Op::kOutWarps output warps: 16, or 8 with twice the row elements per thread (the per-row work of
// a warp that does not depend on its element count -- waits, row scalars, addresses -- is then
// paid by half as many warps).
template <class Op>
__global__ void __launch_bounds__((Op::kOutWarps + kWsServiceWarps) * 32, 1)
ws_row_kernel(NormParams prm, StagedArgs a) {
    using T = typename Op::Elem;
    constexpr int NIN = Op::kInputs;
    constexpr int OUT_WARPS = Op::kOutWarps;
    constexpr int THREADS = OUT_WARPS * 32;
    constexpr int VPT = Op::kVectors;
    constexpr bool FULL = Op::kFull;
    constexpr int E = PairVec<T>::kElems;
    constexpr int KP = Op::kPartials;          // floats per partial record
    constexpr int L = Op::kLocalBuffers;       // CTA-local record buffers (a power of two)
    using Control = WsControl<KP, L, THREADS>;
    static_assert(sizeof(Control) <= kWsControlBytes, "control block overflows its reservation");
    static_assert(KP == 2 || KP == 4 || KP == 8, "records travel as 8- or 16-byte messages");

    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<Control*>(smem);
    unsigned char* data = smem + kWsControlBytes;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const int nvec = g.local / E;
    const int my_rows = cluster < a.rows ? (a.rows - cluster + a.num_clusters - 1) / a.num_clusters : 0;
    const int stages = a.stages;
    const int ahead = min(ws_rows_ahead(stages), L - 1);
    if (Op::kRegisterSlice && (FULL ? nvec != VPT * THREADS : nvec > VPT * THREADS) && threadIdx.x == 0)
        atomicOr(a.status, kStatusBadGeometry);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&ctl.full[s]), 1);
            mbar_init(smem_u32(&ctl.empty[s]), OUT_WARPS);
        }
        for (int b = 0; b < L; ++b) mbar_init(smem_u32(&ctl.local_bar[b]), OUT_WARPS);
        for (int b = 0; b < kWsSlotBuffers; ++b) {
            mbar_init(smem_u32(&ctl.ex_bar[b]), 1);
            mbar_init(smem_u32(&ctl.ready_bar[b]), 1);
            mbar_init(smem_u32(&ctl.info_bar[b]), 1);
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
            const T* src[NIN];
            Op::sources(prm, src);
            const T* const(&csrc)[NIN] = src;
            int stage = 0;
            uint32_t parity = 1;   // parity of the phase the LAST use of the stage completed
            for (int it = 0; it < my_rows; ++it) {
                if (it >= stages) mbar_wait_parked_bounded(smem_u32(&ctl.empty[stage]), parity, a.status);
                issue_slice_fill<T, NIN>(csrc, data, ctl.full, stage, cluster + it * a.num_clusters, a, g);
                if (++stage == stages) {
                    stage = 0;
                    parity ^= 1u;
                }
            }
        }
        return;
    }

    // ---- collector: the output threads' pairs of a row -> one pair -> every CTA of the cluster;
    // lane 0 also publishes the rows' scalars ahead of the output warps
    if (warp == OUT_WARPS + 1) {
        auto publish = [&](int r, const WsRow& info) {
            const int ib = r & (kWsSlotBuffers - 1);
            ctl.row_info[ib] = Op::publish_row(info);
            mbar_arrive(smem_u32(&ctl.info_bar[ib]));   // release
        };
        WsRow next_info{};
        if (Op::kRowInfo && lane == 0) {
            for (int r = 0; r < kWsInfoLead && r < my_rows; ++r)
                publish(r, Op::fetch_row(prm, cluster + r * a.num_clusters, a.cols));
            if (kWsInfoLead < my_rows) next_info = Op::fetch_row(prm, cluster + kWsInfoLead * a.num_clusters, a.cols);
        }
        for (int it = 0; it < my_rows; ++it) {
            if (Op::kRowInfo && lane == 0) {
                // row it + lead was loaded one iteration ago; row it + lead + 1 is requested now. Buffer
                // (it + lead) % 8 last held row it + lead - 8, which every output warp finished before it
                // delivered the row the previous iteration waited for.
                if (it + kWsInfoLead < my_rows) publish(it + kWsInfoLead, next_info);
                if (it + kWsInfoLead + 1 < my_rows)
                    next_info = Op::fetch_row(prm, cluster + (it + kWsInfoLead + 1) * a.num_clusters, a.cols);
            }
            const int lb = it & (L - 1);
            const int xb = it & (kWsSlotBuffers - 1);
            mbar_wait_parked_bounded(smem_u32(&ctl.local_bar[lb]), (static_cast<uint32_t>(it) / L) & 1u, a.status);
            const uint32_t bar = smem_u32(&ctl.ex_bar[xb]);
            if (lane == 0) mbar_arrive_expect_tx(bar, nranks * static_cast<uint32_t>(KP * sizeof(float)));
            float rec[KP];
            if constexpr (KP == 2 && Op::kAdditive) {
                const float4* parts = reinterpret_cast<const float4*>(&ctl.thread_part[lb][0][0]);   // two records each
                float2 acc0 = splat(0.0f), acc1 = splat(0.0f);
#pragma unroll
                for (int k = 0; k < THREADS / 64; ++k) {
                    const float4 v = parts[lane + 32 * k];
                    acc0 = __fadd2_rn(acc0, make_float2(v.x, v.y));
                    acc1 = __fadd2_rn(acc1, make_float2(v.z, v.w));
                }
                const float2 mine = __fadd2_rn(acc0, acc1);
                // both sums over the warp in one tree (warp_sum_split): the first ends in lanes 0..15,
                // the second in lanes 16..31
                const float t = warp_sum_split(mine.x, mine.y);
                rec[0] = __shfl_sync(0xffffffffu, t, 0);
                rec[1] = __shfl_sync(0xffffffffu, t, 16);
            } else {
                Op::identity(rec);
#pragma unroll
                for (int k = 0; k < THREADS / 32; ++k) {
                    float v[KP];
                    ws_load_record<KP>(&ctl.thread_part[lb][lane + 32 * k][0], v);
                    Op::combine(rec, v);
                }
#pragma unroll
                for (int offset = 16; offset > 0; offset >>= 1) {
                    float o[KP];
#pragma unroll
                    for (int k = 0; k < KP; ++k) o[k] = __shfl_xor_sync(0xffffffffu, rec[k], offset);
                    Op::combine(rec, o);
                }
            }
            if (lane < nranks) ws_send_record<KP>(smem_u32(&ctl.slot[xb][rank][0]), lane, rec, bar);
        }
        return;
    }

    // ---- receiver: the cluster's P pairs of a row -> the row's two sums, published to the output warps
    if (warp == OUT_WARPS + 2) {
        for (int it = 0; it < my_rows; ++it) {
            const int xb = it & (kWsSlotBuffers - 1);
            mbar_wait_parked_bounded(smem_u32(&ctl.ex_bar[xb]), (static_cast<uint32_t>(it) / kWsSlotBuffers) & 1u, a.status);
            float rec[KP];
            if constexpr (KP == 2 && Op::kAdditive) {
                const uint32_t half = lane >> 4, idx = lane & 15;
                float t = idx < nranks ? ctl.slot[xb][idx][half] : 0.0f;
#pragma unroll
                for (int offset = 8; offset > 0; offset >>= 1) t += __shfl_xor_sync(0xffffffffu, t, offset);
                rec[0] = t;
                rec[1] = __shfl_sync(0xffffffffu, t, 16);
            } else {
                Op::identity(rec);
                if (lane < nranks) ws_load_record<KP>(&ctl.slot[xb][lane][0], rec);
#pragma unroll
                for (int offset = 8; offset > 0; offset >>= 1) {   // ranks sit in lanes 0..15
                    float o[KP];
#pragma unroll
                    for (int k = 0; k < KP; ++k) o[k] = __shfl_xor_sync(0xffffffffu, rec[k], offset);
                    Op::combine(rec, o);
                }
            }
            if (lane == 0) {
                ws_store_record<KP>(&ctl.total[xb][0], rec);
                mbar_arrive(smem_u32(&ctl.ready_bar[xb]));   // release: the record is visible to whoever sees the phase
            }
        }
        return;
    }

    // ---- output warps
    typename Op::State st;
    Op::init(st, prm, g.start, nvec);

    int stage1 = 0;               // ring stage of pass 1's row
    uint32_t parity1 = 0;
    int stage2 = 0;               // ring stage of pass 2's row

    for (int it = 0; it < my_rows + ahead; ++it) {
        // ---- pass 1 of row `it`: this thread's share of the row's sums
        if (it < my_rows) {
            if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[stage1]), parity1, a.status);
            const uint4* tiles[NIN];
#pragma unroll
            for (int n = 0; n < NIN; ++n)
                tiles[n] = reinterpret_cast<const uint4*>(stage_tile<T, NIN>(data, stage1, n, a.slice_elems));
            const int lb = it & (L - 1);
            float4 info = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (Op::kRowInfo) {
                const int ib = it & (kWsSlotBuffers - 1);
                mbar_wait_bounded(smem_u32(&ctl.info_bar[ib]), (static_cast<uint32_t>(it) / kWsSlotBuffers) & 1u, a.status);
                info = ctl.row_info[ib];
            }
            float part[KP];
            Op::pass1(st, tiles, nvec, info, part);
            ws_store_record<KP>(&ctl.thread_part[lb][threadIdx.x][0], part);
            __syncwarp();   // the other lanes' stores are ordered before lane 0's release
            if (lane == 0) mbar_arrive(smem_u32(&ctl.local_bar[lb]));
            if (++stage1 == stages) {
                stage1 = 0;
                parity1 ^= 1u;
            }
        }

        // ---- pass 2 of row `it - ahead`: outputs from the staged slice
        if (it >= ahead) {
            const int it2 = it - ahead;
            const int row = cluster + it2 * a.num_clusters;
            const int xb = it2 & (kWsSlotBuffers - 1);
            mbar_wait_bounded(smem_u32(&ctl.ready_bar[xb]), (static_cast<uint32_t>(it2) / kWsSlotBuffers) & 1u, a.status);
            float sums[KP];
            ws_load_record<KP>(&ctl.total[xb][0], sums);
            // the row's scalars were published before its pass 1, which this warp has run
            const float4 info = Op::kRowInfo ? ctl.row_info[xb] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const uint4* tiles[NIN];
#pragma unroll
            for (int n = 0; n < NIN; ++n)
                tiles[n] = reinterpret_cast<const uint4*>(stage_tile<T, NIN>(data, stage2, n, a.slice_elems));
            Op::pass2(st, tiles, nvec, info, sums, prm, row, a.cols, g.start, rank);
            if (g.local > 0) {
                __syncwarp();   // every lane has read its vectors of the stage
                if (lane == 0) mbar_arrive(smem_u32(&ctl.empty[stage2]));
            }
            if (++stage2 == stages) stage2 = 0;
        }
    }
    Op::finish(st, prm, cluster, a.cols, g.start, nvec);
}

// ---------------------------------------------------------------------------
// RMSNorm forward: y = x * rsqrt(mean(x^2) + eps) * gamma. One sum per row.
// ---------------------------------------------------------------------------
template <typename T, int OUT_WARPS, int VPT, bool FULL>
struct RmsNormFwdOp {
    using Elem = T;
    static constexpr int kInputs = 1, kOutWarps = OUT_WARPS, kVectors = VPT, THREADS = OUT_WARPS * 32;
    static constexpr bool kFull = FULL;
    static constexpr int E = PairVec<T>::kElems, PAIRS = PairVec<T>::kPairs;
    // a record of two sums; the thread owns fixed vectors of the slice (register-resident parameters)
    static constexpr int kPartials = 2, kLocalBuffers = 4;
    static constexpr bool kAdditive = true, kRegisterSlice = true;
    __device__ __forceinline__ static void identity(float (&v)[2]) { v[0] = v[1] = 0.0f; }
    __device__ __forceinline__ static void combine(float (&v)[2], const float (&o)[2]) { v[0] += o[0]; v[1] += o[1]; }
    struct State {
        float2 gam[VPT][PAIRS];
    };
    __device__ __forceinline__ static void sources(const NormParams& p, const T* (&src)[1]) {
        src[0] = static_cast<const T*>(p.x);
    }
    static constexpr bool kRowInfo = false;
    __device__ __forceinline__ static WsRow fetch_row(const NormParams&, int, int) { return WsRow{0.0f, 0.0f, 0.0f}; }
    __device__ __forceinline__ static float4 publish_row(const WsRow&) { return make_float4(0.0f, 0.0f, 0.0f, 0.0f); }
    __device__ __forceinline__ static void init(State& st, const NormParams& p, int col0, int nvec) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) st.gam[i][j] = splat(0.0f);
            if (FULL || v < nvec) load_param_pairs<PAIRS>(p.gamma + col0 + v * E, st.gam[i]);
        }
    }
    __device__ __forceinline__ static void pass1(State&, const uint4* const (&tiles)[1], int nvec, const float4&,
                                                 float (&part)[2]) {
        float2 q[2] = {splat(0.0f), splat(0.0f)};
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (FULL || v < nvec) {
                float2 xv[PAIRS];
                PairVec<T>::unpack(tiles[0][v], xv);
#pragma unroll
                for (int j = 0; j < PAIRS; ++j) q[j & 1] = __ffma2_rn(xv[j], xv[j], q[j & 1]);
            }
        }
        const float2 t = __fadd2_rn(q[0], q[1]);
        part[0] = t.x + t.y;
        part[1] = 0.0f;
    }
    __device__ __forceinline__ static void pass2(State& st, const uint4* const (&tiles)[1], int nvec, const float4&,
                                                 const float (&sums)[2], const NormParams& p, int row, int cols, int col0,
                                                 uint32_t) {
        const float2 scale = splat(rsqrtf(sums[0] * (1.0f / static_cast<float>(cols)) + p.eps));
        uint4* out = reinterpret_cast<uint4*>(static_cast<T*>(p.y) + static_cast<size_t>(row) * cols + col0);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (FULL || v < nvec) {
                float2 xv[PAIRS];
                PairVec<T>::unpack(tiles[0][v], xv);
#pragma unroll
                for (int j = 0; j < PAIRS; ++j) xv[j] = __fmul2_rn(__fmul2_rn(xv[j], scale), st.gam[i][j]);
                __stcs(out + v, PairVec<T>::pack(xv));
            }
        }
    }
    __device__ __forceinline__ static void finish(State&, const NormParams&, int, int, int, int) {}
};

// ---------------------------------------------------------------------------
// LayerNorm forward: y = (x - mean) * rstd * gamma + beta, plus mean and rstd. Shifted one-pass
// sums S = sum(x - K), Q = sum((x - K)^2) with K = row_shift_sample (median of three elements of
// the row, the same in every CTA).
// ---------------------------------------------------------------------------
template <typename T, int OUT_WARPS, int VPT, bool FULL>
struct LayerNormFwdOp {
    using Elem = T;
    static constexpr int kInputs = 1, kOutWarps = OUT_WARPS, kVectors = VPT, THREADS = OUT_WARPS * 32;
    static constexpr bool kFull = FULL;
    static constexpr int E = PairVec<T>::kElems, PAIRS = PairVec<T>::kPairs;
    // a record of two sums; the thread owns fixed vectors of the slice (register-resident parameters)
    static constexpr int kPartials = 2, kLocalBuffers = 4;
    static constexpr bool kAdditive = true, kRegisterSlice = true;
    __device__ __forceinline__ static void identity(float (&v)[2]) { v[0] = v[1] = 0.0f; }
    __device__ __forceinline__ static void combine(float (&v)[2], const float (&o)[2]) { v[0] += o[0]; v[1] += o[1]; }
    struct State {
        float2 gam[VPT][PAIRS], bet[VPT][PAIRS];
    };
    __device__ __forceinline__ static void sources(const NormParams& p, const T* (&src)[1]) {
        src[0] = static_cast<const T*>(p.x);
    }
    __device__ __forceinline__ static WsRow fetch_row(const NormParams& p, int row, int cols) {
        const T* r = static_cast<const T*>(p.x) + static_cast<size_t>(row) * cols;
        return WsRow{RowVec<T>::to_float(__ldg(r)), RowVec<T>::to_float(__ldg(r + (cols >> 1))),
                     RowVec<T>::to_float(__ldg(r + (cols - 1)))};
    }
    static constexpr bool kRowInfo = true;
    // the row's shift: the median of its three samples (see row_shift_sample)
    __device__ __forceinline__ static float4 publish_row(const WsRow& r) {
        return make_float4(fmaxf(fminf(r.a, r.b), fminf(fmaxf(r.a, r.b), r.c)), 0.0f, 0.0f, 0.0f);
    }
    __device__ __forceinline__ static void init(State& st, const NormParams& p, int col0, int nvec) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                st.gam[i][j] = splat(0.0f);
                st.bet[i][j] = splat(0.0f);
            }
            if (FULL || v < nvec) {
                load_param_pairs<PAIRS>(p.gamma + col0 + v * E, st.gam[i]);
                load_param_pairs<PAIRS>(p.beta + col0 + v * E, st.bet[i]);
            }
        }
    }
    __device__ __forceinline__ static void pass1(State&, const uint4* const (&tiles)[1], int nvec, const float4& r,
                                                 float (&part)[2]) {
        const float2 neg_shift = splat(-r.x);
        float2 s[2] = {splat(0.0f), splat(0.0f)}, q[2] = {splat(0.0f), splat(0.0f)};
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (FULL || v < nvec) {
                float2 xv[PAIRS];
                PairVec<T>::unpack(tiles[0][v], xv);
#pragma unroll
                for (int j = 0; j < PAIRS; ++j) {
                    const float2 d = __fadd2_rn(xv[j], neg_shift);
                    s[j & 1] = __fadd2_rn(s[j & 1], d);
                    q[j & 1] = __ffma2_rn(d, d, q[j & 1]);
                }
            }
        }
        const float2 st = __fadd2_rn(s[0], s[1]), qt = __fadd2_rn(q[0], q[1]);
        part[0] = st.x + st.y;
        part[1] = qt.x + qt.y;
    }
    __device__ __forceinline__ static void pass2(State& st, const uint4* const (&tiles)[1], int nvec, const float4& r,
                                                 const float (&sums)[2], const NormParams& p, int row, int cols, int col0,
                                                 uint32_t rank) {
        float mean, var;
        moments_from_shifted(sums[0], sums[1], r.x, cols, mean, var);
        const float rstd = rsqrtf(var + p.eps);
        if (rank == 0 && threadIdx.x == 0) {
            p.mean_out[row] = mean;
            p.rstd_out[row] = rstd;
        }
        const float2 neg_mean = splat(-mean), rstd2 = splat(rstd);
        // 16-bit rows: xhat = x * rstd - mean * rstd in one fused operation (the rounding of the
        // constant costs |mean| / std * 6e-8 on xhat, far below the output's own 2^-9); fp32 rows
        // keep the exact (x - mean) * rstd.
        const float2 shift2 = splat(-mean * rstd);
        uint4* out = reinterpret_cast<uint4*>(static_cast<T*>(p.y) + static_cast<size_t>(row) * cols + col0);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (FULL || v < nvec) {
                float2 xv[PAIRS];
                PairVec<T>::unpack(tiles[0][v], xv);
#pragma unroll
                for (int j = 0; j < PAIRS; ++j) {
                    const float2 xhat = sizeof(T) == 2 ? __ffma2_rn(xv[j], rstd2, shift2)
                                                       : __fmul2_rn(__fadd2_rn(xv[j], neg_mean), rstd2);
                    xv[j] = __ffma2_rn(xhat, st.gam[i][j], st.bet[i][j]);
                }
                __stcs(out + v, PairVec<T>::pack(xv));
            }
        }
    }
    __device__ __forceinline__ static void finish(State&, const NormParams&, int, int, int, int) {}
};

// ---------------------------------------------------------------------------
// LayerNorm backward with given statistics: dx, and the column sums dgamma / dbeta of the rows
// this cluster handled (written at the end to partials[cluster][2][cols]). With c = x - mean,
// xhat = c * rstd, g = dy * gamma, S1 = sum_row g and S2 = sum_row g * c:
//   dx = g * rstd + c * (-rstd^3 * S2 / N) + (-rstd * S1 / N)
// ---------------------------------------------------------------------------
template <typename T, int OUT_WARPS, int VPT, bool FULL, bool GRADS>
struct LayerNormBwdGivenOp {
    using Elem = T;
    static constexpr int kInputs = 2, kOutWarps = OUT_WARPS, kVectors = VPT, THREADS = OUT_WARPS * 32;
    static constexpr bool kFull = FULL;
    static constexpr int E = PairVec<T>::kElems, PAIRS = PairVec<T>::kPairs;
    // a record of two sums; the thread owns fixed vectors of the slice (register-resident parameters)
    static constexpr int kPartials = 2, kLocalBuffers = 4;
    static constexpr bool kAdditive = true, kRegisterSlice = true;
    __device__ __forceinline__ static void identity(float (&v)[2]) { v[0] = v[1] = 0.0f; }
    __device__ __forceinline__ static void combine(float (&v)[2], const float (&o)[2]) { v[0] += o[0]; v[1] += o[1]; }
    static constexpr int GV = GRADS ? VPT : 1;   // without column sums their registers shrink to a stub
    struct State {
        float2 gam[VPT][PAIRS], dgam[GV][PAIRS], dbet[GV][PAIRS];
    };
    __device__ __forceinline__ static void sources(const NormParams& p, const T* (&src)[2]) {
        src[0] = static_cast<const T*>(p.x);
        src[1] = static_cast<const T*>(p.dy);
    }
    __device__ __forceinline__ static WsRow fetch_row(const NormParams& p, int row, int) {
        return WsRow{__ldg(p.mean_in + row), __ldg(p.rstd_in + row), 0.0f};
    }
    static constexpr bool kRowInfo = true;
    __device__ __forceinline__ static float4 publish_row(const WsRow& r) { return make_float4(r.a, r.b, 0.0f, 0.0f); }
    __device__ __forceinline__ static void init(State& st, const NormParams& p, int col0, int nvec) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                st.gam[i][j] = splat(0.0f);
                if constexpr (GRADS) {
                    st.dgam[i][j] = splat(0.0f);
                    st.dbet[i][j] = splat(0.0f);
                }
            }
            if (FULL || v < nvec) load_param_pairs<PAIRS>(p.gamma + col0 + v * E, st.gam[i]);
        }
    }
    // this thread's share of S1 = sum g and S2 = sum g * (x - mean)
    __device__ __forceinline__ static void pass1(State& st, const uint4* const (&tiles)[2], int nvec, const float4& r,
                                                 float (&part)[2]) {
        const float mean = r.x;
        const float2 neg_mean = splat(-mean);
        float2 s1[2] = {splat(0.0f), splat(0.0f)}, s2[2] = {splat(0.0f), splat(0.0f)};   // two chains each
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (FULL || v < nvec) {
                float2 xv[PAIRS], dv[PAIRS];
                PairVec<T>::unpack(tiles[0][v], xv);
                PairVec<T>::unpack(tiles[1][v], dv);
#pragma unroll
                for (int j = 0; j < PAIRS; ++j) {
                    const float2 gg = __fmul2_rn(dv[j], st.gam[i][j]);
                    s1[j & 1] = __fadd2_rn(s1[j & 1], gg);
                    // 16-bit rows: sum g * x here, mean * sum g comes off once per row below
                    s2[j & 1] = sizeof(T) == 2 ? __ffma2_rn(gg, xv[j], s2[j & 1])
                                               : __ffma2_rn(gg, __fadd2_rn(xv[j], neg_mean), s2[j & 1]);
                }
            }
        }
        const float2 s1t = __fadd2_rn(s1[0], s1[1]), s2t = __fadd2_rn(s2[0], s2[1]);
        const float t1 = s1t.x + s1t.y, t2 = s2t.x + s2t.y;
        part[0] = t1;
        part[1] = sizeof(T) == 2 ? fmaf(-mean, t1, t2) : t2;
    }
    __device__ __forceinline__ static void pass2(State& st, const uint4* const (&tiles)[2], int nvec, const float4& r,
                                                 const float (&sums)[2], const NormParams& p, int row, int cols, int col0,
                                                 uint32_t) {
        const float mean = r.x, rstd = r.y;
        const float inv_cols = 1.0f / static_cast<float>(cols);
        const float2 neg_mean = splat(-mean), rstd2 = splat(rstd);
        const float2 ca = splat(-rstd * rstd * rstd * (sums[1] * inv_cols));
        const float2 cb = splat(-rstd * (sums[0] * inv_cols));
        // 16-bit rows work on xhat = x * rstd - mean * rstd (one fused operation; the rounding of
        // the constant is far below the output's 2^-9): dx = xhat * ca_hat + g * rstd + cb and
        // dgamma += dy * xhat, one operation less per pair than the (x - mean) form fp32 rows keep.
        const float2 shift2 = splat(-mean * rstd);
        const float2 ca_hat = splat(-rstd * rstd * (sums[1] * inv_cols));
        uint4* out = reinterpret_cast<uint4*>(static_cast<T*>(p.y) + static_cast<size_t>(row) * cols + col0);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (FULL || v < nvec) {
                float2 xv[PAIRS], dv[PAIRS], o[PAIRS];
                PairVec<T>::unpack(tiles[0][v], xv);
                PairVec<T>::unpack(tiles[1][v], dv);
#pragma unroll
                for (int j = 0; j < PAIRS; ++j) {
                    const float2 gg = __fmul2_rn(dv[j], st.gam[i][j]);
                    if (sizeof(T) == 2) {
                        const float2 xhat = __ffma2_rn(xv[j], rstd2, shift2);
                        o[j] = __ffma2_rn(xhat, ca_hat, __ffma2_rn(gg, rstd2, cb));
                        if constexpr (GRADS) st.dgam[i][j] = __ffma2_rn(dv[j], xhat, st.dgam[i][j]);
                    } else {
                        const float2 c = __fadd2_rn(xv[j], neg_mean);
                        o[j] = __ffma2_rn(c, ca, __ffma2_rn(gg, rstd2, cb));
                        if constexpr (GRADS) st.dgam[i][j] = __ffma2_rn(__fmul2_rn(dv[j], c), rstd2, st.dgam[i][j]);
                    }
                    if constexpr (GRADS) st.dbet[i][j] = __fadd2_rn(st.dbet[i][j], dv[j]);
                }
                __stcs(out + v, PairVec<T>::pack(o));
            }
        }
    }
    __device__ __forceinline__ static void finish(State& st, const NormParams& p, int cluster, int cols, int col0, int nvec) {
        if constexpr (!GRADS) return;
        float* out_g = p.partials + (static_cast<size_t>(cluster) * 2 + 0) * cols + col0;
        float* out_b = p.partials + (static_cast<size_t>(cluster) * 2 + 1) * cols + col0;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (FULL || v < nvec) {
#pragma unroll
                for (int j = 0; j < PAIRS; j += 2) {
                    *reinterpret_cast<float4*>(out_g + v * E + 2 * j) =
                        make_float4(st.dgam[i][j].x, st.dgam[i][j].y, st.dgam[i][j + 1].x, st.dgam[i][j + 1].y);
                    *reinterpret_cast<float4*>(out_b + v * E + 2 * j) =
                        make_float4(st.dbet[i][j].x, st.dbet[i][j].y, st.dbet[i][j + 1].x, st.dbet[i][j + 1].y);
                }
            }
        }
    }
};

template <typename T, int OUT_WARPS, int VPT, bool FULL>
using LayerNormBwdOp = LayerNormBwdGivenOp<T, OUT_WARPS, VPT, FULL, true>;
template <typename T, int OUT_WARPS, int VPT, bool FULL>
using LayerNormBwdDxOp = LayerNormBwdGivenOp<T, OUT_WARPS, VPT, FULL, false>;

// ---------------------------------------------------------------------------
// LayerNorm backward as the reference states it (dsmem_eval/workloads.py:53-61): the row's mean
// and variance are recomputed from x and only dx is written. One pass over the staged slice
// gathers a record of four sums about the row's shift K (the median of three samples, published
// by the collector warp): with d = x - K and g = dy * gamma,
//   A = sum d, B = sum d^2, C = sum g, D = sum g * d.
// Then m = A / N, mean = K + m, var = B / N - m^2, S1 = C, S2 = sum g * (x - mean) = D - m * C and
//   dx = g * rstd + (d - m) * (-rstd^3 * S2 / N) + (-rstd * S1 / N).
// The record of four floats per thread bounds the kernel to 8 output warps (control block size).
// ---------------------------------------------------------------------------
template <typename T, int OUT_WARPS, int VPT, bool FULL>
struct LayerNormBwdRecomputeOp {
    using Elem = T;
    static constexpr int kInputs = 2, kOutWarps = OUT_WARPS, kVectors = VPT, THREADS = OUT_WARPS * 32;
    static constexpr bool kFull = FULL;
    static constexpr int E = PairVec<T>::kElems, PAIRS = PairVec<T>::kPairs;
    static constexpr int kPartials = 4, kLocalBuffers = 4;
    static constexpr bool kAdditive = true, kRegisterSlice = true;
    __device__ __forceinline__ static void identity(float (&v)[4]) { v[0] = v[1] = v[2] = v[3] = 0.0f; }
    __device__ __forceinline__ static void combine(float (&v)[4], const float (&o)[4]) {
#pragma unroll
        for (int k = 0; k < 4; ++k) v[k] += o[k];
    }
    struct State {
        float2 gam[VPT][PAIRS];
    };
    __device__ __forceinline__ static void sources(const NormParams& p, const T* (&src)[2]) {
        src[0] = static_cast<const T*>(p.x);
        src[1] = static_cast<const T*>(p.dy);
    }
    __device__ __forceinline__ static WsRow fetch_row(const NormParams& p, int row, int cols) {
        const T* r = static_cast<const T*>(p.x) + static_cast<size_t>(row) * cols;
        return WsRow{RowVec<T>::to_float(__ldg(r)), RowVec<T>::to_float(__ldg(r + (cols >> 1))),
                     RowVec<T>::to_float(__ldg(r + (cols - 1)))};
    }
    static constexpr bool kRowInfo = true;
    __device__ __forceinline__ static float4 publish_row(const WsRow& r) {
        return make_float4(fmaxf(fminf(r.a, r.b), fminf(fmaxf(r.a, r.b), r.c)), 0.0f, 0.0f, 0.0f);
    }
    __device__ __forceinline__ static void init(State& st, const NormParams& p, int col0, int nvec) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) st.gam[i][j] = splat(0.0f);
            if (FULL || v < nvec) load_param_pairs<PAIRS>(p.gamma + col0 + v * E, st.gam[i]);
        }
    }
    __device__ __forceinline__ static void pass1(State& st, const uint4* const (&tiles)[2], int nvec, const float4& r,
                                                 float (&part)[4]) {
        const float2 neg_shift = splat(-r.x);
        float2 sa = splat(0.0f), sb = splat(0.0f), sc = splat(0.0f), sd = splat(0.0f);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (FULL || v < nvec) {
                float2 xv[PAIRS], dv[PAIRS];
                PairVec<T>::unpack(tiles[0][v], xv);
                PairVec<T>::unpack(tiles[1][v], dv);
#pragma unroll
                for (int j = 0; j < PAIRS; ++j) {
                    const float2 d = __fadd2_rn(xv[j], neg_shift);
                    const float2 gg = __fmul2_rn(dv[j], st.gam[i][j]);
                    sa = __fadd2_rn(sa, d);
                    sb = __ffma2_rn(d, d, sb);
                    sc = __fadd2_rn(sc, gg);
                    sd = __ffma2_rn(gg, d, sd);
                }
            }
        }
        part[0] = sa.x + sa.y;
        part[1] = sb.x + sb.y;
        part[2] = sc.x + sc.y;
        part[3] = sd.x + sd.y;
    }
    __device__ __forceinline__ static void pass2(State& st, const uint4* const (&tiles)[2], int nvec, const float4& r,
                                                 const float (&sums)[4], const NormParams& p, int row, int cols, int col0,
                                                 uint32_t) {
        const float inv_cols = 1.0f / static_cast<float>(cols);
        const float m = sums[0] * inv_cols;
        const float var = fmaxf(sums[1] * inv_cols - m * m, 0.0f);
        const float rstd = rsqrtf(var + p.eps);
        const float s2 = fmaf(-m, sums[2], sums[3]);
        const float2 neg_center = splat(-(r.x + m)), rstd2 = splat(rstd);
        const float2 ca = splat(-rstd * rstd * rstd * (s2 * inv_cols));
        const float2 cb = splat(-rstd * (sums[2] * inv_cols));
        uint4* out = reinterpret_cast<uint4*>(static_cast<T*>(p.y) + static_cast<size_t>(row) * cols + col0);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (FULL || v < nvec) {
                float2 xv[PAIRS], dv[PAIRS], o[PAIRS];
                PairVec<T>::unpack(tiles[0][v], xv);
                PairVec<T>::unpack(tiles[1][v], dv);
#pragma unroll
                for (int j = 0; j < PAIRS; ++j) {
                    const float2 gg = __fmul2_rn(dv[j], st.gam[i][j]);
                    const float2 c = __fadd2_rn(xv[j], neg_center);
                    o[j] = __ffma2_rn(c, ca, __ffma2_rn(gg, rstd2, cb));
                }
                __stcs(out + v, PairVec<T>::pack(o));
            }
        }
    }
    __device__ __forceinline__ static void finish(State&, const NormParams&, int, int, int, int) {}
};

}  // namespace credit
