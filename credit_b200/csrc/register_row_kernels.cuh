// Register-resident wide-row kernels: the fast path of RMSNorm forward,
// LayerNorm forward and LayerNorm backward for 16-byte aligned rows whose
// per-CTA slice fits VPT 16-byte vectors per thread.
//
// Data flow per row and CTA:
//   HBM --bulk-async copy (TMA)--> shared-memory ring --one LDS.128 per vector-->
//   registers --> partial statistics --> DSMEM exchange --> outputs from
//   registers --128-bit stores--> HBM
// Thread t owns vectors t, t+THREADS, ... of the slice for every row its cluster
// handles, so gamma/beta (and the running dgamma/dbeta sums)
// for those columns stay in registers for the whole kernel.
//
// Nothing in the row loop is a block-wide or cluster-wide barrier; every warp runs
// its own pipeline and only meets the others through mbarriers:
//   * one lane of the last warp keeps the ring full: before the warp starts row i
//     it waits on empty[stage of row i-1] (one arrival per warp, made as soon as a
//     warp has its vectors of that row in registers) and issues the bulk copies of
//     row i-1+stages, which complete on full[stage];
//   * every warp reduces its partials with shuffles, leaves them in shared memory
//     and arrives on a CTA-local mbarrier; warp 0 alone waits for the W arrivals,
//     folds the W values and pushes the CTA's totals into slot[row % 4][k][rank] of
//     EVERY CTA of the cluster with st.async, which signals the receiver's mbarrier
//     by byte count (no barrier.cluster, whose release has to drain the thread's
//     outstanding global stores, and no fence);
//   * a warp waits on its own CTA's mbarrier until all P contributions of the row
//     have landed, folds them itself (same order in every warp of every CTA, so all
//     agree bit for bit) and produces its outputs.
// Rows are software-pipelined two deep per warp. One step of a warp: wait for row
// i+1 in the ring, load it into registers, compute this thread's partial sums;
// wait for row i's exchange; run the warp reduction of row i+1's partials and the
// fold of row i's slots as two shuffle trees side by side (independent, so they
// cost the latency of one); deliver row i+1's partials; write row i's outputs
// from the registers that still hold row i. The DSMEM round trip of one row thus
// overlaps the loads and arithmetic of the next, and other warps' work. Waits
// poll (mbarrier.test_wait): a suspended try_wait wakes late.
// Slot buffer and mbarrier of row i are number i mod 4. A CTA sends row i+4 only
// after all its warps have delivered row i+4, each of which has by then received
// row i+3, which every CTA sent only after all its warps had delivered row i+3,
// i.e. after they had read the slots of row i+2 and, earlier, of row i: a buffer
// is never overwritten while it is read, and its mbarrier is never re-armed
// before every waiter has seen its previous phase complete (a peer's bytes may
// land before the local arming arrival; the phase cannot complete without it).
// The same argument, one level down, covers the two CTA-local partial buffers.
//
// Same arithmetic as the reference's cluster_bwd_staged_kernel family
// (src/workloads/layernorm_backward.cu:376-438), re-designed for sm_100a.
#pragma once

#include "cluster_primitives.cuh"
#include "norm_kernels.cuh"

namespace credit {

constexpr int kExchangeBuffers = 4;

template <int K>
struct alignas(16) ExchangeStream {
    uint64_t bar[kExchangeBuffers];                      // cluster level: one mbarrier per slot buffer
    uint64_t local_bar[2];                               // CTA level: W arrivals per row
    float warp_part[2][K][kMaxWarpsPerCta];              // [row parity][partial][warp]
    float slot[kExchangeBuffers][K][kMaxClusterSize];    // [buffer][partial][source rank]
};

// Control block at the start of dynamic shared memory (kControlBytes reserved).
template <int K>
struct alignas(16) AsyncControl {
    uint64_t full[kMaxStages];    // stage has landed (1 arrival + transaction bytes)
    uint64_t empty[kMaxStages];   // stage is in registers everywhere (W arrivals)
    ExchangeStream<K> ex;
    ExchangeStream<K> ex2;        // second reduction of kernels with two dependent ones
};
static_assert(sizeof(AsyncControl<2>) <= kControlBytes, "control block overflows its reservation");

// Delivers this warp's K warp-reduced partials of row `it`; warp 0 then collects
// the W deliveries of the CTA, folds them and sends the CTA's totals to every CTA
// of the cluster (arming its own mbarrier for the P * K floats it will receive).
// Called by all 32 lanes of every warp; only warp 0 waits, and only for the
// partials of this same row from its own CTA.
template <int K, int W>
__device__ __forceinline__ void exchange_send(const float (&vals)[K], ExchangeStream<K>& s, int it,
                                              uint32_t rank, uint32_t nranks, int* status) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = threadIdx.x >> 5;
    const int par = it & 1;
    const uint32_t local_bar = smem_u32(&s.local_bar[par]);
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) s.warp_part[par][k][warp] = vals[k];
        mbar_arrive(local_bar);   // release: the partials are visible to whoever sees the phase complete
    }
    if (warp != 0) return;
    mbar_wait_bounded(local_bar, (static_cast<uint32_t>(it) >> 1) & 1u, status);
    const int buf = it & (kExchangeBuffers - 1);
    const uint32_t bar = smem_u32(&s.bar[buf]);
    if (lane == 0) mbar_arrive_expect_tx(bar, nranks * K * static_cast<uint32_t>(sizeof(float)));
    const uint32_t remote_bar = map_to_rank(bar, lane < nranks ? lane : 0);
#pragma unroll
    for (int k = 0; k < K; ++k) {
        float t = lane < W ? s.warp_part[par][k][lane] : 0.0f;
#pragma unroll
        for (int offset = (W > 16 ? 16 : W / 2); offset > 0; offset >>= 1) t += __shfl_xor_sync(0xffffffffu, t, offset);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (lane < nranks)
            st_async_f32(map_to_rank(smem_u32(&s.slot[buf][k][rank]), lane), t, remote_bar);
    }
}

// Waits until the P contributions of row `it` have landed in this CTA and returns
// the K sums over them (identical in every lane, warp and CTA).
template <int K>
__device__ __forceinline__ void exchange_receive(ExchangeStream<K>& s, int it, uint32_t nranks,
                                                 int* status, float (&total)[K]) {
    const int buf = it & (kExchangeBuffers - 1);
    const uint32_t phase = (static_cast<uint32_t>(it) / kExchangeBuffers) & 1u;
    mbar_wait_bounded(smem_u32(&s.bar[buf]), phase, status);
    const uint32_t lane = threadIdx.x & 31;
#pragma unroll
    for (int k = 0; k < K; ++k) {
        float t = lane < nranks ? s.slot[buf][k][lane] : 0.0f;
#pragma unroll
        for (int offset = kMaxClusterSize / 2; offset > 0; offset >>= 1) t += __shfl_xor_sync(0xffffffffu, t, offset);
        total[k] = __shfl_sync(0xffffffffu, t, 0);
    }
}

// Two sums over the warp in five exchange rounds instead of ten: after the first round lanes
// 0..15 carry `a` and lanes 16..31 carry `b`. Returns the total of a in lanes 0..15 and the total
// of b in lanes 16..31.
__device__ __forceinline__ float warp_sum_split(float a, float b) {
    const bool upper = (threadIdx.x & 16u) != 0;
    float keep = upper ? b : a;
    const float give = upper ? a : b;
    keep += __shfl_xor_sync(0xffffffffu, give, 16);
#pragma unroll
    for (int offset = 8; offset > 0; offset >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, offset);
    return keep;
}

// exchange_send for two partials in the split form of warp_sum_split (`keep`: partial 0 in lanes
// 0..15, partial 1 in lanes 16..31). The collector folds both partials in one shuffle tree, the
// halves of the warp working on one partial each. W <= 16.
template <int W, int SLEEP_NS = 0>
__device__ __forceinline__ void exchange_send_split(float keep, ExchangeStream<2>& s, int it, uint32_t rank,
                                                    uint32_t nranks, int* status) {
    static_assert(W <= 16, "one half of the collecting warp folds one partial of every warp");
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t half = lane >> 4, idx = lane & 15;
    const int par = it & 1;
    const uint32_t local_bar = smem_u32(&s.local_bar[par]);
    if (idx == 0) s.warp_part[par][half][warp] = keep;
    __syncwarp();                           // lane 16's store is ordered before lane 0's release
    if (lane == 0) mbar_arrive(local_bar);
    if (warp != 0) return;
    mbar_wait_bounded<SLEEP_NS>(local_bar, (static_cast<uint32_t>(it) >> 1) & 1u, status);
    const int buf = it & (kExchangeBuffers - 1);
    const uint32_t bar = smem_u32(&s.bar[buf]);
    if (lane == 0) mbar_arrive_expect_tx(bar, nranks * 2u * static_cast<uint32_t>(sizeof(float)));
    float t = idx < W ? s.warp_part[par][half][idx] : 0.0f;
#pragma unroll
    for (int offset = W / 2; offset > 0; offset >>= 1) t += __shfl_xor_sync(0xffffffffu, t, offset);
    const float t0 = __shfl_sync(0xffffffffu, t, 0);
    const float t1 = __shfl_sync(0xffffffffu, t, 16);
    // the slots of a buffer are laid out [source rank][partial] here: one 8-byte message per peer
    if (lane < nranks)
        st_async_f32x2(map_to_rank(smem_u32(&s.slot[buf][0][0] + 2 * rank), lane), t0, t1, map_to_rank(bar, lane));
}

// exchange_receive for two partials, both folded in one shuffle tree.
template <int SLEEP_NS = 0>
__device__ __forceinline__ void exchange_receive_split(ExchangeStream<2>& s, int it, uint32_t nranks, int* status,
                                                       float (&total)[2]) {
    static_assert(kMaxClusterSize == 16, "one half of the warp reads the slots of one partial");
    const int buf = it & (kExchangeBuffers - 1);
    const uint32_t phase = (static_cast<uint32_t>(it) / kExchangeBuffers) & 1u;
    mbar_wait_bounded<SLEEP_NS>(smem_u32(&s.bar[buf]), phase, status);
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t half = lane >> 4, idx = lane & 15;
    float t = idx < nranks ? (&s.slot[buf][0][0])[2 * idx + half] : 0.0f;
#pragma unroll
    for (int offset = 8; offset > 0; offset >>= 1) t += __shfl_xor_sync(0xffffffffu, t, offset);
    total[0] = __shfl_sync(0xffffffffu, t, 0);
    total[1] = __shfl_sync(0xffffffffu, t, 16);
}

// One partial per row: warp_sum of the NEXT row's partial and exchange_receive<1> of THIS row with
// the two shuffle trees side by side (see reduce_and_receive_split).
__device__ __forceinline__ float reduce_and_receive_one(float a, ExchangeStream<1>& s, int it_recv, uint32_t nranks,
                                                        int* status, float& total) {
    const int buf = it_recv & (kExchangeBuffers - 1);
    const uint32_t phase = (static_cast<uint32_t>(it_recv) / kExchangeBuffers) & 1u;
    mbar_wait_bounded(smem_u32(&s.bar[buf]), phase, status);
    const uint32_t lane = threadIdx.x & 31;
    float t = lane < nranks ? s.slot[buf][0][lane] : 0.0f;
    a += __shfl_xor_sync(0xffffffffu, a, 16);
#pragma unroll
    for (int offset = kMaxClusterSize / 2; offset > 0; offset >>= 1) {
        t += __shfl_xor_sync(0xffffffffu, t, offset);
        a += __shfl_xor_sync(0xffffffffu, a, offset);
    }
    total = __shfl_sync(0xffffffffu, t, 0);
    return a;
}

// warp_sum_split of the NEXT row's two partials and exchange_receive_split of THIS row in one
// step. The two shuffle trees are independent; issued round by round side by side they cost the
// latency of one, and that latency is on every warp's per-row chain. Returns `keep` as
// warp_sum_split does; `total` as exchange_receive_split does.
template <int SLEEP_NS = 0>
__device__ __forceinline__ float reduce_and_receive_split(float a, float b, ExchangeStream<2>& s, int it_recv,
                                                          uint32_t nranks, int* status, float (&total)[2]) {
    const int buf = it_recv & (kExchangeBuffers - 1);
    const uint32_t phase = (static_cast<uint32_t>(it_recv) / kExchangeBuffers) & 1u;
    mbar_wait_bounded<SLEEP_NS>(smem_u32(&s.bar[buf]), phase, status);
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t half = lane >> 4, idx = lane & 15;
    float t = idx < nranks ? (&s.slot[buf][0][0])[2 * idx + half] : 0.0f;
    float keep = half != 0 ? b : a;
    const float give = half != 0 ? a : b;
    keep += __shfl_xor_sync(0xffffffffu, give, 16);
#pragma unroll
    for (int offset = 8; offset > 0; offset >>= 1) {
        t += __shfl_xor_sync(0xffffffffu, t, offset);
        keep += __shfl_xor_sync(0xffffffffu, keep, offset);
    }
    total[0] = __shfl_sync(0xffffffffu, t, 0);
    total[1] = __shfl_sync(0xffffffffu, t, 16);
    return keep;
}

// A 16-byte vector of row elements as packed fp32 pairs, so that the elementwise
// arithmetic can use the two-wide fp32 instructions of sm_100
// (fma/add/mul.rn.f32x2 through __ffma2_rn, __fadd2_rn, __fmul2_rn): half the
// issue slots of scalar fp32 for the same work.
template <typename T>
struct PairVec;
template <>
struct PairVec<float> {
    static constexpr int kElems = 4;
    static constexpr int kPairs = 2;
    __device__ __forceinline__ static void unpack(const uint4& r, float2 (&p)[2]) {
        p[0] = make_float2(__uint_as_float(r.x), __uint_as_float(r.y));
        p[1] = make_float2(__uint_as_float(r.z), __uint_as_float(r.w));
    }
    __device__ __forceinline__ static uint4 pack(const float2 (&p)[2]) {
        return make_uint4(__float_as_uint(p[0].x), __float_as_uint(p[0].y), __float_as_uint(p[1].x),
                          __float_as_uint(p[1].y));
    }
    __device__ __forceinline__ static float first(const void* tile) {
        return *reinterpret_cast<const float*>(tile);
    }
};
template <>
struct PairVec<__nv_bfloat16> {
    static constexpr int kElems = 8;
    static constexpr int kPairs = 4;
    __device__ __forceinline__ static float2 widen(uint32_t w) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
    __device__ __forceinline__ static void unpack(const uint4& r, float2 (&p)[4]) {
        p[0] = widen(r.x); p[1] = widen(r.y); p[2] = widen(r.z); p[3] = widen(r.w);
    }
    __device__ __forceinline__ static uint32_t narrow(const float2& v) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v.x, v.y);
        return *reinterpret_cast<const uint32_t*>(&h);
    }
    __device__ __forceinline__ static uint4 pack(const float2 (&p)[4]) {
        return make_uint4(narrow(p[0]), narrow(p[1]), narrow(p[2]), narrow(p[3]));
    }
    __device__ __forceinline__ static float first(const void* tile) {
        return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(tile));
    }
};

__device__ __forceinline__ float2 splat(float v) { return make_float2(v, v); }

// gamma / beta of one vector as pairs.
template <int PAIRS>
__device__ __forceinline__ void load_param_pairs(const float* p, float2 (&out)[PAIRS]) {
#pragma unroll
    for (int j = 0; j < PAIRS; j += 2) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p + 2 * j));
        out[j] = make_float2(v.x, v.y);
        out[j + 1] = make_float2(v.z, v.w);
    }
}

// Barriers initialised and every CTA of the cluster running (a CTA's shared memory
// may only be written by its peers once it has started). All threads call this.
template <int K, int W>
__device__ __forceinline__ void async_prologue(AsyncControl<K>& ctl, int stages) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&ctl.full[s]), 1);
            mbar_init(smem_u32(&ctl.empty[s]), W);
        }
        for (int b = 0; b < kExchangeBuffers; ++b) {
            mbar_init(smem_u32(&ctl.ex.bar[b]), 1);
            mbar_init(smem_u32(&ctl.ex2.bar[b]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&ctl.ex.local_bar[b]), W);
            mbar_init(smem_u32(&ctl.ex2.local_bar[b]), W);
        }
        fence_mbar_init();
    }
    __syncthreads();
    cluster_sync_all();
}

// Ring maintenance, done by lane 0 of the last warp. prime: the first `stages` rows.
// recycle(it), called before that warp starts row `it` >= 1: the stage that held
// row it-1 is refilled with row it-1+stages once every warp has arrived on its
// empty barrier (its vectors are in registers and every value read has been used,
// so the bulk copy cannot overtake a read). The warps this waits for never wait for
// this warp's row `it`, so the wait always ends.
template <typename T, int NIN, int K>
struct RingFiller {
    AsyncControl<K>& ctl;
    const T* const (&src)[NIN];
    unsigned char* data;
    int cluster;
    int my_rows;
    const StagedArgs& a;
    const SliceGeom& g;

    __device__ __forceinline__ void prime() const {
        if (g.local == 0) return;
        for (int n = 0; n < a.stages && n < my_rows; ++n)
            issue_slice_fill<T, NIN>(src, data, ctl.full, n, cluster + n * a.num_clusters, a, g);
    }
    // `lag`: how many rows back the stage to refill was used. 1: stages are released as soon as
    // a row is in registers; 2: a row's stage stays in use until its outputs are written (kernels
    // that read the row from shared memory twice), so the one to refill is that of row it - 2.
    __device__ __forceinline__ void recycle(int it, int lag = 1) const {
        const int freed = it - lag;
        const int n = freed + a.stages;
        if (g.local == 0 || freed < 0 || n >= my_rows) return;
        const int stage = freed % a.stages;
        const uint32_t parity = static_cast<uint32_t>(freed / a.stages) & 1u;
        mbar_wait_bounded(smem_u32(&ctl.empty[stage]), parity, a.status);
        issue_slice_fill<T, NIN>(src, data, ctl.full, stage, cluster + n * a.num_clusters, a, g);
    }
};

// Copies this thread's vectors of a staged slice into registers. FULL: every
// thread owns exactly VPT vectors, no bounds checks.
template <int THREADS, int VPT, bool FULL>
__device__ __forceinline__ void load_raw(const uint4* tile, int nvec, uint4 (&raw)[VPT]) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
        raw[i] = (FULL || v < nvec) ? tile[v] : make_uint4(0u, 0u, 0u, 0u);
    }
}

// The two-deep software pipeline every compute warp runs, for kernels with one reduction per
// row. `front` ends with the row's partials delivered, `back` starts by waiting for the row's
// exchange; `fused(next, it + 1, current, it)` is front(next) and back(current) in one step with
// their two shuffle trees side by side:
//   front(0); { fused(i+1, i); } ... back(last)
template <typename Regs, typename Front, typename Fused, typename Back>
__device__ __forceinline__ void pipeline_rows_fused(int my_rows, Regs& r0, Regs& r1, Front front, Fused fused,
                                                    Back back) {
    if (my_rows > 0) front(r0, 0);
    for (int it = 0; it < my_rows; it += 2) {
        if (it + 1 < my_rows) fused(r1, it + 1, r0, it);
        else back(r0, it);
        if (it + 1 < my_rows) {
            if (it + 2 < my_rows) fused(r0, it + 2, r1, it + 1);
            else back(r1, it + 1);
        }
    }
}

// Kernels with two dependent reductions per row: middle(i) finishes the first, and front(i+1)
// and back(i) are again one fused step.
template <typename Regs, typename Front, typename Middle, typename Fused, typename Back>
__device__ __forceinline__ void pipeline_rows_middle_fused(int my_rows, Regs& r0, Regs& r1, Front front,
                                                           Middle middle, Fused fused, Back back) {
    if (my_rows > 0) front(r0, 0);
    for (int it = 0; it < my_rows; it += 2) {
        middle(r0, it);
        if (it + 1 < my_rows) fused(r1, it + 1, r0, it);
        else back(r0, it);
        if (it + 1 < my_rows) {
            middle(r1, it + 1);
            if (it + 2 < my_rows) fused(r0, it + 2, r1, it + 1);
            else back(r1, it + 1);
        }
    }
}

// ---------------------------------------------------------------------------
// RMSNorm forward
// ---------------------------------------------------------------------------
template <typename T, int THREADS, int VPT, bool FULL>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_reg_kernel(const T* __restrict__ x, const float* __restrict__ gamma, T* __restrict__ y,
                       float eps, StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<AsyncControl<1>*>(smem);
    unsigned char* data = smem + kControlBytes;
    constexpr int E = PairVec<T>::kElems;
    constexpr int PAIRS = PairVec<T>::kPairs;
    constexpr int W = THREADS / 32;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const int nvec = g.local / E;
    const T* const src[1] = {x};
    const int my_rows = cluster < a.rows ? (a.rows - cluster + a.num_clusters - 1) / a.num_clusters : 0;
    if ((FULL ? nvec != VPT * THREADS : nvec > VPT * THREADS) && threadIdx.x == 0)
        atomicOr(a.status, kStatusBadGeometry);

    async_prologue<1, W>(ctl, a.stages);
    const RingFiller<T, 1, 1> filler{ctl, src, data, cluster, my_rows, a, g};
    const bool fills_ring = threadIdx.x == THREADS - 32;
    if (fills_ring) filler.prime();

    float2 gam[VPT][PAIRS];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) gam[i][j] = splat(0.0f);
        if (FULL || v < nvec) load_param_pairs<PAIRS>(gamma + g.start + v * E, gam[i]);
    }

    RingCursor ring{0, 0u};
    const float inv_cols = 1.0f / static_cast<float>(a.cols);
    struct Regs { uint4 raw[VPT]; };

    // the row into registers; returns this thread's sum of squares
    auto front_load = [&](Regs& r, int it) -> float {
        if (fills_ring && it > 0) filler.recycle(it);
        if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[ring.stage]), ring.parity, a.status);
        load_raw<THREADS, VPT, FULL>(
            reinterpret_cast<const uint4*>(stage_tile<T, 1>(data, ring.stage, 0, a.slice_elems)), nvec, r.raw);
        float2 q0 = splat(0.0f), q1 = splat(0.0f);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            float2 xv[PAIRS];
            PairVec<T>::unpack(r.raw[i], xv);
#pragma unroll
            for (int j = 0; j < PAIRS; j += 2) {
                q0 = __ffma2_rn(xv[j], xv[j], q0);
                q1 = __ffma2_rn(xv[j + 1], xv[j + 1], q1);
            }
        }
        if (g.local > 0 && (threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&ctl.empty[ring.stage]));
        return (q0.x + q0.y) + (q1.x + q1.y);
    };
    auto front_send = [&](float warp_total, int it) {
        const float part[1] = {warp_total};
        exchange_send<1, W>(part, ctl.ex, it, rank, nranks, a.status);
        ring.advance(a.stages);
    };
    auto front = [&](Regs& r, int it) { front_send(warp_sum(front_load(r, it)), it); };
    auto back_store = [&](const Regs& r, int it, float sumsq) {
        const int row = cluster + it * a.num_clusters;
        const float2 scale = splat(rsqrtf(sumsq * inv_cols + eps));
        uint4* out = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * a.cols + g.start);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            float2 xv[PAIRS];
            PairVec<T>::unpack(r.raw[i], xv);
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) xv[j] = __fmul2_rn(__fmul2_rn(xv[j], scale), gam[i][j]);
            if (FULL || v < nvec) __stcs(out + v, PairVec<T>::pack(xv));
        }
    };
    auto back = [&](const Regs& r, int it) {
        float sumsq[1];
        exchange_receive<1>(ctl.ex, it, nranks, a.status, sumsq);
        back_store(r, it, sumsq[0]);
    };
    // front(next) and back(current) with the two shuffle trees side by side
    auto fused = [&](Regs& rn, int itn, const Regs& ro, int ito) {
        float sumsq;
        const float warp_total = reduce_and_receive_one(front_load(rn, itn), ctl.ex, ito, nranks, a.status, sumsq);
        front_send(warp_total, itn);
        back_store(ro, ito, sumsq);
    };
    Regs r0, r1;
    pipeline_rows_fused(my_rows, r0, r1, front, fused, back);
}

// Shifted one-pass statistics of the vectors held in `raw`: with K = a sample of
// the ROW (row_shift_sample: the same K in every CTA, so the partials of all CTAs
// simply add), accumulates sum(x-K) and sum((x-K)^2). K is within a few standard
// deviations of the mean, so the final subtraction loses about one digit instead
// of log10(mean^2/var). Outputs the per-thread partials.
template <typename T, int THREADS, int VPT, bool FULL>
__device__ __forceinline__ void shifted_partials(const uint4 (&raw)[VPT], int nvec, float shift,
                                                 float& s, float& q) {
    constexpr int PAIRS = PairVec<T>::kPairs;
    const float2 neg_shift = splat(-shift);
    float2 s2 = splat(0.0f), q2 = splat(0.0f);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (FULL || v < nvec) {
            float2 xv[PAIRS];
            PairVec<T>::unpack(raw[i], xv);
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const float2 d = __fadd2_rn(xv[j], neg_shift);
                s2 = __fadd2_rn(s2, d);
                q2 = __ffma2_rn(d, d, q2);
            }
        }
    }
    s = s2.x + s2.y;
    q = q2.x + q2.y;
}

// Row mean and biased variance from the cluster-wide sums S = sum(x-K), Q = sum((x-K)^2).
__device__ __forceinline__ void moments_from_shifted(float S, float Q, float shift, int cols,
                                                     float& mean, float& var) {
    const float inv_n = 1.0f / static_cast<float>(cols);
    const float ds = S * inv_n;
    mean = shift + ds;
    var = fmaxf(Q * inv_n - ds * ds, 0.0f);
}

// The shift of a row: the median of three of its elements (first, middle, last). Any shift
// within about ten standard deviations of the mean keeps the relative error of the variance
// below 1e-5 in fp32 (the error is eps * (shift - mean)^2 / var); a single element can be an
// outlier far outside that range, the median of three is not unless two of them are. Every
// thread of every CTA of the cluster reads the same three elements, so all use the same shift.
template <typename T>
__device__ __forceinline__ float row_shift_sample(const T* x, int row, int cols) {
    const T* p = x + static_cast<size_t>(row) * cols;
    const float a = RowVec<T>::to_float(__ldg(p));
    const float b = RowVec<T>::to_float(__ldg(p + (cols >> 1)));
    const float c = RowVec<T>::to_float(__ldg(p + (cols - 1)));
    return fmaxf(fminf(a, b), fminf(fmaxf(a, b), c));
}

// ---------------------------------------------------------------------------
// LayerNorm forward
// ---------------------------------------------------------------------------
// 256-thread CTAs are held to 128 registers so that two of them (of different clusters, whose
// phases drift apart) share an SM.
template <typename T, int THREADS, int VPT, bool FULL>
__global__ void __launch_bounds__(THREADS, THREADS == 256 ? 2 : 1)
layernorm_fwd_reg_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                         const float* __restrict__ beta, T* __restrict__ y,
                         float* __restrict__ mean_out, float* __restrict__ rstd_out, float eps,
                         StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<AsyncControl<2>*>(smem);
    unsigned char* data = smem + kControlBytes;
    constexpr int E = PairVec<T>::kElems;
    constexpr int PAIRS = PairVec<T>::kPairs;
    constexpr int W = THREADS / 32;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const int nvec = g.local / E;
    const T* const src[1] = {x};
    const int my_rows = cluster < a.rows ? (a.rows - cluster + a.num_clusters - 1) / a.num_clusters : 0;
    if ((FULL ? nvec != VPT * THREADS : nvec > VPT * THREADS) && threadIdx.x == 0)
        atomicOr(a.status, kStatusBadGeometry);

    async_prologue<2, W>(ctl, a.stages);
    const RingFiller<T, 1, 2> filler{ctl, src, data, cluster, my_rows, a, g};
    const bool fills_ring = threadIdx.x == THREADS - 32;
    if (fills_ring) filler.prime();

    float2 gam[VPT][PAIRS], bet[VPT][PAIRS];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) {
            gam[i][j] = splat(0.0f);
            bet[i][j] = splat(0.0f);
        }
        if (FULL || v < nvec) {
            load_param_pairs<PAIRS>(gamma + g.start + v * E, gam[i]);
            load_param_pairs<PAIRS>(beta + g.start + v * E, bet[i]);
        }
    }

    RingCursor ring{0, 0u};
    struct Regs { uint4 raw[VPT]; float shift; };
    // the shift of the next row is fetched one step ahead so its latency is hidden
    float next_shift = my_rows > 0 ? row_shift_sample(x, cluster, a.cols) : 0.0f;

    // the row into registers and this thread's two partial sums of it
    auto front_load = [&](Regs& r, int it, float (&part)[2]) {
        if (fills_ring && it > 0) filler.recycle(it);
        r.shift = next_shift;
        if (it + 1 < my_rows) next_shift = row_shift_sample(x, cluster + (it + 1) * a.num_clusters, a.cols);
        if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[ring.stage]), ring.parity, a.status);
        load_raw<THREADS, VPT, FULL>(
            reinterpret_cast<const uint4*>(stage_tile<T, 1>(data, ring.stage, 0, a.slice_elems)), nvec, r.raw);
        shifted_partials<T, THREADS, VPT, FULL>(r.raw, nvec, r.shift, part[0], part[1]);
        if (g.local > 0 && (threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&ctl.empty[ring.stage]));
    };
    auto front_send = [&](float keep, int it) {
        exchange_send_split<W>(keep, ctl.ex, it, rank, nranks, a.status);
        ring.advance(a.stages);
    };
    auto front = [&](Regs& r, int it) {
        float part[2];
        front_load(r, it, part);
        front_send(warp_sum_split(part[0], part[1]), it);
    };
    auto back_store = [&](const Regs& r, int it, const float (&sq)[2]) {
        const int row = cluster + it * a.num_clusters;
        float mean, var;
        moments_from_shifted(sq[0], sq[1], r.shift, a.cols, mean, var);
        const float rstd = rsqrtf(var + eps);
        if (rank == 0 && threadIdx.x == 0) {
            mean_out[row] = mean;
            rstd_out[row] = rstd;
        }
        const float2 neg_mean = splat(-mean), rstd2 = splat(rstd);
        // 16-bit rows: xhat = x * rstd - mean * rstd in one fused operation. The rounding of the
        // constant costs |mean| / std * 6e-8 on xhat, far below the output's own 2^-9; fp32 rows
        // keep the exact (x - mean) * rstd.
        const float2 shift2 = splat(-mean * rstd);
        uint4* out = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * a.cols + g.start);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            float2 xv[PAIRS];
            PairVec<T>::unpack(r.raw[i], xv);
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const float2 xhat = sizeof(T) == 2 ? __ffma2_rn(xv[j], rstd2, shift2)
                                                   : __fmul2_rn(__fadd2_rn(xv[j], neg_mean), rstd2);
                xv[j] = __ffma2_rn(xhat, gam[i][j], bet[i][j]);
            }
            if (FULL || v < nvec) __stcs(out + v, PairVec<T>::pack(xv));
        }
    };
    auto back = [&](const Regs& r, int it) {
        float sq[2];
        exchange_receive_split(ctl.ex, it, nranks, a.status, sq);
        back_store(r, it, sq);
    };
    // front(next) and back(current) with the two shuffle trees side by side
    auto fused = [&](Regs& rn, int itn, const Regs& ro, int ito) {
        float part[2], sq[2];
        front_load(rn, itn, part);
        const float keep = reduce_and_receive_split(part[0], part[1], ctl.ex, ito, nranks, a.status, sq);
        front_send(keep, itn);
        back_store(ro, ito, sq);
    };
    Regs r0, r1;
    pipeline_rows_fused(my_rows, r0, r1, front, fused, back);
}

// ---------------------------------------------------------------------------
// LayerNorm backward. With c = x - mean, xhat = c * rstd, g = dy * gamma,
// S1 = sum_row g and S2 = sum_row g * c:
//   dx = (g - mean_row(g) - xhat * mean_row(g * xhat)) * rstd
//      = g * rstd + c * (-rstd^3 * S2 / N) + (-rstd * S1 / N)
//   dgamma[col] = sum_rows dy * c * rstd,  dbeta[col] = sum_rows dy    (PARAM_GRADS)
// HAS_STATS: mean/rstd are inputs (one exchange per row); otherwise they are
// computed from the staged x first (two dependent exchanges per row, each covered
// by work on the neighbouring row), the form of the reference kernel
// (layernorm_backward.cu:401-437) and of dsmem_eval/workloads.py:53-61. x and dy
// are both staged, so dy crosses HBM once (the reference reads it twice, :418 and
// :434). Column sums live in registers and are written at the end to `partials`
// laid out [num_clusters][2][cols]; a finishing kernel adds the clusters in a
// fixed order (deterministic, no atomics).
// ---------------------------------------------------------------------------
template <typename T, int THREADS, int VPT, bool FULL, bool HAS_STATS, bool PARAM_GRADS>
__global__ void __launch_bounds__(THREADS, THREADS == 256 ? 2 : 1)
layernorm_bwd_reg_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                         const float* __restrict__ gamma, const float* __restrict__ mean_in,
                         const float* __restrict__ rstd_in, T* __restrict__ dx,
                         float* __restrict__ partials, float eps, StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<AsyncControl<2>*>(smem);
    unsigned char* data = smem + kControlBytes;
    constexpr int E = PairVec<T>::kElems;
    constexpr int PAIRS = PairVec<T>::kPairs;
    constexpr int W = THREADS / 32;
    // More than 16 row elements per thread do not fit next to gamma and the column sums: such
    // slices are not kept in registers across the exchange but read from the shared-memory stage
    // a second time (the stage is then held until the row's outputs are written). Twice the
    // elements per thread means half the cluster size for the same row: more co-resident
    // clusters, and the per-row overhead is spread over twice the work.
    constexpr bool REREAD = VPT * E > 16;
    constexpr int HELD = REREAD ? 1 : VPT;
    // with the column sums this kernel is the one shortest of issue slots: its waiting warps sleep
    // between polls (see mbar_wait_bounded)
    constexpr int SLEEP = (HAS_STATS && PARAM_GRADS) ? 150 : 0;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const int nvec = g.local / E;
    const T* const src[2] = {x, dy};
    const int my_rows = cluster < a.rows ? (a.rows - cluster + a.num_clusters - 1) / a.num_clusters : 0;
    if ((FULL ? nvec != VPT * THREADS : nvec > VPT * THREADS) && threadIdx.x == 0)
        atomicOr(a.status, kStatusBadGeometry);

    async_prologue<2, W>(ctl, a.stages);
    const RingFiller<T, 2, 2> filler{ctl, src, data, cluster, my_rows, a, g};
    const bool fills_ring = threadIdx.x == THREADS - 32;
    if (fills_ring) filler.prime();

    float2 gam[VPT][PAIRS];
    float2 dgam[PARAM_GRADS ? VPT : 1][PAIRS];
    float2 dbet[PARAM_GRADS ? VPT : 1][PAIRS];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
#pragma unroll
        for (int j = 0; j < PAIRS; ++j) gam[i][j] = splat(0.0f);
        if (FULL || v < nvec) load_param_pairs<PAIRS>(gamma + g.start + v * E, gam[i]);
        if (PARAM_GRADS) {
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                dgam[i][j] = splat(0.0f);
                dbet[i][j] = splat(0.0f);
            }
        }
    }

    RingCursor ring{0, 0u};
    const float inv_cols = 1.0f / static_cast<float>(a.cols);

    struct Regs {
        uint4 x[HELD];
        uint4 dy[HELD];
        float mean;    // HAS_STATS: given; else the shift first, the mean after `middle`
        float rstd;
        int stage;     // REREAD: the ring stage that holds the row
    };
    // vector i of this thread's part of the row: from registers, or again from the stage
    auto fetch = [&](const Regs& r, int i, uint4& xr, uint4& dr) {
        if (REREAD) {
            const int v = threadIdx.x + i * THREADS;
            const bool live = FULL || v < nvec;
            const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
            xr = live ? reinterpret_cast<const uint4*>(stage_tile<T, 2>(data, r.stage, 0, a.slice_elems))[v] : zero;
            dr = live ? reinterpret_cast<const uint4*>(stage_tile<T, 2>(data, r.stage, 1, a.slice_elems))[v] : zero;
        } else {
            xr = r.x[REREAD ? 0 : i];
            dr = r.dy[REREAD ? 0 : i];
        }
    };
    float next_shift = (!HAS_STATS && my_rows > 0) ? row_shift_sample(x, cluster, a.cols) : 0.0f;

    // warp-reduced S1 = sum g and S2 = sum g * (x - mean) over this warp's columns
    auto partials_of_g = [&](const Regs& r, float (&part)[2]) {
        const float2 neg_mean = splat(-r.mean);
        float2 s1 = splat(0.0f), s2 = splat(0.0f);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            float2 xv[PAIRS], dv[PAIRS];
            uint4 xr, dr;
            fetch(r, i, xr, dr);
            PairVec<T>::unpack(xr, xv);
            PairVec<T>::unpack(dr, dv);
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const float2 gg = __fmul2_rn(dv[j], gam[i][j]);   // 0 past the slice: dy = gamma = 0
                s1 = __fadd2_rn(s1, gg);
                // 16-bit rows: sum g * x here and take mean * sum g off once per row below (a mean
                // that dwarfs the spread cannot be stored in 16 bits in the first place)
                s2 = sizeof(T) == 2 ? __ffma2_rn(gg, xv[j], s2) : __ffma2_rn(gg, __fadd2_rn(xv[j], neg_mean), s2);
            }
        }
        const float t1 = s1.x + s1.y, t2 = s2.x + s2.y;
        part[0] = t1;
        part[1] = sizeof(T) == 2 ? fmaf(-r.mean, t1, t2) : t2;
    };
    auto sums_of_g = [&](const Regs& r) -> float {
        float part[2];
        partials_of_g(r, part);
        return warp_sum_split(part[0], part[1]);
    };
    // the row into registers (or located in its stage) and this thread's two partial sums of it
    auto front_load = [&](Regs& r, int it, float (&part)[2]) {
        const int row = cluster + it * a.num_clusters;
        if (fills_ring && it > 0) filler.recycle(it, REREAD ? 2 : 1);
        if (HAS_STATS) {
            r.mean = __ldg(mean_in + row);
            r.rstd = __ldg(rstd_in + row);
        } else {
            r.mean = next_shift;
            if (it + 1 < my_rows) next_shift = row_shift_sample(x, row + a.num_clusters, a.cols);
        }
        if (g.local > 0) mbar_wait_bounded<SLEEP>(smem_u32(&ctl.full[ring.stage]), ring.parity, a.status);
        r.stage = ring.stage;
        if (!REREAD) {
            load_raw<THREADS, HELD, FULL>(
                reinterpret_cast<const uint4*>(stage_tile<T, 2>(data, ring.stage, 0, a.slice_elems)), nvec, r.x);
            load_raw<THREADS, HELD, FULL>(
                reinterpret_cast<const uint4*>(stage_tile<T, 2>(data, ring.stage, 1, a.slice_elems)), nvec, r.dy);
        }
        if (HAS_STATS) {
            partials_of_g(r, part);
        } else if (REREAD) {
            uint4 raw[VPT];
            load_raw<THREADS, VPT, FULL>(
                reinterpret_cast<const uint4*>(stage_tile<T, 2>(data, ring.stage, 0, a.slice_elems)), nvec, raw);
            shifted_partials<T, THREADS, VPT, FULL>(raw, nvec, r.mean, part[0], part[1]);
        } else {
            shifted_partials<T, THREADS, HELD, FULL>(r.x, nvec, r.mean, part[0], part[1]);
        }
        // the stage is free once the row is in registers, or (REREAD) once its outputs are written
        if (!REREAD && g.local > 0 && (threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&ctl.empty[ring.stage]));
    };
    auto front_send = [&](float keep, int it) {   // keep: the two partials split over the halves of the warp
        exchange_send_split<W, SLEEP>(keep, ctl.ex, it, rank, nranks, a.status);
        ring.advance(a.stages);
    };
    auto front = [&](Regs& r, int it) {
        float part[2];
        front_load(r, it, part);
        front_send(warp_sum_split(part[0], part[1]), it);
    };
    // stats recomputed only: finish the statistics, start the exchange of S1, S2
    auto middle = [&](Regs& r, int it) {
        float sq[2];
        exchange_receive_split(ctl.ex, it, nranks, a.status, sq);
        float mean, var;
        moments_from_shifted(sq[0], sq[1], r.mean, a.cols, mean, var);
        r.mean = mean;
        r.rstd = rsqrtf(var + eps);
        exchange_send_split<W>(sums_of_g(r), ctl.ex2, it, rank, nranks, a.status);
    };
    auto back_store = [&](const Regs& r, int it, const float (&sums)[2]) {
        const int row = cluster + it * a.num_clusters;
        const float2 neg_mean = splat(-r.mean), rstd2 = splat(r.rstd);
        const float2 ca = splat(-r.rstd * r.rstd * r.rstd * (sums[1] * inv_cols));
        const float2 cb = splat(-r.rstd * (sums[0] * inv_cols));
        // 16-bit rows work on xhat = x * rstd - mean * rstd (one fused operation; the rounding of
        // the constant is far below the output's 2^-9): dx = xhat * ca_hat + g * rstd + cb and
        // dgamma += dy * xhat, one operation less per pair than the (x - mean) form fp32 rows keep.
        const float2 shift2 = splat(-r.mean * r.rstd);
        const float2 ca_hat = splat(-r.rstd * r.rstd * (sums[1] * inv_cols));
        uint4* out = reinterpret_cast<uint4*>(dx + static_cast<size_t>(row) * a.cols + g.start);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            float2 xv[PAIRS], dv[PAIRS], o[PAIRS];
            uint4 xr, dr;
            fetch(r, i, xr, dr);
            PairVec<T>::unpack(xr, xv);
            PairVec<T>::unpack(dr, dv);
#pragma unroll
            for (int j = 0; j < PAIRS; ++j) {
                const float2 gg = __fmul2_rn(dv[j], gam[i][j]);
                if (sizeof(T) == 2) {
                    const float2 xhat = __ffma2_rn(xv[j], rstd2, shift2);
                    o[j] = __ffma2_rn(xhat, ca_hat, __ffma2_rn(gg, rstd2, cb));
                    if (PARAM_GRADS) dgam[i][j] = __ffma2_rn(dv[j], xhat, dgam[i][j]);   // dy = 0 past the slice
                } else {
                    const float2 c = __fadd2_rn(xv[j], neg_mean);
                    o[j] = __ffma2_rn(c, ca, __ffma2_rn(gg, rstd2, cb));
                    if (PARAM_GRADS) dgam[i][j] = __ffma2_rn(__fmul2_rn(dv[j], c), rstd2, dgam[i][j]);
                }
                if (PARAM_GRADS) dbet[i][j] = __fadd2_rn(dbet[i][j], dv[j]);
            }
            if (FULL || v < nvec) __stcs(out + v, PairVec<T>::pack(o));
        }
        if (REREAD && g.local > 0) {
            __syncwarp();   // every lane has read its vectors of the stage
            if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&ctl.empty[r.stage]));
        }
    };
    auto back = [&](const Regs& r, int it) {
        float sums[2];
        exchange_receive_split<SLEEP>(HAS_STATS ? ctl.ex : ctl.ex2, it, nranks, a.status, sums);
        back_store(r, it, sums);
    };
    // front(next) and back(current) with the two shuffle trees side by side
    auto fused = [&](Regs& rn, int itn, const Regs& ro, int ito) {
        float part[2], sums[2];
        front_load(rn, itn, part);
        const float keep = reduce_and_receive_split<SLEEP>(part[0], part[1], HAS_STATS ? ctl.ex : ctl.ex2, ito, nranks,
                                                           a.status, sums);
        front_send(keep, itn);
        back_store(ro, ito, sums);
    };

    Regs r0, r1;
    r0.mean = r0.rstd = r1.mean = r1.rstd = 0.0f;
    if (HAS_STATS) pipeline_rows_fused(my_rows, r0, r1, front, fused, back);
    else pipeline_rows_middle_fused(my_rows, r0, r1, front, middle, fused, back);

    if (PARAM_GRADS) {
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
}

}  // namespace credit
