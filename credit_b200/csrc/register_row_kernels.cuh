// Register-resident wide-row kernels: the fast path of RMSNorm forward,
// LayerNorm forward and LayerNorm backward for 16-byte aligned rows whose
// per-CTA slice fits VPT 16-byte vectors per thread.
//
// Data flow per row and CTA:
//   HBM --bulk-async copy (TMA)--> shared-memory ring --one LDS.128 per vector-->
//   registers --> partial statistics --> DSMEM exchange --> outputs from
//   registers --128-bit stores--> HBM
// Thread t owns vectors t, t+THREADS, ... of the slice for every row its cluster
// handles, so gamma/beta (and the running dgamma/dbeta sums) for those columns
// stay in registers for the whole kernel, and a ring stage is free again as soon
// as its vectors are in registers: the refill for the row `stages` steps ahead
// is issued before the statistics are even exchanged.
//
// The exchange uses no cluster barrier and no fence. Every CTA owns two
// mbarriers (one per slot buffer); warp 0 pushes the CTA's partials into the
// slot of every CTA of the cluster with st.async, which signals the receiver's
// mbarrier by byte count; each CTA then waits on its own mbarrier only. (A
// barrier.cluster.arrive.release has to drain the thread's outstanding global
// stores first, which serialises the previous row's output with this row's
// statistics.) Slot buffers and mbarrier phases alternate between successive
// exchanges; a peer can only be two exchanges ahead after it has received this
// CTA's contribution to the exchange in between, which this CTA sends after it
// has read the older slots, so a buffer is never overwritten while it is read.
//
// Same arithmetic as the reference's cluster_bwd_staged_kernel family
// (src/workloads/layernorm_backward.cu:376-438), re-designed for sm_100a.
#pragma once

#include "cluster_primitives.cuh"
#include "norm_kernels.cuh"

namespace credit {

template <int K>
struct alignas(16) ExchangeScratch {
    uint64_t bar[2];                          // one mbarrier per slot buffer
    float warp_part[K][kMaxWarpsPerCta];
    float slot[2][K][kMaxClusterSize];        // [buffer][partial][source rank]
};

struct ExchangeCursor {
    uint32_t buf;
    uint32_t phase;
    __device__ __forceinline__ void advance() {
        buf ^= 1u;
        if (buf == 0u) phase ^= 1u;
    }
};

__device__ __forceinline__ void st_async_f32(uint32_t remote_addr, float v, uint32_t remote_bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];" ::"r"(
                     remote_addr),
                 "f"(v), "r"(remote_bar)
                 : "memory");
}

// Step 1 (all threads): warp sums into shared memory. Follow with __syncthreads().
template <int K>
__device__ __forceinline__ void exchange_local(float (&v)[K], ExchangeScratch<K>& s) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = warp_sum(v[k]);
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) s.warp_part[k][warp] = v[k];
    }
}

// Step 2 (warp 0, after the __syncthreads): CTA totals in every lane of warp 0.
template <int K, int THREADS>
__device__ __forceinline__ void exchange_fold(ExchangeScratch<K>& s, float (&total)[K]) {
    constexpr int kWarps = THREADS / 32;
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int k = 0; k < K; ++k) {
        const float t = lane < kWarps ? s.warp_part[k][lane] : 0.0f;
        total[k] = warp_sum(t);
    }
}

// Step 3 (warp 0): arm the local mbarrier for P*K floats and send this CTA's K
// values to slot[buf][k][rank] of every CTA of the cluster.
template <int K>
__device__ __forceinline__ void exchange_push(const float (&vals)[K], ExchangeScratch<K>& s,
                                              const ExchangeCursor& cur, uint32_t rank,
                                              uint32_t nranks) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t bar = smem_u32(&s.bar[cur.buf]);
    if (lane == 0) mbar_arrive_expect_tx(bar, nranks * K * static_cast<uint32_t>(sizeof(float)));
    if (lane < nranks) {
        const uint32_t remote_bar = map_to_rank(bar, lane);
#pragma unroll
        for (int k = 0; k < K; ++k)
            st_async_f32(map_to_rank(smem_u32(&s.slot[cur.buf][k][rank]), lane), vals[k], remote_bar);
    }
}

// Step 4 (all threads): wait until all P contributions have landed here.
template <int K>
__device__ __forceinline__ void exchange_wait(ExchangeScratch<K>& s, const ExchangeCursor& cur,
                                              int* status) {
    mbar_wait_bounded(smem_u32(&s.bar[cur.buf]), cur.phase, status);
}

// Control block of the register-path kernels.
template <int K>
struct alignas(16) RegControl {
    uint64_t full[kMaxStages];
    ExchangeScratch<K> ex;
};

template <typename T>
struct RawVec;
template <>
struct RawVec<float> {
    static constexpr int kElems = 4;
    __device__ __forceinline__ static void unpack(const uint4& r, float (&o)[4]) {
        o[0] = __uint_as_float(r.x); o[1] = __uint_as_float(r.y);
        o[2] = __uint_as_float(r.z); o[3] = __uint_as_float(r.w);
    }
    __device__ __forceinline__ static uint4 pack(const float (&v)[4]) {
        return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]),
                          __float_as_uint(v[3]));
    }
    __device__ __forceinline__ static float first(const void* tile) {
        return *reinterpret_cast<const float*>(tile);
    }
};
template <>
struct RawVec<__nv_bfloat16> {
    static constexpr int kElems = 8;
    __device__ __forceinline__ static void unpack(const uint4& r, float (&o)[8]) {
        RowVec<__nv_bfloat16>::unpack(r, o);
    }
    __device__ __forceinline__ static uint4 pack(const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    __device__ __forceinline__ static float first(const void* tile) {
        return __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(tile));
    }
};

template <int E>
__device__ __forceinline__ void load_params(const float* p, float (&out)[E]) {
#pragma unroll
    for (int j = 0; j < E; j += 4) ldg_f32x4(p + j, &out[j]);
}

// Barriers initialised, cluster running, ring primed.
template <typename T, int NIN, int K>
__device__ __forceinline__ void reg_prologue(RegControl<K>& ctl, const T* const (&src)[NIN],
                                             unsigned char* data, int cluster, const StagedArgs& a,
                                             const SliceGeom& g) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) mbar_init(smem_u32(&ctl.full[s]), 1);
        mbar_init(smem_u32(&ctl.ex.bar[0]), 1);
        mbar_init(smem_u32(&ctl.ex.bar[1]), 1);
        fence_mbar_init();
    }
    __syncthreads();
    cluster_sync_all();
    if (threadIdx.x == 0 && g.local > 0) {
        for (int s = 0; s < a.stages; ++s) {
            const long long row = static_cast<long long>(cluster) + 1ll * s * a.num_clusters;
            if (row < a.rows)
                issue_slice_fill<T, NIN>(src, data, ctl.full, s, static_cast<int>(row), a, g);
        }
    }
}

// Called by thread 0 once every thread has copied its vectors of `stage` to
// registers (i.e. after a __syncthreads).
template <typename T, int NIN, int K>
__device__ __forceinline__ void reg_refill(RegControl<K>& ctl, const T* const (&src)[NIN],
                                           unsigned char* data, int stage, int row,
                                           const StagedArgs& a, const SliceGeom& g) {
    if (g.local > 0) {
        const long long next = static_cast<long long>(row) + 1ll * a.stages * a.num_clusters;
        if (next < a.rows) {
            fence_proxy_async_smem();
            issue_slice_fill<T, NIN>(src, data, ctl.full, stage, static_cast<int>(next), a, g);
        }
    }
}

// ---------------------------------------------------------------------------
// RMSNorm forward
// ---------------------------------------------------------------------------
template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
rmsnorm_fwd_reg_kernel(const T* __restrict__ x, const float* __restrict__ gamma, T* __restrict__ y,
                       float eps, StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<RegControl<1>*>(smem);
    unsigned char* data = smem + kControlBytes;
    constexpr int E = RawVec<T>::kElems;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const int nvec = g.local / E;
    const T* const src[1] = {x};
    if (nvec > VPT * THREADS && threadIdx.x == 0) atomicOr(a.status, kStatusBadGeometry);

    reg_prologue<T, 1, 1>(ctl, src, data, cluster, a, g);

    float gam[VPT][E];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (v < nvec) load_params<E>(gamma + g.start + v * E, gam[i]);
    }

    RingCursor ring{0, 0u};
    ExchangeCursor exc{0u, 0u};
    const float inv_cols = 1.0f / static_cast<float>(a.cols);

    for (int row = cluster; row < a.rows; row += a.num_clusters) {
        if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[ring.stage]), ring.parity, a.status);
        const uint4* tile = reinterpret_cast<const uint4*>(stage_tile<T, 1>(data, ring.stage, 0, a.slice_elems));
        uint4 raw[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            raw[i] = v < nvec ? tile[v] : make_uint4(0u, 0u, 0u, 0u);
        }
        float part[1] = {0.0f};
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            float xv[E];
            RawVec<T>::unpack(raw[i], xv);
#pragma unroll
            for (int j = 0; j < E; ++j) part[0] = fmaf(xv[j], xv[j], part[0]);
        }
        exchange_local<1>(part, ctl.ex);
        __syncthreads();
        if (threadIdx.x == 0) reg_refill<T, 1, 1>(ctl, src, data, ring.stage, row, a, g);
        if (threadIdx.x < 32) {
            float total[1];
            exchange_fold<1, THREADS>(ctl.ex, total);
            exchange_push<1>(total, ctl.ex, exc, rank, nranks);
        }
        exchange_wait<1>(ctl.ex, exc, a.status);
        float sumsq = 0.0f;
        for (uint32_t r = 0; r < nranks; ++r) sumsq += ctl.ex.slot[exc.buf][0][r];
        exc.advance();
        const float scale = rsqrtf(sumsq * inv_cols + eps);

        T* out = y + static_cast<size_t>(row) * a.cols + g.start;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (v < nvec) {
                float xv[E];
                RawVec<T>::unpack(raw[i], xv);
#pragma unroll
                for (int j = 0; j < E; ++j) xv[j] = xv[j] * scale * gam[i][j];
                __stcs(reinterpret_cast<uint4*>(out) + v, RawVec<T>::pack(xv));
            }
        }
        ring.advance(a.stages);
    }
}

// Shifted one-pass statistics of the slice held in `raw`: with K = first element
// of the slice, accumulates sum(x-K) and sum((x-K)^2); K is within a few standard
// deviations of the mean, so the later subtraction loses about one digit instead
// of log10(mean^2/var). Outputs the per-thread partials.
template <typename T, int THREADS, int VPT>
__device__ __forceinline__ void shifted_partials(const uint4 (&raw)[VPT], int nvec, float shift,
                                                 float& s, float& q) {
    constexpr int E = RawVec<T>::kElems;
    s = 0.0f;
    q = 0.0f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (v < nvec) {
            float xv[E];
            RawVec<T>::unpack(raw[i], xv);
#pragma unroll
            for (int j = 0; j < E; ++j) {
                const float d = xv[j] - shift;
                s += d;
                q = fmaf(d, d, q);
            }
        }
    }
}

// Warp 0: CTA totals of (sum(x-K), sum((x-K)^2)) -> (slice mean, slice M2).
__device__ __forceinline__ void slice_moments(float (&tot)[2], float shift, int local) {
    const float n = static_cast<float>(local > 0 ? local : 1);
    const float ds = tot[0] / n;
    const float m2 = fmaxf(tot[1] - tot[0] * ds, 0.0f);
    tot[0] = shift + ds;   // slice mean
    tot[1] = m2;           // sum of squared deviations about it
}

// All threads: merge the P (mean_i, M2_i) pairs (parallel-variance formula).
__device__ __forceinline__ void merge_moments(const float (&slot)[2][kMaxClusterSize], int cols,
                                              int slice_elems, uint32_t nranks, float& mean,
                                              float& var) {
    float weighted = 0.0f;
    for (uint32_t r = 0; r < nranks; ++r) {
        const SliceGeom gr = slice_geometry(cols, slice_elems, r);
        weighted += slot[0][r] * static_cast<float>(gr.local);
    }
    mean = weighted / static_cast<float>(cols);
    float m2 = 0.0f;
    for (uint32_t r = 0; r < nranks; ++r) {
        const SliceGeom gr = slice_geometry(cols, slice_elems, r);
        const float d = slot[0][r] - mean;
        m2 += slot[1][r] + static_cast<float>(gr.local) * d * d;
    }
    var = m2 / static_cast<float>(cols);
}

// ---------------------------------------------------------------------------
// LayerNorm forward
// ---------------------------------------------------------------------------
template <typename T, int THREADS, int VPT>
__global__ void __launch_bounds__(THREADS)
layernorm_fwd_reg_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                         const float* __restrict__ beta, T* __restrict__ y,
                         float* __restrict__ mean_out, float* __restrict__ rstd_out, float eps,
                         StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<RegControl<2>*>(smem);
    unsigned char* data = smem + kControlBytes;
    constexpr int E = RawVec<T>::kElems;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const int nvec = g.local / E;
    const T* const src[1] = {x};
    if (nvec > VPT * THREADS && threadIdx.x == 0) atomicOr(a.status, kStatusBadGeometry);

    reg_prologue<T, 1, 2>(ctl, src, data, cluster, a, g);

    float gam[VPT][E], bet[VPT][E];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
        if (v < nvec) {
            load_params<E>(gamma + g.start + v * E, gam[i]);
            load_params<E>(beta + g.start + v * E, bet[i]);
        }
    }

    RingCursor ring{0, 0u};
    ExchangeCursor exc{0u, 0u};

    for (int row = cluster; row < a.rows; row += a.num_clusters) {
        if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[ring.stage]), ring.parity, a.status);
        const void* tile_base = stage_tile<T, 1>(data, ring.stage, 0, a.slice_elems);
        const uint4* tile = reinterpret_cast<const uint4*>(tile_base);
        const float shift = g.local > 0 ? RawVec<T>::first(tile_base) : 0.0f;
        uint4 raw[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            raw[i] = v < nvec ? tile[v] : make_uint4(0u, 0u, 0u, 0u);
        }
        float part[2];
        shifted_partials<T, THREADS, VPT>(raw, nvec, shift, part[0], part[1]);
        exchange_local<2>(part, ctl.ex);
        __syncthreads();
        if (threadIdx.x == 0) reg_refill<T, 1, 2>(ctl, src, data, ring.stage, row, a, g);
        if (threadIdx.x < 32) {
            float total[2];
            exchange_fold<2, THREADS>(ctl.ex, total);
            slice_moments(total, shift, g.local);
            exchange_push<2>(total, ctl.ex, exc, rank, nranks);
        }
        exchange_wait<2>(ctl.ex, exc, a.status);
        float mean, var;
        merge_moments(ctl.ex.slot[exc.buf], a.cols, a.slice_elems, nranks, mean, var);
        exc.advance();
        const float rstd = rsqrtf(var + eps);
        if (rank == 0 && threadIdx.x == 0) {
            mean_out[row] = mean;
            rstd_out[row] = rstd;
        }
        const float offset = -mean * rstd;

        T* out = y + static_cast<size_t>(row) * a.cols + g.start;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (v < nvec) {
                float xv[E];
                RawVec<T>::unpack(raw[i], xv);
#pragma unroll
                for (int j = 0; j < E; ++j)
                    xv[j] = fmaf(fmaf(xv[j], rstd, offset), gam[i][j], bet[i][j]);
                __stcs(reinterpret_cast<uint4*>(out) + v, RawVec<T>::pack(xv));
            }
        }
        ring.advance(a.stages);
    }
}

// ---------------------------------------------------------------------------
// LayerNorm backward
//   xhat = (x - mean) * rstd,  g = dy * gamma
//   dx   = (g - mean_row(g) - xhat * mean_row(g * xhat)) * rstd
//        = fma(xhat, -rstd * mean_row(g xhat), fma(g, rstd, -rstd * mean_row(g)))
//   dgamma[c] = sum_rows dy * xhat,  dbeta[c] = sum_rows dy           (PARAM_GRADS)
// HAS_STATS: mean/rstd are inputs (one exchange per row); otherwise they are
// computed from the staged x first (two exchanges), the form of the reference
// kernel (layernorm_backward.cu:401-437) and of dsmem_eval/workloads.py:53-61.
// x and dy are both staged, so dy crosses HBM once (the reference reads it twice,
// :418 and :434). Column sums live in registers and are written at the end to
// `partials` laid out [num_clusters][2][cols]; a finishing kernel adds the
// clusters in a fixed order (deterministic, no atomics).
// ---------------------------------------------------------------------------
template <typename T, int THREADS, int VPT, bool HAS_STATS, bool PARAM_GRADS>
__global__ void __launch_bounds__(THREADS)
layernorm_bwd_reg_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                         const float* __restrict__ gamma, const float* __restrict__ mean_in,
                         const float* __restrict__ rstd_in, T* __restrict__ dx,
                         float* __restrict__ partials, float eps, StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<RegControl<2>*>(smem);
    unsigned char* data = smem + kControlBytes;
    constexpr int E = RawVec<T>::kElems;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const int nvec = g.local / E;
    const T* const src[2] = {x, dy};
    if (nvec > VPT * THREADS && threadIdx.x == 0) atomicOr(a.status, kStatusBadGeometry);

    reg_prologue<T, 2, 2>(ctl, src, data, cluster, a, g);

    float gam[VPT][E];
    float dgam[PARAM_GRADS ? VPT : 1][E];
    float dbet[PARAM_GRADS ? VPT : 1][E];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * THREADS;
#pragma unroll
        for (int j = 0; j < E; ++j) gam[i][j] = 0.0f;
        if (v < nvec) load_params<E>(gamma + g.start + v * E, gam[i]);
        if (PARAM_GRADS) {
#pragma unroll
            for (int j = 0; j < E; ++j) {
                dgam[i][j] = 0.0f;
                dbet[i][j] = 0.0f;
            }
        }
    }

    RingCursor ring{0, 0u};
    ExchangeCursor exc{0u, 0u};
    const float inv_cols = 1.0f / static_cast<float>(a.cols);

    for (int row = cluster; row < a.rows; row += a.num_clusters) {
        float mean = 0.0f, rstd = 0.0f;
        if (HAS_STATS) {
            mean = __ldg(mean_in + row);
            rstd = __ldg(rstd_in + row);
        }
        if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[ring.stage]), ring.parity, a.status);
        const void* x_base = stage_tile<T, 2>(data, ring.stage, 0, a.slice_elems);
        const uint4* xt = reinterpret_cast<const uint4*>(x_base);
        const uint4* dyt = reinterpret_cast<const uint4*>(stage_tile<T, 2>(data, ring.stage, 1, a.slice_elems));
        uint4 xraw[VPT], dyraw[VPT];
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            xraw[i] = v < nvec ? xt[v] : make_uint4(0u, 0u, 0u, 0u);
            dyraw[i] = v < nvec ? dyt[v] : make_uint4(0u, 0u, 0u, 0u);
        }
        bool stage_released = false;
        if (!HAS_STATS) {
            const float shift = g.local > 0 ? RawVec<T>::first(x_base) : 0.0f;
            float sp[2];
            shifted_partials<T, THREADS, VPT>(xraw, nvec, shift, sp[0], sp[1]);
            exchange_local<2>(sp, ctl.ex);
            __syncthreads();
            if (threadIdx.x == 0) reg_refill<T, 2, 2>(ctl, src, data, ring.stage, row, a, g);
            stage_released = true;
            if (threadIdx.x < 32) {
                float total[2];
                exchange_fold<2, THREADS>(ctl.ex, total);
                slice_moments(total, shift, g.local);
                exchange_push<2>(total, ctl.ex, exc, rank, nranks);
            }
            exchange_wait<2>(ctl.ex, exc, a.status);
            float var;
            merge_moments(ctl.ex.slot[exc.buf], a.cols, a.slice_elems, nranks, mean, var);
            exc.advance();
            rstd = rsqrtf(var + eps);
        }
        const float offset = -mean * rstd;

        // xhat and g for this thread's columns stay in registers for the dx pass
        float xh[VPT][E], gg[VPT][E];
        float part[2] = {0.0f, 0.0f};
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            float xv[E], dv[E];
            RawVec<T>::unpack(xraw[i], xv);
            RawVec<T>::unpack(dyraw[i], dv);
#pragma unroll
            for (int j = 0; j < E; ++j) {
                xh[i][j] = fmaf(xv[j], rstd, offset);
                gg[i][j] = dv[j] * gam[i][j];     // 0 for vectors past the slice (dy = gamma = 0)
                part[0] += gg[i][j];
                part[1] = fmaf(gg[i][j], xh[i][j], part[1]);
                if (PARAM_GRADS) {
                    dgam[i][j] = fmaf(dv[j], xh[i][j], dgam[i][j]);
                    dbet[i][j] += dv[j];
                }
            }
        }
        exchange_local<2>(part, ctl.ex);
        __syncthreads();
        if (!stage_released && threadIdx.x == 0)
            reg_refill<T, 2, 2>(ctl, src, data, ring.stage, row, a, g);
        if (threadIdx.x < 32) {
            float total[2];
            exchange_fold<2, THREADS>(ctl.ex, total);
            exchange_push<2>(total, ctl.ex, exc, rank, nranks);
        }
        exchange_wait<2>(ctl.ex, exc, a.status);
        float sum_g = 0.0f, sum_gx = 0.0f;
        for (uint32_t r = 0; r < nranks; ++r) {
            sum_g += ctl.ex.slot[exc.buf][0][r];
            sum_gx += ctl.ex.slot[exc.buf][1][r];
        }
        exc.advance();
        const float c1 = -rstd * (sum_g * inv_cols);
        const float c2 = -rstd * (sum_gx * inv_cols);

        T* out = dx + static_cast<size_t>(row) * a.cols + g.start;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (v < nvec) {
                float o[E];
#pragma unroll
                for (int j = 0; j < E; ++j) o[j] = fmaf(xh[i][j], c2, fmaf(gg[i][j], rstd, c1));
                __stcs(reinterpret_cast<uint4*>(out) + v, RawVec<T>::pack(o));
            }
        }
        ring.advance(a.stages);
    }

    if (PARAM_GRADS) {
        float* out_g = partials + (static_cast<size_t>(cluster) * 2 + 0) * a.cols + g.start;
        float* out_b = partials + (static_cast<size_t>(cluster) * 2 + 1) * a.cols + g.start;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * THREADS;
            if (v < nvec) {
#pragma unroll
                for (int j = 0; j < E; j += 4) {
                    *reinterpret_cast<float4*>(out_g + v * E + j) =
                        make_float4(dgam[i][j], dgam[i][j + 1], dgam[i][j + 2], dgam[i][j + 3]);
                    *reinterpret_cast<float4*>(out_b + v * E + j) =
                        make_float4(dbet[i][j], dbet[i][j + 1], dbet[i][j + 2], dbet[i][j + 3]);
                }
            }
        }
    }
}

}  // namespace credit
