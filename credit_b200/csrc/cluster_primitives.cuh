// Device-side building blocks shared by every wide-row kernel: PTX wrappers for
// thread-block clusters (rank, mapa, st.shared::cluster, split arrive/wait
// barrier), mbarrier + bulk-async (TMA) global->shared copies with bounded
// waits, 128-bit vector access for fp32 and bf16 rows, and the two-level
// (warp shuffle -> CTA -> cluster DSMEM push) all-reduce that replaces the
// reference's block_reduce_* / cluster_reduce_* helper pairs
// (src/workloads/layernorm_backward.cu:177-251, rowwise_quant.cu:174-237).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "launch_args.h"

namespace credit {

// ---------------------------------------------------------------------------
// addressing
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ uint32_t cluster_cta_count() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}

// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(remote)
                 : "r"(local_smem_addr), "r"(rank));
    return remote;
}

__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ void st_cluster_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ void st_cluster_u64(uint32_t addr, uint64_t v) {
    asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}

__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

// ---------------------------------------------------------------------------
// cluster barrier, split so work can sit between arrive and wait
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cluster_arrive_release() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_wait_acquire() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_sync_all() {
    cluster_arrive_release();
    cluster_wait_acquire();
}

// ---------------------------------------------------------------------------
// mbarrier + bulk async copies
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders earlier generic-proxy accesses to shared memory before later
// async-proxy (bulk copy) accesses issued by this thread.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

// One arrival on a barrier of this CTA (release semantics).
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Remote store of one float into a peer CTA's shared memory; the peer's mbarrier
// `remote_bar` is credited with the 4 bytes when they have landed, so data and
// notification travel as one message (no cluster barrier, no fence).
__device__ __forceinline__ void st_async_f32(uint32_t remote_addr, float v, uint32_t remote_bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];" ::"r"(
                     remote_addr),
                 "f"(v), "r"(remote_bar)
                 : "memory");
}

// Two floats (8-byte aligned destination) in one message.
__device__ __forceinline__ void st_async_f32x2(uint32_t remote_addr, float v0, float v1, uint32_t remote_bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];" ::"r"(
                     remote_addr),
                 "f"(v0), "f"(v1), "r"(remote_bar)
                 : "memory");
}

// Four floats (16-byte aligned destination) in one message.
__device__ __forceinline__ void st_async_f32x4(uint32_t remote_addr, float v0, float v1, float v2, float v3,
                                               uint32_t remote_bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(
                     remote_addr),
                 "f"(v0), "f"(v1), "f"(v2), "f"(v3), "r"(remote_bar)
                 : "memory");
}

// One poll, never suspends: true when the phase with this parity has completed. The suspending
// form (mbarrier.try_wait) wakes a warp late when the phase completes shortly after the first
// look, which is the usual case on the row path: measured on one GPU, polling is 0.8 % (LayerNorm
// backward with column sums) to 3 % (LayerNorm forward) faster, and 0.4 % on the FFN.
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait: gives up after ~2^31 SM cycles (about a second) or 2^24 polls,
// records the failure in *status and returns false; the caller keeps going so
// that every CTA of the cluster still reaches the same barriers and the launch
// ends instead of hanging.
// SLEEP_NS > 0: the warp sleeps that long between unsuccessful polls. Polls take issue slots from
// the warps that have work; a kernel short of issue slots gains more from the sleep than it loses
// by waking late (LayerNorm backward with column sums: 760 -> 743 us with 150 ns), the others
// lose, so it is a per-kernel choice. A tighter poll loop than this one (no clock read) is
// slower everywhere.
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status) {
    if (mbar_poll(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t i = 0; i < (1u << 24); ++i) {
        if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
        if (mbar_poll(bar, parity)) return true;
        if (clock64() - t0 > (1ll << 31)) break;
    }
    if (status != nullptr) atomicOr(status, kStatusWaitTimeout);
    return false;
}

// Suspending wait for warps that have nothing else to do (the producer and collector warps of the
// warp-specialised kernels): mbarrier.try_wait parks the warp in hardware until the phase completes
// or a time limit passes, so the waiting warp issues a handful of instructions per wake-up instead
// of competing for issue slots with the warps that have work. Bounded like mbar_wait_bounded.
__device__ __forceinline__ bool mbar_wait_parked_bounded(uint32_t bar, uint32_t parity, int* status) {
    const long long t0 = clock64();
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t"
            "}"
            : "=r"(done)
            : "r"(bar), "r"(parity), "r"(100000u)   // suspend-time hint in ns
            : "memory");
        if (done != 0) return true;
        if (clock64() - t0 > (1ll << 31)) break;
    }
    if (status != nullptr) atomicOr(status, kStatusWaitTimeout);
    return false;
}

// One bulk copy global -> this CTA's shared memory, completion counted in bytes
// on `bar`. src, dst and bytes must all be multiples of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src_gmem, uint32_t bytes,
                                          uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(dst_smem),
        "l"(src_gmem), "r"(bytes), "r"(bar)
        : "memory");
}

// Splits a long contiguous copy into pieces so several copy engines can work on
// one slice; all pieces complete on the same barrier.
__device__ __forceinline__ void bulk_load_chunked(uint32_t dst_smem, const void* src_gmem,
                                                  uint32_t bytes, uint32_t bar) {
    constexpr uint32_t kPiece = 8192;
    const char* src = static_cast<const char*>(src_gmem);
    while (bytes > 0) {
        const uint32_t n = bytes < kPiece ? bytes : kPiece;
        bulk_load(dst_smem, src, n, bar);
        dst_smem += n;
        src += n;
        bytes -= n;
    }
}

// Position in a ring of shared-memory stages and the mbarrier phase parity that
// goes with it.
struct RingCursor {
    int stage;
    uint32_t parity;
    __device__ __forceinline__ void advance(int stages) {
        if (++stage == stages) {
            stage = 0;
            parity ^= 1u;
        }
    }
};

// ---------------------------------------------------------------------------
// 16-byte vectors of row elements
// ---------------------------------------------------------------------------
template <typename T>
struct RowVec;

template <>
struct RowVec<float> {
    static constexpr int kElems = 4;
    __device__ __forceinline__ static void from_smem(const void* base, int vec, float (&out)[4]) {
        const float4 v = reinterpret_cast<const float4*>(base)[vec];
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
    __device__ __forceinline__ static void from_global(const float* p, float (&out)[4]) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p));
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
    __device__ __forceinline__ static void to_global(float* p, const float (&in)[4]) {
        __stcs(reinterpret_cast<float4*>(p), make_float4(in[0], in[1], in[2], in[3]));
    }
    __device__ __forceinline__ static float to_float(float v) { return v; }
    __device__ __forceinline__ static float from_float(float v) { return v; }
};

template <>
struct RowVec<__nv_bfloat16> {
    static constexpr int kElems = 8;
    __device__ __forceinline__ static void unpack(const uint4& v, float (&out)[8]) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ static void from_smem(const void* base, int vec, float (&out)[8]) {
        unpack(reinterpret_cast<const uint4*>(base)[vec], out);
    }
    __device__ __forceinline__ static void from_global(const __nv_bfloat16* p, float (&out)[8]) {
        unpack(__ldg(reinterpret_cast<const uint4*>(p)), out);
    }
    __device__ __forceinline__ static void to_global(__nv_bfloat16* p, const float (&in)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        __stcs(reinterpret_cast<uint4*>(p), make_uint4(w[0], w[1], w[2], w[3]));
    }
    __device__ __forceinline__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ __forceinline__ static __nv_bfloat16 from_float(float v) {
        return __float2bfloat16_rn(v);
    }
};

// Four consecutive fp32 parameters (gamma, beta) through the read-only path.
__device__ __forceinline__ void ldg_f32x4(const float* p, float* out) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(p));
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}

// ---------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

// Scratch used by the reductions; lives in the control block of shared memory.
template <int K>
struct ReduceScratch {
    float warp_part[K][kMaxWarpsPerCta];
    float slot[2][K][kMaxClusterSize];   // double-buffered: [parity][partial][source rank]
};

// Sum of K per-thread partials over the CTA only. Every thread returns the same
// totals. Two __syncthreads.
template <int K, int THREADS>
__device__ __forceinline__ void cta_allreduce_sum(float (&v)[K], ReduceScratch<K>& s) {
    constexpr int kWarps = THREADS / 32;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = warp_sum(v[k]);
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) s.warp_part[k][warp] = v[k];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < K; ++k) {
        float t = lane < kWarps ? s.warp_part[k][lane] : 0.0f;
        v[k] = warp_sum(t);
    }
    __syncthreads();
}

// Sum of K per-thread partials over all threads of all CTAs of the cluster.
// Warp shuffles -> one value per warp in shared memory -> warp 0 folds them and
// pushes the CTA total into slot[parity][k][my rank] of every CTA of the cluster
// (st.shared::cluster) -> ONE cluster barrier (arrive.release / wait.acquire) ->
// every thread adds the P slots in rank order, so all CTAs get bit-identical
// totals. `parity` must alternate between successive calls: the slots a peer is
// still reading belong to the other parity, which is what makes the second
// barrier of the reference's cluster_reduce_* unnecessary.
template <int K, int THREADS>
__device__ __forceinline__ void cluster_allreduce_sum(float (&v)[K], ReduceScratch<K>& s,
                                                      uint32_t parity, uint32_t rank,
                                                      uint32_t nranks) {
    constexpr int kWarps = THREADS / 32;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = warp_sum(v[k]);
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) s.warp_part[k][warp] = v[k];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) {
            float t = lane < kWarps ? s.warp_part[k][lane] : 0.0f;
            t = warp_sum(t);
            if (static_cast<uint32_t>(lane) < nranks) {
                const uint32_t mine = smem_u32(&s.slot[parity][k][rank]);
                st_cluster_f32(map_to_rank(mine, static_cast<uint32_t>(lane)), t);
            }
        }
    }
    cluster_arrive_release();
    cluster_wait_acquire();
#pragma unroll
    for (int k = 0; k < K; ++k) {
        float t = 0.0f;
        for (uint32_t r = 0; r < nranks; ++r) t += s.slot[parity][k][r];
        v[k] = t;
    }
}

// ---------------------------------------------------------------------------
// slice geometry: CTA `rank` of a cluster owns columns [rank*slice, rank*slice+local)
// ---------------------------------------------------------------------------
struct SliceGeom {
    int start;   // first column of this CTA's slice
    int local;   // columns in this CTA's slice (0 when the row is narrower than the cluster)
};

__device__ __forceinline__ SliceGeom slice_geometry(int cols, int slice_elems, uint32_t rank) {
    SliceGeom g;
    g.start = static_cast<int>(rank) * slice_elems;
    int local = cols - g.start;
    if (local > slice_elems) local = slice_elems;
    if (local < 0) local = 0;
    g.local = local;
    return g;
}

}  // namespace credit
