// Device micro-benchmarks behind the cluster-size cost model, for sm_100a.
//
// Prints the labelled lines that the reference's primitive_benchmark prints
// (src/primitive_benchmark.cu:628-976; parsed by dsmem_eval/profile.py:27-103) and,
// after them, B200 extensions: every DSMEM figure per cluster size 2..16, the
// shared::cluster store / mbarrier exchange this library uses next to the
// barrier.cluster exchange of the reference, and bulk-async (TMA) load latency.
//
// Every wait on another CTA is bounded: a spin that runs out records a timeout in
// the result block and the kernel still reaches all its barriers.
//
//   primitive_benchmark [--quick]

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "cluster_primitives.cuh"

using namespace credit;

#define CHECK(expr)                                                                     \
    do {                                                                                \
        cudaError_t e__ = (expr);                                                       \
        if (e__ != cudaSuccess) {                                                       \
            std::fprintf(stderr, "error: %s -> %s\n", #expr, cudaGetErrorString(e__));  \
            return 1;                                                                   \
        }                                                                               \
    } while (0)

namespace {

constexpr int kTrials = 9;
constexpr int kThreads = 256;

// ------------------------------------------------------------------ global memory
template <bool L1>
__global__ void chase_kernel(const int* __restrict__ data, int iterations, long long* cycles,
                             int* sink) {
    int idx = 0;
    // warm the line set
    for (int i = 0; i < 1024; ++i) {
        if (L1) asm volatile("ld.global.ca.s32 %0, [%1];" : "=r"(idx) : "l"(data + idx) : "memory");
        else asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(idx) : "l"(data + idx) : "memory");
    }
    const long long t0 = clock64();
    for (int i = 0; i < iterations; ++i) {
        if (L1) asm volatile("ld.global.ca.s32 %0, [%1];" : "=r"(idx) : "l"(data + idx) : "memory");
        else asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(idx) : "l"(data + idx) : "memory");
    }
    const long long t1 = clock64();
    *cycles = t1 - t0;
    *sink = idx;
}

template <bool L1>
__global__ void scan_kernel(const int4* __restrict__ data, size_t vecs, int repeats, int* sink) {
    int acc = 0;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (int r = 0; r < repeats; ++r) {
        for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += stride) {
            int4 v;
            if (L1)
                asm volatile("ld.global.ca.v4.s32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(data + i) : "memory");
            else
                asm volatile("ld.global.cg.v4.s32 {%0,%1,%2,%3}, [%4];"
                             : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(data + i) : "memory");
            acc += v.x ^ v.y ^ v.z ^ v.w;
        }
    }
    if (acc == 0x7fffffff) *sink = acc;
}

__global__ void copy_kernel(const int4* __restrict__ src, int4* __restrict__ dst, size_t vecs) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += stride)
        dst[i] = src[i];
}

// ------------------------------------------------------------------ cluster / DSMEM
struct ClusterResults {
    long long sync_cycles[kTrials];            // barrier.cluster arrive.release + wait.acquire
    long long barrier_exchange_cycles[kTrials]; // st.shared::cluster all-to-all + barrier.cluster
    long long async_exchange_cycles[kTrials];   // st.async all-to-all + own mbarrier wait
    long long local_latency_cycles[kTrials];
    long long remote_latency_cycles[kTrials];
    long long local_read_cycles[kTrials];
    long long remote_read_cycles[kTrials];
    long long local_store_cycles[kTrials];
    long long remote_store_cycles[kTrials];
    long long roundtrip_cycles[kTrials];
    unsigned smid[kMaxClusterSize];
    int timeouts;
};

constexpr int kSyncIters = 1000;
constexpr int kExchangeIters = 1000;
constexpr int kLatencyIters = 4096;
constexpr int kThroughputIters = 2048;
constexpr int kRoundtripIters = 500;
constexpr int kChaseWords = 4096;   // 16 KiB payload, as the reference uses

__device__ __forceinline__ unsigned smid() {
    unsigned id;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(id));
    return id;
}

__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t ld_cluster_volatile_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.volatile.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void st_async_u32(uint32_t remote_addr, uint32_t v, uint32_t remote_bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.u32 [%0], %1, [%2];" ::"r"(
                     remote_addr), "r"(v), "r"(remote_bar) : "memory");
}

// One cluster of P CTAs (P from the launch attribute); dynamic shared memory is
// sized by the host so that every CTA sits on its own SM.
__global__ void __launch_bounds__(kThreads) cluster_bench_kernel(ClusterResults* out, int* sink) {
    extern __shared__ __align__(16) unsigned char dyn[];
    uint32_t* chase = reinterpret_cast<uint32_t*>(dyn);                    // kChaseWords
    uint32_t* slots = chase + kChaseWords;                                 // 2 x 16
    uint64_t* bars = reinterpret_cast<uint64_t*>(slots + 2 * kMaxClusterSize);  // 2 mbarriers
    volatile uint32_t* flag = reinterpret_cast<volatile uint32_t*>(bars + 2);   // ping-pong cells

    const uint32_t rank = cluster_cta_rank();
    const uint32_t P = cluster_cta_count();
    const uint32_t peer = (rank + 1) % P;
    const int tid = threadIdx.x;

    for (int i = tid; i < kChaseWords; i += kThreads) chase[i] = (i + 257) % kChaseWords;
    if (tid == 0) {
        mbar_init(smem_u32(&bars[0]), 1);
        mbar_init(smem_u32(&bars[1]), 1);
        fence_mbar_init();
        flag[0] = 0;
        flag[1] = 0;
        out->smid[rank] = smid();
    }
    __syncthreads();
    cluster_sync_all();

    int acc = 0;
    for (int trial = 0; trial < kTrials; ++trial) {
        // 1. cluster barrier
        long long t0 = clock64();
        for (int i = 0; i < kSyncIters; ++i) cluster_sync_all();
        long long t1 = clock64();
        if (rank == 0 && tid == 0) out->sync_cycles[trial] = t1 - t0;

        // 2. all-to-all exchange through shared::cluster stores + one cluster barrier
        t0 = clock64();
        for (int i = 0; i < kExchangeIters; ++i) {
            const int buf = i & 1;
            if (tid < static_cast<int>(P))
                st_cluster_u32(map_to_rank(smem_u32(&slots[buf * kMaxClusterSize + rank]), tid), i + rank);
            cluster_sync_all();
            if (tid < static_cast<int>(P)) acc += slots[buf * kMaxClusterSize + tid];
        }
        t1 = clock64();
        if (rank == 0 && tid == 0) out->barrier_exchange_cycles[trial] = t1 - t0;
        cluster_sync_all();

        // 3. all-to-all exchange through st.async + the receiver's mbarrier (warp 0 only)
        t0 = clock64();
        if (tid < 32) {
            for (int i = 0; i < kExchangeIters; ++i) {
                const int buf = i & 1;
                const uint32_t bar = smem_u32(&bars[buf]);
                if (tid == 0) mbar_arrive_expect_tx(bar, P * 4u);
                if (tid < static_cast<int>(P))
                    st_async_u32(map_to_rank(smem_u32(&slots[buf * kMaxClusterSize + rank]), tid), i + rank,
                                 map_to_rank(bar, tid));
                const uint32_t phase = (static_cast<uint32_t>(trial * kExchangeIters + i) >> 1) & 1u;
                if (!mbar_wait_bounded(bar, phase, &out->timeouts)) break;
                if (tid < static_cast<int>(P)) acc += slots[buf * kMaxClusterSize + tid];
            }
        }
        t1 = clock64();
        if (rank == 0 && tid == 0) out->async_exchange_cycles[trial] = t1 - t0;
        __syncthreads();
        cluster_sync_all();

        // 4. dependent-load latency: own shared memory vs the next CTA's
        if (tid == 0) {
            uint32_t idx = 0;
            const uint32_t local_base = smem_u32(chase);
            t0 = clock64();
            for (int i = 0; i < kLatencyIters; ++i) idx = ld_cluster_u32(local_base + idx * 4u);
            t1 = clock64();
            acc += idx;
            if (rank == 0) out->local_latency_cycles[trial] = t1 - t0;
            const uint32_t remote_base = map_to_rank(local_base, peer);
            idx = 0;
            t0 = clock64();
            for (int i = 0; i < kLatencyIters; ++i) idx = ld_cluster_u32(remote_base + idx * 4u);
            t1 = clock64();
            acc += idx;
            if (rank == 0) out->remote_latency_cycles[trial] = t1 - t0;
        }
        cluster_sync_all();

        // 5. throughput of 4-byte reads and stores, local and remote, all threads
        {
            const uint32_t local_addr = smem_u32(chase) + (tid % kChaseWords) * 4u;
            const uint32_t remote_addr = map_to_rank(local_addr, peer);
            __syncthreads();
            t0 = clock64();
#pragma unroll 8
            for (int i = 0; i < kThroughputIters; ++i) acc += ld_cluster_u32(local_addr + ((i & 7) << 10));
            __syncthreads();
            t1 = clock64();
            if (rank == 0 && tid == 0) out->local_read_cycles[trial] = t1 - t0;
            t0 = clock64();
#pragma unroll 8
            for (int i = 0; i < kThroughputIters; ++i) acc += ld_cluster_u32(remote_addr + ((i & 7) << 10));
            __syncthreads();
            t1 = clock64();
            if (rank == 0 && tid == 0) out->remote_read_cycles[trial] = t1 - t0;
            cluster_sync_all();
            t0 = clock64();
#pragma unroll 8
            for (int i = 0; i < kThroughputIters; ++i) st_cluster_u32(local_addr + ((i & 7) << 10), i);
            __syncthreads();
            t1 = clock64();
            if (rank == 0 && tid == 0) out->local_store_cycles[trial] = t1 - t0;
            t0 = clock64();
#pragma unroll 8
            for (int i = 0; i < kThroughputIters; ++i) st_cluster_u32(remote_addr + ((i & 7) << 10), i);
            __syncthreads();
            t1 = clock64();
            if (rank == 0 && tid == 0) out->remote_store_cycles[trial] = t1 - t0;
            cluster_sync_all();
            for (int i = tid; i < kChaseWords; i += kThreads) chase[i] = (i + 257) % kChaseWords;
            __syncthreads();
            cluster_sync_all();
        }

        // 6. store -> visibility round trip between rank 0 and rank 1 (bounded spins)
        if (tid == 0 && rank < 2 && P >= 2) {
            const uint32_t other = 1 - rank;
            const uint32_t my_req = smem_u32(const_cast<uint32_t*>(&flag[0]));
            const uint32_t my_ack = smem_u32(const_cast<uint32_t*>(&flag[1]));
            const uint32_t their_req = map_to_rank(my_req, other);
            const uint32_t their_ack = map_to_rank(my_ack, other);
            bool ok = true;
            t0 = clock64();
            for (int i = 0; i < kRoundtripIters && ok; ++i) {
                const uint32_t token = trial * kRoundtripIters + i + 1;
                if (rank == 0) {
                    st_cluster_u32(their_req, token);
                    uint32_t spins = 0;
                    while (ld_cluster_volatile_u32(my_ack) != token)
                        if (++spins > (1u << 22)) { ok = false; break; }
                } else {
                    uint32_t spins = 0;
                    while (ld_cluster_volatile_u32(my_req) != token)
                        if (++spins > (1u << 22)) { ok = false; break; }
                    st_cluster_u32(their_ack, token);
                }
            }
            t1 = clock64();
            if (!ok) atomicOr(&out->timeouts, 2);
            if (rank == 0) out->roundtrip_cycles[trial] = t1 - t0;
        }
        cluster_sync_all();
    }
    if (acc == 0x7fffffff) *sink = acc;
    cluster_sync_all();
}

// Bulk-async load latency: one thread requests `bytes` from a cold global address
// and waits on the mbarrier; repeated over distinct addresses.
__global__ void tma_latency_kernel(const unsigned char* __restrict__ src, size_t stride, int bytes,
                                   int repeats, long long* cycles, int* status) {
    extern __shared__ __align__(128) unsigned char dyn[];
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        fence_mbar_init();
        long long total = 0;
        for (int r = 0; r < repeats; ++r) {
            const long long t0 = clock64();
            mbar_arrive_expect_tx(smem_u32(&bar), bytes);
            bulk_load(smem_u32(dyn), src + static_cast<size_t>(r) * stride, bytes, smem_u32(&bar));
            mbar_wait_bounded(smem_u32(&bar), r & 1, status);
            total += clock64() - t0;
        }
        *cycles = total;
    }
}

// DSMEM bulk copy: the CTAs of the cluster work in pairs (ranks 2i, 2i + 1); each copies `bytes` from
// its own shared memory into its partner's with cp.async.bulk (shared::cta -> shared::cluster),
// completion counted in bytes on the RECEIVER's mbarrier, and a step ends when the partner's copy
// has landed here. A CTA can be at most one step ahead of its partner (its next step needs the
// partner's copy of this one), and two buffers and two barriers alternate, so a copy never meets a
// barrier phase that is still in use.
// cycles[0]: one copy in flight per step (latency of arm + copy + wait); cycles[1]: kBulkDepth
// copies of `bytes` in flight per step (throughput).
constexpr int kBulkIters = 256;
constexpr int kBulkDepth = 4;
constexpr int kBulkMaxBytes = 16384;

__device__ __forceinline__ void bulk_copy_to_peer(uint32_t remote_dst, uint32_t local_src, uint32_t bytes,
                                                  uint32_t remote_bar) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     remote_dst),
                 "r"(local_src), "r"(bytes), "r"(remote_bar)
                 : "memory");
}

__global__ void __launch_bounds__(32) dsmem_bulk_kernel(int bytes, long long* cycles, int* status) {
    extern __shared__ __align__(128) unsigned char dyn[];   // source | 2 x kBulkDepth landing buffers
    __shared__ uint64_t bars[2];
    const uint32_t rank = cluster_cta_rank();
    const uint32_t next = rank ^ 1u;   // the partner (cluster sizes are even)
    unsigned char* src = dyn;
    unsigned char* landing = dyn + kBulkMaxBytes;
    for (int i = threadIdx.x; i < kBulkMaxBytes / 4; i += 32) reinterpret_cast<uint32_t*>(src)[i] = i + rank;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars[0]), 1);
        mbar_init(smem_u32(&bars[1]), 1);
        fence_mbar_init();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the source is read by the async proxy
    __syncthreads();
    cluster_sync_all();
    if (threadIdx.x == 0) {
        uint32_t step = 0;
        bool ok = true;
        for (int mode = 0; mode < 2; ++mode) {
            const int depth = mode == 0 ? 1 : kBulkDepth;
            const long long t0 = clock64();
            for (int i = 0; i < kBulkIters && ok; ++i, ++step) {
                const uint32_t b = step & 1u;
                const uint32_t my_bar = smem_u32(&bars[b]);
                mbar_arrive_expect_tx(my_bar, static_cast<uint32_t>(depth * bytes));
                for (int d = 0; d < depth; ++d)
                    bulk_copy_to_peer(map_to_rank(smem_u32(landing + (b * kBulkDepth + d) * kBulkMaxBytes), next),
                                      smem_u32(src), static_cast<uint32_t>(bytes), map_to_rank(my_bar, next));
                ok = mbar_wait_bounded(my_bar, (step >> 1) & 1u, status);
            }
            if (rank == 0) cycles[mode] = clock64() - t0;
        }
    }
    __syncthreads();
    cluster_sync_all();   // nobody leaves while a peer may still copy into it
}

// ------------------------------------------------------------------ host helpers
struct Summary { double lo, med, hi; };

Summary summarize(const long long* samples, double scale, bool invert = false, double numer = 0.0) {
    std::vector<double> v(kTrials);
    for (int i = 0; i < kTrials; ++i)
        v[i] = invert ? numer / static_cast<double>(samples[i]) : static_cast<double>(samples[i]) * scale;
    std::sort(v.begin(), v.end());
    return {v.front(), v[kTrials / 2], v.back()};
}

void print_metric(const char* label, const char* unit, const Summary& s) {
    std::printf("%-34s : %9.2f %s  (min %.2f, max %.2f)\n", label, s.med, unit, s.lo, s.hi);
}

void make_cycle(std::vector<int>& data, int stride) {
    const int n = static_cast<int>(data.size());
    int cur = 0;
    for (int i = 0; i < n; ++i) {
        data[cur] = (cur + stride) % n;
        cur = data[cur];
    }
}

int run_cluster_bench(int P, int smem_bytes, ClusterResults* host) {
    ClusterResults* d_res = nullptr;
    int* d_sink = nullptr;
    CHECK(cudaMalloc(&d_res, sizeof(ClusterResults)));
    CHECK(cudaMalloc(&d_sink, sizeof(int)));
    CHECK(cudaMemset(d_res, 0, sizeof(ClusterResults)));
    CHECK(cudaFuncSetAttribute(cluster_bench_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    CHECK(cudaFuncSetAttribute(cluster_bench_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(P);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = P;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int possible = 0;
    if (cudaOccupancyMaxActiveClusters(&possible, cluster_bench_kernel, &cfg) != cudaSuccess || possible < 1) {
        cudaGetLastError();
        cudaFree(d_res);
        cudaFree(d_sink);
        return 2;   // this cluster size cannot be scheduled
    }
    CHECK(cudaLaunchKernelEx(&cfg, cluster_bench_kernel, d_res, d_sink));
    CHECK(cudaDeviceSynchronize());
    CHECK(cudaMemcpy(host, d_res, sizeof(ClusterResults), cudaMemcpyDeviceToHost));
    cudaFree(d_res);
    cudaFree(d_sink);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    bool quick = false;
    for (int i = 1; i < argc; ++i) {
        if (!std::strcmp(argv[i], "--quick")) quick = true;
        else if (!std::strcmp(argv[i], "--help") || !std::strcmp(argv[i], "-h")) {
            std::printf("Usage: primitive_benchmark [--quick]\n");
            return 0;
        } else {
            std::fprintf(stderr, "error: unknown argument: %s\n", argv[i]);
            return 1;
        }
    }
    cudaDeviceProp prop{};
    CHECK(cudaGetDeviceProperties(&prop, 0));
    int clock_khz = 0;
    CHECK(cudaDeviceGetAttribute(&clock_khz, cudaDevAttrClockRate, 0));
    const double clock_ghz = clock_khz / 1.0e6;
    std::printf("GPU Model: %s\n", prop.name);
    std::printf("Clock frequency: %.2f GHz\n", clock_ghz);
    std::printf("SM count: %d\n", prop.multiProcessorCount);
    std::printf("===== Profiling ======\n");

    long long* d_cycles = nullptr;
    int* d_sink = nullptr;
    CHECK(cudaMalloc(&d_cycles, sizeof(long long)));
    CHECK(cudaMalloc(&d_sink, sizeof(int)));

    // ---- latencies: pointer chases sized for L1, L2 and DRAM
    const int lat_iters = quick ? 20000 : 100000;
    auto chase = [&](int elems, int stride, bool l1, double* out) -> int {
        std::vector<int> h(elems);
        make_cycle(h, stride);
        int* d = nullptr;
        CHECK(cudaMalloc(&d, sizeof(int) * static_cast<size_t>(elems)));
        CHECK(cudaMemcpy(d, h.data(), sizeof(int) * static_cast<size_t>(elems), cudaMemcpyHostToDevice));
        if (l1) chase_kernel<true><<<1, 1>>>(d, lat_iters, d_cycles, d_sink);
        else chase_kernel<false><<<1, 1>>>(d, lat_iters, d_cycles, d_sink);
        CHECK(cudaDeviceSynchronize());
        long long c = 0;
        CHECK(cudaMemcpy(&c, d_cycles, sizeof(c), cudaMemcpyDeviceToHost));
        *out = static_cast<double>(c) / lat_iters;
        cudaFree(d);
        return 0;
    };
    double l1_lat = 0, l2_lat = 0, dram_lat = 0;
    if (chase(1 << 13, 257, true, &l1_lat)) return 1;
    if (chase(1 << 21, 257, false, &l2_lat)) return 1;
    if (chase(1 << 26, (1 << 21) + 1, false, &dram_lat)) return 1;
    std::printf("L1 read latency   : %.2f cycles (%.2f ns)\n", l1_lat, l1_lat / clock_ghz);
    std::printf("L2 read latency   : %.2f cycles (%.2f ns)\n", l2_lat, l2_lat / clock_ghz);
    std::printf("DRAM read latency : %.2f cycles (%.2f ns)\n", dram_lat, dram_lat / clock_ghz);

    // ---- bandwidths
    cudaEvent_t e0, e1;
    CHECK(cudaEventCreate(&e0));
    CHECK(cudaEventCreate(&e1));
    auto elapsed = [&](float* ms) -> int {
        CHECK(cudaEventSynchronize(e1));
        CHECK(cudaEventElapsedTime(ms, e0, e1));
        return 0;
    };
    double l1_bw = 0, l2_bw = 0, dram_bw = 0;
    {
        const size_t l1_vecs = (16 << 10) / 16, l2_vecs = (32u << 20) / 16;
        int4* d = nullptr;
        CHECK(cudaMalloc(&d, l2_vecs * 16));
        CHECK(cudaMemset(d, 1, l2_vecs * 16));
        const int blocks = prop.multiProcessorCount * 4;
        const int reps1 = quick ? 2000 : 8000;
        scan_kernel<true><<<blocks, 256>>>(d, l1_vecs, 10, d_sink);
        CHECK(cudaEventRecord(e0));
        scan_kernel<true><<<blocks, 256>>>(d, l1_vecs, reps1, d_sink);
        CHECK(cudaEventRecord(e1));
        float ms = 0;
        if (elapsed(&ms)) return 1;
        // every block reads the same 16 KiB from its own L1
        l1_bw = static_cast<double>(l1_vecs) * 16 * reps1 * blocks / (ms * clock_khz) / prop.multiProcessorCount;
        const int reps2 = quick ? 10 : 40;
        scan_kernel<false><<<blocks * 2, 256>>>(d, l2_vecs, 2, d_sink);
        CHECK(cudaEventRecord(e0));
        scan_kernel<false><<<blocks * 2, 256>>>(d, l2_vecs, reps2, d_sink);
        CHECK(cudaEventRecord(e1));
        if (elapsed(&ms)) return 1;
        l2_bw = static_cast<double>(l2_vecs) * 16 * reps2 / (ms * clock_khz);
        cudaFree(d);
        const size_t copy_vecs = (quick ? 256u << 20 : 1024u << 20) / 16;
        int4 *src = nullptr, *dst = nullptr;
        CHECK(cudaMalloc(&src, copy_vecs * 16));
        CHECK(cudaMalloc(&dst, copy_vecs * 16));
        CHECK(cudaMemset(src, 1, copy_vecs * 16));
        copy_kernel<<<prop.multiProcessorCount * 8, 256>>>(src, dst, copy_vecs);
        CHECK(cudaEventRecord(e0));
        for (int i = 0; i < 5; ++i) copy_kernel<<<prop.multiProcessorCount * 8, 256>>>(src, dst, copy_vecs);
        CHECK(cudaEventRecord(e1));
        if (elapsed(&ms)) return 1;
        dram_bw = 2.0 * copy_vecs * 16 * 5 / (ms * 1.0e6);
        cudaFree(src);
        cudaFree(dst);
    }
    std::printf("L1 cache bandwidth      : %.2f B/cycle/SM\n", l1_bw);
    std::printf("L2 cache bandwidth      : %.2f B/cycle\n", l2_bw);
    std::printf("Global memory bandwidth : %.2f GB/s\n", dram_bw);

    // ---- DSMEM, per cluster size; the P = 2 block carries the reference's labels
    // more than half of an SM's shared memory per CTA, so no two CTAs share an SM
    const int smem_bytes = std::min<int>(static_cast<int>(prop.sharedMemPerBlockOptin),
                                         static_cast<int>(prop.sharedMemPerMultiprocessor) / 2 + 8192);
    const int sizes[] = {2, 4, 8, 16};
    std::vector<std::pair<int, ClusterResults>> all;
    for (int P : sizes) {
        ClusterResults r{};
        const int rc = run_cluster_bench(P, smem_bytes, &r);
        if (rc == 1) return 1;
        if (rc == 2) {
            std::printf("Cluster size %d: cannot be scheduled on this device\n", P);
            continue;
        }
        all.emplace_back(P, r);
    }
    const double tp_bytes = static_cast<double>(kThreads) * kThroughputIters * 4.0;
    for (auto& pr : all) {
        const int P = pr.first;
        const ClusterResults& r = pr.second;
        if (P == 2) {
            std::printf("----- Inter-SM DSMEM (2 CTAs, %d threads/CTA) -----\n", kThreads);
            std::printf("Dynamic shared memory/CTA         : %d bytes\n", smem_bytes);
            std::printf("%-34s : SM %u -> SM %u\n", "Cluster placement", r.smid[0], r.smid[1]);
            print_metric("Cluster sync latency", "cycles/sync", summarize(r.sync_cycles, 1.0 / kSyncIters));
            print_metric("Local SMEM read latency", "cycles/load", summarize(r.local_latency_cycles, 1.0 / kLatencyIters));
            print_metric("DSMEM read latency", "cycles/load", summarize(r.remote_latency_cycles, 1.0 / kLatencyIters));
            print_metric("Local SMEM read throughput", "B/cycle/CTA", summarize(r.local_read_cycles, 0, true, tp_bytes));
            print_metric("DSMEM read throughput", "B/cycle/CTA", summarize(r.remote_read_cycles, 0, true, tp_bytes));
            print_metric("Local SMEM store throughput", "B/cycle/CTA", summarize(r.local_store_cycles, 0, true, tp_bytes));
            print_metric("DSMEM store issue throughput", "B/cycle/CTA", summarize(r.remote_store_cycles, 0, true, tp_bytes));
            const Summary rt = summarize(r.roundtrip_cycles, 1.0 / kRoundtripIters);
            print_metric("Store visibility round trip", "cycles/roundtrip", rt);
            print_metric("One-way visibility estimate", "cycles", {rt.lo / 2, rt.med / 2, rt.hi / 2});
        }
    }
    std::printf("----- B200 extensions: per cluster size -----\n");
    for (auto& pr : all) {
        const int P = pr.first;
        const ClusterResults& r = pr.second;
        char label[96];
        bool distinct = true;
        for (int i = 0; i < P; ++i)
            for (int j = i + 1; j < P; ++j) distinct = distinct && r.smid[i] != r.smid[j];
        std::printf("Cluster %2d placement               : %s SMs%s\n", P, distinct ? "distinct" : "SHARED",
                    r.timeouts ? "  (TIMEOUTS RECORDED)" : "");
        std::snprintf(label, sizeof(label), "Cluster %2d sync latency", P);
        print_metric(label, "cycles/sync", summarize(r.sync_cycles, 1.0 / kSyncIters));
        std::snprintf(label, sizeof(label), "Cluster %2d barrier exchange", P);
        print_metric(label, "cycles/exchange", summarize(r.barrier_exchange_cycles, 1.0 / kExchangeIters));
        std::snprintf(label, sizeof(label), "Cluster %2d mbarrier exchange", P);
        print_metric(label, "cycles/exchange", summarize(r.async_exchange_cycles, 1.0 / kExchangeIters));
        std::snprintf(label, sizeof(label), "Cluster %2d DSMEM read latency", P);
        print_metric(label, "cycles/load", summarize(r.remote_latency_cycles, 1.0 / kLatencyIters));
        std::snprintf(label, sizeof(label), "Cluster %2d DSMEM read throughput", P);
        print_metric(label, "B/cycle/CTA", summarize(r.remote_read_cycles, 0, true, tp_bytes));
        std::snprintf(label, sizeof(label), "Cluster %2d DSMEM store throughput", P);
        print_metric(label, "B/cycle/CTA", summarize(r.remote_store_cycles, 0, true, tp_bytes));
    }

    // ---- DSMEM bulk copy (shared memory of one CTA -> shared memory of the next CTA of the cluster)
    {
        const int bulk_smem = kBulkMaxBytes * (1 + 2 * kBulkDepth);
        CHECK(cudaFuncSetAttribute(dsmem_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bulk_smem));
        CHECK(cudaFuncSetAttribute(dsmem_bulk_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        long long* d_bulk = nullptr;
        int* d_status = nullptr;
        CHECK(cudaMalloc(&d_bulk, 2 * sizeof(long long)));
        CHECK(cudaMalloc(&d_status, sizeof(int)));
        CHECK(cudaMemset(d_status, 0, sizeof(int)));
        for (auto& pr : all) {
            const int P = pr.first;
            if (P != 2 && P != 8 && P != 16) continue;
            for (int bytes : {256, 1024, 4096, 16384}) {
                cudaLaunchConfig_t cfg{};
                cfg.gridDim = dim3(P);
                cfg.blockDim = dim3(32);
                cfg.dynamicSmemBytes = bulk_smem;
                cudaLaunchAttribute attr{};
                attr.id = cudaLaunchAttributeClusterDimension;
                attr.val.clusterDim.x = P;
                attr.val.clusterDim.y = 1;
                attr.val.clusterDim.z = 1;
                cfg.attrs = &attr;
                cfg.numAttrs = 1;
                CHECK(cudaMemset(d_bulk, 0, 2 * sizeof(long long)));
                CHECK(cudaLaunchKernelEx(&cfg, dsmem_bulk_kernel, bytes, d_bulk, d_status));
                CHECK(cudaDeviceSynchronize());
                long long c[2] = {0, 0};
                CHECK(cudaMemcpy(c, d_bulk, sizeof(c), cudaMemcpyDeviceToHost));
                char label[96];
                std::snprintf(label, sizeof(label), "Cluster %2d DSMEM bulk %5d B step", P, bytes);
                std::printf("%-34s : %9.2f cycles  (%.2f B/cycle/CTA with %d copies in flight)\n", label,
                            static_cast<double>(c[0]) / kBulkIters,
                            c[1] > 0 ? static_cast<double>(kBulkDepth) * bytes * kBulkIters / static_cast<double>(c[1]) : 0.0,
                            kBulkDepth);
            }
        }
        int st = 0;
        CHECK(cudaMemcpy(&st, d_status, sizeof(int), cudaMemcpyDeviceToHost));
        if (st) std::printf("DSMEM bulk copy waits timed out (status %d)\n", st);
        cudaFree(d_bulk);
        cudaFree(d_status);
    }

    // ---- bulk-async load latency from DRAM
    {
        const size_t stride = 8u << 20;
        const int repeats = 32;
        unsigned char* d = nullptr;
        CHECK(cudaMalloc(&d, stride * repeats));
        CHECK(cudaMemset(d, 1, stride * repeats));
        // written before every measurement so that the lines of `d` leave the L2
        const size_t flush_bytes = 512u << 20;
        unsigned char* d_flush = nullptr;
        CHECK(cudaMalloc(&d_flush, flush_bytes));
        int* d_status = nullptr;
        CHECK(cudaMalloc(&d_status, sizeof(int)));
        CHECK(cudaMemset(d_status, 0, sizeof(int)));
        CHECK(cudaFuncSetAttribute(tma_latency_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));
        const int sizes_b[] = {1024, 4096, 16384, 32768, 65536};
        for (int bytes : sizes_b) {
            CHECK(cudaMemset(d_flush, bytes & 0xff, flush_bytes));
            tma_latency_kernel<<<1, 32, 65536>>>(d, stride, bytes, repeats, d_cycles, d_status);
            CHECK(cudaDeviceSynchronize());
            long long c = 0;
            CHECK(cudaMemcpy(&c, d_cycles, sizeof(c), cudaMemcpyDeviceToHost));
            char label[96];
            std::snprintf(label, sizeof(label), "Bulk copy %5d B latency", bytes);
            std::printf("%-34s : %9.2f cycles  (%.2f ns)\n", label, static_cast<double>(c) / repeats,
                        static_cast<double>(c) / repeats / clock_ghz);
        }
        cudaFree(d_flush);
        int st = 0;
        CHECK(cudaMemcpy(&st, d_status, sizeof(int), cudaMemcpyDeviceToHost));
        if (st) std::printf("Bulk copy waits timed out (status %d)\n", st);
        cudaFree(d);
        cudaFree(d_status);
    }

    std::printf("==================== SUMMARY ====================\n");
    std::printf("L1   read latency       : %8.2f cycles\n", l1_lat);
    std::printf("L2   read latency       : %8.2f cycles\n", l2_lat);
    std::printf("DRAM read latency       : %8.2f cycles\n", dram_lat);
    std::printf("L1   bandwidth          : %8.2f B/cycle/SM\n", l1_bw);
    std::printf("L2   bandwidth          : %8.2f B/cycle\n", l2_bw);
    std::printf("DRAM bandwidth          : %8.2f GB/s\n", dram_bw);
    std::printf("=================================================\n");
    cudaFree(d_cycles);
    cudaFree(d_sink);
    return 0;
}
