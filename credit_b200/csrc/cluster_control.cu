// Launch-and-barrier overhead of an empty cluster kernel against an empty block
// kernel: the control term of the cluster-size cost model. Same flags and the same
// CONTROL / UNSUPPORTED output lines as the reference tool
// (src/cluster_control.cu:20-66, 114-180), extended to cluster sizes 1..16 and to
// the mbarrier exchange this library uses instead of barrier.cluster.
//
//   cluster_control --rows R --cluster-size P --barriers B --shared-bytes S
//                   [--warmup W] [--iters I] [--threads T] [--exchange barrier|mbarrier]
//   -> CONTROL,rows,P,barriers,shared_bytes,block_ms,cluster_ms,delta_ms

#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "cluster_primitives.cuh"

using namespace credit;

namespace {

__global__ void block_control_kernel(unsigned* sink) {
    if (threadIdx.x == 0) sink[blockIdx.x] = blockIdx.x;
}

// `barriers` cluster-wide synchronisations with `shared_bytes` of dynamic shared
// memory claimed, nothing else. use_mbarrier: each synchronisation is the
// st.async all-to-all of one float per CTA plus a wait on the CTA's own mbarrier.
__global__ void cluster_control_kernel(unsigned* sink, int barriers, int shared_bytes, int use_mbarrier,
                                       int* status) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ uint64_t bars[2];
    __shared__ float slots[2][kMaxClusterSize];
    const uint32_t rank = cluster_cta_rank();
    const uint32_t P = cluster_cta_count();
    if (threadIdx.x == 0) {
        if (shared_bytes > 0) dyn[0] = static_cast<unsigned char>(rank);
        mbar_init(smem_u32(&bars[0]), 1);
        mbar_init(smem_u32(&bars[1]), 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (use_mbarrier) {
        cluster_sync_all();   // peers must be running before their shared memory is written
        for (int i = 0; i < barriers; ++i) {
            const int buf = i & 1;
            const uint32_t bar = smem_u32(&bars[buf]);
            if (threadIdx.x < 32) {
                if (threadIdx.x == 0) mbar_arrive_expect_tx(bar, P * 4u);
                if (threadIdx.x < P)
                    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];" ::
                                     "r"(map_to_rank(smem_u32(&slots[buf][rank]), threadIdx.x)),
                                 "f"(1.0f), "r"(map_to_rank(bar, threadIdx.x))
                                 : "memory");
                mbar_wait_bounded(bar, (static_cast<uint32_t>(i) >> 1) & 1u, status);
            }
            __syncthreads();
        }
    } else {
        for (int i = 0; i < barriers; ++i) cluster_sync_all();
    }
    if (threadIdx.x == 0) sink[blockIdx.x] = (shared_bytes > 0 ? dyn[0] : 0u) + static_cast<unsigned>(barriers);
}

struct Options {
    int rows = 4096, cluster_size = 8, barriers = 4, shared_bytes = 0, warmup = 5, iters = 20, threads = 256;
    bool mbarrier = false;
};

bool parse(int argc, char** argv, Options* o, std::string* err) {
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto need = [&](int* dst) {
            if (i + 1 >= argc) { *err = "missing value for " + a; return false; }
            *dst = std::atoi(argv[++i]);
            return true;
        };
        if (a == "--rows") { if (!need(&o->rows)) return false; }
        else if (a == "--cluster-size") { if (!need(&o->cluster_size)) return false; }
        else if (a == "--barriers") { if (!need(&o->barriers)) return false; }
        else if (a == "--shared-bytes") { if (!need(&o->shared_bytes)) return false; }
        else if (a == "--warmup") { if (!need(&o->warmup)) return false; }
        else if (a == "--iters") { if (!need(&o->iters)) return false; }
        else if (a == "--threads") { if (!need(&o->threads)) return false; }
        else if (a == "--exchange") {
            if (i + 1 >= argc) { *err = "missing value for --exchange"; return false; }
            const std::string v = argv[++i];
            if (v != "barrier" && v != "mbarrier") { *err = "--exchange must be barrier or mbarrier"; return false; }
            o->mbarrier = v == "mbarrier";
        } else if (a == "--help" || a == "-h") {
            std::printf("Usage: cluster_control --rows N --cluster-size N --barriers N --shared-bytes N "
                        "[--warmup N] [--iters N] [--threads N] [--exchange barrier|mbarrier]\n");
            std::exit(0);
        } else { *err = "unknown argument: " + a; return false; }
    }
    if (o->rows <= 0 || o->barriers < 0 || o->shared_bytes < 0 || o->warmup < 0 || o->iters <= 0) {
        *err = "numeric arguments must be positive";
        return false;
    }
    const int p = o->cluster_size;
    if (p != 1 && p != 2 && p != 4 && p != 8 && p != 16) { *err = "cluster size must be 1, 2, 4, 8 or 16"; return false; }
    if (o->threads < 32 || o->threads > 1024 || o->threads % 32) { *err = "threads must be a multiple of 32 up to 1024"; return false; }
    return true;
}

#define CHECK(expr)                                                                         \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess) {                                                           \
            std::fprintf(stderr, "error: %s -> %s\n", #expr, cudaGetErrorString(e__));      \
            return 1;                                                                       \
        }                                                                                   \
    } while (0)

}  // namespace

int main(int argc, char** argv) {
    Options o;
    std::string err;
    if (!parse(argc, argv, &o, &err)) {
        std::fprintf(stderr, "error: %s\n", err.c_str());
        return 1;
    }
    cudaDeviceProp prop{};
    CHECK(cudaGetDeviceProperties(&prop, 0));
    int cluster_launch = 0;
    CHECK(cudaDeviceGetAttribute(&cluster_launch, cudaDevAttrClusterLaunch, 0));
    if (!cluster_launch) {
        std::fprintf(stderr, "error: device does not support cluster launch\n");
        return 1;
    }
    if (static_cast<size_t>(o.shared_bytes) > prop.sharedMemPerBlockOptin) {
        std::printf("UNSUPPORTED,%d,%d,%d,%d,shared-memory-limit\n", o.rows, o.cluster_size, o.barriers, o.shared_bytes);
        return 0;
    }
    CHECK(cudaFuncSetAttribute(cluster_control_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, o.shared_bytes));
    CHECK(cudaFuncSetAttribute(cluster_control_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    const int blocks = o.rows * o.cluster_size;
    unsigned* sink = nullptr;
    int* status = nullptr;
    CHECK(cudaMalloc(&sink, sizeof(unsigned) * static_cast<size_t>(blocks)));
    CHECK(cudaMalloc(&status, sizeof(int)));
    CHECK(cudaMemset(status, 0, sizeof(int)));

    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(o.threads);
    cfg.dynamicSmemBytes = o.shared_bytes;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = o.cluster_size;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int resident = 0;
    if (cudaOccupancyMaxActiveClusters(&resident, cluster_control_kernel, &cfg) != cudaSuccess || resident < 1) {
        cudaGetLastError();
        std::printf("UNSUPPORTED,%d,%d,%d,%d,cluster-cannot-be-scheduled\n", o.rows, o.cluster_size, o.barriers,
                    o.shared_bytes);
        return 0;
    }
    cudaEvent_t e0, e1;
    CHECK(cudaEventCreate(&e0));
    CHECK(cudaEventCreate(&e1));
    auto time_it = [&](bool cluster, double* ms) -> int {
        for (int i = 0; i < o.warmup + o.iters; ++i) {
            if (i == o.warmup) CHECK(cudaEventRecord(e0));
            if (cluster)
                CHECK(cudaLaunchKernelEx(&cfg, cluster_control_kernel, sink, o.barriers, o.shared_bytes,
                                         o.mbarrier ? 1 : 0, status));
            else
                block_control_kernel<<<o.rows, o.threads>>>(sink);
        }
        CHECK(cudaEventRecord(e1));
        CHECK(cudaEventSynchronize(e1));
        float t = 0;
        CHECK(cudaEventElapsedTime(&t, e0, e1));
        *ms = static_cast<double>(t) / o.iters;
        return 0;
    };
    double block_ms = 0, cluster_ms = 0;
    if (time_it(false, &block_ms)) return 1;
    if (time_it(true, &cluster_ms)) return 1;
    int st = 0;
    CHECK(cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != 0) {
        std::fprintf(stderr, "error: an exchange wait timed out (status %d)\n", st);
        return 1;
    }
    std::printf("CONTROL,%d,%d,%d,%d,%g,%g,%g\n", o.rows, o.cluster_size, o.barriers, o.shared_bytes, block_ms,
                cluster_ms, cluster_ms - block_ms);
    cudaFree(sink);
    cudaFree(status);
    return 0;
}
