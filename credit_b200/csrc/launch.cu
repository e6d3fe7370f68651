// Host side of the C ABI declared in include/credit_b200.h: argument checks,
// launch planning (cluster size, slice, ring depth, grid), cached function
// attributes and the cluster launches themselves. This is the one shared
// launcher that replaces the host glue every reference binary carries a copy of
// (query_device_info, benchmark_block_*, benchmark_cluster;
// src/workloads/layernorm_backward.cu:440-593).

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

#include "../../include/credit_b200.h"
#include "cluster_primitives.cuh"
#include "error_state.h"
#include "kernel_tables.h"
#include "launch_args.h"

namespace credit {

// Device status word: kernels OR their failure bits into it.
__device__ int g_status_word;

namespace {

thread_local char t_last_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_last_error, sizeof(t_last_error), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t err, const char* what) {
    return fail(CREDIT_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
}

}  // namespace

int report_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_last_error, sizeof(t_last_error), fmt, ap);
    va_end(ap);
    return code;
}

namespace {

#define CREDIT_CUDA_TRY(expr)                                  \
    do {                                                       \
        cudaError_t err__ = (expr);                            \
        if (err__ != cudaSuccess) return cuda_fail(err__, #expr); \
    } while (0)

struct DeviceState {
    bool ready = false;
    credit_device_info info{};
    int* status_ptr = nullptr;
};

std::mutex g_mutex;
std::map<int, DeviceState> g_devices;
// (device, function) pairs whose attributes are already set.
std::map<std::pair<int, const void*>, bool> g_prepared;
// (device, function, cluster, smem, threads) -> co-resident clusters
std::map<std::tuple<int, const void*, int, int, int>, int> g_active_clusters;

int load_device(int device, DeviceState** out) {
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState& st = g_devices[device];
    if (!st.ready) {
        cudaDeviceProp prop{};
        CREDIT_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
        std::memset(&st.info, 0, sizeof(st.info));
        std::snprintf(st.info.name, sizeof(st.info.name), "%s", prop.name);
        st.info.sm_major = prop.major;
        st.info.sm_minor = prop.minor;
        st.info.sm_count = prop.multiProcessorCount;
        int cluster_launch = 0;
        CREDIT_CUDA_TRY(cudaDeviceGetAttribute(&cluster_launch, cudaDevAttrClusterLaunch, device));
        st.info.cluster_launch = cluster_launch;
        st.info.max_cluster_size = cluster_launch ? kMaxClusterSize : 1;
        st.info.max_dynamic_smem_per_block = static_cast<int>(prop.sharedMemPerBlockOptin);
        st.info.smem_per_sm = static_cast<int>(prop.sharedMemPerMultiprocessor);
        st.info.l2_bytes = prop.l2CacheSize;
        int khz = 0;
        CREDIT_CUDA_TRY(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device));
        st.info.clock_khz = khz;
        CREDIT_CUDA_TRY(cudaDeviceGetAttribute(&khz, cudaDevAttrMemoryClockRate, device));
        st.info.mem_clock_khz = khz;
        int bits = 0;
        CREDIT_CUDA_TRY(cudaDeviceGetAttribute(&bits, cudaDevAttrGlobalMemoryBusWidth, device));
        st.info.mem_bus_bits = bits;
        int current = 0;
        CREDIT_CUDA_TRY(cudaGetDevice(&current));
        if (current != device) CREDIT_CUDA_TRY(cudaSetDevice(device));
        void* sym = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&sym, g_status_word);
        if (err == cudaSuccess) err = cudaMemset(sym, 0, sizeof(int));
        if (current != device) cudaSetDevice(current);
        if (err != cudaSuccess) return cuda_fail(err, "status word set-up");
        st.status_ptr = static_cast<int*>(sym);
        st.ready = true;
    }
    *out = &st;
    return CREDIT_OK;
}

int current_device_state(DeviceState** out) {
    int device = 0;
    CREDIT_CUDA_TRY(cudaGetDevice(&device));
    return load_device(device, out);
}

int prepare_function(int device, const void* func, int max_smem) {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto key = std::make_pair(device, func);
    if (g_prepared.count(key)) return CREDIT_OK;
    cudaFuncAttributes fa{};
    CREDIT_CUDA_TRY(cudaFuncGetAttributes(&fa, func));
    // static + dynamic shared memory together must stay within the opt-in limit
    const int max_dynamic = max_smem - static_cast<int>(fa.sharedSizeBytes);
    CREDIT_CUDA_TRY(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, max_dynamic));
    CREDIT_CUDA_TRY(cudaFuncSetAttribute(func, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
    g_prepared[key] = true;
    return CREDIT_OK;
}

struct Launch {
    const void* func = nullptr;
    int grid = 0;
    int threads = 0;
    int cluster = 1;
    int smem = 0;
    cudaStream_t stream = nullptr;
};

void fill_config(const Launch& l, cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr) {
    std::memset(cfg, 0, sizeof(*cfg));
    cfg->gridDim = dim3(static_cast<unsigned>(l.grid));
    cfg->blockDim = dim3(static_cast<unsigned>(l.threads));
    cfg->dynamicSmemBytes = static_cast<size_t>(l.smem);
    cfg->stream = l.stream;
    attr->id = cudaLaunchAttributeClusterDimension;
    attr->val.clusterDim.x = static_cast<unsigned>(l.cluster);
    attr->val.clusterDim.y = 1;
    attr->val.clusterDim.z = 1;
    cfg->attrs = attr;
    cfg->numAttrs = 1;
}

int launch_cluster_kernel(const Launch& l, void** args) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    fill_config(l, &cfg, &attr);
    CREDIT_CUDA_TRY(cudaLaunchKernelExC(&cfg, l.func, args));
    return CREDIT_OK;
}

// Clusters of this shape that can be resident at once on the device.
int max_active_clusters(int device, const void* func, int cluster, int smem, int threads,
                        int* out) {
    auto key = std::make_tuple(device, func, cluster, smem, threads);
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        auto it = g_active_clusters.find(key);
        if (it != g_active_clusters.end()) {
            *out = it->second;
            return CREDIT_OK;
        }
    }
    Launch l;
    l.func = func;
    l.grid = cluster;
    l.threads = threads;
    l.cluster = cluster;
    l.smem = smem;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr;
    fill_config(l, &cfg, &attr);
    int n = 0;
    cudaError_t err = cudaOccupancyMaxActiveClusters(&n, func, &cfg);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(CREDIT_ERR_UNSUPPORTED,
                    "cluster size %d with %d B shared memory and %d threads cannot be scheduled: %s",
                    cluster, smem, threads, cudaGetErrorString(err));
    }
    if (n <= 0) {
        return fail(CREDIT_ERR_UNSUPPORTED,
                    "cluster size %d with %d B shared memory and %d threads: no resident cluster",
                    cluster, smem, threads);
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    g_active_clusters[key] = n;
    *out = n;
    return CREDIT_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int round_up(int v, int m) { return (v + m - 1) / m * m; }

bool valid_cluster_size(int p) { return p == 1 || p == 2 || p == 4 || p == 8 || p == 16; }

struct Shape {
    int rows;
    int cols;
    int elem_bytes;
    int vec_elems;
};

int check_shape(int64_t rows, int64_t cols, int dtype, Shape* s) {
    if (dtype != CREDIT_F32 && dtype != CREDIT_BF16)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
    if (rows < 0 || rows > (1ll << 30))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "rows=%lld out of range [0, 2^30]",
                    static_cast<long long>(rows));
    if (cols < 1 || cols > (1ll << 30))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "cols=%lld out of range [1, 2^30]",
                    static_cast<long long>(cols));
    s->rows = static_cast<int>(rows);
    s->cols = static_cast<int>(cols);
    s->elem_bytes = dtype == CREDIT_F32 ? 4 : 2;
    s->vec_elems = 16 / s->elem_bytes;
    return CREDIT_OK;
}

int check_opts(const credit_launch_opts* o, credit_launch_opts* out) {
    credit_launch_opts z{};
    if (o != nullptr) z = *o;
    if (z.cluster_size != 0 && !valid_cluster_size(z.cluster_size))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "cluster_size must be 0, 1, 2, 4, 8 or 16 (got %d)",
                    z.cluster_size);
    if (z.variant < CREDIT_VARIANT_AUTO || z.variant > CREDIT_VARIANT_CLUSTER_SMEM)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "unknown variant %d", z.variant);
    if (z.stages < 0 || z.stages > kWsMaxStages)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "stages must be in [0, %d] (got %d)", kWsMaxStages,
                    z.stages);
    if (z.threads != 0 && z.threads != 256 && z.threads != 512 && z.threads != kWsThreadsPerCta &&
        z.threads != kWsThreadsPerCtaWide)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "threads must be 0, 256, 512, %d or %d (got %d)",
                    kWsThreadsPerCtaWide, kWsThreadsPerCta, z.threads);
    if (z.schedule < CREDIT_SCHEDULE_AUTO || z.schedule > CREDIT_SCHEDULE_PERSISTENT)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "unknown schedule %d", z.schedule);
    if (z.load_path < CREDIT_LOAD_AUTO || z.load_path > CREDIT_LOAD_LDG)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "unknown load_path %d", z.load_path);
    if (z.chunk_bytes < 0 || z.chunk_bytes % 1024 != 0 || z.chunk_bytes > 65536)
        return fail(CREDIT_ERR_INVALID_ARGUMENT,
                    "chunk_bytes must be a multiple of 1024 up to 65536 (got %d)", z.chunk_bytes);
    if (z.flags & ~CREDIT_FLAG_NO_REGISTER_PATH)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "unknown flags 0x%x", z.flags);
    if (z.variant == CREDIT_VARIANT_BLOCK_SMEM || z.variant == CREDIT_VARIANT_BLOCK_READ) {
        if (z.cluster_size > 1)
            return fail(CREDIT_ERR_INVALID_ARGUMENT, "block variants run with cluster_size 1 (got %d)",
                        z.cluster_size);
        z.cluster_size = 1;
    }
    if (z.variant == CREDIT_VARIANT_CLUSTER_SMEM && z.cluster_size == 1)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "the cluster variant needs cluster_size >= 2");
    *out = z;
    return CREDIT_OK;
}

// ---------------------------------------------------------------------------
// kernel selection (the tables live in one translation unit per kernel family)
// ---------------------------------------------------------------------------
bool is_row_op(int workload) {
    return workload >= CREDIT_WL_WEIGHTED_VAR_BACKWARD && workload <= CREDIT_WL_ROWWISE_QUANT;
}

const void* workload_func(int workload, int dtype, const credit_plan_info& p, bool want_grads) {
    const bool al = p.aligned != 0;
    if (is_row_op(workload) && (p.threads == kWsThreadsPerCta || p.threads == kWsThreadsPerCtaWide))
        return ws_row_op_kernel_for(workload);
    if (is_row_op(workload)) return row_op_kernel_for(workload, p.threads, al, p.variant != CREDIT_VARIANT_BLOCK_READ);
    if (p.variant == CREDIT_VARIANT_BLOCK_READ) return block_read_kernel_for(workload, dtype, al);
    const int vpt = p.vectors_per_thread;
    const bool full = p.full_tiles != 0;
    if (p.threads == kWsThreadsPerCta || p.threads == kWsThreadsPerCtaWide) {
        const int out_warps = p.threads / 32 - 3;   // three service warps
        switch (workload) {
            case CREDIT_WL_RMSNORM_FORWARD: return ws_rmsnorm_kernel_for(dtype, out_warps, vpt, full);
            case CREDIT_WL_LAYERNORM_FORWARD: return ws_layernorm_fwd_kernel_for(dtype, out_warps, vpt, full);
            case CREDIT_WL_LAYERNORM_BACKWARD: return ws_layernorm_bwd_dx_kernel_for(dtype, out_warps, vpt, full, true);
            case CREDIT_WL_LAYERNORM_BACKWARD_STATS:
                return want_grads ? ws_layernorm_bwd_kernel_for(dtype, out_warps, vpt, full)
                                  : ws_layernorm_bwd_dx_kernel_for(dtype, out_warps, vpt, full, false);
            default: return nullptr;
        }
    }
    switch (workload) {
        case CREDIT_WL_RMSNORM_FORWARD:
            return rmsnorm_kernel_for(dtype, p.threads, vpt, full, al);
        case CREDIT_WL_ROW_REDUCE:
            return row_reduce_kernel_for(p.load_path, p.threads, al);
        case CREDIT_WL_LAYERNORM_FORWARD:
            return layernorm_fwd_kernel_for(dtype, p.threads, vpt, full, al);
        case CREDIT_WL_LAYERNORM_BACKWARD:
            return layernorm_bwd_kernel_for(dtype, p.threads, vpt, full, al, false, false);
        case CREDIT_WL_LAYERNORM_BACKWARD_STATS:
            return layernorm_bwd_kernel_for(dtype, p.threads, vpt, full, al, true, want_grads);
        default:
            return nullptr;
    }
}

// ---------------------------------------------------------------------------
// planning
// ---------------------------------------------------------------------------
constexpr int kColsumRowsPerBlock = 128;   // fallback column-sum kernel: rows per partial ...
constexpr int kColsumMaxBlocks = 1024;     // ... unless that would make more partials than this
constexpr int kAutoStageBytes = 32 * 1024; // automatic cluster size aims at this much per stage
constexpr int kAutoRingBytes = 96 * 1024;  // and at this much ring per CTA

// Row elements a thread of the register path may own: what it keeps per element
// in registers (raw data, gamma/beta, xhat and g, running column sums) bounds it.
int max_elems_per_thread(int workload, bool grads) {
    switch (workload) {
        case CREDIT_WL_RMSNORM_FORWARD: return 32;
        case CREDIT_WL_LAYERNORM_FORWARD: return 32;
        // up to 16 elements are held in registers across the exchange; 17..32 are read from the
        // shared-memory stage a second time instead (the stage then lives one row longer)
        // (with the column sums in registers as well, 32 elements spill: measured slower)
        case CREDIT_WL_LAYERNORM_BACKWARD: return 32;
        case CREDIT_WL_LAYERNORM_BACKWARD_STATS: return grads ? 16 : 32;
        default: return 0;
    }
}

int inputs_staged(int workload) {
    switch (workload) {
        case CREDIT_WL_LAYERNORM_BACKWARD:
        case CREDIT_WL_LAYERNORM_BACKWARD_STATS:
        case CREDIT_WL_PEARSON_BACKWARD:
        case CREDIT_WL_SOFTMAX_LOGITS_BACKWARD:
            return 2;
        case CREDIT_WL_WEIGHTED_VAR_BACKWARD:
        case CREDIT_WL_LARS_MOMENTUM:
            return 3;
        default:
            return 1;
    }
}

// Resolves everything that does not need the occupancy query. `want_grads`
// only matters for CREDIT_WL_LAYERNORM_BACKWARD_STATS.
int plan_static(int workload, const Shape& s, int dtype, const credit_launch_opts& o,
                bool pointers_aligned, bool want_grads, const credit_device_info& dev,
                credit_plan_info* p) {
    std::memset(p, 0, sizeof(*p));
    if (workload < CREDIT_WL_RMSNORM_FORWARD || workload > CREDIT_WL_ROWWISE_QUANT)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "unknown workload %d", workload);
    if (is_row_op(workload) && dtype != CREDIT_F32)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "the reference-sweep workloads take fp32 data");
    if (workload == CREDIT_WL_ROW_REDUCE && dtype != CREDIT_F32)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "row_reduce takes fp32 input");
    if (o.variant == CREDIT_VARIANT_BLOCK_READ && workload == CREDIT_WL_ROW_REDUCE)
        return fail(CREDIT_ERR_UNSUPPORTED,
                    "row_reduce reads its input once in every variant; use cluster_size 1 for the block form");
    if (!dev.cluster_launch && o.cluster_size > 1)
        return fail(CREDIT_ERR_UNSUPPORTED, "device cannot launch thread-block clusters");

    const int max_smem = dev.max_dynamic_smem_per_block;
    const int max_cluster = dev.cluster_launch ? kMaxClusterSize : 1;
    p->aligned = (pointers_aligned && s.cols % s.vec_elems == 0) ? 1 : 0;
    p->variant = o.variant;
    p->kernel_launches = 1;

    if (workload == CREDIT_WL_ROW_REDUCE) {
        // measured on B200 (512 x 1M fp32): unrolled 128-bit loads 300 us, best bulk-copy ring 305 us
        p->load_path = o.load_path != CREDIT_LOAD_AUTO ? o.load_path : CREDIT_LOAD_LDG;
        if (p->load_path == CREDIT_LOAD_TMA && !p->aligned)
            return fail(CREDIT_ERR_UNSUPPORTED,
                        "bulk-copy path needs 16-byte aligned rows (cols %% 4 == 0, aligned base)");
        p->threads = o.threads ? o.threads : 256;
        int cluster = o.cluster_size;
        if (cluster == 0) {
            // One CTA per row unless the rows are too few to cover the device twice (measured: at 512
            // rows one CTA per row wins from 4 K to 1 M columns); slices of at least 64 KiB.
            cluster = 1;
            while (cluster < max_cluster && 1ll * s.rows * cluster < 2ll * dev.sm_count &&
                   1ll * s.cols * 4 / (cluster * 2) >= 65536)
                cluster *= 2;
            if (o.variant == CREDIT_VARIANT_CLUSTER_SMEM && cluster < 2) cluster = 2;
        }
        p->cluster_size = cluster;
        p->slice_elems = round_up((s.cols + cluster - 1) / cluster, 64);
        if (p->load_path == CREDIT_LOAD_TMA) {
            int chunk_bytes = o.chunk_bytes ? o.chunk_bytes : 16384;
            chunk_bytes = std::min(chunk_bytes, round_up(p->slice_elems * 4, 1024));
            p->chunk_elems = chunk_bytes / 4;
            if (o.stages > kMaxStages)
                return fail(CREDIT_ERR_UNSUPPORTED, "the row reduction takes rings of at most %d stages", kMaxStages);
            p->stages = o.stages ? o.stages : 3;
            p->smem_bytes = kControlBytes + p->stages * chunk_bytes;
            if (p->smem_bytes > max_smem)
                return fail(CREDIT_ERR_UNSUPPORTED, "ring of %d x %d B exceeds %d B of shared memory",
                            p->stages, chunk_bytes, max_smem);
            p->schedule = o.schedule ? o.schedule : CREDIT_SCHEDULE_ROW_PER_CLUSTER;
        } else {
            p->stages = 0;
            p->chunk_elems = 0;
            p->smem_bytes = 0;
            p->schedule = o.schedule ? o.schedule : CREDIT_SCHEDULE_ROW_PER_CLUSTER;
        }
        return CREDIT_OK;
    }

    if (o.variant == CREDIT_VARIANT_BLOCK_READ) {
        // one CTA of 512 threads per row, no shared-memory staging, no cluster
        p->cluster_size = 1;
        p->threads = is_row_op(workload) ? (o.threads ? o.threads : 256) : 512;
        p->schedule = CREDIT_SCHEDULE_ROW_PER_CLUSTER;
        p->load_path = CREDIT_LOAD_LDG;
        p->slice_elems = round_up(s.cols, 64);
        p->stages = 0;
        p->smem_bytes = is_row_op(workload) ? kControlBytes : 0;   // reduction scratch
        return CREDIT_OK;
    }

    // staged kernels
    const int nin = inputs_staged(workload);
    const bool grads = workload == CREDIT_WL_LAYERNORM_BACKWARD_STATS && want_grads;
    p->load_path = p->aligned ? CREDIT_LOAD_TMA : CREDIT_LOAD_LDG;
    if (o.load_path == CREDIT_LOAD_TMA && !p->aligned)
        return fail(CREDIT_ERR_UNSUPPORTED,
                    "bulk-copy path needs 16-byte aligned rows and base pointers");

    auto stage_bytes_for = [&](int cluster) {
        return nin * round_up((s.cols + cluster - 1) / cluster, 64) * s.elem_bytes;
    };

    // The warp-specialised kernels (ws_row_kernels.cuh: 16 or 8 output warps plus producer, collector
    // and receiver warps) serve RMSNorm forward, LayerNorm forward and every form of LayerNorm
    // backward whenever the rows are 16-byte aligned, the slice fits the output threads' registers
    // and a ring of at least three stages fits shared memory. threads = 256 / 512 keep the lock-step
    // register kernels. (LayerNorm backward with recomputed statistics sends records of four sums:
    // like the reference-sweep workloads it has the 8-output-warp form only.)
    const bool ws_threads = o.threads == kWsThreadsPerCta || o.threads == kWsThreadsPerCtaWide;
    const bool row_op = is_row_op(workload);   // no per-column registers: any slice length, 8 output warps only
    const bool wide_only = row_op || workload == CREDIT_WL_LAYERNORM_BACKWARD;
    const bool ws_workload = wide_only ? o.threads != kWsThreadsPerCta
                                       : (workload == CREDIT_WL_RMSNORM_FORWARD || workload == CREDIT_WL_LAYERNORM_FORWARD ||
                                          workload == CREDIT_WL_LAYERNORM_BACKWARD_STATS);
    // fp32 RMSNorm keeps the lock-step register kernel unless threads asks otherwise: with 512 threads
    // and the smallest cluster whose slice fits them it ran 1024 x 32768 in 45.1 us against 46.4 - 50.3 us
    // for every warp-specialised form (4096 x 32768: 163 us against 170 - 184 us), and within 4 % of the
    // best form at the other row lengths from 4096 to 65536.
    const bool lock_step_default = workload == CREDIT_WL_RMSNORM_FORWARD && dtype == CREDIT_F32 && o.threads == 0;
    if (ws_workload && !lock_step_default && p->aligned && !(o.flags & CREDIT_FLAG_NO_REGISTER_PATH) &&
        (o.threads == 0 || ws_threads) &&
        o.schedule != CREDIT_SCHEDULE_ROW_PER_CLUSTER && (o.stages == 0 || o.stages >= 3) &&
        o.variant != CREDIT_VARIANT_BLOCK_SMEM) {
        // measured at the target shapes: 8 output warps with twice the elements per thread win over 16
        // (the per-row work of a warp is paid by half as many warps)
        const int threads = o.threads ? o.threads : kWsThreadsPerCtaWide;
        const bool wide = threads == kWsThreadsPerCtaWide;
        const int out_threads = threads - 96;   // three service warps
        const int max_slice = row_op ? (1 << 30) : out_threads * ws_max_elems_per_thread(grads, wide);
        // Automatic choice, from a sweep of cluster size x ring depth on B200 (four workloads, row
        // lengths 4096 ... 65536): the smallest cluster that fits wins or is within 2 % of the winner
        // nearly everywhere, because small clusters cover more SMs (148, 148, 132, 120, 112 for sizes
        // 1 ... 16) and spread a row's fixed costs over longer slices. A ring of three stages runs the
        // two passes one row apart and costs 5 - 20 %, so a cluster that only fits three yields to the
        // next size, except that 16 never replaces 8. The row-period model picked clusters too large
        // (15 % mean loss on the same sweep, against 1.7 % for this rule).
        auto ws_fits = [&](int c, int min_stages) {
            return round_up((s.cols + c - 1) / c, 64) <= max_slice &&
                   kWsControlBytes + min_stages * stage_bytes_for(c) <= max_smem;
        };
        // Ring depth a cluster size must reach to be taken over the next one, from the same sweeps:
        // four for the normalisation workloads and Pearson, six for LARS (three inputs and two
        // outputs per row: its best size always had stages of 24 KiB), three for the others.
        const int wanted_stages = workload == CREDIT_WL_LARS_MOMENTUM ? 6
                                  : (row_op && workload != CREDIT_WL_PEARSON_BACKWARD) ? 3 : 4;
        int c = o.cluster_size;
        if (c == 0) {
            const int first = o.variant == CREDIT_VARIANT_CLUSTER_SMEM ? 2 : 1;
            int with3 = 0, with4 = 0;
            for (int t = first; t <= max_cluster; t *= 2) {
                if (with3 == 0 && ws_fits(t, 3)) with3 = t;
                if (with4 == 0 && ws_fits(t, wanted_stages)) with4 = t;
            }
            c = with4 != 0 ? with4 : with3;
            if (c == 16 && with3 != 0 && with3 <= 8) c = with3;
            if (c == 0) c = 2 * max_cluster;   // nothing fits: fall through to the other kernels
        }
        if (c <= max_cluster && ws_fits(c, 3)) {
            p->cluster_size = c;
            p->slice_elems = round_up((s.cols + c - 1) / c, 64);
            const int nvec = p->slice_elems / s.vec_elems;
            int vpt = 1;
            while (vpt * out_threads < nvec && !row_op) vpt *= 2;
            if (row_op) vpt = std::max(1, (nvec + out_threads - 1) / out_threads);
            const int stage_bytes = stage_bytes_for(c);
            // Ring depth: up to 8 stages. Where six or more fit half of the SM's shared memory the
            // ring stays inside that half, so that two CTAs share an SM (short slices: 2 x 8 stages
            // measured faster than 1 x 12 or 1 x 16); otherwise whatever fits, up to 8.
            auto most_stages = [&](int limit) { return std::min(8, (limit - kWsControlBytes) / std::max(stage_bytes, 1)); };
            const int half_smem = (max_smem - 2048) / 2;
            int stages = o.stages ? o.stages
                         : row_op ? 6   // as swept for the reference workloads
                                  : (most_stages(half_smem) >= 6 ? most_stages(half_smem) : most_stages(max_smem));
            while (stages > 3 && kWsControlBytes + stages * stage_bytes > max_smem) --stages;
            p->threads = threads;
            p->vectors_per_thread = vpt;
            p->full_tiles = (vpt * out_threads == nvec && 1ll * p->slice_elems * c == s.cols) ? 1 : 0;
            p->schedule = CREDIT_SCHEDULE_PERSISTENT;
            p->stages = stages;
            p->smem_bytes = kWsControlBytes + stages * stage_bytes;
            return CREDIT_OK;
        }
        if (ws_threads)
            return fail(CREDIT_ERR_UNSUPPORTED,
                        "the warp-specialised kernel needs slices of at most %d elements and three stages of %d B",
                        max_slice, stage_bytes_for(std::max(o.cluster_size, 1)));
    } else if (ws_threads) {
        return fail(CREDIT_ERR_UNSUPPORTED,
                    "threads = %d selects a warp-specialised kernel: 16-byte aligned rows, persistent schedule, at "
                    "least three stages (LayerNorm backward with recomputed statistics and the reference-sweep "
                    "workloads: 352 only)",
                    o.threads);
    }
    if (o.stages > kMaxStages)
        return fail(CREDIT_ERR_UNSUPPORTED, "only the warp-specialised kernels take rings deeper than %d stages", kMaxStages);
    int cluster = o.cluster_size;
    if (cluster == 0) {
        // Smallest cluster whose slice fits the stage budget and, for aligned rows,
        // the register path at 512 threads.
        cluster = o.variant == CREDIT_VARIANT_CLUSTER_SMEM ? 2 : 1;
        // LayerNorm backward without column sums: measured best (fp32 and bf16, N = 16K ... 128K) is
        // the smallest cluster whose slice fits 256 threads x 32 elements, read twice from its stage
        const bool two_reads = nin == 2 && !grads && p->aligned && !(o.flags & CREDIT_FLAG_NO_REGISTER_PATH);
        auto fits = [&](int c) {
            if (stage_bytes_for(c) > (two_reads ? 2 : 1) * kAutoStageBytes) return false;
            if (!p->aligned || (o.flags & CREDIT_FLAG_NO_REGISTER_PATH)) return true;
            const int nvec = round_up((s.cols + c - 1) / c, 64) / s.vec_elems;
            const int threads = o.threads ? o.threads : (two_reads ? 256 : 512);
            return nvec <= threads * (max_elems_per_thread(workload, grads) / s.vec_elems);
        };
        while (cluster < max_cluster && !fits(cluster)) cluster *= 2;
    }
    if (cluster > max_cluster)
        return fail(CREDIT_ERR_UNSUPPORTED, "cluster size %d not available on this device", cluster);
    p->cluster_size = cluster;
    p->slice_elems = round_up((s.cols + cluster - 1) / cluster, 64);
    const int stage_bytes = stage_bytes_for(cluster);
    if (kControlBytes + stage_bytes > max_smem)
        return fail(CREDIT_ERR_UNSUPPORTED,
                    "a slice of %d B per CTA (cluster size %d) exceeds %d B of shared memory",
                    stage_bytes, cluster, max_smem);

    p->threads = o.threads ? o.threads : 256;
    p->vectors_per_thread = 0;
    if (p->aligned && !(o.flags & CREDIT_FLAG_NO_REGISTER_PATH)) {
        // Register path: the slice must fit `vpt` 16-byte vectors per thread, with
        // vpt bounded by the registers the workload keeps per element.
        const int max_vpt = max_elems_per_thread(workload, grads) / s.vec_elems;
        const int nvec = p->slice_elems / s.vec_elems;
        int threads = o.threads;
        if (threads == 0) threads = (nvec > 256 * max_vpt || (lock_step_default && nvec >= 512)) ? 512 : 256;
        int vpt = 1;
        while (vpt * threads < nvec) vpt *= 2;
        // slices read twice from their stage need three stages; a caller who asks for fewer gets
        // the shared-memory kernels instead
        const bool two_reads = inputs_staged(workload) == 2 && vpt * s.vec_elems > 16;
        const bool three_fit = kControlBytes + 3 * stage_bytes <= max_smem;
        if (vpt <= max_vpt && !(two_reads && (o.stages == 1 || o.stages == 2 || !three_fit))) {
            p->threads = threads;
            p->vectors_per_thread = vpt;
            p->full_tiles = (vpt * threads == nvec && 1ll * p->slice_elems * cluster == s.cols) ? 1 : 0;
        }
    }

    p->schedule = o.schedule;
    if (p->schedule == CREDIT_SCHEDULE_AUTO)
        p->schedule = p->aligned ? CREDIT_SCHEDULE_PERSISTENT : CREDIT_SCHEDULE_ROW_PER_CLUSTER;
    if (grads && p->vectors_per_thread > 0 && p->schedule != CREDIT_SCHEDULE_PERSISTENT)
        return fail(CREDIT_ERR_INVALID_ARGUMENT,
                    "column sums are accumulated by persistent clusters; schedule must be persistent");

    const int control_bytes = kControlBytes;
    int stages = o.stages;
    if (!p->aligned || p->schedule == CREDIT_SCHEDULE_ROW_PER_CLUSTER) {
        stages = 1;
    } else if (stages == 0) {
        // measured on B200: three stages, except two where two fp32 arrays (or two 16-bit arrays
        // without the column sums) are staged
        stages = p->vectors_per_thread > 0 ? ((nin == 2 && !(grads && s.elem_bytes == 2)) ? 2 : 3)
                                           : std::max(1, std::min(4, kAutoRingBytes / stage_bytes));
        while (stages > 1 && control_bytes + stages * stage_bytes > max_smem) --stages;
    }
    const bool backward = workload == CREDIT_WL_LAYERNORM_BACKWARD || workload == CREDIT_WL_LAYERNORM_BACKWARD_STATS;
    if (backward && p->vectors_per_thread * s.vec_elems > 16 && stages < 3) stages = 3;
    p->stages = stages;
    p->smem_bytes = control_bytes + stages * stage_bytes;
    if (p->smem_bytes > max_smem)
        return fail(CREDIT_ERR_UNSUPPORTED, "%d stages of %d B exceed %d B of shared memory", stages,
                    stage_bytes, max_smem);
    return CREDIT_OK;
}

// Grid size; needs the device for the occupancy query when persistent.
int plan_grid(int device, const void* func, const Shape& s, credit_plan_info* p) {
    int clusters = s.rows;
    if (p->schedule == CREDIT_SCHEDULE_PERSISTENT && s.rows > 0) {
        int resident = 0;
        int rc = max_active_clusters(device, func, p->cluster_size, p->smem_bytes, p->threads,
                                     &resident);
        if (rc != CREDIT_OK) return rc;
        clusters = std::min(s.rows, resident);
    }
    if (1ll * clusters * p->cluster_size > 0x7fffffffll)
        return fail(CREDIT_ERR_UNSUPPORTED, "%d rows x cluster size %d exceeds the grid limit", clusters,
                    p->cluster_size);
    p->num_clusters = clusters;
    p->grid_ctas = clusters * p->cluster_size;
    return CREDIT_OK;
}

int colsum_blocks(int rows) {
    return std::max(1, std::min((rows + kColsumRowsPerBlock - 1) / kColsumRowsPerBlock, kColsumMaxBlocks));
}

size_t grads_workspace_bytes(const Shape& s, const credit_plan_info& p) {
    const size_t partials = p.vectors_per_thread > 0 ? static_cast<size_t>(p.num_clusters)
                                                     : static_cast<size_t>(colsum_blocks(s.rows));
    return partials * 2 * static_cast<size_t>(s.cols) * sizeof(float);
}

bool is_ws_plan_threads(int threads) { return threads == kWsThreadsPerCta || threads == kWsThreadsPerCtaWide; }
bool is_ws_plan(const credit_plan_info& p) { return is_ws_plan_threads(p.threads); }

struct Resolved {
    DeviceState* dev = nullptr;
    int device = 0;
    Shape shape{};
    credit_plan_info plan{};
    const void* func = nullptr;
};

// ---------------------------------------------------------------------------
// automatic cluster size: the B200 row-period model (same constants and formula as
// credit_b200/cost_model.py: predict_cluster_ms), evaluated over the admissible sizes
//   time(P) = sqrt(hbm^2 + latency^2),  latency = ceil(rows / resident(P)) * row_period(P)
// with resident(P) from the driver's occupancy query. Calibrated on B200 (copy ceiling
// 6538.6 GB/s, 1.93 GHz under these kernels, exchange cycles from primitive_benchmark).
// ---------------------------------------------------------------------------
// The copy ceiling the planner's models divide by: 6538.6 GB/s was measured on B200; a host that
// has measured its own device sets CREDIT_HBM_GBPS (read once).
double calibrated_hbm_gbps() {
    static const double value = [] {
        const char* text = std::getenv("CREDIT_HBM_GBPS");
        const double v = text != nullptr ? std::atof(text) : 0.0;
        return v > 100.0 ? v : 6538.6;
    }();
    return value;
}

double compulsory_bytes(int workload, const Shape& s, bool grads) {
    const double rc = static_cast<double>(s.rows) * s.cols, e = s.elem_bytes;
    switch (workload) {
        case CREDIT_WL_RMSNORM_FORWARD: return 2 * rc * e + s.cols * 4.0;
        case CREDIT_WL_LAYERNORM_FORWARD: return 2 * rc * e + 2 * s.cols * 4.0 + 2 * s.rows * 4.0;
        case CREDIT_WL_LAYERNORM_BACKWARD: return 3 * rc * e + s.cols * 4.0;
        default: return 3 * rc * e + 2 * s.rows * 4.0 + (grads ? 3 : 1) * s.cols * 4.0;
    }
}

double predicted_ms(int workload, const Shape& s, const credit_plan_info& p, bool grads) {
    const double hbm_ms = compulsory_bytes(workload, s, grads) / (calibrated_hbm_gbps() * 1.0e6);
    if (p.vectors_per_thread == 0) return hbm_ms / 0.5;   // shared-memory re-read kernels
    static const double kExchange[5] = {150.0, 315.0, 322.0, 351.0, 420.0};   // P = 1, 2, 4, 8, 16
    int log2p = 0;
    while ((1 << log2p) < p.cluster_size) ++log2p;
    const int stages = workload == CREDIT_WL_LAYERNORM_BACKWARD ? 2 : 1;
    const double elems = std::ceil(static_cast<double>(s.cols) / p.cluster_size / p.threads);
    const double chain = 1600.0 + (stages - 1) * 200.0 + stages * (20.0 * (p.threads / 32) + kExchange[log2p]) +
                         4.0 * elems;
    const double rows_per_cluster = std::ceil(static_cast<double>(s.rows) / std::max(p.num_clusters, 1));
    const double latency_ms = rows_per_cluster * chain / (1.93 * 1.0e6);
    return std::sqrt(hbm_ms * hbm_ms + latency_ms * latency_ms);
}

// The warp-specialised kernels: a cluster's row period is the larger of its CTAs' share of the HBM
// bandwidth (the SMs the co-resident clusters cover share the copy ceiling; one SM pulls at most
// about 58 GB/s through bulk copies) and the output warps' issue time for one row (a fixed part per
// row plus a part per row element a thread owns); a kernel costs rows-per-cluster + 3 such periods
// (ring fill, the rows between the two passes, the last cluster's extra row). Constants measured on
// B200 with 8 output warps: fixed part 550 cycles, 28 cycles per element forward, 36 backward and 40 backward with column sums,
// 12 % more with a ring too short to run the passes two rows apart, 15 % more in clusters of 16
// (7 of them are co-resident, and they ran that much slower than the terms above say), and a row
// period of at least 1.5 us / (ring stages that are loads in flight).
double predicted_ws_ms(int workload, const Shape& s, const credit_plan_info& p, bool grads) {
    const int nin = inputs_staged(workload);
    double nout = 1.0;   // output arrays of the element type written per row
    if (workload == CREDIT_WL_PEARSON_BACKWARD || workload == CREDIT_WL_LARS_MOMENTUM) nout = 2.0;
    if (workload == CREDIT_WL_ROWWISE_QUANT) nout = 0.25;
    const double bytes_per_cta_row = (nin + nout) * p.slice_elems * s.elem_bytes;
    const double sms = static_cast<double>(std::max(p.num_clusters, 1)) * p.cluster_size;
    const double per_sm_gbps = std::min(calibrated_hbm_gbps() / sms, 58.0);
    const double hbm_us = bytes_per_cta_row / (per_sm_gbps * 1.0e3);
    const int out_threads = p.threads - 96;
    const double elems = std::ceil(static_cast<double>(p.slice_elems) / out_threads);
    const double per_elem = grads ? 40.0 : (is_row_op(workload) ? 12.0 * (nin + nout) : (nin == 2 ? 36.0 : 28.0));
    const double issue_us = (550.0 + per_elem * elems) / 1930.0;
    // loads in flight: three stages (two with a short ring) sit between the passes, the others are
    // requests that take about 1.5 us to land, one row each
    const int in_flight = std::max(1, p.stages - (p.stages >= 5 ? 3 : 2));
    double row_us = std::max(std::max(hbm_us, issue_us), 1.5 / in_flight);
    if (p.stages < 5) row_us *= 1.12;
    if (p.cluster_size >= 16) row_us *= 1.15;
    const double rows_per_cluster = std::ceil(static_cast<double>(s.rows) / std::max(p.num_clusters, 1));
    return row_us * (rows_per_cluster + 3.0) * 1.0e-3;
}

// (device, workload, rows, cols, dtype, aligned, grads, variant, threads, stages, flags) -> chosen size
std::map<std::tuple<int, int, int, int, int, bool, bool, int, int, int, int>, int> g_auto_cluster;

// Fills o->cluster_size for the staged workloads when the caller left it at 0. On any failure the
// planner's own rule (smallest cluster that fits) stays in charge.
void choose_cluster_by_model(int device, const DeviceState& dev, int workload, const Shape& s, int dtype,
                             bool pointers_aligned, bool grads, credit_launch_opts* o) {
    if (o->cluster_size != 0 || s.rows == 0 || !dev.info.cluster_launch) return;
    if (workload == CREDIT_WL_ROW_REDUCE) return;
    // fp32 RMSNorm: plan_static's smallest-fit rule for the lock-step kernel (see there)
    if (workload == CREDIT_WL_RMSNORM_FORWARD && dtype == CREDIT_F32 && o->threads == 0) return;
    // Reference-sweep workloads: plan_static's measured rule (the smallest cluster whose ring is deep
    // enough) decides for both of their kernel families.
    if (is_row_op(workload)) return;
    if (o->variant == CREDIT_VARIANT_BLOCK_READ || o->variant == CREDIT_VARIANT_BLOCK_SMEM) return;
    if (o->schedule == CREDIT_SCHEDULE_ROW_PER_CLUSTER) return;
    {
        // the warp-specialised kernels choose by plan_static's measured rule, not by the model
        credit_plan_info plan;
        if (plan_static(workload, s, dtype, *o, pointers_aligned, grads, dev.info, &plan) == CREDIT_OK && is_ws_plan(plan)) return;
        t_last_error[0] = '\0';
    }
    const auto key = std::make_tuple(device, workload, s.rows, s.cols, dtype, pointers_aligned, grads, o->variant,
                                     o->threads, o->stages, o->flags);
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        auto it = g_auto_cluster.find(key);
        if (it != g_auto_cluster.end()) {
            o->cluster_size = it->second;
            return;
        }
    }
    // two passes, as cost_model.best_cluster_size does: the fastest prediction, then the smallest
    // cluster within 1 % of it
    int sizes[8];
    double times[8];
    int candidates = 0;
    for (int c = o->variant == CREDIT_VARIANT_CLUSTER_SMEM ? 2 : 1; c <= kMaxClusterSize; c *= 2) {
        credit_launch_opts trial = *o;
        trial.cluster_size = c;
        credit_plan_info plan;
        if (plan_static(workload, s, dtype, trial, pointers_aligned, grads, dev.info, &plan) != CREDIT_OK) continue;
        if (plan.schedule != CREDIT_SCHEDULE_PERSISTENT) continue;
        // never below the smallest cluster whose stage fits the budget (larger stages measured
        // slower with inputs that are not in L2); the model decides whether to go above it
        const bool two_reads = inputs_staged(workload) == 2 && !grads;
        if (!is_ws_plan(plan) && c < kMaxClusterSize &&
            inputs_staged(workload) * plan.slice_elems * s.elem_bytes > (two_reads ? 2 : 1) * kAutoStageBytes)
            continue;
        const void* func = workload_func(workload, dtype, plan, grads);
        if (func == nullptr || prepare_function(device, func, dev.info.max_dynamic_smem_per_block) != CREDIT_OK) continue;
        if (plan_grid(device, func, s, &plan) != CREDIT_OK) continue;
        sizes[candidates] = c;
        times[candidates] = is_ws_plan(plan) ? predicted_ws_ms(workload, s, plan, grads) : predicted_ms(workload, s, plan, grads);
        ++candidates;
    }
    int best = 0;
    if (candidates > 0) {
        const double fastest = *std::min_element(times, times + candidates);
        for (int i = 0; i < candidates && best == 0; ++i)
            if (times[i] <= fastest * 1.01) best = sizes[i];
    }
    t_last_error[0] = '\0';   // failed trials are not errors of this call
    if (best == 0) return;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        g_auto_cluster[key] = best;
    }
    o->cluster_size = best;
}

int resolve(int workload, int64_t rows, int64_t cols, int dtype, const credit_launch_opts* opts,
            bool pointers_aligned, bool want_grads, Resolved* r) {
    int rc = check_shape(rows, cols, dtype, &r->shape);
    if (rc != CREDIT_OK) return rc;
    credit_launch_opts o;
    rc = check_opts(opts, &o);
    if (rc != CREDIT_OK) return rc;
    CREDIT_CUDA_TRY(cudaGetDevice(&r->device));
    rc = load_device(r->device, &r->dev);
    if (rc != CREDIT_OK) return rc;
    if (workload >= CREDIT_WL_RMSNORM_FORWARD && workload <= CREDIT_WL_ROWWISE_QUANT)
        choose_cluster_by_model(r->device, *r->dev, workload, r->shape, dtype, pointers_aligned, want_grads, &o);
    rc = plan_static(workload, r->shape, dtype, o, pointers_aligned, want_grads, r->dev->info, &r->plan);
    if (rc != CREDIT_OK) return rc;
    r->func = workload_func(workload, dtype, r->plan, want_grads);
    if (r->func == nullptr) return fail(CREDIT_ERR_INVALID_ARGUMENT, "no kernel for workload %d", workload);
    rc = prepare_function(r->device, r->func, r->dev->info.max_dynamic_smem_per_block);
    if (rc != CREDIT_OK) return rc;
    rc = plan_grid(r->device, r->func, r->shape, &r->plan);
    if (rc != CREDIT_OK) return rc;
    if (workload == CREDIT_WL_LAYERNORM_BACKWARD_STATS && want_grads) {
        r->plan.workspace_bytes = grads_workspace_bytes(r->shape, r->plan);
        r->plan.kernel_launches = r->plan.vectors_per_thread > 0 ? 2 : 3;  // (+ column sums) + finish
    }
    return CREDIT_OK;
}

Launch make_launch(const Resolved& r, void* stream) {
    Launch l;
    l.func = r.func;
    l.grid = r.plan.grid_ctas;
    l.threads = r.plan.threads;
    l.cluster = r.plan.cluster_size;
    l.smem = r.plan.smem_bytes;
    l.stream = static_cast<cudaStream_t>(stream);
    return l;
}

StagedArgs staged_args(const Resolved& r) {
    StagedArgs a;
    a.rows = r.shape.rows;
    a.cols = r.shape.cols;
    a.slice_elems = r.plan.slice_elems;
    a.num_clusters = r.plan.num_clusters;
    a.stages = r.plan.stages;
    a.status = r.dev->status_ptr;
    return a;
}

}  // namespace
}  // namespace credit

using namespace credit;

extern "C" {

const char* credit_last_error(void) { return t_last_error; }

int credit_query_device(int device, credit_device_info* info) {
    if (info == nullptr) return fail(CREDIT_ERR_INVALID_ARGUMENT, "info is NULL");
    if (device < 0) CREDIT_CUDA_TRY(cudaGetDevice(&device));
    DeviceState* st = nullptr;
    int rc = load_device(device, &st);
    if (rc != CREDIT_OK) return rc;
    *info = st->info;
    return CREDIT_OK;
}

int credit_device_status(int* status_out, int reset) {
    DeviceState* st = nullptr;
    int rc = current_device_state(&st);
    if (rc != CREDIT_OK) return rc;
    CREDIT_CUDA_TRY(cudaDeviceSynchronize());
    int word = 0;
    CREDIT_CUDA_TRY(cudaMemcpy(&word, st->status_ptr, sizeof(int), cudaMemcpyDeviceToHost));
    if (reset && word != 0) CREDIT_CUDA_TRY(cudaMemset(st->status_ptr, 0, sizeof(int)));
    if (status_out != nullptr) *status_out = word;
    if (word != 0)
        return fail(CREDIT_ERR_DEVICE_STATUS, "device status word = %d (1: wait timed out, 2: bad geometry)",
                    word);
    return CREDIT_OK;
}

int credit_plan(int workload, int64_t rows, int64_t cols, int dtype, const credit_launch_opts* opts,
                credit_plan_info* plan) {
    if (plan == nullptr) return fail(CREDIT_ERR_INVALID_ARGUMENT, "plan is NULL");
    Resolved r;
    int rc = resolve(workload, rows, cols, dtype, opts, true, true, &r);
    if (rc != CREDIT_OK) return rc;
    *plan = r.plan;
    return CREDIT_OK;
}

int credit_rmsnorm_forward(const void* x, const float* gamma, void* y, int64_t rows, int64_t cols,
                           float eps, int dtype, const credit_launch_opts* opts, void* stream) {
    if (rows != 0 && (x == nullptr || gamma == nullptr || y == nullptr))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "x, gamma and y must not be NULL");
    Resolved r;
    int rc = resolve(CREDIT_WL_RMSNORM_FORWARD, rows, cols, dtype, opts,
                     aligned16(x) && aligned16(gamma) && aligned16(y), false, &r);
    if (rc != CREDIT_OK) return rc;
    if (r.shape.rows == 0) return CREDIT_OK;
    if (r.plan.variant == CREDIT_VARIANT_BLOCK_READ) {
        void* args[] = {&x, &gamma, &y, &eps, &r.shape.rows, &r.shape.cols};
        return launch_cluster_kernel(make_launch(r, stream), args);
    }
    StagedArgs a = staged_args(r);
    if (is_ws_plan(r.plan)) {
        NormParams prm{};
        prm.x = x;
        prm.gamma = gamma;
        prm.y = y;
        prm.eps = eps;
        void* args[] = {&prm, &a};
        return launch_cluster_kernel(make_launch(r, stream), args);
    }
    void* args[] = {&x, &gamma, &y, &eps, &a};
    return launch_cluster_kernel(make_launch(r, stream), args);
}

int credit_row_reduce(const float* x, float* out_sum, float* out_max, int64_t* out_argmax,
                      int64_t rows, int64_t cols, const credit_launch_opts* opts, void* stream) {
    if (rows != 0 && (x == nullptr || out_sum == nullptr || out_max == nullptr || out_argmax == nullptr))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "x and the three outputs must not be NULL");
    Resolved r;
    int rc = resolve(CREDIT_WL_ROW_REDUCE, rows, cols, CREDIT_F32, opts, aligned16(x), false, &r);
    if (rc != CREDIT_OK) return rc;
    if (r.shape.rows == 0) return CREDIT_OK;
    ReduceArgs a;
    a.rows = r.shape.rows;
    a.cols = r.shape.cols;
    a.slice_elems = r.plan.slice_elems;
    a.num_clusters = r.plan.num_clusters;
    a.stages = r.plan.stages;
    a.chunk_elems = r.plan.chunk_elems;
    a.status = r.dev->status_ptr;
    long long* argmax = reinterpret_cast<long long*>(out_argmax);
    void* args[] = {&x, &out_sum, &out_max, &argmax, &a};
    return launch_cluster_kernel(make_launch(r, stream), args);
}

int credit_layernorm_forward(const void* x, const float* gamma, const float* beta, void* y,
                             float* mean, float* rstd, int64_t rows, int64_t cols, float eps,
                             int dtype, const credit_launch_opts* opts, void* stream) {
    if (rows != 0 && (x == nullptr || gamma == nullptr || beta == nullptr || y == nullptr ||
                      mean == nullptr || rstd == nullptr))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "x, gamma, beta, y, mean and rstd must not be NULL");
    Resolved r;
    int rc = resolve(CREDIT_WL_LAYERNORM_FORWARD, rows, cols, dtype, opts,
                     aligned16(x) && aligned16(gamma) && aligned16(beta) && aligned16(y), false, &r);
    if (rc != CREDIT_OK) return rc;
    if (r.shape.rows == 0) return CREDIT_OK;
    if (r.plan.variant == CREDIT_VARIANT_BLOCK_READ) {
        void* args[] = {&x, &gamma, &beta, &y, &mean, &rstd, &eps, &r.shape.rows, &r.shape.cols};
        return launch_cluster_kernel(make_launch(r, stream), args);
    }
    StagedArgs a = staged_args(r);
    if (is_ws_plan(r.plan)) {
        NormParams prm{};
        prm.x = x;
        prm.gamma = gamma;
        prm.beta = beta;
        prm.y = y;
        prm.mean_out = mean;
        prm.rstd_out = rstd;
        prm.eps = eps;
        void* args[] = {&prm, &a};
        return launch_cluster_kernel(make_launch(r, stream), args);
    }
    void* args[] = {&x, &gamma, &beta, &y, &mean, &rstd, &eps, &a};
    return launch_cluster_kernel(make_launch(r, stream), args);
}

int credit_layernorm_backward(const void* x, const void* dy, const float* gamma, void* dx,
                              int64_t rows, int64_t cols, float eps, int dtype,
                              const credit_launch_opts* opts, void* stream) {
    if (rows != 0 && (x == nullptr || dy == nullptr || gamma == nullptr || dx == nullptr))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "x, dy, gamma and dx must not be NULL");
    Resolved r;
    int rc = resolve(CREDIT_WL_LAYERNORM_BACKWARD, rows, cols, dtype, opts,
                     aligned16(x) && aligned16(dy) && aligned16(gamma) && aligned16(dx), false, &r);
    if (rc != CREDIT_OK) return rc;
    if (r.shape.rows == 0) return CREDIT_OK;
    const float* no_stats = nullptr;
    float* no_partials = nullptr;
    if (r.plan.variant == CREDIT_VARIANT_BLOCK_READ) {
        void* args[] = {&x, &dy, &gamma, &no_stats, &no_stats, &dx, &eps, &r.shape.rows, &r.shape.cols};
        return launch_cluster_kernel(make_launch(r, stream), args);
    }
    StagedArgs a = staged_args(r);
    if (is_ws_plan(r.plan)) {
        NormParams prm{};
        prm.x = x;
        prm.dy = dy;
        prm.gamma = gamma;
        prm.y = dx;
        prm.eps = eps;
        void* args[] = {&prm, &a};
        return launch_cluster_kernel(make_launch(r, stream), args);
    }
    if (r.plan.vectors_per_thread > 0) {
        void* args[] = {&x, &dy, &gamma, &no_stats, &no_stats, &dx, &no_partials, &eps, &a};
        return launch_cluster_kernel(make_launch(r, stream), args);
    }
    void* args[] = {&x, &dy, &gamma, &no_stats, &no_stats, &dx, &eps, &a};
    return launch_cluster_kernel(make_launch(r, stream), args);
}

size_t credit_layernorm_backward_stats_workspace_bytes(int64_t rows, int64_t cols, int dtype,
                                                       const credit_launch_opts* opts) {
    Resolved r;
    int rc = resolve(CREDIT_WL_LAYERNORM_BACKWARD_STATS, rows, cols, dtype, opts, true, true, &r);
    if (rc != CREDIT_OK) return 0;
    // Unaligned base pointers fall back to the column-sum kernel, whose partial
    // count differs: report the larger of the two so either path fits.
    Shape s = r.shape;
    credit_plan_info fallback = r.plan;
    fallback.vectors_per_thread = 0;
    return std::max(r.plan.workspace_bytes, grads_workspace_bytes(s, fallback));
}

int credit_layernorm_backward_stats(const void* x, const void* dy, const float* gamma,
                                    const float* mean, const float* rstd, void* dx, float* dgamma,
                                    float* dbeta, int64_t rows, int64_t cols, int dtype,
                                    const credit_launch_opts* opts, void* workspace,
                                    size_t workspace_bytes, void* stream) {
    if (rows != 0 && (x == nullptr || dy == nullptr || gamma == nullptr || mean == nullptr ||
                      rstd == nullptr || dx == nullptr))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "x, dy, gamma, mean, rstd and dx must not be NULL");
    if ((dgamma == nullptr) != (dbeta == nullptr))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "dgamma and dbeta must both be given or both be NULL");
    const bool want_grads = dgamma != nullptr;
    Resolved r;
    int rc = resolve(CREDIT_WL_LAYERNORM_BACKWARD_STATS, rows, cols, dtype, opts,
                     aligned16(x) && aligned16(dy) && aligned16(gamma) && aligned16(dx) &&
                         (!want_grads || aligned16(workspace)),
                     want_grads, &r);
    if (rc != CREDIT_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (want_grads) {
        if (workspace == nullptr || workspace_bytes < r.plan.workspace_bytes)
            return fail(CREDIT_ERR_WORKSPACE, "workspace of %zu B given, %zu B needed", workspace_bytes,
                        r.plan.workspace_bytes);
    }
    if (r.shape.rows == 0) {
        if (want_grads) {
            CREDIT_CUDA_TRY(cudaMemsetAsync(dgamma, 0, sizeof(float) * r.shape.cols, s));
            CREDIT_CUDA_TRY(cudaMemsetAsync(dbeta, 0, sizeof(float) * r.shape.cols, s));
        }
        return CREDIT_OK;
    }
    StagedArgs a = staged_args(r);
    float* partials = static_cast<float*>(workspace);
    float eps = 0.0f;
    if (r.plan.variant == CREDIT_VARIANT_BLOCK_READ) {
        void* args[] = {&x, &dy, &gamma, &mean, &rstd, &dx, &eps, &r.shape.rows, &r.shape.cols};
        rc = launch_cluster_kernel(make_launch(r, stream), args);
    } else if (is_ws_plan(r.plan)) {
        NormParams prm{};
        prm.x = x;
        prm.dy = dy;
        prm.gamma = gamma;
        prm.mean_in = mean;
        prm.rstd_in = rstd;
        prm.y = dx;
        prm.partials = partials;
        void* args[] = {&prm, &a};
        rc = launch_cluster_kernel(make_launch(r, stream), args);
    } else if (r.plan.vectors_per_thread > 0) {
        void* args[] = {&x, &dy, &gamma, &mean, &rstd, &dx, &partials, &eps, &a};
        rc = launch_cluster_kernel(make_launch(r, stream), args);
    } else {
        void* args[] = {&x, &dy, &gamma, &mean, &rstd, &dx, &eps, &a};
        rc = launch_cluster_kernel(make_launch(r, stream), args);
    }
    if (rc != CREDIT_OK) return rc;
    if (!want_grads) return CREDIT_OK;

    int num_partials = r.plan.num_clusters;
    if (r.plan.vectors_per_thread == 0) {
        num_partials = colsum_blocks(r.shape.rows);
        CREDIT_CUDA_TRY(launch_layernorm_bwd_colsum(dtype, x, dy, mean, rstd, partials, r.shape.rows,
                                                    r.shape.cols, num_partials, s));
    }
    CREDIT_CUDA_TRY(launch_layernorm_bwd_finish(partials, dgamma, dbeta, r.shape.cols, num_partials, s));
    return CREDIT_OK;
}

// ---------------------------------------------------------------------------
// reference-sweep workloads
// ---------------------------------------------------------------------------
int credit_row_op(int workload, const float* in0, const float* in1, const float* in2, const float* row_in,
                  void* out0, void* out1, float* row_out, int64_t rows, int64_t cols,
                  const credit_launch_opts* opts, void* stream) {
    if (!is_row_op(workload))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "credit_row_op: workload %d is not one of the reference-sweep workloads",
                    workload);
    const int nin = inputs_staged(workload);
    const bool two_out = workload == CREDIT_WL_PEARSON_BACKWARD || workload == CREDIT_WL_LARS_MOMENTUM;
    const bool needs_row_in = workload == CREDIT_WL_PEARSON_BACKWARD;
    const bool needs_row_out = workload == CREDIT_WL_ROWWISE_QUANT;
    const float* ins[3] = {in0, in1, in2};
    for (int n = 0; n < 3; ++n) {
        if (rows != 0 && (n < nin) != (ins[n] != nullptr))
            return fail(CREDIT_ERR_INVALID_ARGUMENT, "credit_row_op: workload %d takes %d input arrays (in%d is %s)",
                        workload, nin, n, ins[n] ? "given" : "NULL");
    }
    if (rows != 0 && (out0 == nullptr || two_out != (out1 != nullptr) || needs_row_in != (row_in != nullptr) ||
                      needs_row_out != (row_out != nullptr)))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "credit_row_op: wrong set of output / per-row pointers for workload %d",
                    workload);
    const bool al = aligned16(in0) && aligned16(in1) && aligned16(in2) && aligned16(out0) && aligned16(out1);
    Resolved r;
    int rc = resolve(workload, rows, cols, CREDIT_F32, opts, al, false, &r);
    if (rc != CREDIT_OK) return rc;
    if (r.shape.rows == 0) return CREDIT_OK;
    if (is_ws_plan(r.plan)) {
        NormParams prm{};
        prm.x = in0;
        prm.dy = in1;
        prm.in2 = in2;
        prm.row_in = row_in;
        prm.y = out0;
        prm.out1 = out1;
        prm.row_out = row_out;
        StagedArgs a = staged_args(r);
        void* args[] = {&prm, &a};
        return launch_cluster_kernel(make_launch(r, stream), args);
    }
    RowOpArgs io;
    for (int n = 0; n < 3; ++n) io.in[n] = ins[n];
    io.row_in = row_in;
    io.out[0] = out0;
    io.out[1] = out1;
    io.row_out = row_out;
    StagedArgs a = staged_args(r);
    void* args[] = {&io, &a};
    return launch_cluster_kernel(make_launch(r, stream), args);
}

// ---------------------------------------------------------------------------
// fused FFN
// ---------------------------------------------------------------------------
int credit_ffn_pack_weight(const void* w, void* packed, int64_t k, int64_t n, void* stream) {
    if (w == nullptr || packed == nullptr)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "w and packed must not be NULL");
    if (k <= 0 || n <= 0 || k > (1 << 24) || n > (1 << 24))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "k=%lld, n=%lld out of range", static_cast<long long>(k),
                    static_cast<long long>(n));
    CREDIT_CUDA_TRY(launch_ffn_pack_weight(w, packed, static_cast<int>(k), static_cast<int>(n),
                                           static_cast<cudaStream_t>(stream)));
    return CREDIT_OK;
}

size_t credit_ffn_workspace_bytes(int64_t m, int64_t d, int64_t h) {
    if (ffn_check_shape(m, d, h) != nullptr) return 0;
    // the hidden activations (bf16), then the scratch of the second GEMM
    return static_cast<size_t>(m) * static_cast<size_t>(h) * 2 + ffn_scratch_bytes(d);
}

int credit_ffn_forward(const void* x, const void* w1_packed, const void* w2_packed, const float* gamma,
                       void* y, int64_t m, int64_t d, int64_t h, float eps, void* workspace,
                       size_t workspace_bytes, void* stream) {
    const char* why = ffn_check_shape(m, d, h);
    if (why != nullptr) return fail(CREDIT_ERR_UNSUPPORTED, "ffn shape m=%lld d=%lld h=%lld: %s",
                                    static_cast<long long>(m), static_cast<long long>(d),
                                    static_cast<long long>(h), why);
    if (x == nullptr || w1_packed == nullptr || w2_packed == nullptr || gamma == nullptr || y == nullptr)
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "x, the packed weights, gamma and y must not be NULL");
    if (!aligned16(x) || !aligned16(w1_packed) || !aligned16(w2_packed) || !aligned16(gamma) || !aligned16(y) ||
        !aligned16(workspace))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "all ffn pointers must be 16-byte aligned");
    const size_t need = credit_ffn_workspace_bytes(m, d, h);
    if (workspace == nullptr || workspace_bytes < need)
        return fail(CREDIT_ERR_WORKSPACE, "workspace of %zu B given, %zu B needed", workspace_bytes, need);
    DeviceState* st = nullptr;
    int rc = current_device_state(&st);
    if (rc != CREDIT_OK) return rc;
    if (st->info.sm_major != 10)
        return fail(CREDIT_ERR_UNSUPPORTED, "the FFN kernels need an sm_100 device (tcgen05)");
    bool bad_map = false;
    void* scratch = static_cast<unsigned char*>(workspace) + static_cast<size_t>(m) * static_cast<size_t>(h) * 2;
    cudaError_t err = launch_ffn_forward(x, w1_packed, w2_packed, gamma, y, workspace, scratch, static_cast<int>(m),
                                         static_cast<int>(d), static_cast<int>(h), eps, st->status_ptr,
                                         static_cast<cudaStream_t>(stream), &bad_map);
    if (bad_map) return fail(CREDIT_ERR_CUDA, "could not encode a TMA tensor map for the FFN operands");
    if (err != cudaSuccess) return cuda_fail(err, "ffn launch");
    return CREDIT_OK;
}

// ---------------------------------------------------------------------------
// LayerNorm backward with library-owned scratch
// ---------------------------------------------------------------------------
namespace {

// Scratch for the per-cluster partial column sums of
// credit_layernorm_backward_stats_static. It is part of the loaded library image:
// every GPU that loads the library holds these 16 MiB until the process exits.
constexpr size_t kStaticScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch per device. In host code the array's name is
// only a handle for the runtime, not something a kernel can dereference, so the
// address is looked up once per device (with that device current) and cached.
std::map<int, void*> g_static_scratch_ptr;

int static_scratch_for_current_device(void** out) {
    int device = 0;
    CREDIT_CUDA_TRY(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_static_scratch_ptr.find(device);
    if (it == g_static_scratch_ptr.end()) {
        void* ptr = nullptr;
        CREDIT_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch));
        it = g_static_scratch_ptr.emplace(device, ptr).first;
    }
    *out = it->second;
    return CREDIT_OK;
}

}  // namespace

size_t credit_layernorm_backward_stats_static_capacity(void) { return kStaticScratchBytes; }

int credit_layernorm_backward_stats_static(const void* x, const void* dy, const float* gamma,
                                           const float* mean, const float* rstd, void* dx,
                                           float* dgamma, float* dbeta, int64_t rows, int64_t cols,
                                           int dtype, const credit_launch_opts* opts, void* stream) {
    if ((dgamma == nullptr) != (dbeta == nullptr))
        return fail(CREDIT_ERR_INVALID_ARGUMENT, "dgamma and dbeta must both be given or both be NULL");
    // Without the column sums no scratch is used at all.
    if (dgamma == nullptr)
        return credit_layernorm_backward_stats(x, dy, gamma, mean, rstd, dx, nullptr, nullptr, rows, cols, dtype,
                                               opts, nullptr, 0, stream);
    // Size first: a shape whose partial sums do not fit is refused before any pointer is
    // dereferenced. What counts is the path this very call would take: the built-in array is
    // 256-byte aligned, so only the caller's own pointers decide between the register path
    // (one partial per resident cluster) and the column-sum fallback (one per block of rows).
    Resolved r;
    int rc = resolve(CREDIT_WL_LAYERNORM_BACKWARD_STATS, rows, cols, dtype, opts,
                     aligned16(x) && aligned16(dy) && aligned16(gamma) && aligned16(dx), true, &r);
    if (rc != CREDIT_OK) return rc;
    if (r.plan.workspace_bytes > kStaticScratchBytes)
        return fail(CREDIT_ERR_WORKSPACE,
                    "this shape needs %zu B of scratch but the built-in scratch holds %zu B; use "
                    "credit_layernorm_backward_stats with a caller workspace",
                    r.plan.workspace_bytes, kStaticScratchBytes);
    void* scratch = nullptr;
    rc = static_scratch_for_current_device(&scratch);
    if (rc != CREDIT_OK) return rc;
    // Nothing in the scratch has to start at zero: every partial sum the finishing
    // kernel reads is written earlier in this same call.
    return credit_layernorm_backward_stats(x, dy, gamma, mean, rstd, dx, dgamma, dbeta, rows, cols,
                                           dtype, opts, scratch, kStaticScratchBytes, stream);
}

}  // extern "C"
