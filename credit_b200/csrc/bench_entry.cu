// credit_bench: event timing of one workload on buffers the library allocates and
// fills itself, for callers that only want a number (the counterpart of
// time_kernel + benchmark_block_* / benchmark_cluster in the reference binaries,
// src/workloads/layernorm_backward.cu:150-175, 480-593). Built on the public entry
// points; nothing here is on a hot path.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <vector>

#include "../../include/credit_b200.h"

namespace {

struct BenchWorkload {
    const char* name;
    int id;
};
const BenchWorkload kBenchWorkloads[] = {
    {"rmsnorm_forward", CREDIT_WL_RMSNORM_FORWARD},
    {"row_reduce", CREDIT_WL_ROW_REDUCE},
    {"layernorm_forward", CREDIT_WL_LAYERNORM_FORWARD},
    {"layernorm_backward", CREDIT_WL_LAYERNORM_BACKWARD},
    {"layernorm_backward_stats", CREDIT_WL_LAYERNORM_BACKWARD_STATS},
    {"weighted_var_backward", CREDIT_WL_WEIGHTED_VAR_BACKWARD},
    {"pearson_backward", CREDIT_WL_PEARSON_BACKWARD},
    {"softmax_logits_backward", CREDIT_WL_SOFTMAX_LOGITS_BACKWARD},
    {"lars_momentum", CREDIT_WL_LARS_MOMENTUM},
    {"rowwise_quant", CREDIT_WL_ROWWISE_QUANT},
};

// Values in [low, high) from an index hash, stored as fp32 or bf16.
template <typename T>
__global__ void bench_fill_kernel(T* out, size_t n, float low, float high, unsigned salt) {
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned h = static_cast<unsigned>(((i + salt) * 1103515245ull + 12345ull) >> 16);
    const float v = low + static_cast<float>(h & 2047u) * ((high - low) / 2048.0f);
    if (sizeof(T) == 4) reinterpret_cast<float*>(out)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
}

struct Arena {
    std::vector<void*> blocks;
    bool failed = false;
    void* get(size_t bytes) {
        void* p = nullptr;
        if (cudaMalloc(&p, bytes ? bytes : 16) != cudaSuccess) {
            failed = true;
            return nullptr;
        }
        blocks.push_back(p);
        return p;
    }
    ~Arena() {
        for (void* p : blocks) cudaFree(p);
    }
};

void fill(void* p, size_t n, int dtype, float low, float high, unsigned salt) {
    const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
    if (n == 0) return;
    if (dtype == CREDIT_F32) bench_fill_kernel<float><<<blocks, 256>>>(static_cast<float*>(p), n, low, high, salt);
    else bench_fill_kernel<__nv_bfloat16><<<blocks, 256>>>(static_cast<__nv_bfloat16*>(p), n, low, high, salt);
}

}  // namespace

extern "C" int credit_bench(const char* workload, int64_t rows, int64_t cols, int dtype, int cluster_size,
                            int variant, int warmup, int iters, double* avg_ms) {
    if (workload == nullptr || avg_ms == nullptr || rows <= 0 || cols <= 0 || warmup < 0 || iters <= 0)
        return CREDIT_ERR_INVALID_ARGUMENT;
    int id = -1;
    for (const BenchWorkload& w : kBenchWorkloads)
        if (std::strcmp(w.name, workload) == 0) id = w.id;
    if (id < 0) return CREDIT_ERR_INVALID_ARGUMENT;
    if (dtype != CREDIT_F32 && dtype != CREDIT_BF16) return CREDIT_ERR_INVALID_ARGUMENT;
    const bool row_op = id >= CREDIT_WL_WEIGHTED_VAR_BACKWARD;
    if ((row_op || id == CREDIT_WL_ROW_REDUCE) && dtype != CREDIT_F32) return CREDIT_ERR_INVALID_ARGUMENT;

    credit_launch_opts o{};
    o.cluster_size = cluster_size;
    o.variant = variant;
    const size_t elem = dtype == CREDIT_F32 ? 4 : 2;
    const size_t n = static_cast<size_t>(rows) * static_cast<size_t>(cols);
    Arena arena;
    void* in[3] = {nullptr, nullptr, nullptr};
    void* out[2] = {nullptr, nullptr};
    int nin = 1, nout = 1;
    switch (id) {
        case CREDIT_WL_LAYERNORM_BACKWARD:
        case CREDIT_WL_LAYERNORM_BACKWARD_STATS:
        case CREDIT_WL_SOFTMAX_LOGITS_BACKWARD: nin = 2; break;
        case CREDIT_WL_PEARSON_BACKWARD: nin = 2; nout = 2; break;
        case CREDIT_WL_WEIGHTED_VAR_BACKWARD: nin = 3; break;
        case CREDIT_WL_LARS_MOMENTUM: nin = 3; nout = 2; break;
        default: break;
    }
    for (int i = 0; i < nin; ++i) {
        in[i] = arena.get(n * elem);
        if (in[i]) fill(in[i], n, dtype, id == CREDIT_WL_WEIGHTED_VAR_BACKWARD && i == 1 ? 0.5f : -1.0f,
                        id == CREDIT_WL_WEIGHTED_VAR_BACKWARD && i == 1 ? 1.5f : 1.0f, 31u * i + 1u);
    }
    if (id != CREDIT_WL_ROW_REDUCE)
        for (int i = 0; i < nout; ++i) out[i] = arena.get(id == CREDIT_WL_ROWWISE_QUANT ? n : n * elem);
    float* gamma = static_cast<float*>(arena.get(cols * sizeof(float)));
    float* beta = static_cast<float*>(arena.get(cols * sizeof(float)));
    float* per_row_a = static_cast<float*>(arena.get(rows * sizeof(float)));   // mean / sums / grad / scale
    float* per_row_b = static_cast<float*>(arena.get(rows * sizeof(float)));   // rstd / maxima
    long long* per_row_i = static_cast<long long*>(arena.get(rows * sizeof(long long)));
    float* dgamma = static_cast<float*>(arena.get(cols * sizeof(float)));
    float* dbeta = static_cast<float*>(arena.get(cols * sizeof(float)));
    size_t ws_bytes = 0;
    void* ws = nullptr;
    if (id == CREDIT_WL_LAYERNORM_BACKWARD_STATS) {
        ws_bytes = credit_layernorm_backward_stats_workspace_bytes(rows, cols, dtype, &o);
        ws = arena.get(ws_bytes);
    }
    if (arena.failed) return CREDIT_ERR_CUDA;
    fill(gamma, cols, CREDIT_F32, 0.75f, 1.25f, 7u);
    fill(beta, cols, CREDIT_F32, -0.1f, 0.1f, 11u);
    fill(per_row_a, rows, CREDIT_F32, id == CREDIT_WL_PEARSON_BACKWARD ? 0.75f : -0.01f,
         id == CREDIT_WL_PEARSON_BACKWARD ? 1.25f : 0.01f, 13u);
    fill(per_row_b, rows, CREDIT_F32, 1.7f, 1.8f, 17u);   // a plausible rstd for inputs uniform in [-1, 1)
    if (cudaDeviceSynchronize() != cudaSuccess) return CREDIT_ERR_CUDA;

    auto call = [&]() -> int {
        switch (id) {
            case CREDIT_WL_RMSNORM_FORWARD:
                return credit_rmsnorm_forward(in[0], gamma, out[0], rows, cols, 1.0e-6f, dtype, &o, nullptr);
            case CREDIT_WL_ROW_REDUCE:
                return credit_row_reduce(static_cast<const float*>(in[0]), per_row_a, per_row_b,
                                         reinterpret_cast<int64_t*>(per_row_i), rows, cols, &o, nullptr);
            case CREDIT_WL_LAYERNORM_FORWARD:
                return credit_layernorm_forward(in[0], gamma, beta, out[0], per_row_a, per_row_b, rows, cols, 1.0e-5f,
                                                dtype, &o, nullptr);
            case CREDIT_WL_LAYERNORM_BACKWARD:
                return credit_layernorm_backward(in[0], in[1], gamma, out[0], rows, cols, 1.0e-5f, dtype, &o, nullptr);
            case CREDIT_WL_LAYERNORM_BACKWARD_STATS:
                return credit_layernorm_backward_stats(in[0], in[1], gamma, per_row_a, per_row_b, out[0], dgamma, dbeta,
                                                       rows, cols, dtype, &o, ws, ws_bytes, nullptr);
            default:
                return credit_row_op(id, static_cast<const float*>(in[0]), static_cast<const float*>(in[1]),
                                     static_cast<const float*>(in[2]),
                                     id == CREDIT_WL_PEARSON_BACKWARD ? per_row_a : nullptr, out[0], out[1],
                                     id == CREDIT_WL_ROWWISE_QUANT ? per_row_b : nullptr, rows, cols, &o, nullptr);
        }
    };
    int rc = call();
    if (rc != CREDIT_OK) return rc;
    for (int i = 1; i < warmup; ++i) call();
    cudaEvent_t start, stop;
    if (cudaEventCreate(&start) != cudaSuccess || cudaEventCreate(&stop) != cudaSuccess) return CREDIT_ERR_CUDA;
    cudaDeviceSynchronize();
    cudaEventRecord(start);
    for (int i = 0; i < iters; ++i) call();
    cudaEventRecord(stop);
    const cudaError_t sync = cudaEventSynchronize(stop);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, start, stop);
    cudaEventDestroy(start);
    cudaEventDestroy(stop);
    if (sync != cudaSuccess) return CREDIT_ERR_CUDA;
    int status = 0;
    rc = credit_device_status(&status, 1);
    if (rc != CREDIT_OK) return rc;
    *avg_ms = static_cast<double>(ms) / iters;
    return CREDIT_OK;
}
