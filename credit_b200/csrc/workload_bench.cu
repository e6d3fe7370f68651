// Command-line front end of the wide-row workloads: one executable, installed under
// the name of each workload (the workload is taken from the program name, or from
// --workload), speaking the reference's benchmark protocol
// (src/workloads/layernorm_backward.cu:87-140 flags, :707-765 META / RESULT lines)
// so that dsmem_eval/runner.py-style drivers can spawn it unchanged:
//
//   <workload> [--csv] [--warmup N] [--iters N] [--rows N | --batch-size N]
//              [--cluster-size N] [--n-values a,b,c] [--profile-variant all|block|cluster]
//              [--no-verify] [--dtype f32|bf16] [--workload NAME]
//   RESULT,cols,rows,block_variant,block_ms,block_gbps,cluster_variant,cluster_ms,
//          cluster_gbps,cluster_size,cluster_vs_block      ("n/a" for a variant that does not fit)
//
// All kernels come from libcredit_b200 through its C ABI; this file only owns the
// device buffers, the deterministic inputs (the index hashes of the reference,
// layernorm_backward.cu:253-272), the event timing (time_kernel, :150-175) and the
// sampled fp64 self-check (verify_output_samples, :608-674). GB/s figures use the
// algorithmic bytes of a call (each input read once, each output written once).

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <limits>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/credit_b200.h"

namespace {

#define CUDA_OK(expr)                                                                          \
    do {                                                                                       \
        cudaError_t e__ = (expr);                                                              \
        if (e__ != cudaSuccess)                                                                \
            throw std::runtime_error(std::string(#expr) + ": " + cudaGetErrorString(e__));     \
    } while (0)

struct Options {
    int warmup = 2, iters = 5, rows = 0, requested_cluster_size = 8;
    bool csv = false, verify = true;
    std::string profile_variant = "all", workload, dtype;
    std::vector<int> n_values{4096, 8192, 16384, 32768, 65536};
};

struct Workload {
    const char* name;
    int id;            // credit_workload
    int default_rows;  // the reference's WorkloadSpec.rows where it has one
    int default_dtype;
};
const Workload kWorkloads[] = {
    {"layernorm_backward", CREDIT_WL_LAYERNORM_BACKWARD, 2048, CREDIT_F32},
    {"rmsnorm_forward", CREDIT_WL_RMSNORM_FORWARD, 1024, CREDIT_F32},
    {"row_reduce", CREDIT_WL_ROW_REDUCE, 512, CREDIT_F32},
    {"layernorm_forward", CREDIT_WL_LAYERNORM_FORWARD, 4096, CREDIT_BF16},
    {"layernorm_backward_stats", CREDIT_WL_LAYERNORM_BACKWARD_STATS, 8192, CREDIT_BF16},
    // the rest of the reference sweep (rows as in dsmem_eval/workloads.py:164-210), fp32 only
    {"weighted_var_backward", CREDIT_WL_WEIGHTED_VAR_BACKWARD, 4096, CREDIT_F32},
    {"pearson_backward", CREDIT_WL_PEARSON_BACKWARD, 4096, CREDIT_F32},
    {"softmax_logits_backward", CREDIT_WL_SOFTMAX_LOGITS_BACKWARD, 4096, CREDIT_F32},
    {"lars_momentum", CREDIT_WL_LARS_MOMENTUM, 4096, CREDIT_F32},
    {"rowwise_quant", CREDIT_WL_ROWWISE_QUANT, 4096, CREDIT_F32},
};

bool is_row_op(int id) { return id >= CREDIT_WL_WEIGHTED_VAR_BACKWARD && id <= CREDIT_WL_ROWWISE_QUANT; }

std::vector<int> parse_int_list(const std::string& text) {
    std::vector<int> values;
    std::stringstream ss(text);
    std::string part;
    while (std::getline(ss, part, ','))
        if (!part.empty()) values.push_back(std::stoi(part));
    if (values.empty()) throw std::runtime_error("integer list cannot be empty");
    return values;
}

Options parse_options(int argc, char** argv) {
    Options o;
    std::string base = argv[0];
    const size_t slash = base.find_last_of('/');
    if (slash != std::string::npos) base = base.substr(slash + 1);
    o.workload = base;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto value = [&](const char* name) -> std::string {
            if (i + 1 >= argc) throw std::runtime_error(std::string("missing value for ") + name);
            return argv[++i];
        };
        if (a == "--warmup") o.warmup = std::stoi(value("--warmup"));
        else if (a == "--iters") o.iters = std::stoi(value("--iters"));
        else if (a == "--rows" || a == "--batch-size") o.rows = std::stoi(value(a.c_str()));
        else if (a == "--cluster-size") o.requested_cluster_size = std::stoi(value("--cluster-size"));
        else if (a == "--n-values") o.n_values = parse_int_list(value("--n-values"));
        else if (a == "--profile-variant") o.profile_variant = value("--profile-variant");
        else if (a == "--workload") o.workload = value("--workload");
        else if (a == "--dtype") o.dtype = value("--dtype");
        else if (a == "--csv") o.csv = true;
        else if (a == "--no-verify") o.verify = false;
        else if (a == "--help" || a == "-h") {
            std::printf("Usage: %s [--csv] [--warmup N] [--iters N] [--rows N] [--cluster-size N] "
                        "[--n-values list] [--profile-variant all|block|cluster] [--no-verify] "
                        "[--dtype f32|bf16] [--workload NAME]\n", base.c_str());
            std::exit(EXIT_SUCCESS);
        } else throw std::runtime_error("unknown argument: " + a);
    }
    if (o.warmup < 0 || o.iters <= 0 || o.rows < 0 || o.requested_cluster_size < 1)
        throw std::runtime_error("numeric arguments must be positive");
    if (o.profile_variant != "all" && o.profile_variant != "block" && o.profile_variant != "cluster")
        throw std::runtime_error("--profile-variant must be all, block, or cluster");
    if (!o.dtype.empty() && o.dtype != "f32" && o.dtype != "bf16")
        throw std::runtime_error("--dtype must be f32 or bf16");
    return o;
}

// ---- deterministic inputs ----------------------------------------------------------
template <typename T>
__device__ T to_elem(float v);
template <> __device__ float to_elem<float>(float v) { return v; }
template <> __device__ __nv_bfloat16 to_elem<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Two streams of values in [-1, 1) with 1/1024 granularity from two index hashes.
template <typename T>
__global__ void init_pair_kernel(T* a, T* b, size_t elements) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= elements) return;
    const unsigned ha = static_cast<unsigned>((idx * 1103515245ull + 12345ull) >> 16);
    const unsigned hb = static_cast<unsigned>((idx * 1664525ull + 1013904223ull) >> 16);
    a[idx] = to_elem<T>(static_cast<float>(ha & 2047u) * (1.0f / 1024.0f) - 1.0f);
    if (b != nullptr) b[idx] = to_elem<T>(static_cast<float>(hb & 2047u) * (1.0f / 1024.0f) - 1.0f);
}

__global__ void init_param_kernel(float* gamma, float* beta, int cols) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    gamma[c] = 0.75f + static_cast<float>(c % 31) * 0.015625f;
    if (beta != nullptr) beta[c] = static_cast<float>(c % 17) * 0.01f - 0.08f;
}

// One distinct maximum per row for the reduction workload.
__global__ void plant_max_kernel(float* x, int rows, int cols) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    const unsigned col = (static_cast<unsigned>(r) * 2654435761u) % static_cast<unsigned>(cols);
    x[static_cast<size_t>(r) * cols + col] = 10.0f;
}

struct VariantResult {
    bool valid = false;
    std::string name = "n/a";
    double avg_ms = std::numeric_limits<double>::quiet_NaN();
    double gbps = std::numeric_limits<double>::quiet_NaN();
};

struct Buffers {
    void *x = nullptr, *dy = nullptr, *out = nullptr, *workspace = nullptr;
    float *gamma = nullptr, *beta = nullptr, *mean = nullptr, *rstd = nullptr, *dgamma = nullptr, *dbeta = nullptr;
    float *rsum = nullptr, *rmax = nullptr;
    int64_t* rarg = nullptr;
    size_t workspace_bytes = 0;
};

double algorithmic_bytes(int id, int rows, int cols, int elem) {
    const double rc = static_cast<double>(rows) * cols;
    switch (id) {
        case CREDIT_WL_RMSNORM_FORWARD: return 2 * rc * elem + cols * 4.0;
        case CREDIT_WL_ROW_REDUCE: return rc * 4 + rows * 16.0;
        case CREDIT_WL_LAYERNORM_FORWARD: return 2 * rc * elem + 2 * cols * 4.0 + 2 * rows * 4.0;
        case CREDIT_WL_LAYERNORM_BACKWARD: return 3 * rc * elem + cols * 4.0;
        default: return 3 * rc * elem + 2 * rows * 4.0 + 3 * cols * 4.0;
    }
}

// One call of the workload with the given options; returns the library status.
int call_workload(int id, int dtype, const Buffers& b, int rows, int cols, const credit_launch_opts& o) {
    switch (id) {
        case CREDIT_WL_RMSNORM_FORWARD:
            return credit_rmsnorm_forward(b.x, b.gamma, b.out, rows, cols, 1.0e-6f, dtype, &o, nullptr);
        case CREDIT_WL_ROW_REDUCE:
            return credit_row_reduce(static_cast<const float*>(b.x), b.rsum, b.rmax, b.rarg, rows, cols, &o, nullptr);
        case CREDIT_WL_LAYERNORM_FORWARD:
            return credit_layernorm_forward(b.x, b.gamma, b.beta, b.out, b.mean, b.rstd, rows, cols, 1.0e-5f, dtype,
                                            &o, nullptr);
        case CREDIT_WL_LAYERNORM_BACKWARD:
            return credit_layernorm_backward(b.x, b.dy, b.gamma, b.out, rows, cols, 1.0e-5f, dtype, &o, nullptr);
        default:
            return credit_layernorm_backward_stats(b.x, b.dy, b.gamma, b.mean, b.rstd, b.out, b.dgamma, b.dbeta, rows,
                                                   cols, dtype, &o, b.workspace, b.workspace_bytes, nullptr);
    }
}

// Event timing of `iters` back-to-back calls after `warmup` calls (time_kernel of the reference).
VariantResult time_variant(const char* name, int id, int dtype, const Buffers& b, int rows, int cols,
                           const credit_launch_opts& o, const Options& opts, int elem) {
    VariantResult r;
    r.name = name;
    int rc = call_workload(id, dtype, b, rows, cols, o);
    if (rc == CREDIT_ERR_UNSUPPORTED || rc == CREDIT_ERR_WORKSPACE) return r;   // does not fit: n/a
    if (rc != CREDIT_OK) throw std::runtime_error(std::string(name) + ": " + credit_last_error());
    for (int i = 1; i < opts.warmup; ++i) call_workload(id, dtype, b, rows, cols, o);
    CUDA_OK(cudaDeviceSynchronize());
    cudaEvent_t start, stop;
    CUDA_OK(cudaEventCreate(&start));
    CUDA_OK(cudaEventCreate(&stop));
    CUDA_OK(cudaEventRecord(start));
    for (int i = 0; i < opts.iters; ++i) call_workload(id, dtype, b, rows, cols, o);
    CUDA_OK(cudaEventRecord(stop));
    CUDA_OK(cudaEventSynchronize(stop));
    float ms = 0.0f;
    CUDA_OK(cudaEventElapsedTime(&ms, start, stop));
    CUDA_OK(cudaEventDestroy(start));
    CUDA_OK(cudaEventDestroy(stop));
    int status = 0;
    if (credit_device_status(&status, 1) != CREDIT_OK)
        throw std::runtime_error(std::string(name) + ": " + credit_last_error());
    r.valid = true;
    r.avg_ms = static_cast<double>(ms) / opts.iters;
    r.gbps = algorithmic_bytes(id, rows, cols, elem) / (r.avg_ms / 1000.0) / 1.0e9;
    return r;
}

// ---- sampled fp64 verification -------------------------------------------------------
std::vector<int> unique_samples(std::initializer_list<int> values, int limit) {
    std::vector<int> out;
    for (int v : values)
        if (v >= 0 && v < limit && std::find(out.begin(), out.end(), v) == out.end()) out.push_back(v);
    return out;
}

std::vector<double> fetch_row(const void* dev, int dtype, size_t row, int cols) {
    std::vector<double> out(cols);
    if (dtype == CREDIT_F32) {
        std::vector<float> h(cols);
        CUDA_OK(cudaMemcpy(h.data(), static_cast<const float*>(dev) + row * cols, sizeof(float) * cols, cudaMemcpyDeviceToHost));
        for (int i = 0; i < cols; ++i) out[i] = h[i];
    } else {
        std::vector<__nv_bfloat16> h(cols);
        CUDA_OK(cudaMemcpy(h.data(), static_cast<const __nv_bfloat16*>(dev) + row * cols, sizeof(__nv_bfloat16) * cols,
                           cudaMemcpyDeviceToHost));
        for (int i = 0; i < cols; ++i) out[i] = __bfloat162float(h[i]);
    }
    return out;
}

std::vector<double> fetch_floats(const float* dev, size_t n) {
    std::vector<float> h(n);
    CUDA_OK(cudaMemcpy(h.data(), dev, sizeof(float) * n, cudaMemcpyDeviceToHost));
    return std::vector<double>(h.begin(), h.end());
}

void expect_close(double got, double ref, double tol, const char* label, const char* what, int row, int col) {
    const double err = std::abs(got - ref);
    if (!(err <= tol + tol * std::abs(ref))) {
        std::ostringstream oss;
        oss << label << " verification failed for " << what << " row=" << row << " col=" << col << " got=" << got
            << " ref=" << ref << " err=" << err;
        throw std::runtime_error(oss.str());
    }
}

void verify_outputs(int id, int dtype, const Buffers& b, int rows, int cols, const char* label) {
    const double tol = dtype == CREDIT_F32 ? 2.0e-4 : 2.0e-2;
    const auto sample_rows = unique_samples({0, rows / 2, rows - 1}, rows);
    const auto sample_cols = unique_samples({0, cols / 7, cols / 2, cols - 1}, cols);
    std::vector<double> gamma, beta;
    if (id != CREDIT_WL_ROW_REDUCE) gamma = fetch_floats(b.gamma, cols);
    if (id == CREDIT_WL_LAYERNORM_FORWARD) beta = fetch_floats(b.beta, cols);
    for (int row : sample_rows) {
        const auto x = fetch_row(b.x, dtype, row, cols);
        if (id == CREDIT_WL_ROW_REDUCE) {
            double sum = 0.0, best = -std::numeric_limits<double>::infinity();
            int arg = 0;
            for (int c = 0; c < cols; ++c) {
                sum += x[c];
                if (x[c] > best) { best = x[c]; arg = c; }
            }
            float s = 0, m = 0;
            int64_t a = -1;
            CUDA_OK(cudaMemcpy(&s, b.rsum + row, sizeof(float), cudaMemcpyDeviceToHost));
            CUDA_OK(cudaMemcpy(&m, b.rmax + row, sizeof(float), cudaMemcpyDeviceToHost));
            CUDA_OK(cudaMemcpy(&a, b.rarg + row, sizeof(int64_t), cudaMemcpyDeviceToHost));
            if (std::abs(s - sum) > 1.0e-5 * std::abs(sum) + 1.0e-5 * std::sqrt(static_cast<double>(cols)))
                expect_close(s, sum, 0.0, label, "sum", row, 0);
            if (m != static_cast<float>(best) || a != arg)
                throw std::runtime_error(std::string(label) + " verification failed for max/argmax row=" + std::to_string(row));
            continue;
        }
        const auto out = fetch_row(b.out, dtype, row, cols);
        double sum = 0.0, sumsq = 0.0;
        for (double v : x) { sum += v; sumsq += v * v; }
        if (id == CREDIT_WL_RMSNORM_FORWARD) {
            const double scale = 1.0 / std::sqrt(sumsq / cols + 1.0e-6);
            for (int c : sample_cols) expect_close(out[c], x[c] * scale * gamma[c], tol, label, "y", row, c);
            continue;
        }
        double mean = sum / cols, var = 0.0;
        for (double v : x) var += (v - mean) * (v - mean);
        var /= cols;
        double rstd = 1.0 / std::sqrt(var + 1.0e-5);
        if (id == CREDIT_WL_LAYERNORM_FORWARD) {
            for (int c : sample_cols)
                expect_close(out[c], (x[c] - mean) * rstd * gamma[c] + beta[c], tol, label, "y", row, c);
            continue;
        }
        if (id == CREDIT_WL_LAYERNORM_BACKWARD_STATS) {   // statistics are inputs
            mean = fetch_floats(b.mean + row, 1)[0];
            rstd = fetch_floats(b.rstd + row, 1)[0];
        }
        const auto dy = fetch_row(b.dy, dtype, row, cols);
        double sg = 0.0, sgx = 0.0;
        for (int c = 0; c < cols; ++c) {
            const double g = dy[c] * gamma[c];
            sg += g;
            sgx += g * (x[c] - mean) * rstd;
        }
        for (int c : sample_cols) {
            const double xhat = (x[c] - mean) * rstd;
            expect_close(out[c], (dy[c] * gamma[c] - sg / cols - xhat * sgx / cols) * rstd, tol, label, "dx", row, c);
        }
    }
    if (id == CREDIT_WL_LAYERNORM_BACKWARD_STATS) {
        // column sums over all rows at the sampled columns
        const auto mean = fetch_floats(b.mean, rows), rstd = fetch_floats(b.rstd, rows);
        const auto dg = fetch_floats(b.dgamma, cols), db = fetch_floats(b.dbeta, cols);
        const size_t elem = dtype == CREDIT_F32 ? 4 : 2;
        for (int c : sample_cols) {
            std::vector<unsigned char> xc(rows * elem), dc(rows * elem);
            CUDA_OK(cudaMemcpy2D(xc.data(), elem, static_cast<const char*>(b.x) + c * elem, cols * elem, elem, rows,
                                 cudaMemcpyDeviceToHost));
            CUDA_OK(cudaMemcpy2D(dc.data(), elem, static_cast<const char*>(b.dy) + c * elem, cols * elem, elem, rows,
                                 cudaMemcpyDeviceToHost));
            double rg = 0.0, rb = 0.0;
            for (int r = 0; r < rows; ++r) {
                const double xv = dtype == CREDIT_F32 ? reinterpret_cast<float*>(xc.data())[r]
                                                      : __bfloat162float(reinterpret_cast<__nv_bfloat16*>(xc.data())[r]);
                const double dv = dtype == CREDIT_F32 ? reinterpret_cast<float*>(dc.data())[r]
                                                      : __bfloat162float(reinterpret_cast<__nv_bfloat16*>(dc.data())[r]);
                rg += dv * (xv - mean[r]) * rstd[r];
                rb += dv;
            }
            const double scale = 1.0e-5 * 4.0 * std::sqrt(static_cast<double>(rows));
            if (std::abs(dg[c] - rg) > 1.0e-5 * std::abs(rg) + scale) expect_close(dg[c], rg, 0.0, label, "dgamma", -1, c);
            if (std::abs(db[c] - rb) > 1.0e-5 * std::abs(rb) + scale) expect_close(db[c], rb, 0.0, label, "dbeta", -1, c);
        }
    }
}

void print_result(int cols, int rows, const VariantResult& block, const VariantResult& cluster, int chosen, bool csv) {
    const double ratio = (block.valid && cluster.valid) ? block.avg_ms / cluster.avg_ms
                                                        : std::numeric_limits<double>::quiet_NaN();
    if (!csv) {
        std::printf("%8d%14s%12.5f%14s%12.5f%12.4f\n", cols, block.name.c_str(), block.avg_ms, cluster.name.c_str(),
                    cluster.avg_ms, ratio);
        return;
    }
    std::printf("RESULT,%d,%d,", cols, rows);
    if (block.valid) std::printf("%s,%g,%g,", block.name.c_str(), block.avg_ms, block.gbps);
    else std::printf("n/a,n/a,n/a,");
    if (cluster.valid) std::printf("%s,%g,%g,%d,", cluster.name.c_str(), cluster.avg_ms, cluster.gbps, chosen);
    else std::printf("n/a,n/a,n/a,%d,", chosen);
    if (std::isnan(ratio)) std::printf("n/a\n");
    else std::printf("%g\n", ratio);
}

// ---- the reference sweep's other workloads (credit_row_op) ---------------------------------
// Values in [low, high) with 1/2048 granularity from an index hash; `salt` separates the arrays.
__global__ void init_uniform_kernel(float* a, size_t elements, float low, float high, unsigned salt) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= elements) return;
    const unsigned h = static_cast<unsigned>(((idx + salt) * 1103515245ull + 12345ull + 7919ull * salt) >> 16);
    a[idx] = low + static_cast<float>(h & 2047u) * ((high - low) / 2048.0f);
}

struct RowOpShape {
    int nin, nout;
    bool row_in, row_out;
    float low[3], high[3];     // input ranges of the reference factories (workloads.py:64-150)
    double bytes_per_elem;     // compulsory traffic: every input read once, every output written once
    double tol;
};

RowOpShape row_op_shape(int id) {
    switch (id) {
        case CREDIT_WL_WEIGHTED_VAR_BACKWARD: return {3, 1, false, false, {-2.0f, 0.5f, -1.0f}, {2.0f, 1.5f, 1.0f}, 16.0, 3.0e-2};
        case CREDIT_WL_PEARSON_BACKWARD: return {2, 2, true, false, {-1.0f, -1.0f, 0.0f}, {1.0f, 1.0f, 0.0f}, 16.0, 3.0e-3};
        case CREDIT_WL_SOFTMAX_LOGITS_BACKWARD: return {2, 1, false, false, {-4.0f, -1.0f, 0.0f}, {4.0f, 1.0f, 0.0f}, 12.0, 3.0e-3};
        case CREDIT_WL_LARS_MOMENTUM: return {3, 2, false, false, {-1.0f, -1.0f, -1.0f}, {1.0f, 1.0f, 1.0f}, 20.0, 3.0e-3};
        default: return {1, 1, false, true, {-1.0f, 0.0f, 0.0f}, {1.0f, 0.0f, 0.0f}, 5.0, 1.0e-6};
    }
}

struct RowOpBuffers {
    float* in[3] = {nullptr, nullptr, nullptr};
    void* out[2] = {nullptr, nullptr};
    float *row_in = nullptr, *row_out = nullptr;
};

int call_row_op(int id, const RowOpBuffers& b, int rows, int cols, const credit_launch_opts& o) {
    return credit_row_op(id, b.in[0], b.in[1], b.in[2], b.row_in, b.out[0], b.out[1], b.row_out, rows, cols, &o, nullptr);
}

VariantResult time_row_op(const char* name, int id, const RowOpBuffers& b, int rows, int cols,
                          const credit_launch_opts& o, const Options& opts, double bytes) {
    VariantResult r;
    r.name = name;
    int rc = call_row_op(id, b, rows, cols, o);
    if (rc == CREDIT_ERR_UNSUPPORTED) return r;
    if (rc != CREDIT_OK) throw std::runtime_error(std::string(name) + ": " + credit_last_error());
    for (int i = 1; i < opts.warmup; ++i) call_row_op(id, b, rows, cols, o);
    CUDA_OK(cudaDeviceSynchronize());
    cudaEvent_t start, stop;
    CUDA_OK(cudaEventCreate(&start));
    CUDA_OK(cudaEventCreate(&stop));
    CUDA_OK(cudaEventRecord(start));
    for (int i = 0; i < opts.iters; ++i) call_row_op(id, b, rows, cols, o);
    CUDA_OK(cudaEventRecord(stop));
    CUDA_OK(cudaEventSynchronize(stop));
    float ms = 0.0f;
    CUDA_OK(cudaEventElapsedTime(&ms, start, stop));
    CUDA_OK(cudaEventDestroy(start));
    CUDA_OK(cudaEventDestroy(stop));
    int status = 0;
    if (credit_device_status(&status, 1) != CREDIT_OK)
        throw std::runtime_error(std::string(name) + ": " + credit_last_error());
    r.valid = true;
    r.avg_ms = static_cast<double>(ms) / opts.iters;
    r.gbps = bytes / (r.avg_ms / 1000.0) / 1.0e9;
    return r;
}

// fp64 recomputation of sampled rows on the host (verify_output_samples of the reference binaries).
void verify_row_op(int id, const RowOpBuffers& b, const RowOpShape& sh, int rows, int cols, const char* label) {
    const auto sample_rows = unique_samples({0, rows / 2, rows - 1}, rows);
    const auto sample_cols = unique_samples({0, cols / 7, cols / 2, cols - 1}, cols);
    for (int row : sample_rows) {
        std::vector<double> in[3], out[2];
        for (int n = 0; n < sh.nin; ++n) in[n] = fetch_row(b.in[n], CREDIT_F32, row, cols);
        const auto& x = in[0];
        auto check = [&](int k, int c, double ref) {
            float got = 0.0f;
            CUDA_OK(cudaMemcpy(&got, static_cast<const float*>(b.out[k]) + static_cast<size_t>(row) * cols + c,
                               sizeof(float), cudaMemcpyDeviceToHost));
            expect_close(got, ref, sh.tol, label, k == 0 ? "out0" : "out1", row, c);
        };
        if (id == CREDIT_WL_WEIGHTED_VAR_BACKWARD) {
            const auto &w = in[1], &dy = in[2];
            double sw = 0, swx = 0;
            for (int c = 0; c < cols; ++c) { sw += w[c]; swx += w[c] * x[c]; }
            const double inv_w = 1.0 / (sw + 1.0e-5), mean = swx * inv_w;
            double var = 0, s_dy = 0, s_dyd = 0;
            for (int c = 0; c < cols; ++c) {
                const double d = x[c] - mean;
                var += w[c] * d * d; s_dy += dy[c]; s_dyd += dy[c] * d;
            }
            const double rstd = 1.0 / std::sqrt(var * inv_w + 1.0e-5);
            for (int c : sample_cols) {
                const double d = x[c] - mean;
                check(0, c, rstd * (dy[c] - w[c] * inv_w * s_dy - w[c] * d * rstd * rstd * inv_w * s_dyd));
            }
        } else if (id == CREDIT_WL_PEARSON_BACKWARD) {
            const auto& y = in[1];
            const double grad = fetch_floats(b.row_in + row, 1)[0];
            double mx = 0, my = 0;
            for (int c = 0; c < cols; ++c) { mx += x[c]; my += y[c]; }
            mx /= cols; my /= cols;
            double vx = 0, vy = 0, cov = 0;
            for (int c = 0; c < cols; ++c) {
                const double xc = x[c] - mx, yc = y[c] - my;
                vx += xc * xc; vy += yc * yc; cov += xc * yc;
            }
            const double ix = 1.0 / std::sqrt(vx + 1.0e-6), iy = 1.0 / std::sqrt(vy + 1.0e-6);
            for (int c : sample_cols) {
                const double xc = x[c] - mx, yc = y[c] - my;
                check(0, c, grad * (yc * ix * iy - xc * cov * ix * ix * ix * iy));
                check(1, c, grad * (xc * ix * iy - yc * cov * ix * iy * iy * iy));
            }
        } else if (id == CREDIT_WL_SOFTMAX_LOGITS_BACKWARD) {
            const auto& dy = in[1];
            double mx = -std::numeric_limits<double>::infinity();
            for (double v : x) mx = std::max(mx, v);
            double sum = 0, dot = 0;
            for (int c = 0; c < cols; ++c) sum += std::exp(x[c] - mx);
            for (int c = 0; c < cols; ++c) dot += std::exp(x[c] - mx) / sum * dy[c];
            for (int c : sample_cols) check(0, c, std::exp(x[c] - mx) / sum * (dy[c] - dot));
        } else if (id == CREDIT_WL_LARS_MOMENTUM) {
            const auto &g = in[1], &m = in[2];
            double wn = 0, un = 0;
            for (int c = 0; c < cols; ++c) {
                const double u = 0.9 * m[c] + g[c] + 0.01 * x[c];
                wn += x[c] * x[c]; un += u * u;
            }
            const double trust = 0.02 * std::sqrt(wn) / (std::sqrt(un) + 1.0e-6);
            for (int c : sample_cols) {
                const double u = 0.9 * m[c] + g[c] + 0.01 * x[c];
                check(0, c, x[c] - 1.0e-3 * trust * u);
                check(1, c, u);
            }
        } else {
            double mx = 0;
            for (double v : x) mx = std::max(mx, std::abs(v));
            const double scale = fetch_floats(b.row_out + row, 1)[0];
            expect_close(scale, mx / 127.0, 1.0e-6, label, "scale", row, 0);
            const float inv = mx > 0 ? 127.0f / static_cast<float>(mx) : 0.0f;
            for (int c : sample_cols) {
                signed char q = 0;
                CUDA_OK(cudaMemcpy(&q, static_cast<const signed char*>(b.out[0]) + static_cast<size_t>(row) * cols + c, 1,
                                   cudaMemcpyDeviceToHost));
                const float want = std::min(std::max(std::nearbyint(static_cast<float>(x[c]) * inv), -127.0f), 127.0f);
                if (std::abs(static_cast<int>(q) - static_cast<int>(want)) > 1)
                    throw std::runtime_error(std::string(label) + " verification failed for q row=" + std::to_string(row));
            }
        }
    }
}

void run_row_op_shape(const Workload& w, int rows, int cols, int chosen, const Options& opts) {
    const RowOpShape sh = row_op_shape(w.id);
    const size_t elements = static_cast<size_t>(rows) * cols;
    RowOpBuffers b;
    const unsigned init_blocks = static_cast<unsigned>((elements + 255) / 256);
    for (int n = 0; n < sh.nin; ++n) {
        CUDA_OK(cudaMalloc(&b.in[n], elements * sizeof(float)));
        init_uniform_kernel<<<init_blocks, 256>>>(b.in[n], elements, sh.low[n], sh.high[n], 17u * n + 1u);
    }
    const size_t out_elem = w.id == CREDIT_WL_ROWWISE_QUANT ? 1 : sizeof(float);
    for (int k = 0; k < sh.nout; ++k) CUDA_OK(cudaMalloc(&b.out[k], elements * out_elem));
    if (sh.row_in) {
        CUDA_OK(cudaMalloc(&b.row_in, sizeof(float) * rows));
        init_uniform_kernel<<<(rows + 255) / 256, 256>>>(b.row_in, rows, 0.75f, 1.25f, 101u);
    }
    if (sh.row_out) CUDA_OK(cudaMalloc(&b.row_out, sizeof(float) * rows));
    CUDA_OK(cudaGetLastError());
    CUDA_OK(cudaDeviceSynchronize());
    const double bytes = sh.bytes_per_elem * static_cast<double>(elements);

    VariantResult block, cluster;
    credit_launch_opts o{};
    if (opts.profile_variant != "cluster") {
        o.variant = CREDIT_VARIANT_BLOCK_READ;
        block = time_row_op("block_read", w.id, b, rows, cols, o, opts, bytes);
        o = credit_launch_opts{};
        o.variant = CREDIT_VARIANT_BLOCK_SMEM;
        const VariantResult staged = time_row_op("block_smem", w.id, b, rows, cols, o, opts, bytes);
        if (staged.valid && (!block.valid || staged.avg_ms < block.avg_ms)) block = staged;
        if (block.valid && opts.verify) {
            o = credit_launch_opts{};
            o.variant = block.name == "block_smem" ? CREDIT_VARIANT_BLOCK_SMEM : CREDIT_VARIANT_BLOCK_READ;
            call_row_op(w.id, b, rows, cols, o);
            CUDA_OK(cudaDeviceSynchronize());
            verify_row_op(w.id, b, sh, rows, cols, "block");
        }
    }
    // --cluster-size 1 (an extension: the reference prints n/a there) puts the same pipeline with one
    // CTA per row in the cluster column, so that a sweep can cover the size the planner often picks
    if (opts.profile_variant != "block" && chosen >= 1) {
        o = credit_launch_opts{};
        o.variant = chosen >= 2 ? CREDIT_VARIANT_CLUSTER_SMEM : CREDIT_VARIANT_AUTO;
        o.cluster_size = chosen;
        cluster = time_row_op("cluster_smem", w.id, b, rows, cols, o, opts, bytes);
        if (cluster.valid && opts.verify) {
            call_row_op(w.id, b, rows, cols, o);
            CUDA_OK(cudaDeviceSynchronize());
            verify_row_op(w.id, b, sh, rows, cols, "cluster");
        }
    }
    cluster.name = "cluster_smem";
    print_result(cols, rows, block, cluster, chosen, opts.csv);
    for (void* p : {static_cast<void*>(b.in[0]), static_cast<void*>(b.in[1]), static_cast<void*>(b.in[2]), b.out[0],
                    b.out[1], static_cast<void*>(b.row_in), static_cast<void*>(b.row_out)})
        if (p != nullptr) cudaFree(p);
}

void run_shape(const Workload& w, int dtype, int rows, int cols, int chosen, const Options& opts) {
    const int elem = dtype == CREDIT_F32 ? 4 : 2;
    const size_t elements = static_cast<size_t>(rows) * cols;
    Buffers b;
    CUDA_OK(cudaMalloc(&b.x, elements * elem));
    const bool backward = w.id == CREDIT_WL_LAYERNORM_BACKWARD || w.id == CREDIT_WL_LAYERNORM_BACKWARD_STATS;
    if (backward) CUDA_OK(cudaMalloc(&b.dy, elements * elem));
    if (w.id != CREDIT_WL_ROW_REDUCE) {
        CUDA_OK(cudaMalloc(&b.out, elements * elem));
        CUDA_OK(cudaMalloc(&b.gamma, sizeof(float) * cols));
        CUDA_OK(cudaMalloc(&b.beta, sizeof(float) * cols));
        CUDA_OK(cudaMalloc(&b.mean, sizeof(float) * rows));
        CUDA_OK(cudaMalloc(&b.rstd, sizeof(float) * rows));
        CUDA_OK(cudaMalloc(&b.dgamma, sizeof(float) * cols));
        CUDA_OK(cudaMalloc(&b.dbeta, sizeof(float) * cols));
        init_param_kernel<<<(cols + 255) / 256, 256>>>(b.gamma, b.beta, cols);
    } else {
        CUDA_OK(cudaMalloc(&b.rsum, sizeof(float) * rows));
        CUDA_OK(cudaMalloc(&b.rmax, sizeof(float) * rows));
        CUDA_OK(cudaMalloc(&b.rarg, sizeof(int64_t) * rows));
    }
    const unsigned init_blocks = static_cast<unsigned>((elements + 255) / 256);
    if (dtype == CREDIT_F32)
        init_pair_kernel<float><<<init_blocks, 256>>>(static_cast<float*>(b.x), static_cast<float*>(b.dy), elements);
    else
        init_pair_kernel<__nv_bfloat16><<<init_blocks, 256>>>(static_cast<__nv_bfloat16*>(b.x),
                                                             static_cast<__nv_bfloat16*>(b.dy), elements);
    if (w.id == CREDIT_WL_ROW_REDUCE) plant_max_kernel<<<(rows + 255) / 256, 256>>>(static_cast<float*>(b.x), rows, cols);
    CUDA_OK(cudaGetLastError());
    if (w.id == CREDIT_WL_LAYERNORM_BACKWARD_STATS) {
        // the saved statistics come from this library's own forward pass (output discarded)
        if (credit_layernorm_forward(b.x, b.gamma, b.beta, b.out, b.mean, b.rstd, rows, cols, 1.0e-5f, dtype, nullptr,
                                     nullptr) != CREDIT_OK)
            throw std::runtime_error(std::string("statistics: ") + credit_last_error());
        credit_launch_opts gen{};
        gen.variant = CREDIT_VARIANT_BLOCK_READ;   // the variant with the largest workspace
        b.workspace_bytes = credit_layernorm_backward_stats_workspace_bytes(rows, cols, dtype, &gen);
        credit_launch_opts any{};
        for (int p : {1, 2, 4, 8, 16}) {
            any.cluster_size = p;
            b.workspace_bytes = std::max(b.workspace_bytes,
                                         credit_layernorm_backward_stats_workspace_bytes(rows, cols, dtype, &any));
        }
        CUDA_OK(cudaMalloc(&b.workspace, std::max<size_t>(b.workspace_bytes, 16)));
    }
    CUDA_OK(cudaDeviceSynchronize());

    VariantResult block, cluster;
    credit_launch_opts o{};
    if (opts.profile_variant != "cluster") {
        if (w.id != CREDIT_WL_ROW_REDUCE) {
            o = credit_launch_opts{};
            o.variant = CREDIT_VARIANT_BLOCK_READ;
            block = time_variant("block_read", w.id, dtype, b, rows, cols, o, opts, elem);
        }
        o = credit_launch_opts{};
        o.variant = CREDIT_VARIANT_BLOCK_SMEM;
        const VariantResult staged = time_variant("block_smem", w.id, dtype, b, rows, cols, o, opts, elem);
        if (staged.valid && (!block.valid || staged.avg_ms < block.avg_ms)) block = staged;
        if (block.valid && opts.verify) {
            o = credit_launch_opts{};
            o.variant = block.name == "block_smem" ? CREDIT_VARIANT_BLOCK_SMEM : CREDIT_VARIANT_BLOCK_READ;
            call_workload(w.id, dtype, b, rows, cols, o);
            CUDA_OK(cudaDeviceSynchronize());
            verify_outputs(w.id, dtype, b, rows, cols, "block");
        }
    }
    // --cluster-size 1 (an extension: the reference prints n/a there) puts the same pipeline with one
    // CTA per row in the cluster column, so that a sweep can cover the size the planner often picks
    if (opts.profile_variant != "block" && chosen >= 1) {
        o = credit_launch_opts{};
        o.variant = chosen >= 2 ? CREDIT_VARIANT_CLUSTER_SMEM : CREDIT_VARIANT_AUTO;
        o.cluster_size = chosen;
        cluster = time_variant("cluster_smem", w.id, dtype, b, rows, cols, o, opts, elem);
        if (cluster.valid && opts.verify) {
            call_workload(w.id, dtype, b, rows, cols, o);
            CUDA_OK(cudaDeviceSynchronize());
            verify_outputs(w.id, dtype, b, rows, cols, "cluster");
        }
    }
    cluster.name = "cluster_smem";
    print_result(cols, rows, block, cluster, chosen, opts.csv);

    for (void* p : {b.x, b.dy, b.out, b.workspace, static_cast<void*>(b.gamma), static_cast<void*>(b.beta),
                    static_cast<void*>(b.mean), static_cast<void*>(b.rstd), static_cast<void*>(b.dgamma),
                    static_cast<void*>(b.dbeta), static_cast<void*>(b.rsum), static_cast<void*>(b.rmax),
                    static_cast<void*>(b.rarg)})
        if (p != nullptr) cudaFree(p);
}

}  // namespace

int main(int argc, char** argv) {
    try {
        const Options opts = parse_options(argc, argv);
        const Workload* w = nullptr;
        for (const Workload& cand : kWorkloads)
            if (opts.workload == cand.name) w = &cand;
        if (w == nullptr) throw std::runtime_error("unknown workload: " + opts.workload);
        int dtype = w->default_dtype;
        if (!opts.dtype.empty()) dtype = opts.dtype == "f32" ? CREDIT_F32 : CREDIT_BF16;
        if ((w->id == CREDIT_WL_ROW_REDUCE || is_row_op(w->id)) && dtype != CREDIT_F32)
            throw std::runtime_error(std::string(w->name) + " takes f32");
        const int rows = opts.rows > 0 ? opts.rows : w->default_rows;

        credit_device_info info{};
        if (credit_query_device(0, &info) != CREDIT_OK) throw std::runtime_error(credit_last_error());
        int chosen = info.cluster_launch ? std::min(opts.requested_cluster_size, info.max_cluster_size) : 0;
        while (chosen > 1 && (chosen & (chosen - 1))) --chosen;   // 1, 2, 4, 8 or 16

        if (opts.csv) {
            std::printf("META,device_name,%s\n", info.name);
            std::printf("META,sm,%d.%d\n", info.sm_major, info.sm_minor);
            std::printf("META,workload,%s\n", w->name);
            std::printf("META,dtype,%s\n", dtype == CREDIT_F32 ? "f32" : "bf16");
            std::printf("META,rows,%d\n", rows);
            std::printf("META,warmup,%d\n", opts.warmup);
            std::printf("META,iters,%d\n", opts.iters);
            std::printf("META,cluster_launch,%d\n", info.cluster_launch);
            std::printf("META,requested_cluster_size,%d\n", opts.requested_cluster_size);
            std::printf("META,max_cluster_size,%d\n", info.max_cluster_size);
            std::printf("META,chosen_cluster_size,%d\n", chosen);
            std::printf("META,gbps_basis,algorithmic\n");
        } else {
            std::printf("Device: %s sm_%d%d\n", info.name, info.sm_major, info.sm_minor);
            std::printf("Workload: %s (%s), rows: %d, warmup: %d, iters: %d, cluster size: %d\n", w->name,
                        dtype == CREDIT_F32 ? "f32" : "bf16", rows, opts.warmup, opts.iters, chosen);
            std::printf("%8s%14s%12s%14s%12s%12s\n", "N", "block", "ms", "cluster", "ms", "c/b");
        }
        for (int cols : opts.n_values) {
            if (is_row_op(w->id)) run_row_op_shape(*w, rows, cols, chosen, opts);
            else run_shape(*w, dtype, rows, cols, chosen, opts);
        }
        CUDA_OK(cudaDeviceSynchronize());
    } catch (const std::exception& exc) {
        std::fprintf(stderr, "error: %s\n", exc.what());
        return EXIT_FAILURE;
    }
    return EXIT_SUCCESS;
}
