// Host-buffer entry points: the workloads of the C ABI on data that lives in HOST
// memory. A matrix is streamed through caller-owned device scratch in row blocks on
// three streams, so that the upload of block k+1, the kernels of block k and the
// download of block k-1 overlap (rows are independent in every workload; the only
// quantity that spans blocks, LayerNorm backward's column sums, is kept per block and
// added up at the end by the library's own finishing kernel).
//
// This is the shape of run_shape in the reference executables
// (src/workloads/layernorm_backward.cu:767-805), which own their device buffers and
// copy sampled rows back (:608-674), with the allocation moved to the caller and the
// copies pipelined. Everything here goes through the public device-pointer entry
// points; there is no second implementation of any kernel.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <map>
#include <mutex>

#include "../../include/credit_b200.h"
#include "error_state.h"
#include "kernel_tables.h"

namespace {

using credit::report_error;

#define HOST_CUDA_TRY(expr)                                                                          \
    do {                                                                                             \
        cudaError_t err__ = (expr);                                                                  \
        if (err__ != cudaSuccess) return report_error(CREDIT_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(err__)); \
    } while (0)

constexpr size_t kAlign = 256;
size_t align_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

// A block is at least this many bytes over all of its arrays (or the whole matrix if that is
// smaller): large enough that a copy runs at the full rate of the link.
constexpr size_t kMinBlockBytes = 64ull << 20;

// One array that is cut into row blocks: an input (host_src) or an output (host_dst).
struct BlockArray {
    const void* host_src;
    void* host_dst;
    size_t row_bytes;
};

// Per-device streams and events of the pipeline. One call at a time uses them: the mutex is
// held for the whole call, so concurrent calls on one device run one after the other.
struct Pipe {
    std::mutex busy;
    bool ready = false;
    cudaStream_t upload = nullptr, download = nullptr;
    cudaEvent_t start = nullptr;
    cudaEvent_t loaded[2] = {nullptr, nullptr};     // inputs of a block are on the device
    cudaEvent_t computed[2] = {nullptr, nullptr};   // kernels of a block are done
    cudaEvent_t drained[2] = {nullptr, nullptr};    // outputs of a block are in host memory
};
std::mutex g_pipes_mutex;
std::map<int, Pipe> g_pipes;

void destroy(Pipe& p) {
    if (p.upload) cudaStreamDestroy(p.upload);
    if (p.download) cudaStreamDestroy(p.download);
    if (p.start) cudaEventDestroy(p.start);
    for (int i = 0; i < 2; ++i) {
        if (p.loaded[i]) cudaEventDestroy(p.loaded[i]);
        if (p.computed[i]) cudaEventDestroy(p.computed[i]);
        if (p.drained[i]) cudaEventDestroy(p.drained[i]);
    }
    p.upload = p.download = nullptr;
    p.start = nullptr;
    for (int i = 0; i < 2; ++i) p.loaded[i] = p.computed[i] = p.drained[i] = nullptr;
    p.ready = false;
}

int create(Pipe& p) {
    cudaError_t err = cudaStreamCreateWithFlags(&p.upload, cudaStreamNonBlocking);
    if (err == cudaSuccess) err = cudaStreamCreateWithFlags(&p.download, cudaStreamNonBlocking);
    if (err == cudaSuccess) err = cudaEventCreateWithFlags(&p.start, cudaEventDisableTiming);
    for (int i = 0; i < 2 && err == cudaSuccess; ++i) {
        err = cudaEventCreateWithFlags(&p.loaded[i], cudaEventDisableTiming);
        if (err == cudaSuccess) err = cudaEventCreateWithFlags(&p.computed[i], cudaEventDisableTiming);
        if (err == cudaSuccess) err = cudaEventCreateWithFlags(&p.drained[i], cudaEventDisableTiming);
    }
    return err == cudaSuccess ? CREDIT_OK
                              : report_error(CREDIT_ERR_CUDA, "host pipeline set-up: %s", cudaGetErrorString(err));
}

int pipe_for_current_device(Pipe** out) {
    int device = 0;
    HOST_CUDA_TRY(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(g_pipes_mutex);
    *out = &g_pipes[device];   // std::map nodes never move
    return CREDIT_OK;
}

struct BlockLayout {
    int64_t min_block_rows = 0;
    int64_t max_blocks = 0;
};

BlockLayout block_layout(int64_t rows, const BlockArray* arrays, int n) {
    size_t per_row = 0;
    for (int i = 0; i < n; ++i) per_row += arrays[i].row_bytes;
    BlockLayout l;
    l.min_block_rows = std::min<int64_t>(rows, std::max<int64_t>(1, static_cast<int64_t>(kMinBlockBytes / std::max<size_t>(per_row, 1))));
    l.max_blocks = (rows + l.min_block_rows - 1) / l.min_block_rows;
    return l;
}

size_t block_set_bytes(int64_t block_rows, const BlockArray* arrays, int n) {
    size_t total = 0;
    for (int i = 0; i < n; ++i) total += align_up(static_cast<size_t>(block_rows) * arrays[i].row_bytes);
    return total;
}

// Streams `rows` rows through `blocks_base` (two sets of per-array device buffers).
// launch(block, first_row, count, device_arrays, compute_stream) enqueues the kernels of one block.
template <typename Launch>
int run_blocks(int64_t rows, const BlockArray* arrays, int n, unsigned char* blocks_base, size_t blocks_bytes,
               cudaStream_t compute, Launch launch, int64_t* blocks_done) {
    const BlockLayout layout = block_layout(rows, arrays, n);
    // the largest block two sets of which fit
    int64_t block_rows = rows;
    while (block_rows > layout.min_block_rows && 2 * block_set_bytes(block_rows, arrays, n) > blocks_bytes)
        block_rows = std::max<int64_t>(layout.min_block_rows, (block_rows + 1) / 2);
    const size_t set_bytes = block_set_bytes(block_rows, arrays, n);
    if (2 * set_bytes > blocks_bytes)
        return report_error(CREDIT_ERR_WORKSPACE, "scratch cannot hold two blocks of %lld rows",
                            static_cast<long long>(block_rows));
    void* dev[2][8];
    for (int b = 0; b < 2; ++b) {
        unsigned char* at = blocks_base + b * set_bytes;
        for (int i = 0; i < n; ++i) {
            dev[b][i] = at;
            at += align_up(static_cast<size_t>(block_rows) * arrays[i].row_bytes);
        }
    }

    Pipe* pipe = nullptr;
    int rc = pipe_for_current_device(&pipe);
    if (rc != CREDIT_OK) return rc;
    std::lock_guard<std::mutex> busy(pipe->busy);
    if (!pipe->ready) {
        rc = create(*pipe);
        if (rc != CREDIT_OK) {
            destroy(*pipe);
            return rc;
        }
        pipe->ready = true;
    }
    auto drain_all = [&]() {
        cudaStreamSynchronize(pipe->upload);
        cudaStreamSynchronize(compute);
        cudaStreamSynchronize(pipe->download);
    };
#define PIPE_TRY(expr)                                                                                \
    do {                                                                                              \
        cudaError_t err__ = (expr);                                                                   \
        if (err__ != cudaSuccess) {                                                                   \
            drain_all();                                                                              \
            return report_error(CREDIT_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(err__));         \
        }                                                                                             \
    } while (0)

    // the scratch may still be in use by earlier work of the caller on `compute`
    PIPE_TRY(cudaEventRecord(pipe->start, compute));
    PIPE_TRY(cudaStreamWaitEvent(pipe->upload, pipe->start, 0));
    int64_t block = 0;
    for (int64_t r0 = 0; r0 < rows; r0 += block_rows, ++block) {
        const int64_t count = std::min(block_rows, rows - r0);
        const int b = static_cast<int>(block & 1);
        if (block >= 2) PIPE_TRY(cudaStreamWaitEvent(pipe->upload, pipe->computed[b], 0));   // inputs consumed
        for (int i = 0; i < n; ++i) {
            if (arrays[i].host_src == nullptr) continue;
            PIPE_TRY(cudaMemcpyAsync(dev[b][i],
                                     static_cast<const unsigned char*>(arrays[i].host_src) + static_cast<size_t>(r0) * arrays[i].row_bytes,
                                     static_cast<size_t>(count) * arrays[i].row_bytes, cudaMemcpyHostToDevice, pipe->upload));
        }
        PIPE_TRY(cudaEventRecord(pipe->loaded[b], pipe->upload));
        PIPE_TRY(cudaStreamWaitEvent(compute, pipe->loaded[b], 0));
        if (block >= 2) PIPE_TRY(cudaStreamWaitEvent(compute, pipe->drained[b], 0));         // outputs copied out
        rc = launch(block, r0, count, dev[b], compute);
        if (rc != CREDIT_OK) {
            drain_all();
            return rc;
        }
        PIPE_TRY(cudaEventRecord(pipe->computed[b], compute));
        PIPE_TRY(cudaStreamWaitEvent(pipe->download, pipe->computed[b], 0));
        for (int i = 0; i < n; ++i) {
            if (arrays[i].host_dst == nullptr) continue;
            PIPE_TRY(cudaMemcpyAsync(static_cast<unsigned char*>(arrays[i].host_dst) + static_cast<size_t>(r0) * arrays[i].row_bytes,
                                     dev[b][i], static_cast<size_t>(count) * arrays[i].row_bytes, cudaMemcpyDeviceToHost,
                                     pipe->download));
        }
        PIPE_TRY(cudaEventRecord(pipe->drained[b], pipe->download));
    }
    PIPE_TRY(cudaStreamSynchronize(pipe->download));
    PIPE_TRY(cudaStreamSynchronize(compute));
#undef PIPE_TRY
    if (blocks_done != nullptr) *blocks_done = block;
    return CREDIT_OK;
}

int check_common(int64_t rows, int64_t cols, const void* scratch, size_t scratch_bytes, size_t need) {
    if (rows < 0 || rows > (1ll << 30) || cols < 1 || cols > (1ll << 30))
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "rows=%lld, cols=%lld out of range",
                            static_cast<long long>(rows), static_cast<long long>(cols));
    if (rows > 0 && (scratch == nullptr || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255u)))
        return report_error(CREDIT_ERR_WORKSPACE, "scratch of %zu B given, %zu B (256-byte aligned) needed",
                            scratch_bytes, need);
    return CREDIT_OK;
}

size_t elem_bytes(int dtype) { return dtype == CREDIT_BF16 ? 2 : 4; }

// scratch = [fixed region][two block sets]
size_t scratch_need(int64_t rows, size_t fixed, const BlockArray* arrays, int n) {
    if (rows <= 0) return 0;
    return align_up(fixed) + 2 * block_set_bytes(block_layout(rows, arrays, n).min_block_rows, arrays, n);
}

}  // namespace

extern "C" {

// ---- row reduction ---------------------------------------------------------------------------
size_t credit_row_reduce_host_scratch_bytes(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0) return 0;
    const BlockArray arrays[4] = {{nullptr, nullptr, static_cast<size_t>(cols) * 4}, {nullptr, nullptr, 4},
                                  {nullptr, nullptr, 4}, {nullptr, nullptr, 8}};
    return scratch_need(rows, 0, arrays, 4);
}

int credit_row_reduce_host(const float* x_host, float* out_sum_host, float* out_max_host, int64_t* out_argmax_host,
                           int64_t rows, int64_t cols, const credit_launch_opts* opts, void* scratch,
                           size_t scratch_bytes, void* stream) {
    if (x_host == nullptr || out_sum_host == nullptr || out_max_host == nullptr || out_argmax_host == nullptr)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "host input and outputs must not be NULL");
    int rc = check_common(rows, cols, scratch, scratch_bytes, credit_row_reduce_host_scratch_bytes(rows, cols));
    if (rc != CREDIT_OK || rows == 0) return rc;
    const BlockArray arrays[4] = {{x_host, nullptr, static_cast<size_t>(cols) * 4}, {nullptr, out_sum_host, 4},
                                  {nullptr, out_max_host, 4}, {nullptr, out_argmax_host, 8}};
    auto launch = [&](int64_t, int64_t, int64_t count, void* const* dev, cudaStream_t s) {
        return credit_row_reduce(static_cast<const float*>(dev[0]), static_cast<float*>(dev[1]),
                                 static_cast<float*>(dev[2]), static_cast<int64_t*>(dev[3]), count, cols, opts, s);
    };
    return run_blocks(rows, arrays, 4, static_cast<unsigned char*>(scratch), scratch_bytes,
                      static_cast<cudaStream_t>(stream), launch, nullptr);
}

// ---- RMSNorm forward -------------------------------------------------------------------------
size_t credit_rmsnorm_forward_host_scratch_bytes(int64_t rows, int64_t cols, int dtype) {
    if (rows <= 0 || cols <= 0) return 0;
    const size_t row = static_cast<size_t>(cols) * elem_bytes(dtype);
    const BlockArray arrays[2] = {{nullptr, nullptr, row}, {nullptr, nullptr, row}};
    return scratch_need(rows, static_cast<size_t>(cols) * 4, arrays, 2);
}

int credit_rmsnorm_forward_host(const void* x_host, const float* gamma_host, void* y_host, int64_t rows, int64_t cols,
                                float eps, int dtype, const credit_launch_opts* opts, void* scratch,
                                size_t scratch_bytes, void* stream) {
    if (x_host == nullptr || gamma_host == nullptr || y_host == nullptr)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "x, gamma and y must not be NULL");
    if (dtype != CREDIT_F32 && dtype != CREDIT_BF16) return report_error(CREDIT_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
    int rc = check_common(rows, cols, scratch, scratch_bytes, credit_rmsnorm_forward_host_scratch_bytes(rows, cols, dtype));
    if (rc != CREDIT_OK || rows == 0) return rc;
    const size_t row = static_cast<size_t>(cols) * elem_bytes(dtype);
    const BlockArray arrays[2] = {{x_host, nullptr, row}, {nullptr, y_host, row}};
    cudaStream_t compute = static_cast<cudaStream_t>(stream);
    unsigned char* base = static_cast<unsigned char*>(scratch);
    float* gamma = reinterpret_cast<float*>(base);
    const size_t fixed = align_up(static_cast<size_t>(cols) * 4);
    HOST_CUDA_TRY(cudaMemcpyAsync(gamma, gamma_host, static_cast<size_t>(cols) * 4, cudaMemcpyHostToDevice, compute));
    auto launch = [&](int64_t, int64_t, int64_t count, void* const* dev, cudaStream_t s) {
        return credit_rmsnorm_forward(dev[0], gamma, dev[1], count, cols, eps, dtype, opts, s);
    };
    return run_blocks(rows, arrays, 2, base + fixed, scratch_bytes - fixed, compute, launch, nullptr);
}

// ---- LayerNorm forward -----------------------------------------------------------------------
size_t credit_layernorm_forward_host_scratch_bytes(int64_t rows, int64_t cols, int dtype) {
    if (rows <= 0 || cols <= 0) return 0;
    const size_t row = static_cast<size_t>(cols) * elem_bytes(dtype);
    const BlockArray arrays[4] = {{nullptr, nullptr, row}, {nullptr, nullptr, row}, {nullptr, nullptr, 4}, {nullptr, nullptr, 4}};
    return scratch_need(rows, 2 * align_up(static_cast<size_t>(cols) * 4), arrays, 4);
}

int credit_layernorm_forward_host(const void* x_host, const float* gamma_host, const float* beta_host, void* y_host,
                                  float* mean_host, float* rstd_host, int64_t rows, int64_t cols, float eps, int dtype,
                                  const credit_launch_opts* opts, void* scratch, size_t scratch_bytes, void* stream) {
    if (x_host == nullptr || gamma_host == nullptr || beta_host == nullptr || y_host == nullptr || mean_host == nullptr ||
        rstd_host == nullptr)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "x, gamma, beta, y, mean and rstd must not be NULL");
    if (dtype != CREDIT_F32 && dtype != CREDIT_BF16) return report_error(CREDIT_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
    int rc = check_common(rows, cols, scratch, scratch_bytes, credit_layernorm_forward_host_scratch_bytes(rows, cols, dtype));
    if (rc != CREDIT_OK || rows == 0) return rc;
    const size_t row = static_cast<size_t>(cols) * elem_bytes(dtype);
    const BlockArray arrays[4] = {{x_host, nullptr, row}, {nullptr, y_host, row}, {nullptr, mean_host, 4}, {nullptr, rstd_host, 4}};
    cudaStream_t compute = static_cast<cudaStream_t>(stream);
    unsigned char* base = static_cast<unsigned char*>(scratch);
    const size_t vec = align_up(static_cast<size_t>(cols) * 4);
    float* gamma = reinterpret_cast<float*>(base);
    float* beta = reinterpret_cast<float*>(base + vec);
    HOST_CUDA_TRY(cudaMemcpyAsync(gamma, gamma_host, static_cast<size_t>(cols) * 4, cudaMemcpyHostToDevice, compute));
    HOST_CUDA_TRY(cudaMemcpyAsync(beta, beta_host, static_cast<size_t>(cols) * 4, cudaMemcpyHostToDevice, compute));
    auto launch = [&](int64_t, int64_t, int64_t count, void* const* dev, cudaStream_t s) {
        return credit_layernorm_forward(dev[0], gamma, beta, dev[1], static_cast<float*>(dev[2]), static_cast<float*>(dev[3]),
                                        count, cols, eps, dtype, opts, s);
    };
    return run_blocks(rows, arrays, 4, base + 2 * vec, scratch_bytes - 2 * vec, compute, launch, nullptr);
}

// ---- LayerNorm backward with given statistics ------------------------------------------------
namespace {
struct BackwardFixed {
    size_t vec = 0;         // gamma: one [cols] fp32 vector, padded to the alignment
    size_t slots = 0;       // (max_blocks + 1) x [2, cols] fp32, densely packed: per-block column sums, then the total
    size_t workspace = 0;   // the kernels' own workspace for one block
    size_t total() const { return vec + slots + workspace; }
};
BackwardFixed backward_fixed(int64_t rows, int64_t cols, int dtype, const credit_launch_opts* opts, const BlockArray* arrays) {
    BackwardFixed f;
    f.vec = align_up(static_cast<size_t>(cols) * 4);
    const BlockLayout layout = block_layout(rows, arrays, 5);
    f.slots = align_up(static_cast<size_t>(layout.max_blocks + 1) * 2 * static_cast<size_t>(cols) * 4);
    // a block never has more rows than the matrix, and the workspace does not shrink with rows
    f.workspace = align_up(credit_layernorm_backward_stats_workspace_bytes(rows, cols, dtype, opts));
    return f;
}
}  // namespace

namespace {
size_t backward_scratch_need(int64_t rows, int64_t cols, int dtype, const credit_launch_opts* opts) {
    if (rows <= 0 || cols <= 0) return 0;
    const size_t row = static_cast<size_t>(cols) * elem_bytes(dtype);
    const BlockArray arrays[5] = {{nullptr, nullptr, row}, {nullptr, nullptr, row}, {nullptr, nullptr, 4},
                                  {nullptr, nullptr, 4}, {nullptr, nullptr, row}};
    return scratch_need(rows, backward_fixed(rows, cols, dtype, opts, arrays).total(), arrays, 5);
}
}  // namespace

size_t credit_layernorm_backward_stats_host_scratch_bytes(int64_t rows, int64_t cols, int dtype,
                                                          const credit_launch_opts* opts) {
    return backward_scratch_need(rows, cols, dtype, opts);
}

int credit_layernorm_backward_stats_host(const void* x_host, const void* dy_host, const float* gamma_host,
                                         const float* mean_host, const float* rstd_host, void* dx_host,
                                         float* dgamma_host, float* dbeta_host, int64_t rows, int64_t cols, int dtype,
                                         const credit_launch_opts* opts, void* scratch, size_t scratch_bytes, void* stream) {
    if (x_host == nullptr || dy_host == nullptr || gamma_host == nullptr || mean_host == nullptr || rstd_host == nullptr ||
        dx_host == nullptr || dgamma_host == nullptr || dbeta_host == nullptr)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "inputs and outputs must not be NULL");
    if (dtype != CREDIT_F32 && dtype != CREDIT_BF16) return report_error(CREDIT_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
    int rc = check_common(rows, cols, scratch, scratch_bytes, backward_scratch_need(rows, cols, dtype, opts));
    if (rc != CREDIT_OK) return rc;
    cudaStream_t compute = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
        std::fill(dgamma_host, dgamma_host + cols, 0.0f);
        std::fill(dbeta_host, dbeta_host + cols, 0.0f);
        return CREDIT_OK;
    }
    const size_t row = static_cast<size_t>(cols) * elem_bytes(dtype);
    const BlockArray arrays[5] = {{x_host, nullptr, row}, {dy_host, nullptr, row}, {mean_host, nullptr, 4},
                                  {rstd_host, nullptr, 4}, {nullptr, dx_host, row}};
    const BackwardFixed fixed = backward_fixed(rows, cols, dtype, opts, arrays);
    unsigned char* base = static_cast<unsigned char*>(scratch);
    float* gamma = reinterpret_cast<float*>(base);
    unsigned char* slots = base + fixed.vec;
    void* workspace = slots + fixed.slots;
    auto slot = [&](int64_t block, int which) {
        return reinterpret_cast<float*>(slots) + (2 * block + which) * static_cast<size_t>(cols);
    };
    HOST_CUDA_TRY(cudaMemcpyAsync(gamma, gamma_host, static_cast<size_t>(cols) * 4, cudaMemcpyHostToDevice, compute));
    auto launch = [&](int64_t block, int64_t, int64_t count, void* const* dev, cudaStream_t s) {
        return credit_layernorm_backward_stats(dev[0], dev[1], gamma, static_cast<const float*>(dev[2]),
                                               static_cast<const float*>(dev[3]), dev[4], slot(block, 0), slot(block, 1),
                                               count, cols, dtype, opts, workspace, fixed.workspace, s);
    };
    int64_t blocks = 0;
    rc = run_blocks(rows, arrays, 5, base + fixed.total(), scratch_bytes - fixed.total(), compute, launch, &blocks);
    if (rc != CREDIT_OK) return rc;
    // the per-block sums are laid out like per-cluster partials, [blocks][2][cols]: one more pass of the
    // finishing kernel adds them (in block order: deterministic)
    const float* total = slot(0, 0);
    if (blocks > 1) {
        HOST_CUDA_TRY(credit::launch_layernorm_bwd_finish(slot(0, 0), slot(blocks, 0), slot(blocks, 1),
                                                          static_cast<int>(cols), static_cast<int>(blocks), compute));
        total = slot(blocks, 0);
    }
    HOST_CUDA_TRY(cudaMemcpyAsync(dgamma_host, total, static_cast<size_t>(cols) * 4, cudaMemcpyDeviceToHost, compute));
    HOST_CUDA_TRY(cudaMemcpyAsync(dbeta_host, total + cols, static_cast<size_t>(cols) * 4, cudaMemcpyDeviceToHost,
                                  compute));
    HOST_CUDA_TRY(cudaStreamSynchronize(compute));
    return CREDIT_OK;
}

// ---- fused FFN -------------------------------------------------------------------------------
size_t credit_ffn_forward_host_scratch_bytes(int64_t m, int64_t d, int64_t h) {
    const size_t ws = credit_ffn_workspace_bytes(m, d, h);
    if (ws == 0) return 0;
    return align_up(ws) + 2 * align_up(static_cast<size_t>(m) * static_cast<size_t>(d) * 2);
}

int credit_ffn_forward_host(const void* x_host, const void* w1_packed, const void* w2_packed, const float* gamma,
                            void* y_host, int64_t m, int64_t d, int64_t h, float eps, void* scratch,
                            size_t scratch_bytes, void* stream) {
    if (x_host == nullptr || y_host == nullptr)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "x and y must not be NULL");
    const size_t need = credit_ffn_forward_host_scratch_bytes(m, d, h);
    if (need == 0) return report_error(CREDIT_ERR_UNSUPPORTED, "ffn shape m=%lld d=%lld h=%lld is not supported",
                                       static_cast<long long>(m), static_cast<long long>(d), static_cast<long long>(h));
    if (scratch == nullptr || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 255u))
        return report_error(CREDIT_ERR_WORKSPACE, "scratch of %zu B given, %zu B (256-byte aligned) needed", scratch_bytes, need);
    cudaStream_t compute = static_cast<cudaStream_t>(stream);
    unsigned char* base = static_cast<unsigned char*>(scratch);
    const size_t ws = align_up(credit_ffn_workspace_bytes(m, d, h));
    const size_t act = static_cast<size_t>(m) * static_cast<size_t>(d) * 2;
    void* x = base + ws;
    void* y = base + ws + align_up(act);
    // every row needs both weight matrices in full, so the rows are not cut into blocks: a second
    // block would stream the weights through the chip a second time
    HOST_CUDA_TRY(cudaMemcpyAsync(x, x_host, act, cudaMemcpyHostToDevice, compute));
    int rc = credit_ffn_forward(x, w1_packed, w2_packed, gamma, y, m, d, h, eps, base, ws, compute);
    if (rc != CREDIT_OK) {
        cudaStreamSynchronize(compute);
        return rc;
    }
    HOST_CUDA_TRY(cudaMemcpyAsync(y_host, y, act, cudaMemcpyDeviceToHost, compute));
    HOST_CUDA_TRY(cudaStreamSynchronize(compute));
    return CREDIT_OK;
}

}  // extern "C"
