/*
 * credit_b200 -- C ABI of the sm_100a wide-row cluster/DSMEM kernels.
 *
 * The reference project (CREDIT) has no library boundary: its evaluation
 * pipeline spawns one executable per workload (dsmem_eval/runner.py:280-347) and
 * calls Triton through an in-process launcher table
 * (dsmem_eval/triton_kernels.py:300-400). This header is the boundary a
 * maintainer binds with ctypes to add a third, native backend: every entry point
 * below names the reference interface it stands in for.
 *
 * Conventions
 *  - Every function returns CREDIT_OK (0) or a negative credit_status; nothing
 *    exits the process or throws (the reference's CUDA_CHECK calls std::exit,
 *    src/workloads/layernorm_backward.cu:20-28). credit_last_error() gives the
 *    text for the calling thread's last failure.
 *  - Matrix pointers are caller-owned DEVICE pointers to row-major, densely
 *    packed [rows, cols] arrays on the current device. gamma/beta/dgamma/dbeta
 *    are always fp32 [cols]; per-row statistics are fp32 [rows].
 *  - Launches are asynchronous on `stream` (a cudaStream_t passed as void*; NULL
 *    is the default stream). No call allocates device memory or synchronises,
 *    except where stated.
 *  - Rows whose byte length is a multiple of 16 with 16-byte aligned base
 *    pointers take the bulk-copy/128-bit path; anything else is served by scalar
 *    kernels with the same results.
 *  - `opts` may be NULL (all fields 0 = automatic).
 */
#ifndef CREDIT_B200_H
#define CREDIT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum credit_status {
    CREDIT_OK = 0,
    CREDIT_ERR_INVALID_ARGUMENT = -1, /* bad pointer, size, dtype or option */
    CREDIT_ERR_UNSUPPORTED = -2,      /* shape does not fit the requested variant (the
                                         reference prints "n/a" for such a variant,
                                         layernorm_backward.cu:508-511, 563-565) */
    CREDIT_ERR_CUDA = -3,             /* a CUDA runtime call failed */
    CREDIT_ERR_WORKSPACE = -4,        /* workspace missing or too small */
    CREDIT_ERR_DEVICE_STATUS = -5     /* a kernel reported a timeout or bad geometry */
} credit_status;

typedef enum credit_dtype { CREDIT_F32 = 0, CREDIT_BF16 = 1 } credit_dtype;

/* Variant names follow the reference's RESULT lines
 * (layernorm_backward.cu:489, 517, 555). */
typedef enum credit_variant {
    CREDIT_VARIANT_AUTO = 0,
    CREDIT_VARIANT_BLOCK_READ = 1,   /* one CTA per row, no staging, re-reads global memory */
    CREDIT_VARIANT_BLOCK_SMEM = 2,   /* one CTA per row, row staged in shared memory */
    CREDIT_VARIANT_CLUSTER_SMEM = 3  /* row split over a cluster, partials through DSMEM */
} credit_variant;

typedef enum credit_load_path {
    CREDIT_LOAD_AUTO = 0,
    CREDIT_LOAD_TMA = 1,  /* bulk-async copies into a shared-memory ring */
    CREDIT_LOAD_LDG = 2   /* 128-bit read-only loads into registers (streaming kernels) */
} credit_load_path;

typedef enum credit_schedule {
    CREDIT_SCHEDULE_AUTO = 0,
    CREDIT_SCHEDULE_ROW_PER_CLUSTER = 1, /* grid = rows clusters */
    CREDIT_SCHEDULE_PERSISTENT = 2       /* grid = resident clusters, each walks many rows */
} credit_schedule;

typedef enum credit_launch_flags {
    /* Keep aligned rows on the generic shared-memory kernels (every pass re-reads the
     * staged slice, cluster barrier exchange) instead of the register-resident ones. */
    CREDIT_FLAG_NO_REGISTER_PATH = 1
} credit_launch_flags;

typedef struct credit_launch_opts {
    int cluster_size; /* CTAs per row: 1,2,4,8,16; 0 = automatic (the smallest cluster whose ring is deep
                         enough: a rule calibrated on B200 sweeps) */
    int variant;      /* credit_variant */
    int stages;       /* shared-memory ring depth: 1..8, up to 16 for the warp-specialised kernels (which
                         need at least 3); 0 = automatic */
    int threads;      /* threads per CTA selects the kernel form: 352 / 608 = warp-specialised pipeline
                         with 8 / 16 output warps and three service warps (the default for 16-byte
                         aligned rows, except fp32 RMSNorm), 256 / 512 = lock-step kernels; 0 = automatic */
    int schedule;     /* credit_schedule */
    int load_path;    /* credit_load_path (streaming kernels) */
    int chunk_bytes;  /* ring chunk of the streaming kernels, multiple of 1024; 0 = automatic */
    int flags;        /* credit_launch_flags, OR-ed */
} credit_launch_opts;

/* The fields of DeviceInfo in the reference binaries
 * (layernorm_backward.cu:50-58, query_device_info :440-468) plus what the cost
 * model needs. */
typedef struct credit_device_info {
    char name[256];
    int sm_major;
    int sm_minor;
    int sm_count;
    int cluster_launch;            /* cudaDevAttrClusterLaunch */
    int max_cluster_size;          /* largest cluster this library will launch (16 on sm_100) */
    int max_dynamic_smem_per_block; /* sharedMemPerBlockOptin */
    int smem_per_sm;
    int l2_bytes;
    int clock_khz;                 /* maximum SM clock */
    int mem_clock_khz;
    int mem_bus_bits;
} credit_device_info;

typedef enum credit_workload {
    CREDIT_WL_RMSNORM_FORWARD = 0,
    CREDIT_WL_ROW_REDUCE = 1,
    CREDIT_WL_LAYERNORM_FORWARD = 2,
    CREDIT_WL_LAYERNORM_BACKWARD = 3,      /* statistics recomputed, dx only */
    CREDIT_WL_LAYERNORM_BACKWARD_STATS = 4, /* statistics given, dx + dgamma + dbeta */
    /* the other workloads of the reference sweep (fp32), through credit_row_op */
    CREDIT_WL_WEIGHTED_VAR_BACKWARD = 5,
    CREDIT_WL_PEARSON_BACKWARD = 6,
    CREDIT_WL_SOFTMAX_LOGITS_BACKWARD = 7,
    CREDIT_WL_LARS_MOMENTUM = 8,
    CREDIT_WL_ROWWISE_QUANT = 9
} credit_workload;

/* What a call would launch: the resolved form of credit_launch_opts. */
typedef struct credit_plan_info {
    int cluster_size;
    int variant;
    int stages;
    int threads;
    int schedule;
    int load_path;
    int aligned;            /* 1 = 16-byte path */
    int slice_elems;        /* columns per CTA */
    int chunk_elems;        /* streaming kernels: columns per ring chunk */
    int vectors_per_thread; /* register path: 16-byte vectors each thread owns; 0 = generic path */
    int full_tiles;         /* register path: every thread owns exactly that many (no bounds checks) */
    int num_clusters;       /* clusters in the grid */
    int grid_ctas;
    int smem_bytes;         /* dynamic shared memory per CTA */
    int kernel_launches;    /* kernels one call enqueues */
    size_t workspace_bytes;
} credit_plan_info;

/* Library and device ---------------------------------------------------- */

/* Text of the calling thread's last failure ("" if none). */
const char* credit_last_error(void);

/* Replaces query_device_info (layernorm_backward.cu:440-468). device < 0 means
 * the current device. */
int credit_query_device(int device, credit_device_info* info);

/* Reads (and optionally clears) the current device's status word: bit 0 = an
 * mbarrier wait timed out, bit 1 = a kernel refused its launch geometry.
 * Synchronises the device. Returns CREDIT_ERR_DEVICE_STATUS if any bit is set. */
int credit_device_status(int* status_out, int reset);

/* Resolves opts for a workload and shape without launching. Replaces the
 * shape gating in benchmark_block_staged / benchmark_cluster
 * (layernorm_backward.cu:499-593). */
int credit_plan(int workload, int64_t rows, int64_t cols, int dtype,
                const credit_launch_opts* opts, credit_plan_info* plan);

/* Workloads -------------------------------------------------------------- */

/* y = x * rsqrt(mean_row(x^2) + eps) * gamma. x, y: dtype [rows, cols].
 * No reference kernel exists for this workload; it runs on the same cluster
 * core as cluster_bwd_staged_kernel (layernorm_backward.cu:376-438) with one
 * reduction stage of one partial. */
int credit_rmsnorm_forward(const void* x, const float* gamma, void* y, int64_t rows, int64_t cols,
                           float eps, int dtype, const credit_launch_opts* opts, void* stream);

/* Per-row sum, maximum and index of the first maximum of fp32 x [rows, cols].
 * The max-type one-stage reduction of cluster_quant_staged_kernel
 * (rowwise_quant.cu:321-363) with the column index carried along.
 * out_argmax is int64 [rows]. */
int credit_row_reduce(const float* x, float* out_sum, float* out_max, int64_t* out_argmax,
                      int64_t rows, int64_t cols, const credit_launch_opts* opts, void* stream);

/* y = (x - mean) * rstd * gamma + beta, rstd = rsqrt(var + eps) (biased var).
 * mean, rstd: fp32 [rows] outputs. No reference kernel; same cluster core. */
int credit_layernorm_forward(const void* x, const float* gamma, const float* beta, void* y,
                             float* mean, float* rstd, int64_t rows, int64_t cols, float eps,
                             int dtype, const credit_launch_opts* opts, void* stream);

/* dx of LayerNorm with the row statistics recomputed from x. Replaces
 * block_bwd_read_kernel / block_bwd_staged_kernel / cluster_bwd_staged_kernel
 * (layernorm_backward.cu:274-438) and launch_layernorm_backward
 * (dsmem_eval/triton_kernels.py:300-312); formula of
 * dsmem_eval/workloads.py:53-61. */
int credit_layernorm_backward(const void* x, const void* dy, const float* gamma, void* dx,
                              int64_t rows, int64_t cols, float eps, int dtype,
                              const credit_launch_opts* opts, void* stream);

/* LayerNorm backward with given statistics: dx plus the column sums
 * dgamma = sum_rows dy * xhat and dbeta = sum_rows dy (fp32 [cols]); dgamma and
 * dbeta may both be NULL to skip them. Needs a device workspace of at least
 * credit_layernorm_backward_stats_workspace_bytes() (per-cluster partial column
 * sums; contents are overwritten). Extends cluster_bwd_staged_kernel to the
 * bf16 / precomputed-statistics / parameter-gradient form. */
size_t credit_layernorm_backward_stats_workspace_bytes(int64_t rows, int64_t cols, int dtype,
                                                       const credit_launch_opts* opts);
int credit_layernorm_backward_stats(const void* x, const void* dy, const float* gamma,
                                    const float* mean, const float* rstd, void* dx, float* dgamma,
                                    float* dbeta, int64_t rows, int64_t cols, int dtype,
                                    const credit_launch_opts* opts, void* workspace,
                                    size_t workspace_bytes, void* stream);

/* The other five workloads of the reference sweep, fp32, on the same cluster core
 * (slices staged once in shared memory, partial sums / maxima exchanged through
 * DSMEM, 2 to 3 dependent reductions). `workload` selects the formula:
 *   CREDIT_WL_WEIGHTED_VAR_BACKWARD   in0 x, in1 weight, in2 dy        -> out0 dx
 *       (weighted_var_backward.cu:426, dsmem_eval/workloads.py:72-87)
 *   CREDIT_WL_PEARSON_BACKWARD        in0 x, in1 y, row_in grad [rows] -> out0 dx, out1 dy
 *       (pearson_backward.cu:417, workloads.py:98-115)
 *   CREDIT_WL_SOFTMAX_LOGITS_BACKWARD in0 logits, in1 dy               -> out0 dlogits
 *       (softmax_logits_backward.cu:410, workloads.py:125-128)
 *   CREDIT_WL_LARS_MOMENTUM           in0 weight, in1 grad, in2 momentum -> out0 weight', out1 update
 *       (lars_momentum.cu:364, workloads.py:139-147)
 *   CREDIT_WL_ROWWISE_QUANT           in0 x -> out0 int8 q [rows, cols], row_out scale [rows]
 *       (rowwise_quant.cu:321, workloads.py:153-157)
 * Unused pointers must be NULL. Inputs and outputs are [rows, cols] row-major. */
int credit_row_op(int workload, const float* in0, const float* in1, const float* in2, const float* row_in,
                  void* out0, void* out1, float* row_out, int64_t rows, int64_t cols,
                  const credit_launch_opts* opts, void* stream);

/* Times `iters` back-to-back calls of a workload (after `warmup` calls) with CUDA
 * events, on device buffers this call allocates, fills with deterministic values and
 * frees again; *avg_ms receives the time per call. `workload` is one of the ten
 * names ("rmsnorm_forward", "row_reduce", "layernorm_forward", "layernorm_backward",
 * "layernorm_backward_stats", "weighted_var_backward", "pearson_backward",
 * "softmax_logits_backward", "lars_momentum", "rowwise_quant"); cluster_size 0 and
 * variant CREDIT_VARIANT_AUTO let the planner choose. A variant that does not fit
 * the shape returns CREDIT_ERR_UNSUPPORTED (the reference prints n/a). Replaces
 * time_kernel + benchmark_block_read / benchmark_block_staged / benchmark_cluster of
 * the reference binaries (layernorm_backward.cu:150-175, 480-593). Synchronous; not
 * for use on a hot path. */
int credit_bench(const char* workload, int64_t rows, int64_t cols, int dtype, int cluster_size, int variant,
                 int warmup, int iters, double* avg_ms);

/* Fused FFN, bf16 with fp32 accumulation on the tensor cores:
 *   H = GELU(X W1)  (exact erf GELU, b1 = 0),  Y = RMSNorm(H W2 + X) * gamma.
 * X, Y: bf16 [m, d]; gamma fp32 [d]; W1 [d, h] and W2 [h, d] are given PACKED
 * K-major, i.e. transposed once with credit_ffn_pack_weight(w [k, n] -> packed [n, k]):
 * w1_packed is [h, d], w2_packed is [d, h]. `workspace` (credit_ffn_workspace_bytes)
 * holds the hidden activations. Shapes: m % 128 == 0, d % 256 == 0, d <= 4096,
 * h % 256 == 0; anything else returns CREDIT_ERR_UNSUPPORTED. The row statistics
 * of the RMSNorm are reduced across the CTAs of a cluster through DSMEM in the
 * epilogue of the second GEMM. No reference kernel or function exists for this
 * workload; the exchange follows cluster_reduce_pair
 * (src/workloads/layernorm_backward.cu:217-251). */
int credit_ffn_pack_weight(const void* w, void* packed, int64_t k, int64_t n, void* stream);
size_t credit_ffn_workspace_bytes(int64_t m, int64_t d, int64_t h);
int credit_ffn_forward(const void* x, const void* w1_packed, const void* w2_packed, const float* gamma,
                       void* y, int64_t m, int64_t d, int64_t h, float eps, void* workspace,
                       size_t workspace_bytes, void* stream);

/* The same computation as credit_layernorm_backward_stats for callers that cannot
 * obtain device memory for the workspace: code running where the CUDA allocator
 * must not be called (for example between launches of a latency-critical serving
 * loop, where cudaMalloc would stall the device, or in a host that gives a plug-in
 * no allocator of its own). The partial column sums go into a 16 MiB array that
 * is built into the library image, so nothing is allocated or freed by this call
 * or by anything it calls; credit_layernorm_backward_stats_static_capacity()
 * returns that size. The array counts as aligned, so the scratch a call needs is
 * that of the path its own pointers select: for 16-byte aligned x, dy, gamma and dx
 * one [2, cols] fp32 partial per resident cluster (7.5 MiB at bf16 8192 x 65536),
 * otherwise one per block of 128 rows. A call that needs more is refused with
 * CREDIT_ERR_WORKSPACE and a message before any pointer is used; with dgamma and
 * dbeta NULL no scratch is used and no size is checked. Inputs and outputs are
 * still the caller's.
 *
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress) and reads the device's properties, and the CUDA runtime
 * may load the library's device code, which contains the array, at that moment:
 * make that first call before any stream capture begins, and count the 16 MiB as
 * held by every device that has made it. All calls on a device share the one array and
 * it keeps whatever the last call left there; no part of it needs clearing,
 * because a call writes every partial sum it later reads. For the same reason two
 * calls whose kernels overlap on the GPU (different streams, or different host
 * threads) corrupt each other's column sums: run them one after another.
 *
 * This entry point has no counterpart in the reference. */
size_t credit_layernorm_backward_stats_static_capacity(void);
int credit_layernorm_backward_stats_static(const void* x, const void* dy, const float* gamma,
                                           const float* mean, const float* rstd, void* dx,
                                           float* dgamma, float* dbeta, int64_t rows, int64_t cols,
                                           int dtype, const credit_launch_opts* opts, void* stream);

/* Host-buffer entry points ----------------------------------------------- */

/* The workloads above on HOST data. Every matrix and vector argument named *_host is
 * host memory; `scratch` is caller-owned DEVICE memory (256-byte aligned) of at least
 * the matching *_host_scratch_bytes(). A matrix is streamed through the scratch in row
 * blocks on three streams: the upload of block k+1, the kernels of block k and the
 * download of block k-1 overlap. More scratch than the minimum lets the blocks grow,
 * up to the whole matrix. Pinned host memory makes the copies asynchronous to each
 * other; pageable memory works but serialises them. A call returns after its results
 * are in host memory (it synchronises `stream`). Calls on one device run one after
 * the other (the library holds one set of copy streams per device). This is the shape
 * of run_shape in the reference executables (layernorm_backward.cu:767-805), which own
 * their device buffers, with the allocation moved to the caller and the copies
 * pipelined; the kernels are the ones of the device-pointer entry points. */
size_t credit_row_reduce_host_scratch_bytes(int64_t rows, int64_t cols);
int credit_row_reduce_host(const float* x_host, float* out_sum_host, float* out_max_host,
                           int64_t* out_argmax_host, int64_t rows, int64_t cols,
                           const credit_launch_opts* opts, void* scratch, size_t scratch_bytes,
                           void* stream);

size_t credit_rmsnorm_forward_host_scratch_bytes(int64_t rows, int64_t cols, int dtype);
int credit_rmsnorm_forward_host(const void* x_host, const float* gamma_host, void* y_host, int64_t rows,
                                int64_t cols, float eps, int dtype, const credit_launch_opts* opts,
                                void* scratch, size_t scratch_bytes, void* stream);

size_t credit_layernorm_forward_host_scratch_bytes(int64_t rows, int64_t cols, int dtype);
int credit_layernorm_forward_host(const void* x_host, const float* gamma_host, const float* beta_host,
                                  void* y_host, float* mean_host, float* rstd_host, int64_t rows,
                                  int64_t cols, float eps, int dtype, const credit_launch_opts* opts,
                                  void* scratch, size_t scratch_bytes, void* stream);

/* dgamma_host / dbeta_host are required here. Column sums are kept per row block on the
 * device and added in block order at the end (deterministic). */
size_t credit_layernorm_backward_stats_host_scratch_bytes(int64_t rows, int64_t cols, int dtype,
                                                          const credit_launch_opts* opts);
int credit_layernorm_backward_stats_host(const void* x_host, const void* dy_host, const float* gamma_host,
                                         const float* mean_host, const float* rstd_host, void* dx_host,
                                         float* dgamma_host, float* dbeta_host, int64_t rows, int64_t cols,
                                         int dtype, const credit_launch_opts* opts, void* scratch,
                                         size_t scratch_bytes, void* stream);

/* Fused FFN with the activations in host memory: x_host and y_host are bf16 [m, d] on
 * the host; the packed weights and gamma are the DEVICE pointers credit_ffn_forward
 * takes (parameters stay resident between calls). Every row needs both weight matrices
 * in full, so the rows are not cut into blocks. */
size_t credit_ffn_forward_host_scratch_bytes(int64_t m, int64_t d, int64_t h);
int credit_ffn_forward_host(const void* x_host, const void* w1_packed, const void* w2_packed,
                            const float* gamma, void* y_host, int64_t m, int64_t d, int64_t h, float eps,
                            void* scratch, size_t scratch_bytes, void* stream);

/* Multi-GPU: rows sharded over the GPUs of a node ---------------------------- */

/* Rows are independent in every workload, so a matrix is split into contiguous row
 * blocks, one per GPU (one process per GPU), parameters are replicated and outputs
 * stay sharded. The single quantity that spans the shards is LayerNorm backward's
 * dgamma / dbeta (column sums over ALL rows): each rank calls
 * credit_layernorm_backward_stats with dgamma = buf and dbeta = buf + cols of one
 * [2, cols] fp32 device buffer, then credit_layernorm_bwd_allreduce(comm, buf, cols,
 * stream) sums that buffer over the ranks, in place, on the same stream (NCCL over
 * NVLink; no host synchronisation in between). The reference is single-device
 * (device 0 is hard-coded, src/workloads/layernorm_backward.cu:443); these entry
 * points have no counterpart there.
 *
 * Set-up: rank 0 obtains an id (CREDIT_COMM_ID_BYTES bytes) and hands it to the other
 * ranks by whatever channel the host has; every rank then calls credit_comm_init_rank
 * with its own device current (collective: returns when all ranks have called it).
 * NCCL is loaded at run time (libnccl.so.2); where it is absent these calls return
 * CREDIT_ERR_UNSUPPORTED and the rest of the library is unaffected. */
#define CREDIT_COMM_ID_BYTES 128
typedef struct credit_comm credit_comm;
int credit_comm_get_unique_id(void* id_out);
int credit_comm_init_rank(credit_comm** comm, int world_size, int rank, const void* id);
int credit_comm_destroy(credit_comm* comm);
int credit_layernorm_bwd_allreduce(credit_comm* comm, float* dgamma_dbeta, int64_t cols, void* stream);

/* The same sum without a library collective: one kernel per rank that publishes the rank's
 * [2, cols] vector in a window of device memory its peers have mapped (CUDA IPC, plain
 * loads and stores over NVLink), raises a flag in every peer's window, waits for the
 * peers' flags and adds the vectors in rank order, so every rank gets bit-identical
 * sums. The vector is 512 KiB at the target shape: an NCCL all-reduce of it is about
 * 35 us of latency behind a 490 us kernel at 8 ranks, this kernel about a third of that.
 * No reference counterpart (single device).
 *
 * Set-up: every rank (one process per GPU, its device current) calls
 * credit_peer_group_create, which allocates its window and writes a handle of
 * CREDIT_PEER_HANDLE_BYTES bytes; the host gathers the handles of all ranks, in rank
 * order, by whatever channel it has and gives the array to credit_peer_group_connect.
 * At most 16 ranks, all on GPUs of one node with peer access to one another.
 * credit_layernorm_bwd_allreduce_peer is collective: every rank calls it once per step
 * with the same cols, on any stream; calls of one group must not overlap on a device.
 * The wait is bounded (about a second): if a peer never arrives, bit 0 of
 * credit_peer_group_status() is set and the local vector is left unreduced. Ranks of one
 * group must never share a GPU (a kernel that waits for a launch that cannot start).
 * Before credit_peer_group_destroy the host makes sure no rank is still inside a call. */
#define CREDIT_PEER_HANDLE_BYTES 64
typedef struct credit_peer_group credit_peer_group;
int credit_peer_group_create(credit_peer_group** group, int world_size, int rank, int64_t max_cols, void* handle_out);
int credit_peer_group_connect(credit_peer_group* group, const void* handles);
int credit_peer_group_destroy(credit_peer_group* group);
int credit_peer_group_status(credit_peer_group* group);
int credit_layernorm_bwd_allreduce_peer(credit_peer_group* group, float* dgamma_dbeta, int64_t cols, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* CREDIT_B200_H */
