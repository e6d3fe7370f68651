// Constants and kernel-argument structs shared by the host launcher and the
// device code.
#pragma once

namespace credit {

constexpr int kMaxClusterSize = 16;   // 8 portable, 16 with the non-portable opt-in
constexpr int kMaxWarpsPerCta = 32;
constexpr int kMaxStages = 8;
constexpr int kWsMaxStages = 16;      // the warp-specialised kernels: short slices need a deeper ring
// Threads per CTA of the warp-specialised kernels: 16 (or, "wide", 8) output warps plus three
// service warps (producer, collector, receiver); their control block at the start of dynamic
// shared memory holds one pair of partial sums per output thread for four rows.
constexpr int kWsThreadsPerCta = 608;
constexpr int kWsThreadsPerCtaWide = 352;
constexpr int kWsControlBytes = 22528;
// Bytes reserved at the start of dynamic shared memory for barriers and
// reduction scratch; row data starts after it (keeps 1024-byte alignment).
constexpr int kControlBytes = 4096;

// Bits of the device status word (see credit_device_status in the C ABI).
constexpr int kStatusWaitTimeout = 1;      // an mbarrier wait ran out of patience
constexpr int kStatusBadGeometry = 2;      // a kernel saw a launch shape it cannot handle

// Geometry shared by the staged kernels.
struct StagedArgs {
    int rows;
    int cols;
    int slice_elems;    // columns per CTA (multiple of 64); stage stride in elements
    int num_clusters;   // clusters in the grid; cluster c handles rows c, c+num_clusters, ...
    int stages;         // ring depth (1 for the scalar-fill path)
    int* status;        // device status word
};

// Pointers of the normalisation workloads, as the warp-specialised kernels take them (one struct
// for RMSNorm forward, LayerNorm forward and LayerNorm backward; unused members are NULL).
struct NormParams {
    const void* x;           // first staged input
    const void* dy;          // second staged input
    const void* in2;         // third staged input (reference-sweep workloads)
    void* out1;              // second output (reference-sweep workloads)
    const float* row_in;     // per-row input (Pearson: upstream gradient [rows])
    float* row_out;          // per-row output (quantiser: scale [rows])
    const float* gamma;
    const float* beta;
    const float* mean_in;    // given statistics (backward)
    const float* rstd_in;
    void* y;                 // y (forward) or dx (backward)
    float* mean_out;         // computed statistics (LayerNorm forward)
    float* rstd_out;
    float* partials;         // [num_clusters][2][cols] partial column sums (backward)
    float eps;
};

// Row elements one output thread of a warp-specialised kernel may own (what it keeps per element
// in registers bounds it): forward kernels 32 with 16 output warps and 64 with 8; backward with
// column sums 16 and 32.
constexpr int ws_max_elems_per_thread(bool backward, bool wide) { return (backward ? 16 : 32) * (wide ? 2 : 1); }

// Pointers of a reference-sweep workload (weighted variance, Pearson, softmax
// backward, LARS, int8 quantisation).
struct RowOpArgs {
    const float* in[3];     // row-major [rows, cols] inputs
    const float* row_in;    // per-row input (Pearson: upstream gradient [rows]) or NULL
    void* out[2];           // row-major outputs: fp32, or int8 for the quantiser
    float* row_out;         // per-row output (quantiser: scale [rows]) or NULL
};

// Geometry of the streaming row reduction.
struct ReduceArgs {
    int rows;
    int cols;
    int slice_elems;    // columns per CTA, multiple of 64
    int num_clusters;
    int stages;         // ring depth (TMA variant)
    int chunk_elems;    // columns per ring chunk, multiple of 4 (TMA variant)
    int* status;
};

}  // namespace credit
