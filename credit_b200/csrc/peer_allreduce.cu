// One-shot all-reduce of LayerNorm backward's [2, cols] dgamma/dbeta buffer over the GPUs of a node
// through peer memory (plain loads and stores over NVLink, no library collective): the sum is 512 KiB
// at the target shape, so an NCCL call is pure latency (about 35 us at 8 ranks) behind a 490 us
// kernel; here one kernel publishes the rank's vector in a window its peers have mapped, raises a
// flag in every peer's window, waits (bounded) for the peers' flags and adds the vectors in rank
// order, so every rank gets bit-identical sums. The reference is single-device
// (src/workloads/layernorm_backward.cu:443) and has no counterpart.
//
// Windows are cudaMalloc allocations exported with cudaIpcGetMemHandle (one process per GPU); the
// host passes the 64-byte handles between the ranks by whatever channel it has. Layout of a window:
//   [0, 4096)                        uint32 flags[16]: flags[r] = last epoch rank r has published
//   4096 + b * stride, b = 0, 1      data of even / odd epochs, 2 * max_cols floats each
// Two data buffers make one barrier per call enough: a rank overwrites buffer b two calls later, and
// it can only get there after every peer has published the call in between, which a peer does after
// its reads of this call (launches of one rank run in stream order).
//
// Never run two ranks of one group on the same GPU: a kernel that waits for another launch on the
// same device may never see it start.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "../../include/credit_b200.h"
#include "error_state.h"
#include "launch_args.h"

namespace {

using credit::report_error;

constexpr int kMaxPeerRanks = 16;
constexpr size_t kFlagBytes = 4096;
constexpr int kPeerThreads = 256;
constexpr int kPeerMaxCtas = 128;

struct PeerPointers {
    unsigned char* window[kMaxPeerRanks];
};

__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_volatile_f32x4(const float* p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ float ld_volatile_f32(const float* p) {
    float v;
    asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_volatile_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// n floats of `local` are summed over the ranks, result back in `local`. `epoch` counts the calls of
// this group from 1; `arrived` counts the CTA arrivals of all calls so far and reaches
// `arrivals_target` when this call's copies are complete.
__global__ void __launch_bounds__(kPeerThreads)
peer_allreduce_kernel(float* __restrict__ local, PeerPointers peers, int world, int rank, int n, size_t data_stride,
                      uint32_t epoch, unsigned int arrivals_target, unsigned int* arrived, int* status) {
    const size_t data_offset = kFlagBytes + static_cast<size_t>(epoch & 1u) * data_stride;
    float* mine = reinterpret_cast<float*>(peers.window[rank] + data_offset);
    const bool vec = (n & 3) == 0 && (reinterpret_cast<uintptr_t>(local) & 15) == 0;
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    const int nthreads = gridDim.x * blockDim.x;

    // 1. publish this rank's vector
    if (vec) {
        for (int i = tid; i < n / 4; i += nthreads)
            reinterpret_cast<float4*>(mine)[i] = reinterpret_cast<const float4*>(local)[i];
    } else {
        for (int i = tid; i < n; i += nthreads) mine[i] = local[i];
    }
    __threadfence_system();
    __syncthreads();
    __shared__ bool gave_up;
    if (threadIdx.x == 0) {
        gave_up = false;
        const unsigned int before = atomicAdd(arrived, 1u);
        if (before + 1u == arrivals_target) {
            // the last CTA of this rank: every CTA's copy is visible system-wide (each fenced before
            // it arrived); tell every rank, this one included
            __threadfence_system();
            for (int r = 0; r < world; ++r)
                st_volatile_u32(reinterpret_cast<uint32_t*>(peers.window[r]) + rank, epoch);
        }
        // 2. wait for every rank's flag in this rank's own window (bounded: about a second)
        const uint32_t* flags = reinterpret_cast<const uint32_t*>(peers.window[rank]);
        const long long t0 = clock64();
        for (int r = 0; r < world && !gave_up; ++r) {
            while (static_cast<int32_t>(ld_volatile_u32(flags + r) - epoch) < 0) {
                if (clock64() - t0 > (1ll << 31)) {
                    atomicOr(status, credit::kStatusWaitTimeout);
                    gave_up = true;
                    break;
                }
            }
        }
        __threadfence_system();
    }
    __syncthreads();
    if (gave_up) return;   // the sums would be wrong: leave the local vector as it was

    // 3. add the vectors in rank order (the same order on every rank: identical results). All loads of
    // an element are issued before the first add, so their NVLink round trips overlap.
    if (vec) {
        for (int i = tid; i < n / 4; i += nthreads) {
            float4 v[kMaxPeerRanks];
#pragma unroll
            for (int r = 0; r < kMaxPeerRanks; ++r)
                if (r < world) v[r] = ld_volatile_f32x4(reinterpret_cast<const float*>(peers.window[r] + data_offset) + 4 * i);
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int r = 0; r < kMaxPeerRanks; ++r)
                if (r < world) {
                    acc.x += v[r].x;
                    acc.y += v[r].y;
                    acc.z += v[r].z;
                    acc.w += v[r].w;
                }
            reinterpret_cast<float4*>(local)[i] = acc;
        }
    } else {
        for (int i = tid; i < n; i += nthreads) {
            float v[kMaxPeerRanks];
#pragma unroll
            for (int r = 0; r < kMaxPeerRanks; ++r)
                if (r < world) v[r] = ld_volatile_f32(reinterpret_cast<const float*>(peers.window[r] + data_offset) + i);
            float acc = 0.0f;
#pragma unroll
            for (int r = 0; r < kMaxPeerRanks; ++r)
                if (r < world) acc += v[r];
            local[i] = acc;
        }
    }
}

}  // namespace

struct credit_peer_group {
    int world_size = 0;
    int rank = 0;
    int device = 0;
    int64_t max_cols = 0;
    size_t data_stride = 0;        // bytes of one data buffer
    size_t window_bytes = 0;
    unsigned char* window[kMaxPeerRanks] = {};   // own allocation at [rank], mapped peers elsewhere
    unsigned int* arrived = nullptr;
    int* status = nullptr;         // this group's own status word (credit_peer_group_status)
    uint32_t epoch = 0;
    unsigned int arrivals = 0;     // CTA arrivals of all calls so far (wraps with the device counter)
    bool connected = false;
};

extern "C" {

int credit_peer_group_create(credit_peer_group** group_out, int world_size, int rank, int64_t max_cols, void* handle_out) {
    if (group_out == nullptr || handle_out == nullptr)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "group_out and handle_out must not be NULL");
    if (world_size < 1 || world_size > kMaxPeerRanks || rank < 0 || rank >= world_size)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "rank %d outside a world of %d (at most %d ranks)", rank, world_size,
                            kMaxPeerRanks);
    if (max_cols < 1 || max_cols > (1ll << 28))
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "max_cols must be in [1, 2^28]");
    credit_peer_group* g = new credit_peer_group();
    g->world_size = world_size;
    g->rank = rank;
    g->max_cols = max_cols;
    g->data_stride = (static_cast<size_t>(2 * max_cols) * sizeof(float) + 255) / 256 * 256;
    g->window_bytes = kFlagBytes + 2 * g->data_stride;
    cudaError_t err = cudaGetDevice(&g->device);
    if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&g->window[rank]), g->window_bytes);
    if (err == cudaSuccess) err = cudaMemset(g->window[rank], 0, g->window_bytes);
    if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&g->arrived), 256);
    if (err == cudaSuccess) err = cudaMemset(g->arrived, 0, 256);
    if (err == cudaSuccess) {
        g->status = reinterpret_cast<int*>(g->arrived) + 16;
        cudaIpcMemHandle_t handle;
        static_assert(sizeof(handle) == CREDIT_PEER_HANDLE_BYTES, "handles travel as 64 bytes");
        err = cudaIpcGetMemHandle(&handle, g->window[rank]);
        if (err == cudaSuccess) std::memcpy(handle_out, &handle, sizeof(handle));
    }
    if (err == cudaSuccess) err = cudaDeviceSynchronize();
    if (err != cudaSuccess) {
        if (g->window[rank] != nullptr) cudaFree(g->window[rank]);
        if (g->arrived != nullptr) cudaFree(g->arrived);
        delete g;
        return report_error(CREDIT_ERR_CUDA, "peer window: %s", cudaGetErrorString(err));
    }
    g->connected = world_size == 1;
    *group_out = g;
    return CREDIT_OK;
}

int credit_peer_group_connect(credit_peer_group* g, const void* handles) {
    if (g == nullptr || handles == nullptr) return report_error(CREDIT_ERR_INVALID_ARGUMENT, "group and handles must not be NULL");
    if (g->connected) return CREDIT_OK;
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return report_error(CREDIT_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(err));
    if (device != g->device)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "the group belongs to device %d, the current device is %d", g->device,
                            device);
    const unsigned char* bytes = static_cast<const unsigned char*>(handles);
    for (int r = 0; r < g->world_size; ++r) {
        if (r == g->rank) continue;
        cudaIpcMemHandle_t handle;
        std::memcpy(&handle, bytes + static_cast<size_t>(r) * CREDIT_PEER_HANDLE_BYTES, sizeof(handle));
        void* mapped = nullptr;
        err = cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess);
        if (err != cudaSuccess) {
            for (int q = 0; q < r; ++q)
                if (q != g->rank && g->window[q] != nullptr) {
                    cudaIpcCloseMemHandle(g->window[q]);
                    g->window[q] = nullptr;
                }
            return report_error(CREDIT_ERR_CUDA, "cudaIpcOpenMemHandle for rank %d: %s (peers must be other processes on GPUs "
                                "of this node with peer access)", r, cudaGetErrorString(err));
        }
        g->window[r] = static_cast<unsigned char*>(mapped);
    }
    g->connected = true;
    return CREDIT_OK;
}

int credit_peer_group_destroy(credit_peer_group* g) {
    if (g == nullptr) return CREDIT_OK;
    // the caller makes sure no rank is still inside an all-reduce (e.g. a host barrier after the
    // last synchronised call): a window must outlive its peers' reads
    for (int r = 0; r < g->world_size; ++r)
        if (r != g->rank && g->window[r] != nullptr) cudaIpcCloseMemHandle(g->window[r]);
    if (g->window[g->rank] != nullptr) cudaFree(g->window[g->rank]);
    if (g->arrived != nullptr) cudaFree(g->arrived);
    delete g;
    return CREDIT_OK;
}

int credit_peer_group_status(credit_peer_group* g) {
    if (g == nullptr) return report_error(CREDIT_ERR_INVALID_ARGUMENT, "group is NULL");
    int word = 0;
    cudaError_t err = cudaMemcpy(&word, g->status, sizeof(int), cudaMemcpyDeviceToHost);
    if (err != cudaSuccess) return report_error(CREDIT_ERR_CUDA, "cudaMemcpy: %s", cudaGetErrorString(err));
    return word;
}

int credit_layernorm_bwd_allreduce_peer(credit_peer_group* g, float* dgamma_dbeta, int64_t cols, void* stream) {
    if (g == nullptr) return report_error(CREDIT_ERR_INVALID_ARGUMENT, "group is NULL");
    if (!g->connected) return report_error(CREDIT_ERR_INVALID_ARGUMENT, "credit_peer_group_connect has not been called");
    if (dgamma_dbeta == nullptr || cols < 1 || cols > g->max_cols)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "dgamma_dbeta must be a [2, cols] buffer, cols in [1, %lld] for this group",
                            static_cast<long long>(g->max_cols));
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return report_error(CREDIT_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(err));
    if (device != g->device)
        return report_error(CREDIT_ERR_INVALID_ARGUMENT, "the group belongs to device %d, the current device is %d", g->device,
                            device);
    if (g->world_size == 1) return CREDIT_OK;   // nothing to add
    const int n = static_cast<int>(2 * cols);
    int ctas = (n / 4 + kPeerThreads - 1) / kPeerThreads;
    ctas = ctas < 1 ? 1 : (ctas > kPeerMaxCtas ? kPeerMaxCtas : ctas);
    ++g->epoch;
    g->arrivals += static_cast<unsigned int>(ctas);
    PeerPointers peers{};
    for (int r = 0; r < g->world_size; ++r) peers.window[r] = g->window[r];
    peer_allreduce_kernel<<<ctas, kPeerThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        dgamma_dbeta, peers, g->world_size, g->rank, n, g->data_stride, g->epoch, g->arrivals, g->arrived, g->status);
    err = cudaGetLastError();
    if (err != cudaSuccess) return report_error(CREDIT_ERR_CUDA, "peer all-reduce launch: %s", cudaGetErrorString(err));
    return CREDIT_OK;
}

}  // extern "C"
