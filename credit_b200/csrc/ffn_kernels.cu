// Fused FFN for sm_100a: two bf16 GEMMs on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory), operands staged by TMA,
//   H = GELU(X W1)                      (erf GELU, b1 = 0)
//   Y = RMSNorm(H W2 + X) * gamma       (row statistics over the full width d)
// The second GEMM is launched as clusters of d / 256 CTAs along N, so one cluster
// owns complete output rows: after the mainloop every thread holds one row of its
// CTA's 128 x 256 accumulator tile, adds the residual, sums z^2 over its 256
// columns, and the d / 256 per-CTA partials of each row are exchanged through
// distributed shared memory (st.shared::cluster + one cluster barrier) before the
// normalised row is written. The reference project has no GEMM; this file follows
// the cluster/DSMEM reduction scheme of its row kernels
// (src/workloads/layernorm_backward.cu:217-251) in a GEMM epilogue.
//
// Layout: X [m, d], H [m, h], Y [m, d] row-major bf16; weights are taken PACKED
// K-major (W1p [h, d], W2p [d, h], i.e. transposed once by credit_ffn_pack_weight),
// so both operands of both GEMMs are K-major tiles of 64 bf16 (128 bytes) per row,
// the shape the 128-byte swizzle of TMA and of the MMA shared-memory descriptors
// is made for. Every CTA loads its own tiles (no TMA multicast anywhere).
//
// Kernel structure (persistent, 192 threads, one CTA per SM; a CTA walks over
// 128 x 256 output tiles):
//   warp 0   : TMA producer, 4-stage ring of (A 128x64, B 256x64) tiles, runs ahead
//              across tile boundaries
//   warp 1   : allocates all 512 TMEM columns (two 128 x 256 fp32 accumulators),
//              issues tcgen05.mma, commits to mbarriers
//   warps 2-5: epilogue, tcgen05.ld 32 lanes x 32 columns at a time; the epilogue of
//              tile i runs while the MMAs of tile i+1 fill the other accumulator
// In the second GEMM the CTAs of a cluster walk over the same row blocks in step;
// the per-row partial sums travel with st.async and are counted on the receiving
// CTA's mbarrier (two slot buffers), so the producer and MMA warps never stop for
// the exchange. A cluster works on TWO row blocks at a time where it can (one in each
// of a CTA's two accumulators): the B tile of a k block is then staged once for two
// MMAs, a third less traffic into shared memory per FLOP, and W2 passes through the
// chip once per two rounds of row blocks instead of once per round.
// Every mbarrier wait is bounded; a timeout sets the device status word and the
// kernel still releases its tensor memory.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <mutex>

#include "../../include/credit_b200.h"
#include "cluster_primitives.cuh"
#include "kernel_tables.h"

namespace credit {
namespace {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
constexpr int kMaxFfnStages = 6;           // 4 stages of 48 KiB (one CTA per MMA) or 6 of 32 KiB (CTA pair)
constexpr int kUmmaK = 16;
constexpr int kAccCols = kBN;             // one accumulator: 128 lanes x 256 fp32 columns
constexpr int kTmemCols = 2 * kAccCols;   // two accumulators = all of tensor memory
constexpr int kATileBytes = kBM * kBK * 2;   // 16 KiB
constexpr int kRingBytes = 192 * 1024;

// Ring geometry. One CTA per MMA: a stage holds A 128x64 and B 256x64. CTA pair
// (tcgen05 cta_group::2, a 256 x 256 tile per pair): each CTA stages its own 128
// rows of A and HALF of B (128 of the 256 columns of the tile); the tensor cores of
// both SMs read both halves, so a CTA moves a third less through its shared memory
// per MMA, which is what bounds the one-CTA form (TMA writes + MMA reads = 192 bytes
// per clock against 128 available).
// DUAL (second GEMM): a stage holds the A tiles of two row blocks and one B tile, A0 | A1 | B; an
// item of a single row block leaves A1 unused.
template <bool PAIR, bool DUAL = false>
struct Ring {
    static constexpr int kBRows = PAIR ? kBN / 2 : kBN;
    static constexpr int kBTileBytes = kBRows * kBK * 2;
    static constexpr int kBOffset = (DUAL ? 2 : 1) * kATileBytes;
    static constexpr int kStageBytes = kBOffset + kBTileBytes;
    static constexpr int kStages = kRingBytes / kStageBytes;
    static_assert(kStages <= kMaxFfnStages, "control block has too few barriers");
};
constexpr int kEpilogueThreads = 128;
constexpr int kFfnThreads = 64 + kEpilogueThreads;
constexpr int kFfnControlBytes = 1024;
constexpr int kMaxRowClusters = 16;
constexpr int kSlotBufferFloats = kBM * kMaxRowClusters;
// ring + control + alignment slack + two buffers of row-partial slots (second GEMM)
constexpr int kFfnSmemBytes = kRingBytes + kFfnControlBytes + 1024 +
                              2 * kSlotBufferFloats * static_cast<int>(sizeof(float));

struct FfnControl {
    uint64_t full[kMaxFfnStages];   // TMA -> MMA: stage holds its tiles (pair: both CTAs' halves)
    uint64_t empty[kMaxFfnStages];  // MMA -> TMA: stage may be overwritten
    uint64_t acc_full[2];       // MMA -> epilogue: accumulator complete
    uint64_t acc_empty[2];      // epilogue -> MMA: accumulator read out (one arrival per epilogue warp)
    uint64_t slots_ready[2];    // peers -> epilogue: all row partials of a tile have landed
    uint32_t tmem_base;
};
static_assert(sizeof(FfnControl) <= kFfnControlBytes, "control block overflows its reservation");

// ---- PTX wrappers --------------------------------------------------------------
// CG = 1: an MMA of one CTA. CG = 2: an MMA of a CTA pair (cluster ranks 2i, 2i + 1); the even
// CTA (the leader) issues it, and copies, commits and tensor-memory management carry the same
// qualifier.
template <int CG>
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    if (CG == 1)
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
                "r"(dst),
            "l"(map), "r"(bar), "r"(x), "r"(y)
            : "memory");
    else   // `bar` may be the leader's barrier (a shared::cluster address)
        asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
            "%4}], [%2];" ::"r"(dst),
            "l"(map), "r"(bar), "r"(x), "r"(y)
            : "memory");
}

template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    if (CG == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    } else {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
}

template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    if (CG == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
template <int CG>
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    if (CG == 1)
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
}

// The mbarrier (any CTA of the cluster) gets one arrival when every MMA issued so far by this
// thread is done.
template <int CG>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    if (CG == 1)
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                     : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                     : "memory");
}

// Pair form for a barrier that exists at the same shared-memory offset in both CTAs of the pair:
// one commit, one arrival on each CTA's copy (mask: cluster ranks of the receivers).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}

// Arrivals on a barrier that may live in another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: lane i of the warp gets row (lane base + i).
__device__ __forceinline__ void tmem_load_32x32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
          "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
          "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
          "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// (64 bf16), 128-byte swizzled: 8-row groups 1024 bytes apart; version 1 (sm_100),
// layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fffu);
    d |= static_cast<uint64_t>(1) << 16;                    // leading byte offset (unused with swizzle)
    d |= static_cast<uint64_t>(1024 >> 4) << 32;            // stride between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;                    // descriptor version
    d |= static_cast<uint64_t>(2) << 61;                    // SWIZZLE_128B
    return d;
}

// Instruction descriptor: D = fp32, A = B = bf16, both K-major, M x N tile.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)); }

__device__ __forceinline__ uint4 pack8(const float* v) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ void unpack8(const uint4& r, float* o) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        o[2 * i] = __uint_as_float(w[i] << 16);
        o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// Bounded wait that gives up for good after its first timeout, so a broken pipeline
// costs one timeout per thread instead of one per k-block.
__device__ __forceinline__ void wait_or_give_up(uint32_t bar, uint32_t parity, int* status, bool& gave_up) {
    if (!gave_up && !mbar_wait_bounded(bar, parity, status)) gave_up = true;
}

// ---- the GEMM kernel -------------------------------------------------------------
// Output tiles of A [M, K] x B^T with B packed [N, K].
// NORM_EPILOGUE == false: out = GELU(acc) as bf16 [M, N]; CTA b takes tiles b, b + grid, ...
//                         numbered with the row block fastest, so that CTAs running at the
//                         same time share B tiles through L2.
// NORM_EPILOGUE == true : a cluster of n_tiles CTAs along N covers whole rows;
//                         out = (acc + residual) * rsqrt(mean_row((acc+residual)^2) + eps) * gamma.
//   Plain walk : cluster c takes row blocks c, c + clusters, ... All clusters start a row block
//                at the same time and move through k together, so a k block of B is fetched from
//                HBM once and served to the other clusters by L2 (B is as large as L2).
//   Split tail : when the row blocks do not divide evenly among the resident clusters, the L
//                blocks left after the full rounds are each shared by a group of G = clusters / L
//                clusters, which cut the k range into G equal parts (again in step across blocks).
//                The cluster with the first part OWNS the block; the others are HELPERS: they write
//                their raw fp32 partial tile to global memory and raise a flag; the owner adds the
//                partials to its accumulator and runs the epilogue.
struct WorkItem {
    int tile;       // row block (NORM) or tile number
    int tile2;      // >= 0: a second row block worked on at the same time (other accumulator)
    int kb0, kb1;   // k blocks [kb0, kb1)
};

struct TileWalk {
    int m_tiles, k_blocks;
    int fixed_n;           // >= 0: every work item is a row block and the column tile is fixed
    int dual_next, dual_step, dual_end;   // pairs of row blocks (2 * p, 2 * p + 1), p below dual_end
    int next, step, end;   // plain walk
    int tail_tile;         // >= 0: one more item, part of a shared row block
    int tail_kb0, tail_kb1;

    __device__ __forceinline__ bool pop(WorkItem& w) {
        w.tile2 = -1;
        if (dual_next < dual_end) {
            w.tile = 2 * dual_next;
            w.tile2 = 2 * dual_next + 1;
            w.kb0 = 0;
            w.kb1 = k_blocks;
            dual_next += dual_step;
            return true;
        }
        if (next < end) {
            w.tile = next;
            w.kb0 = 0;
            w.kb1 = k_blocks;
            next += step;
            return true;
        }
        if (tail_tile < 0) return false;
        w.tile = tail_tile;
        w.kb0 = tail_kb0;
        w.kb1 = tail_kb1;
        tail_tile = -1;
        return true;
    }
    __device__ __forceinline__ void locate(int tile, int& m_tile, int& n_tile) const {
        if (fixed_n >= 0) {
            m_tile = tile;
            n_tile = fixed_n;
        } else {
            m_tile = tile % m_tiles;
            n_tile = tile / m_tiles;
        }
    }
};

constexpr int kPartialSlots = 16;   // split walk: at most this many clusters (one partial tile each)

// Float offset, inside a partial slot, of the 4 columns [32 * chunk + 4 * g, +4) of row `row` in
// the tile of cluster rank `rank`: rows are the fastest index, so a warp's stores are contiguous.
__device__ __forceinline__ size_t partial_offset(uint32_t rank, int chunk, int g, int row) {
    return ((static_cast<size_t>(rank) * (kBN / 32) + chunk) * 8 + g) * (kBM * 4) + static_cast<size_t>(row) * 4;
}

// Bounded wait for a flag another cluster sets in global memory.
__device__ __forceinline__ void wait_flag(const int* flag, int* status, bool& gave_up) {
    if (gave_up) return;
    const volatile int* f = flag;
    const long long t0 = clock64();
    while (*f == 0) {
        if (clock64() - t0 > (1ll << 31)) {
            atomicOr(status, kStatusWaitTimeout);
            gave_up = true;
            break;
        }
    }
    __threadfence();   // the partial tile written before the flag is visible to the loads after it
}

// PAIR: launched as clusters of two CTAs that share every MMA (NORM_EPILOGUE must be false).
// A work item is then a 256 x 256 tile; CTA `half` of the pair owns rows half * 128 .. + 127 of it
// (its A tile, its accumulators, its epilogue) and stages columns half * 128 .. + 127 of B.
template <bool NORM_EPILOGUE, bool PAIR>
__global__ void __launch_bounds__(kFfnThreads)
ffn_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ residual,
                const float* __restrict__ gamma, int m_tiles, int n_tiles, int n_total, int k_total, float eps,
                float* __restrict__ partials, int* __restrict__ flags, int* status) {
    static_assert(!(NORM_EPILOGUE && PAIR), "the row-norm epilogue uses the cluster for whole rows");
    constexpr int CG = PAIR ? 2 : 1;
    using R = Ring<PAIR, NORM_EPILOGUE>;
    constexpr int kStages = R::kStages;
    constexpr int kStageBytes = R::kStageBytes;
    constexpr int kTileRows = PAIR ? 2 * kBM : kBM;   // rows of a work item

    extern __shared__ unsigned char smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle; the dynamic window starts at the
    // same shared-memory address in every CTA, so both CTAs of a pair get the same offsets
    unsigned char* smem = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char* tiles = smem;
    FfnControl& ctl = *reinterpret_cast<FfnControl*>(smem + kRingBytes);
    float* row_slots = reinterpret_cast<float*>(smem + kRingBytes + kFfnControlBytes);  // [2][kBM][16]

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int k_blocks = k_total / kBK;
    const uint32_t rank = (NORM_EPILOGUE || PAIR) ? cluster_cta_rank() : 0u;
    const uint32_t nranks = NORM_EPILOGUE ? cluster_cta_count() : 1u;
    const int half = PAIR ? static_cast<int>(rank & 1u) : 0;
    const bool leader = half == 0;

    // every role walks over the same sequence of work items with its own copy of this
    TileWalk walk0;
    walk0.m_tiles = m_tiles;
    walk0.k_blocks = k_blocks;
    walk0.tail_tile = -1;
    walk0.tail_kb0 = walk0.tail_kb1 = 0;
    walk0.dual_next = walk0.dual_end = 0;
    walk0.dual_step = 1;
    int group = 1;   // clusters sharing the tail row block of this cluster
    const int cluster_id = static_cast<int>(blockIdx.x / (NORM_EPILOGUE ? nranks : CG));
    const int num_clusters = static_cast<int>(gridDim.x / (NORM_EPILOGUE ? nranks : CG));
    if (NORM_EPILOGUE) {
        // rounds of two row blocks per cluster first, then at most one round of single blocks, then
        // the blocks that are left (fewer than clusters) shared by groups of clusters
        const int dual_rounds = m_tiles / (2 * num_clusters);
        const int dual_blocks = dual_rounds * 2 * num_clusters;
        walk0.dual_next = cluster_id;
        walk0.dual_step = num_clusters;
        walk0.dual_end = dual_rounds * num_clusters;
        walk0.next = dual_blocks + cluster_id;
        walk0.step = num_clusters;
        walk0.end = m_tiles;
        walk0.fixed_n = static_cast<int>(rank);
        const int left = (m_tiles - dual_blocks) % num_clusters;
        // at most 4 clusters per block (the owner reads every helper's tile twice), at least 4 k
        // blocks per part
        int share = left != 0 ? num_clusters / left : 1;
        share = share < 4 ? share : 4;
        share = share < k_blocks / 4 ? share : k_blocks / 4;
        if (partials != nullptr && share >= 2) {
            group = share;
            walk0.end = m_tiles - left;   // full rounds only
            if (cluster_id < left * group) {
                const int part = cluster_id % group;
                walk0.tail_tile = m_tiles - left + cluster_id / group;
                walk0.tail_kb0 = static_cast<int>(static_cast<long long>(k_blocks) * part / group);
                walk0.tail_kb1 = static_cast<int>(static_cast<long long>(k_blocks) * (part + 1) / group);
            }
        }
    } else {
        walk0.next = cluster_id;
        walk0.step = num_clusters;
        walk0.end = m_tiles * n_tiles;
        walk0.fixed_n = -1;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&ctl.full[s]), 1);     // the (leader's) producer's arrive.expect_tx
            mbar_init(smem_u32(&ctl.empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&ctl.acc_full[b]), 1);
            mbar_init(smem_u32(&ctl.acc_empty[b]), CG * (kEpilogueThreads / 32));
            mbar_init(smem_u32(&ctl.slots_ready[b]), 1);
        }
        fence_mbar_init();
    }
    if (warp == 1) tmem_alloc<CG>(smem_u32(&ctl.tmem_base), kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = ctl.tmem_base;
    bool gave_up = false;
    // peers' barriers exist before anything is sent to them
    if (NORM_EPILOGUE || PAIR) cluster_sync_all();

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t parity = 1;   // a fresh barrier passes a wait on the "previous" phase
            TileWalk walk = walk0;
            WorkItem w;
            while (walk.pop(w)) {
                int m_tile, n_tile;
                walk.locate(w.tile, m_tile, n_tile);
                const int a_row = m_tile * kTileRows + half * kBM;
                const int b_row = n_tile * kBN + half * R::kBRows;
                const bool dual = NORM_EPILOGUE && w.tile2 >= 0;
                const uint32_t stage_tx = CG * (kATileBytes + R::kBTileBytes) + (dual ? kATileBytes : 0);
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    wait_or_give_up(smem_u32(&ctl.empty[stage]), parity, status, gave_up);
                    // the stage's "full" barrier is the leader's: its MMA thread consumes both halves
                    // and arms it for the bytes of both CTAs (the peer's copies may complete on it
                    // first: the phase cannot end before this arrival)
                    const uint32_t local_bar = smem_u32(&ctl.full[stage]);
                    const uint32_t bar = PAIR ? map_to_rank(local_bar, rank & ~1u) : local_bar;
                    if (leader) mbar_arrive_expect_tx(local_bar, stage_tx);
                    const uint32_t a_dst = smem_u32(tiles + stage * kStageBytes);
                    tma_load_2d<CG>(a_dst, &map_a, bar, kb * kBK, a_row);
                    if (dual) tma_load_2d<CG>(a_dst + kATileBytes, &map_a, bar, kb * kBK, w.tile2 * kTileRows);
                    tma_load_2d<CG>(a_dst + R::kBOffset, &map_b, bar, kb * kBK, b_row);
                    if (++stage == kStages) {
                        stage = 0;
                        parity ^= 1u;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = instr_desc(kTileRows, kBN);
            const uint16_t pair_mask = static_cast<uint16_t>(3u << (rank & ~1u));
            int stage = 0;
            uint32_t parity = 0;
            TileWalk walk = walk0;
            WorkItem w;
            uint32_t uses[2] = {0u, 0u};   // times each accumulator has been filled so far
            int singles = 0;
            while (walk.pop(w)) {
                const bool dual = NORM_EPILOGUE && w.tile2 >= 0;
                const int buf = dual ? 0 : (singles++ & 1);   // single items alternate; a dual item takes both
                // the epilogue warps (of both CTAs) have read the accumulator(s) out; passes at once
                // the first time
                wait_or_give_up(smem_u32(&ctl.acc_empty[buf]), (uses[buf] & 1u) ^ 1u, status, gave_up);
                if (dual) wait_or_give_up(smem_u32(&ctl.acc_empty[1]), (uses[1] & 1u) ^ 1u, status, gave_up);
                tc_fence_after_sync();
                const uint32_t acc = tmem_base + static_cast<uint32_t>(buf * kAccCols);
                for (int kb = w.kb0; kb < w.kb1; ++kb) {
                    wait_or_give_up(smem_u32(&ctl.full[stage]), parity, status, gave_up);
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_u32(tiles + stage * kStageBytes);
                    const uint64_t desc_a = smem_desc_k_major_sw128(a_addr);
                    const uint64_t desc_b = smem_desc_k_major_sw128(a_addr + R::kBOffset);
#pragma unroll
                    for (int k = 0; k < kBK / kUmmaK; ++k) {
                        // advance 16 bf16 = 32 bytes inside the swizzle row: +2 in the address field
                        umma_bf16<CG>(acc, desc_a + 2u * k, desc_b + 2u * k, idesc, (kb != w.kb0 || k != 0) ? 1u : 0u);
                    }
                    if (dual) {   // the second row block against the same B tile, into the other accumulator
                        const uint64_t desc_a2 = smem_desc_k_major_sw128(a_addr + kATileBytes);
#pragma unroll
                        for (int k = 0; k < kBK / kUmmaK; ++k)
                            umma_bf16<CG>(acc + kAccCols, desc_a2 + 2u * k, desc_b + 2u * k, idesc,
                                          (kb != w.kb0 || k != 0) ? 1u : 0u);
                    }
                    // stage reusable (in both CTAs) when these MMAs are done
                    if (PAIR)
                        umma_commit_pair(smem_u32(&ctl.empty[stage]), pair_mask);
                    else
                        umma_commit<CG>(smem_u32(&ctl.empty[stage]));
                    if (++stage == kStages) {
                        stage = 0;
                        parity ^= 1u;
                    }
                }
                ++uses[buf];
                if (PAIR)   // accumulator complete (in both CTAs)
                    umma_commit_pair(smem_u32(&ctl.acc_full[buf]), pair_mask);
                else
                    umma_commit<CG>(smem_u32(&ctl.acc_full[buf]));
                if (dual) {
                    ++uses[1];
                    umma_commit<CG>(smem_u32(&ctl.acc_full[1]));
                }
            }
        }
        __syncwarp();
    } else {
        // epilogue warps 2..5: warp w may touch TMEM lanes 32 * (w % 4) .. +31
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        TileWalk walk = walk0;
        WorkItem w;
        int exchanges = 0;   // row-norm exchanges done: selects the slot buffer and its barrier phase
        uint32_t uses[2] = {0u, 0u};   // times each accumulator has been read out so far
        int singles = 0;
        while (walk.pop(w)) {
          const bool dual = NORM_EPILOGUE && w.tile2 >= 0;
          const int single_buf = dual ? 0 : (singles++ & 1);
          // a dual item is two row blocks, one per accumulator: the same epilogue twice
          for (int sub = 0; sub < (dual ? 2 : 1); ++sub) {
            int m_tile, n_tile;
            walk.locate(sub == 0 ? w.tile : w.tile2, m_tile, n_tile);
            const int buf = dual ? sub : single_buf;
            const size_t row = static_cast<size_t>(m_tile) * kTileRows + half * kBM + row_in_tile;
            const size_t col0 = static_cast<size_t>(n_tile) * kBN;
            const uint32_t lane_base =
                tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(buf * kAccCols);
            __nv_bfloat16* dst = out + row * n_total + col0;
            wait_or_give_up(smem_u32(&ctl.acc_full[buf]), uses[buf] & 1u, status, gave_up);
            ++uses[buf];
            tc_fence_after_sync();

            if (!NORM_EPILOGUE) {
#pragma unroll 1
                for (int c = 0; c < kBN; c += 32) {
                    float v[32];
                    tmem_load_32x32(lane_base + c, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = gelu_erf(v[i]);
#pragma unroll
                    for (int i = 0; i < 32; i += 8) *reinterpret_cast<uint4*>(dst + c + i) = pack8(v + i);
                }
            } else if (w.kb0 != 0) {
                // HELPER: the raw partial tile goes to this cluster's slot, then the flag of this
                // column tile is raised for the owner's CTA of the same rank
                float* slot = partials + static_cast<size_t>(cluster_id) * nranks * (kBM * kBN);
#pragma unroll 1
                for (int c = 0; c < kBN; c += 32) {
                    float v[32];
                    tmem_load_32x32(lane_base + c, v);
#pragma unroll
                    for (int g = 0; g < 8; ++g)
                        *reinterpret_cast<float4*>(slot + partial_offset(rank, c / 32, g, row_in_tile)) =
                            make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
                }
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");   // the epilogue warps only
                if (threadIdx.x == 64) atomicExch(&flags[cluster_id * kMaxRowClusters + static_cast<int>(rank)], 1);
            } else {
                // FULL tile, or OWNER of a shared one (then the helpers are the next group - 1 clusters)
                const int helpers = w.kb1 != k_blocks ? group - 1 : 0;
                const size_t slot_floats = static_cast<size_t>(nranks) * (kBM * kBN);
                const float* part = partials + static_cast<size_t>(cluster_id + 1) * slot_floats;
                for (int hlp = 1; hlp <= helpers; ++hlp)
                    wait_flag(&flags[(cluster_id + hlp) * kMaxRowClusters + static_cast<int>(rank)], status, gave_up);
                const int sbuf = exchanges & 1;
                const uint32_t sphase = (static_cast<uint32_t>(exchanges) >> 1) & 1u;
                ++exchanges;
                const __nv_bfloat16* res = residual + row * n_total + col0;
                float* slots = row_slots + sbuf * kSlotBufferFloats + row_in_tile * kMaxRowClusters;
                const uint32_t ready = smem_u32(&ctl.slots_ready[sbuf]);
                // this CTA will receive one float per row from every CTA of the cluster (itself included)
                if (threadIdx.x == 64) mbar_arrive_expect_tx(ready, nranks * kBM * static_cast<uint32_t>(sizeof(float)));
                // pass 1: sum of squares of z = acc + residual over this CTA's 256 columns of the row
                float ss = 0.0f;
#pragma unroll 1
                for (int c = 0; c < kBN; c += 32) {
                    float v[32];
                    tmem_load_32x32(lane_base + c, v);
                    for (int hlp = 0; hlp < helpers; ++hlp) {
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            const float4 q = __ldcg(reinterpret_cast<const float4*>(
                                part + hlp * slot_floats + partial_offset(rank, c / 32, g, row_in_tile)));
                            v[4 * g] += q.x;
                            v[4 * g + 1] += q.y;
                            v[4 * g + 2] += q.z;
                            v[4 * g + 3] += q.w;
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float r8[8];
                        unpack8(__ldg(reinterpret_cast<const uint4*>(res + c + i)), r8);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float z = v[i + j] + r8[j];
                            ss = fmaf(z, z, ss);
                        }
                    }
                }
                // every CTA of the cluster gets every CTA's partial of every row
                for (uint32_t p = 0; p < nranks; ++p)
                    st_async_f32(map_to_rank(smem_u32(&slots[rank]), p), ss, map_to_rank(ready, p));
                wait_or_give_up(ready, sphase, status, gave_up);
                float total = 0.0f;
                for (uint32_t p = 0; p < nranks; ++p) total += slots[p];
                const float scale = rsqrtf(total / static_cast<float>(n_total) + eps);
                // pass 2: normalise
#pragma unroll 1
                for (int c = 0; c < kBN; c += 32) {
                    float v[32];
                    tmem_load_32x32(lane_base + c, v);
                    for (int hlp = 0; hlp < helpers; ++hlp) {
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            const float4 q = __ldcg(reinterpret_cast<const float4*>(
                                part + hlp * slot_floats + partial_offset(rank, c / 32, g, row_in_tile)));
                            v[4 * g] += q.x;
                            v[4 * g + 1] += q.y;
                            v[4 * g + 2] += q.z;
                            v[4 * g + 3] += q.w;
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float r8[8], g8[8];
                        unpack8(__ldg(reinterpret_cast<const uint4*>(res + c + i)), r8);
                        ldg_f32x4(gamma + col0 + c + i, g8);
                        ldg_f32x4(gamma + col0 + c + i + 4, g8 + 4);
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[i + j] = (v[i + j] + r8[j]) * scale * g8[j];
                        *reinterpret_cast<uint4*>(dst + c + i) = pack8(v + i);
                    }
                }
            }
            // accumulator `buf` may be overwritten by the MMAs of the next item that uses it: one arrival per warp
            // on the barrier of the CTA that issues them
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                const uint32_t bar = smem_u32(&ctl.acc_empty[buf]);
                if (PAIR)
                    mbar_arrive_cluster(map_to_rank(bar, rank & ~1u));
                else
                    mbar_arrive(bar);
            }
          }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    // no CTA leaves while a peer may still send to it, read its tiles or signal its barriers
    if (NORM_EPILOGUE || PAIR) cluster_sync_all();
    if (warp == 1) tmem_dealloc<CG>(tmem_base, kTmemCols);
}

// Transposes a row-major [k, n] bf16 weight into the K-major [n, k] form the GEMMs take.
__global__ void __launch_bounds__(256)
pack_weight_kernel(const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ packed, int k, int n) {
    __shared__ __nv_bfloat16 tile[32][33];
    const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    for (int j = ty; j < 32; j += 8)
        if (k0 + j < k && n0 + tx < n) tile[j][tx] = w[static_cast<size_t>(k0 + j) * n + n0 + tx];
    __syncthreads();
    for (int j = ty; j < 32; j += 8)
        if (n0 + j < n && k0 + tx < k) packed[static_cast<size_t>(n0 + j) * k + k0 + tx] = tile[tx][j];
}

// ---- host side ---------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Row-major [rows, k] bf16 matrix, boxes of box_rows x 64 elements, 128-byte swizzle.
bool make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t elem_strides[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
              elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

const char* ffn_check_shape(int64_t m, int64_t d, int64_t h) {
    if (m <= 0 || d <= 0 || h <= 0) return "m, d and h must be positive";
    if (m % kBM != 0) return "m must be a multiple of 128";
    if (d % kBN != 0 || h % kBN != 0) return "d and h must be multiples of 256";
    if (d / kBN > kMaxRowClusters) return "d must be at most 4096 (one cluster of up to 16 CTAs spans a row)";
    if (d % kBK != 0 || h % kBK != 0) return "d and h must be multiples of 64";
    if (m > (1 << 24) || d > (1 << 24) || h > (1 << 24)) return "shape too large";
    return nullptr;
}

namespace {
constexpr size_t kFlagBytes = static_cast<size_t>(kPartialSlots + 1) * kMaxRowClusters * sizeof(int);
size_t ffn_partial_bytes(int64_t d) {
    // one 128 x d fp32 partial tile per cluster (+ one never written: the last cluster owns nothing)
    return static_cast<size_t>(kPartialSlots + 1) * kBM * static_cast<size_t>(d) * sizeof(float);
}
}  // namespace

size_t ffn_scratch_bytes(int64_t d) { return ffn_partial_bytes(d) + kFlagBytes; }

cudaError_t launch_ffn_pack_weight(const void* w, void* packed, int k, int n, cudaStream_t stream) {
    dim3 grid(static_cast<unsigned>((n + 31) / 32), static_cast<unsigned>((k + 31) / 32));
    pack_weight_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(w),
                                                static_cast<__nv_bfloat16*>(packed), k, n);
    return cudaGetLastError();
}

namespace {
// Clusters of `cluster_size` CTAs of `kernel` that can be resident at once on the current device
// (cached by the caller in `*cache`, 0 = not asked yet), or -1 if the driver cannot tell. A
// persistent grid must not be larger: the surplus clusters would only start when the first ones
// have finished everything.
int resident_clusters(const void* kernel, int cluster_size, int grid_clusters, int* cache) {
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (*cache == 0) {
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(static_cast<unsigned>(cluster_size * grid_clusters));
        cfg.blockDim = dim3(kFfnThreads);
        cfg.dynamicSmemBytes = kFfnSmemBytes;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = static_cast<unsigned>(cluster_size);
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int q = 0;
        if (cudaOccupancyMaxActiveClusters(&q, kernel, &cfg) != cudaSuccess || q < 1) {
            (void)cudaGetLastError();
            q = -1;
        }
        *cache = q;
    }
    return *cache;
}
// What is set up or asked once per device: kernel attributes live in the device's context, and
// the resident-cluster counts depend on the device.
struct FfnDeviceState {
    cudaError_t attr_err = cudaSuccess;
    int resident_pairs = 0;
    int resident_row_clusters[kMaxRowClusters + 1] = {};
};

// The state of `device`, which must be the current device; kernel attributes are set on first use.
FfnDeviceState& ffn_device_state(int device) {
    static std::mutex mu;
    static std::map<int, FfnDeviceState> states;
    std::lock_guard<std::mutex> lock(mu);
    auto found = states.find(device);
    if (found != states.end()) return found->second;
    FfnDeviceState& st = states[device];
    const void* kernels[3] = {reinterpret_cast<const void*>(ffn_gemm_kernel<false, false>),
                              reinterpret_cast<const void*>(ffn_gemm_kernel<false, true>),
                              reinterpret_cast<const void*>(ffn_gemm_kernel<true, false>)};
    for (const void* k : kernels)
        if (st.attr_err == cudaSuccess)
            st.attr_err = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kFfnSmemBytes);
    if (st.attr_err == cudaSuccess)
        st.attr_err = cudaFuncSetAttribute(ffn_gemm_kernel<true, false>,
                                           cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    return st;
}
}  // namespace

// Returns cudaSuccess, or an error; *bad_map is set when a tensor map could not be encoded.
cudaError_t launch_ffn_forward(const void* x, const void* w1p, const void* w2p, const float* gamma, void* y,
                               void* hidden, void* scratch, int m, int d, int h, float eps, int* status,
                               cudaStream_t stream, bool* bad_map) {
    *bad_map = false;
    // CTA pairs need whole 256-row tiles; otherwise the first GEMM runs one CTA per MMA
    const bool pair = m % (2 * kBM) == 0;
    CUtensorMap map_x, map_w1, map_h, map_w2;
    if (!make_map(&map_x, x, m, d, kBM) || !make_map(&map_w1, w1p, h, d, pair ? kBN / 2 : kBN) ||
        !make_map(&map_h, hidden, m, h, kBM) || !make_map(&map_w2, w2p, d, h, kBN)) {
        *bad_map = true;
        return cudaErrorInvalidValue;
    }
    int device = 0, sms = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err == cudaSuccess) err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (err != cudaSuccess) return err;
    FfnDeviceState& dev = ffn_device_state(device);
    if (dev.attr_err != cudaSuccess) return dev.attr_err;

    const int m_tiles = m / kBM;
    // GEMM 1: H = GELU(X W1); persistent CTAs (pairs of CTAs sharing each MMA when m allows) walk
    // over the tiles
    {
        const int n_tiles = h / kBN;
        __nv_bfloat16* hid = static_cast<__nv_bfloat16*>(hidden);
        if (pair) {
            const int tiles = (m_tiles / 2) * n_tiles;
            int pairs = resident_clusters(reinterpret_cast<const void*>(ffn_gemm_kernel<false, true>), 2, tiles,
                                          &dev.resident_pairs);
            if (pairs < 1) pairs = sms / 2;
            if (pairs > tiles) pairs = tiles;
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
            cfg.blockDim = dim3(kFfnThreads);
            cfg.dynamicSmemBytes = kFfnSmemBytes;
            cfg.stream = stream;
            cudaLaunchAttribute attr{};
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim.x = 2;
            attr.val.clusterDim.y = 1;
            attr.val.clusterDim.z = 1;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            const __nv_bfloat16* no_res = nullptr;
            const float* no_gamma = nullptr;
            float* no_partials = nullptr;
            int* no_flags = nullptr;
            err = cudaLaunchKernelEx(&cfg, ffn_gemm_kernel<false, true>, map_x, map_w1, hid, no_res, no_gamma,
                                     m_tiles / 2, n_tiles, h, d, 0.0f, no_partials, no_flags, status);
        } else {
            const int tiles = m_tiles * n_tiles;
            const unsigned grid = static_cast<unsigned>(tiles < sms ? tiles : sms);
            ffn_gemm_kernel<false, false><<<grid, kFfnThreads, kFfnSmemBytes, stream>>>(
                map_x, map_w1, hid, nullptr, nullptr, m_tiles, n_tiles, h, d, 0.0f, nullptr, nullptr, status);
            err = cudaGetLastError();
        }
        if (err != cudaSuccess) return err;
    }
    // GEMM 2: Y = RMSNorm(H W2 + X) gamma; clusters of d / 256 CTAs, as many as fit on the device
    // at once, each walking over row blocks of 128 rows
    {
        const int n_tiles = d / kBN;
        cudaLaunchConfig_t cfg{};
        cfg.blockDim = dim3(kFfnThreads);
        cfg.dynamicSmemBytes = kFfnSmemBytes;
        cfg.stream = stream;
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = static_cast<unsigned>(n_tiles);
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;

        const int resident = resident_clusters(reinterpret_cast<const void*>(ffn_gemm_kernel<true, false>), n_tiles,
                                               m_tiles, &dev.resident_row_clusters[n_tiles]);
        const int clusters = (resident < 1 || resident > m_tiles) ? m_tiles : resident;
        cfg.gridDim = dim3(static_cast<unsigned>(n_tiles * clusters));
        // Row blocks left over after the full rounds are shared by groups of clusters that split
        // the k range (all clusters are resident, so an owner never waits for a helper that has
        // not started).
        float* partials = nullptr;
        int* flags = nullptr;
        if (resident >= 1 && clusters <= kPartialSlots && m_tiles % clusters != 0) {
            partials = static_cast<float*>(scratch);
            flags = reinterpret_cast<int*>(static_cast<unsigned char*>(scratch) + ffn_partial_bytes(d));
            err = cudaMemsetAsync(flags, 0, kFlagBytes, stream);
            if (err != cudaSuccess) return err;
        }
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(y);
        const __nv_bfloat16* res = static_cast<const __nv_bfloat16*>(x);
        return cudaLaunchKernelEx(&cfg, ffn_gemm_kernel<true, false>, map_h, map_w2, out, res, gamma, m_tiles, n_tiles, d, h,
                                  eps, partials, flags, status);
    }
}

}  // namespace credit
