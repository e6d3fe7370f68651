// The five wide-row workloads that exist only in the reference's sweep
// (weighted-variance backward, Pearson backward, softmax-logits backward, LARS
// momentum, row-wise int8 quantisation), on the same cluster core as the norm
// kernels: a cluster owns a row at a time, every CTA stages its slice of every
// input in shared memory once (bulk-async ring), the per-CTA partials of each
// dependent reduction are exchanged through distributed shared memory, and all
// later passes read the staged copy. fp32 throughout, as in the reference.
//
// One kernel template, one policy struct per workload. Reference kernels and
// formulas: src/workloads/weighted_var_backward.cu:426, pearson_backward.cu:417,
// softmax_logits_backward.cu:410, lars_momentum.cu:364, rowwise_quant.cu:321;
// dsmem_eval/workloads.py:72-157.
//
// STAGED = false gives the reference's block_*_read form (one CTA per row, no
// staging, every pass re-reads global memory), the baseline of the cost model.
#pragma once

#include <cmath>

#include "norm_kernels.cuh"

namespace credit {

template <int NIN>
struct SrcPtrs;
template <>
struct SrcPtrs<1> {
    const float* const p[1];
    __device__ explicit SrcPtrs(const RowOpArgs& io) : p{io.in[0]} {}
};
template <>
struct SrcPtrs<2> {
    const float* const p[2];
    __device__ explicit SrcPtrs(const RowOpArgs& io) : p{io.in[0], io.in[1]} {}
};
template <>
struct SrcPtrs<3> {
    const float* const p[3];
    __device__ explicit SrcPtrs(const RowOpArgs& io) : p{io.in[0], io.in[1], io.in[2]} {}
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// cluster_allreduce_sum with a choice of sum or max (all K partials of a stage
// use the same operation). Same structure: warp shuffles, one value per warp in
// shared memory, warp 0 folds and pushes to every CTA's slot, one cluster
// barrier, every thread folds the P slots in rank order.
template <int K, int THREADS>
__device__ __forceinline__ void cluster_allreduce_op(float (&v)[K], ReduceScratch<K>& s, uint32_t parity,
                                                     uint32_t rank, uint32_t nranks, bool is_max) {
    constexpr int kWarps = THREADS / 32;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const float identity = is_max ? -INFINITY : 0.0f;
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = is_max ? warp_max(v[k]) : warp_sum(v[k]);
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) s.warp_part[k][warp] = v[k];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int k = 0; k < K; ++k) {
            float t = lane < kWarps ? s.warp_part[k][lane] : identity;
            t = is_max ? warp_max(t) : warp_sum(t);
            if (static_cast<uint32_t>(lane) < nranks) {
                const uint32_t mine = smem_u32(&s.slot[parity][k][rank]);
                st_cluster_f32(map_to_rank(mine, static_cast<uint32_t>(lane)), t);
            }
        }
    }
    cluster_arrive_release();
    cluster_wait_acquire();
#pragma unroll
    for (int k = 0; k < K; ++k) {
        float t = identity;
        for (uint32_t r = 0; r < nranks; ++r) t = is_max ? fmaxf(t, s.slot[parity][k][r]) : t + s.slot[parity][k][r];
        v[k] = t;
    }
}

// Calls f(in) for every element of this CTA's slice, `in` holding the element of
// each of the NIN arrays. 128-bit reads when ALIGNED.
template <int NIN, int THREADS, bool ALIGNED, typename F>
__device__ __forceinline__ void for_slice(const float* const (&tile)[NIN], int local, F f) {
    if (ALIGNED) {
        const int nvec = local >> 2;
#pragma unroll 2
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            float4 q[NIN];
#pragma unroll
            for (int n = 0; n < NIN; ++n) q[n] = reinterpret_cast<const float4*>(tile[n])[v];
            float in[NIN];
#pragma unroll
            for (int n = 0; n < NIN; ++n) in[n] = q[n].x;
            f(in);
#pragma unroll
            for (int n = 0; n < NIN; ++n) in[n] = q[n].y;
            f(in);
#pragma unroll
            for (int n = 0; n < NIN; ++n) in[n] = q[n].z;
            f(in);
#pragma unroll
            for (int n = 0; n < NIN; ++n) in[n] = q[n].w;
            f(in);
        }
    } else {
        for (int c = threadIdx.x; c < local; c += THREADS) {
            float in[NIN];
#pragma unroll
            for (int n = 0; n < NIN; ++n) in[n] = tile[n][c];
            f(in);
        }
    }
}

__device__ __forceinline__ int quantised(float v) { return static_cast<int>(v); }

// ---------------------------------------------------------------------------
// Workload policies. accumulate(stage, in, state, part) adds one element to the
// stage's partials; finish(stage, totals, state, cols) turns cluster totals into
// row scalars; emit(in, state, out) produces the element's outputs.
// ---------------------------------------------------------------------------

// dsmem_eval/workloads.py:72-87; inputs x, weight, dy; output dx.
struct WeightedVarOp {
    static constexpr int kInputs = 3, kStages = 2, kOutputs = 1;
    static constexpr bool kInt8 = false;
    struct State { float inv_w, mean, rstd, s_dy, s_dyd; };
    __device__ static bool is_max(int) { return false; }
    __device__ static void init(State&, const RowOpArgs&, int) {}
    __device__ static void accumulate(int stage, const float (&in)[3], const State& st, float (&p)[3]) {
        if (stage == 0) {
            p[0] += in[1];
            p[1] = fmaf(in[1], in[0], p[1]);
        } else {
            const float d = in[0] - st.mean;
            p[0] = fmaf(in[1] * d, d, p[0]);
            p[1] += in[2];
            p[2] = fmaf(in[2], d, p[2]);
        }
    }
    __device__ static void finish(int stage, const float (&t)[3], State& st, int) {
        if (stage == 0) {
            st.inv_w = 1.0f / (t[0] + 1.0e-5f);
            st.mean = t[1] * st.inv_w;
        } else {
            st.rstd = rsqrtf(t[0] * st.inv_w + 1.0e-5f);
            st.s_dy = t[1];
            st.s_dyd = t[2];
        }
    }
    __device__ static void emit(const float (&in)[3], const State& st, float (&o)[2]) {
        const float d = in[0] - st.mean;
        o[0] = st.rstd * (in[2] - in[1] * st.inv_w * st.s_dy -
                          in[1] * d * st.rstd * st.rstd * st.inv_w * st.s_dyd);
    }
    __device__ static void row_result(const State&, const RowOpArgs&, int) {}
};

// dsmem_eval/workloads.py:98-115; inputs x, y (+ per-row grad); outputs dx, dy.
struct PearsonOp {
    static constexpr int kInputs = 2, kStages = 2, kOutputs = 2;
    static constexpr bool kInt8 = false;
    struct State { float grad, mx, my, inv_xy, coeff_x, coeff_y; };
    __device__ static bool is_max(int) { return false; }
    __device__ static void init(State& st, const RowOpArgs& io, int row) { st.grad = __ldg(io.row_in + row); }
    __device__ static void accumulate(int stage, const float (&in)[2], const State& st, float (&p)[3]) {
        if (stage == 0) {
            p[0] += in[0];
            p[1] += in[1];
        } else {
            const float xc = in[0] - st.mx, yc = in[1] - st.my;
            p[0] = fmaf(xc, xc, p[0]);
            p[1] = fmaf(yc, yc, p[1]);
            p[2] = fmaf(xc, yc, p[2]);
        }
    }
    __device__ static void finish(int stage, const float (&t)[3], State& st, int cols) {
        if (stage == 0) {
            const float inv_n = 1.0f / static_cast<float>(cols);
            st.mx = t[0] * inv_n;
            st.my = t[1] * inv_n;
        } else {
            const float ix = rsqrtf(t[0] + 1.0e-6f), iy = rsqrtf(t[1] + 1.0e-6f);
            st.inv_xy = ix * iy;
            st.coeff_x = t[2] * ix * ix * ix * iy;
            st.coeff_y = t[2] * ix * iy * iy * iy;
        }
    }
    __device__ static void emit(const float (&in)[2], const State& st, float (&o)[2]) {
        const float xc = in[0] - st.mx, yc = in[1] - st.my;
        o[0] = st.grad * (yc * st.inv_xy - xc * st.coeff_x);
        o[1] = st.grad * (xc * st.inv_xy - yc * st.coeff_y);
    }
    __device__ static void row_result(const State&, const RowOpArgs&, int) {}
};

// dsmem_eval/workloads.py:125-128; inputs logits, dy; output p * (dy - sum(p * dy)).
struct SoftmaxBwdOp {
    static constexpr int kInputs = 2, kStages = 3, kOutputs = 1;
    static constexpr bool kInt8 = false;
    struct State { float mx, inv_sum, dot; };
    __device__ static bool is_max(int stage) { return stage == 0; }
    __device__ static void init(State&, const RowOpArgs&, int) {}
    __device__ static void accumulate(int stage, const float (&in)[2], const State& st, float (&p)[3]) {
        if (stage == 0) {
            p[0] = fmaxf(p[0], in[0]);
        } else if (stage == 1) {
            p[0] += expf(in[0] - st.mx);
        } else {
            p[0] = fmaf(expf(in[0] - st.mx) * st.inv_sum, in[1], p[0]);
        }
    }
    __device__ static void finish(int stage, const float (&t)[3], State& st, int) {
        if (stage == 0) st.mx = t[0];
        else if (stage == 1) st.inv_sum = 1.0f / t[0];
        else st.dot = t[0];
    }
    __device__ static void emit(const float (&in)[2], const State& st, float (&o)[2]) {
        o[0] = expf(in[0] - st.mx) * st.inv_sum * (in[1] - st.dot);
    }
    __device__ static void row_result(const State&, const RowOpArgs&, int) {}
};

// dsmem_eval/workloads.py:139-147; inputs weight, grad, momentum; outputs new weight, update.
struct LarsOp {
    static constexpr int kInputs = 3, kStages = 1, kOutputs = 2;
    static constexpr bool kInt8 = false;
    struct State { float step; };
    __device__ static bool is_max(int) { return false; }
    __device__ static void init(State&, const RowOpArgs&, int) {}
    __device__ static float update_of(const float (&in)[3]) { return 0.9f * in[2] + in[1] + 0.01f * in[0]; }
    __device__ static void accumulate(int, const float (&in)[3], const State&, float (&p)[3]) {
        const float u = update_of(in);
        p[0] = fmaf(in[0], in[0], p[0]);
        p[1] = fmaf(u, u, p[1]);
    }
    __device__ static void finish(int, const float (&t)[3], State& st, int) {
        const float trust = 0.02f * sqrtf(t[0]) / (sqrtf(t[1]) + 1.0e-6f);
        st.step = 1.0e-3f * trust;
    }
    __device__ static void emit(const float (&in)[3], const State& st, float (&o)[2]) {
        const float u = update_of(in);
        o[0] = in[0] - st.step * u;
        o[1] = u;
    }
    __device__ static void row_result(const State&, const RowOpArgs&, int) {}
};

// dsmem_eval/workloads.py:153-157; input x; outputs int8 q and the per-row scale max|x| / 127.
struct QuantOp {
    static constexpr int kInputs = 1, kStages = 1, kOutputs = 1;
    static constexpr bool kInt8 = true;
    struct State { float max_abs, inv; };
    __device__ static bool is_max(int) { return true; }
    __device__ static void init(State&, const RowOpArgs&, int) {}
    __device__ static void accumulate(int, const float (&in)[1], const State&, float (&p)[3]) {
        p[0] = fmaxf(p[0], fabsf(in[0]));
    }
    __device__ static void finish(int, const float (&t)[3], State& st, int) {
        st.max_abs = t[0];
        st.inv = t[0] > 0.0f ? 127.0f / t[0] : 0.0f;
    }
    __device__ static void emit(const float (&in)[1], const State& st, float (&o)[2]) {
        o[0] = fminf(fmaxf(rintf(in[0] * st.inv), -127.0f), 127.0f);   // round half to even, as torch.round
    }
    __device__ static void row_result(const State& st, const RowOpArgs& io, int row) {
        io.row_out[row] = st.max_abs / 127.0f;
    }
};

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
template <class Op, int THREADS, bool ALIGNED, bool STAGED>
__global__ void __launch_bounds__(THREADS)
row_op_kernel(RowOpArgs io, StagedArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    auto& ctl = *reinterpret_cast<StagedControl<3>*>(smem);
    unsigned char* data = smem + kControlBytes;
    constexpr int NIN = Op::kInputs;

    const uint32_t rank = cluster_cta_rank();
    const uint32_t nranks = cluster_cta_count();
    const int cluster = blockIdx.x / nranks;
    const SliceGeom g = slice_geometry(a.cols, a.slice_elems, rank);
    const SrcPtrs<NIN> src(io);

    if (STAGED) staged_prologue<float, NIN, 3, ALIGNED>(ctl, src.p, data, cluster, a, g);

    RingCursor cur{0, 0u};
    uint32_t red_parity = 0;

    for (int row = cluster; row < a.rows; row += a.num_clusters) {
        const size_t row_base = static_cast<size_t>(row) * a.cols + g.start;
        const float* tile[NIN];
        if (STAGED) {
            if (ALIGNED) {
                if (g.local > 0) mbar_wait_bounded(smem_u32(&ctl.full[cur.stage]), cur.parity, a.status);
            } else {
                scalar_slice_fill<float, NIN, THREADS>(src.p, data, row, a, g);
            }
#pragma unroll
            for (int n = 0; n < NIN; ++n) tile[n] = stage_tile<float, NIN>(data, cur.stage, n, a.slice_elems);
        } else {
#pragma unroll
            for (int n = 0; n < NIN; ++n) tile[n] = io.in[n] + row_base;
        }
        const float* const(&tiles)[NIN] = reinterpret_cast<const float* const(&)[NIN]>(tile);

        typename Op::State st;
        Op::init(st, io, row);
#pragma unroll
        for (int stage = 0; stage < Op::kStages; ++stage) {
            const bool mx = Op::is_max(stage);
            float part[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) part[k] = mx ? -INFINITY : 0.0f;
            for_slice<NIN, THREADS, ALIGNED>(tiles, g.local,
                                             [&](const float(&in)[NIN]) { Op::accumulate(stage, in, st, part); });
            cluster_allreduce_op<3, THREADS>(part, ctl.red, red_parity, rank, nranks, mx);
            red_parity ^= 1u;
            Op::finish(stage, part, st, a.cols);
        }

        if (ALIGNED) {
            const int nvec = g.local >> 2;
#pragma unroll 2
            for (int v = threadIdx.x; v < nvec; v += THREADS) {
                float4 q[NIN];
#pragma unroll
                for (int n = 0; n < NIN; ++n) q[n] = reinterpret_cast<const float4*>(tiles[n])[v];
                float o[4][2];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float in[NIN];
#pragma unroll
                    for (int n = 0; n < NIN; ++n) in[n] = reinterpret_cast<const float*>(&q[n])[j];
                    Op::emit(in, st, o[j]);
                }
                if (Op::kInt8) {
                    const char4 packed = make_char4(static_cast<signed char>(quantised(o[0][0])),
                                                    static_cast<signed char>(quantised(o[1][0])),
                                                    static_cast<signed char>(quantised(o[2][0])),
                                                    static_cast<signed char>(quantised(o[3][0])));
                    reinterpret_cast<char4*>(static_cast<signed char*>(io.out[0]) + row_base)[v] = packed;
                } else {
#pragma unroll
                    for (int k = 0; k < Op::kOutputs; ++k)
                        __stcs(reinterpret_cast<float4*>(static_cast<float*>(io.out[k]) + row_base) + v,
                               make_float4(o[0][k], o[1][k], o[2][k], o[3][k]));
                }
            }
        } else {
            for (int c = threadIdx.x; c < g.local; c += THREADS) {
                float in[NIN], o[2];
#pragma unroll
                for (int n = 0; n < NIN; ++n) in[n] = tiles[n][c];
                Op::emit(in, st, o);
                if (Op::kInt8) {
                    static_cast<signed char*>(io.out[0])[row_base + c] = static_cast<signed char>(quantised(o[0]));
                } else {
#pragma unroll
                    for (int k = 0; k < Op::kOutputs; ++k) static_cast<float*>(io.out[k])[row_base + c] = o[k];
                }
            }
        }
        if (rank == 0 && threadIdx.x == 0) Op::row_result(st, io, row);

        if (STAGED) {
            staged_release<float, NIN, 3, ALIGNED>(ctl, src.p, data, cur.stage, row, a, g);
            cur.advance(a.stages);
        }
    }
}

}  // namespace credit
