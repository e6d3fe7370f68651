// The five workloads that exist only in the reference's sweep (weighted-variance backward,
// Pearson backward, softmax-logits backward, LARS momentum, row-wise int8 quantisation) as
// policies of the warp-specialised pipeline (ws_row_kernels.cuh). fp32, as in the reference.
//
// The pipeline runs ONE reduction per row, so each workload is restated with a single pass of
// partial records where the reference's eager functions (dsmem_eval/workloads.py:72-157) and its
// CUDA kernels use two or three dependent reductions:
//   * Pearson, weighted variance: shifted moments. With K a sample of the row (the median of
//     three elements, the same in every CTA) the record holds sum(x-K), sum((x-K)^2), ... and
//     the centred quantities follow exactly, e.g. sum((x-mean)^2) = Sdd - Sd^2 / n. The
//     reference's own CUDA kernel takes raw moments in one pass (pearson_backward.cu:456-458,
//     var = sum x^2 - sum x * mean); the shift removes that form's cancellation.
//   * softmax backward: online softmax. A record is (m, s, t) with s = sum exp(x - m) and
//     t = sum exp(x - m) * dy for the running maximum m; two records merge by rescaling both to
//     the larger maximum, so max, normaliser and the dot product sum(p * dy) come out of one pass
//     (the reference kernel makes three, recomputing expf each time,
//     softmax_logits_backward.cu:410).
//   * LARS and the quantiser have a single reduction anyway (two sums; one maximum).
// A thread owns no fixed columns here (nothing is kept per column), so slices of any length are
// walked with a strided loop. Exponentials use the fast intrinsic (ex2.approx after a multiply,
// about 2 ulp): the reference accepts 3e-3 for this workload (dsmem_eval/workloads.py:186-190).
#pragma once

#include <cmath>

#include "ws_row_kernels.cuh"

namespace credit {

// Common shape of the reference-sweep policies: fp32, 8 output warps, strided loops.
template <int NIN, int KP>
struct WsRowOpBase {
    using Elem = float;
    static constexpr int kInputs = NIN, kOutWarps = 8, kVectors = 0, THREADS = 256;
    static constexpr bool kFull = false, kRegisterSlice = false;
    static constexpr int kPartials = KP;
    // records of 8 floats leave room for two CTA-local buffers: the passes then run one row apart
    static constexpr int kLocalBuffers = KP == 8 ? 2 : 4;
    struct State {};
    __device__ __forceinline__ static void init(State&, const NormParams&, int, int) {}
    __device__ __forceinline__ static void finish(State&, const NormParams&, int, int, int, int) {}
    __device__ __forceinline__ static void sources(const NormParams& p, const float* (&src)[NIN]) {
        src[0] = static_cast<const float*>(p.x);
        if constexpr (NIN > 1) src[1] = static_cast<const float*>(p.dy);
        if constexpr (NIN > 2) src[2] = static_cast<const float*>(p.in2);
    }
    // median of three samples of a row (first, middle, last element)
    __device__ __forceinline__ static float median3(float a, float b, float c) {
        return fmaxf(fminf(a, b), fminf(fmaxf(a, b), c));
    }
    __device__ __forceinline__ static float4 vec(const uint4* tile, int v) {
        const uint4 r = tile[v];
        return make_float4(__uint_as_float(r.x), __uint_as_float(r.y), __uint_as_float(r.z), __uint_as_float(r.w));
    }
};

// ---------------------------------------------------------------------------
// Row-wise int8 quantisation (workloads.py:153-157): scale = max|x| / 127, q = clamp(rint(x * 127 / max)).
// ---------------------------------------------------------------------------
struct WsQuantOp : WsRowOpBase<1, 2> {
    static constexpr bool kAdditive = false, kRowInfo = false;
    __device__ __forceinline__ static WsRow fetch_row(const NormParams&, int, int) { return WsRow{}; }
    __device__ __forceinline__ static float4 publish_row(const WsRow&) { return make_float4(0.0f, 0.0f, 0.0f, 0.0f); }
    __device__ __forceinline__ static void identity(float (&v)[2]) { v[0] = v[1] = 0.0f; }
    __device__ __forceinline__ static void combine(float (&v)[2], const float (&o)[2]) { v[0] = fmaxf(v[0], o[0]); }
    __device__ __forceinline__ static void pass1(State&, const uint4* const (&tiles)[1], int nvec, const float4&,
                                                 float (&part)[2]) {
        float m0 = 0.0f, m1 = 0.0f;
#pragma unroll 4
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 q = vec(tiles[0], v);
            m0 = fmaxf(m0, fmaxf(fabsf(q.x), fabsf(q.y)));
            m1 = fmaxf(m1, fmaxf(fabsf(q.z), fabsf(q.w)));
        }
        part[0] = fmaxf(m0, m1);
        part[1] = 0.0f;
    }
    __device__ __forceinline__ static void pass2(State&, const uint4* const (&tiles)[1], int nvec, const float4&,
                                                 const float (&tot)[2], const NormParams& p, int row, int cols, int col0,
                                                 uint32_t rank) {
        const float max_abs = tot[0];
        const float inv = max_abs > 0.0f ? 127.0f / max_abs : 0.0f;
        if (rank == 0 && threadIdx.x == 0) p.row_out[row] = max_abs / 127.0f;
        // Round half to even, as torch.round, then clamp: clamp first (same result: the bounds are
        // integers), then add 1.5 * 2^23, whose sum is rounded to a whole number by the adder itself; the
        // low byte of the sum's bit pattern is the two's-complement int8. No conversion instructions
        // (they run at a quarter of the rate of an add), bit-identical to clamp(rint(x * inv)).
        auto q8 = [&](float x) {
            return __float_as_uint(fminf(fmaxf(x * inv, -127.0f), 127.0f) + 12582912.0f);
        };
        uint32_t* out = reinterpret_cast<uint32_t*>(static_cast<signed char*>(p.y) + static_cast<size_t>(row) * cols + col0);
#pragma unroll 4
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 q = vec(tiles[0], v);
            const uint32_t lo = __byte_perm(q8(q.x), q8(q.y), 0x0040);   // bytes: x.b0, y.b0
            const uint32_t hi = __byte_perm(q8(q.z), q8(q.w), 0x0040);
            out[v] = __byte_perm(lo, hi, 0x5410);
        }
    }
};

// ---------------------------------------------------------------------------
// LARS momentum (workloads.py:139-147): u = 0.9 m + g + 0.01 w; trust = 0.02 |w| / (|u| + 1e-6);
// w' = w - 1e-3 trust u. Inputs weight, grad, momentum; outputs w', u.
// ---------------------------------------------------------------------------
struct WsLarsOp : WsRowOpBase<3, 2> {
    static constexpr bool kAdditive = true, kRowInfo = false;
    __device__ __forceinline__ static WsRow fetch_row(const NormParams&, int, int) { return WsRow{}; }
    __device__ __forceinline__ static float4 publish_row(const WsRow&) { return make_float4(0.0f, 0.0f, 0.0f, 0.0f); }
    __device__ __forceinline__ static void identity(float (&v)[2]) { v[0] = v[1] = 0.0f; }
    __device__ __forceinline__ static void combine(float (&v)[2], const float (&o)[2]) { v[0] += o[0]; v[1] += o[1]; }
    __device__ __forceinline__ static float update_of(float w, float g, float m) { return 0.9f * m + g + 0.01f * w; }
    __device__ __forceinline__ static void pass1(State&, const uint4* const (&tiles)[3], int nvec, const float4&,
                                                 float (&part)[2]) {
        float sw[2] = {0.0f, 0.0f}, su[2] = {0.0f, 0.0f};
#pragma unroll 2
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 w = vec(tiles[0], v), g = vec(tiles[1], v), m = vec(tiles[2], v);
            const float u0 = update_of(w.x, g.x, m.x), u1 = update_of(w.y, g.y, m.y);
            const float u2 = update_of(w.z, g.z, m.z), u3 = update_of(w.w, g.w, m.w);
            sw[0] = fmaf(w.x, w.x, sw[0]); sw[1] = fmaf(w.y, w.y, sw[1]);
            sw[0] = fmaf(w.z, w.z, sw[0]); sw[1] = fmaf(w.w, w.w, sw[1]);
            su[0] = fmaf(u0, u0, su[0]); su[1] = fmaf(u1, u1, su[1]);
            su[0] = fmaf(u2, u2, su[0]); su[1] = fmaf(u3, u3, su[1]);
        }
        part[0] = sw[0] + sw[1];
        part[1] = su[0] + su[1];
    }
    __device__ __forceinline__ static void pass2(State&, const uint4* const (&tiles)[3], int nvec, const float4&,
                                                 const float (&tot)[2], const NormParams& p, int row, int cols, int col0,
                                                 uint32_t) {
        const float step = 1.0e-3f * (0.02f * sqrtf(tot[0]) / (sqrtf(tot[1]) + 1.0e-6f));
        const size_t base = static_cast<size_t>(row) * cols + col0;
        float4* out_w = reinterpret_cast<float4*>(static_cast<float*>(p.y) + base);
        float4* out_u = reinterpret_cast<float4*>(static_cast<float*>(p.out1) + base);
#pragma unroll 2
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 w = vec(tiles[0], v), g = vec(tiles[1], v), m = vec(tiles[2], v);
            const float4 u = make_float4(update_of(w.x, g.x, m.x), update_of(w.y, g.y, m.y), update_of(w.z, g.z, m.z),
                                         update_of(w.w, g.w, m.w));
            __stcs(out_w + v, make_float4(w.x - step * u.x, w.y - step * u.y, w.z - step * u.z, w.w - step * u.w));
            __stcs(out_u + v, u);
        }
    }
};

// ---------------------------------------------------------------------------
// Pearson backward (workloads.py:98-115): with xc = x - mean(x), yc = y - mean(y),
// vx = sum xc^2, vy = sum yc^2, cov = sum xc yc, ix = rsqrt(vx + 1e-6), iy likewise:
//   dx = grad (yc ix iy - xc cov ix^3 iy),  dy = grad (xc ix iy - yc cov ix iy^3).
// Record: Sx = sum(x-Kx), Sy = sum(y-Ky), Sxx, Syy, Sxy of the shifted values.
// ---------------------------------------------------------------------------
struct WsPearsonOp : WsRowOpBase<2, 8> {
    static constexpr bool kAdditive = true, kRowInfo = true;
    __device__ __forceinline__ static WsRow fetch_row(const NormParams& p, int row, int cols) {
        const float* x = static_cast<const float*>(p.x) + static_cast<size_t>(row) * cols;
        const float* y = static_cast<const float*>(p.dy) + static_cast<size_t>(row) * cols;
        return WsRow{__ldg(x), __ldg(x + (cols >> 1)), __ldg(x + cols - 1), __ldg(y), __ldg(y + (cols >> 1)),
                     __ldg(y + cols - 1), __ldg(p.row_in + row)};
    }
    __device__ __forceinline__ static float4 publish_row(const WsRow& r) {
        return make_float4(median3(r.a, r.b, r.c), median3(r.d, r.e, r.f), r.g, 0.0f);
    }
    __device__ __forceinline__ static void identity(float (&v)[8]) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = 0.0f;
    }
    __device__ __forceinline__ static void combine(float (&v)[8], const float (&o)[8]) {
#pragma unroll
        for (int k = 0; k < 5; ++k) v[k] += o[k];
    }
    __device__ __forceinline__ static void pass1(State&, const uint4* const (&tiles)[2], int nvec, const float4& info,
                                                 float (&part)[8]) {
        const float kx = info.x, ky = info.y;
        float sx = 0.0f, sy = 0.0f, sxx = 0.0f, syy = 0.0f, sxy = 0.0f;
        auto add = [&](float xv, float yv) {
            const float a = xv - kx, b = yv - ky;
            sx += a;
            sy += b;
            sxx = fmaf(a, a, sxx);
            syy = fmaf(b, b, syy);
            sxy = fmaf(a, b, sxy);
        };
#pragma unroll 2
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 x = vec(tiles[0], v), y = vec(tiles[1], v);
            add(x.x, y.x); add(x.y, y.y); add(x.z, y.z); add(x.w, y.w);
        }
        part[0] = sx; part[1] = sy; part[2] = sxx; part[3] = syy; part[4] = sxy;
        part[5] = part[6] = part[7] = 0.0f;
    }
    __device__ __forceinline__ static void pass2(State&, const uint4* const (&tiles)[2], int nvec, const float4& info,
                                                 const float (&t)[8], const NormParams& p, int row, int cols, int col0,
                                                 uint32_t) {
        const float inv_n = 1.0f / static_cast<float>(cols);
        const float dx_mean = t[0] * inv_n, dy_mean = t[1] * inv_n;       // mean - K
        const float mx = info.x + dx_mean, my = info.y + dy_mean;
        const float vx = fmaxf(t[2] - t[0] * dx_mean, 0.0f), vy = fmaxf(t[3] - t[1] * dy_mean, 0.0f);
        const float cov = t[4] - t[0] * dy_mean;
        const float ix = rsqrtf(vx + 1.0e-6f), iy = rsqrtf(vy + 1.0e-6f);
        const float grad = info.z;
        const float a = grad * ix * iy, cx = grad * cov * ix * ix * ix * iy, cy = grad * cov * ix * iy * iy * iy;
        const size_t base = static_cast<size_t>(row) * cols + col0;
        float4* out_x = reinterpret_cast<float4*>(static_cast<float*>(p.y) + base);
        float4* out_y = reinterpret_cast<float4*>(static_cast<float*>(p.out1) + base);
#pragma unroll 2
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 x = vec(tiles[0], v), y = vec(tiles[1], v);
            const float4 xc = make_float4(x.x - mx, x.y - mx, x.z - mx, x.w - mx);
            const float4 yc = make_float4(y.x - my, y.y - my, y.z - my, y.w - my);
            __stcs(out_x + v, make_float4(yc.x * a - xc.x * cx, yc.y * a - xc.y * cx, yc.z * a - xc.z * cx, yc.w * a - xc.w * cx));
            __stcs(out_y + v, make_float4(xc.x * a - yc.x * cy, xc.y * a - yc.y * cy, xc.z * a - yc.z * cy, xc.w * a - yc.w * cy));
        }
    }
};

// ---------------------------------------------------------------------------
// Weighted-variance backward (workloads.py:72-87): inv_w = 1 / (sum w + 1e-5), mean = sum(w x) inv_w,
// d = x - mean, rstd = rsqrt(sum(w d^2) inv_w + 1e-5):
//   dx = rstd (dy - w inv_w sum(dy) - w d rstd^2 inv_w sum(dy d)).
// Inputs x, weight, dy. Record with e = x - K: Sw, Swe, Swee, Sdy, Sdye.
// ---------------------------------------------------------------------------
struct WsWeightedVarOp : WsRowOpBase<3, 8> {
    static constexpr bool kAdditive = true, kRowInfo = true;
    __device__ __forceinline__ static WsRow fetch_row(const NormParams& p, int row, int cols) {
        const float* x = static_cast<const float*>(p.x) + static_cast<size_t>(row) * cols;
        return WsRow{__ldg(x), __ldg(x + (cols >> 1)), __ldg(x + cols - 1)};
    }
    __device__ __forceinline__ static float4 publish_row(const WsRow& r) {
        return make_float4(median3(r.a, r.b, r.c), 0.0f, 0.0f, 0.0f);
    }
    __device__ __forceinline__ static void identity(float (&v)[8]) {
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = 0.0f;
    }
    __device__ __forceinline__ static void combine(float (&v)[8], const float (&o)[8]) {
#pragma unroll
        for (int k = 0; k < 5; ++k) v[k] += o[k];
    }
    __device__ __forceinline__ static void pass1(State&, const uint4* const (&tiles)[3], int nvec, const float4& info,
                                                 float (&part)[8]) {
        const float k0 = info.x;
        float sw = 0.0f, swe = 0.0f, swee = 0.0f, sdy = 0.0f, sdye = 0.0f;
        auto add = [&](float xv, float wv, float gv) {
            const float e = xv - k0, we = wv * e;
            sw += wv;
            swe += we;
            swee = fmaf(we, e, swee);
            sdy += gv;
            sdye = fmaf(gv, e, sdye);
        };
#pragma unroll 2
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 x = vec(tiles[0], v), w = vec(tiles[1], v), g = vec(tiles[2], v);
            add(x.x, w.x, g.x); add(x.y, w.y, g.y); add(x.z, w.z, g.z); add(x.w, w.w, g.w);
        }
        part[0] = sw; part[1] = swe; part[2] = swee; part[3] = sdy; part[4] = sdye;
        part[5] = part[6] = part[7] = 0.0f;
    }
    __device__ __forceinline__ static void pass2(State&, const uint4* const (&tiles)[3], int nvec, const float4& info,
                                                 const float (&t)[8], const NormParams& p, int row, int cols, int col0,
                                                 uint32_t) {
        const float k0 = info.x;
        const float inv_w = 1.0f / (t[0] + 1.0e-5f);
        // mean = (Swe + K Sw) / (Sw + eps), so mean - K = (Swe - K eps) / (Sw + eps)
        const float delta = (t[1] - k0 * 1.0e-5f) * inv_w;
        const float mean = k0 + delta;
        const float var_num = fmaxf(t[2] - 2.0f * delta * t[1] + delta * delta * t[0], 0.0f);   // sum w (x - mean)^2
        const float rstd = rsqrtf(var_num * inv_w + 1.0e-5f);
        const float s_dy = t[3], s_dyd = t[4] - delta * t[3];
        const float c1 = inv_w * s_dy, c2 = rstd * rstd * inv_w * s_dyd;
        float4* out = reinterpret_cast<float4*>(static_cast<float*>(p.y) + static_cast<size_t>(row) * cols + col0);
        auto dx = [&](float xv, float wv, float gv) { return rstd * (gv - wv * c1 - wv * (xv - mean) * c2); };
#pragma unroll 2
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 x = vec(tiles[0], v), w = vec(tiles[1], v), g = vec(tiles[2], v);
            __stcs(out + v, make_float4(dx(x.x, w.x, g.x), dx(x.y, w.y, g.y), dx(x.z, w.z, g.z), dx(x.w, w.w, g.w)));
        }
    }
};

// ---------------------------------------------------------------------------
// Softmax-logits backward (workloads.py:125-128): p = softmax(logits), out = p (dy - sum(p dy)).
// Record (m, s, t): running maximum, sum exp(x - m), sum exp(x - m) dy.
// ---------------------------------------------------------------------------
struct WsSoftmaxBwdOp : WsRowOpBase<2, 4> {
    static constexpr bool kAdditive = false, kRowInfo = false;
    __device__ __forceinline__ static WsRow fetch_row(const NormParams&, int, int) { return WsRow{}; }
    __device__ __forceinline__ static float4 publish_row(const WsRow&) { return make_float4(0.0f, 0.0f, 0.0f, 0.0f); }
    __device__ __forceinline__ static void identity(float (&v)[4]) {
        v[0] = -INFINITY;
        v[1] = v[2] = v[3] = 0.0f;
    }
    // exp(a - m) for a <= m, 0 for a = -inf even when m = -inf
    __device__ __forceinline__ static float rescale(float a, float m) { return a == m ? (a == -INFINITY ? 0.0f : 1.0f) : __expf(a - m); }
    __device__ __forceinline__ static void combine(float (&v)[4], const float (&o)[4]) {
        const float m = fmaxf(v[0], o[0]);
        const float a = rescale(v[0], m), b = rescale(o[0], m);
        v[1] = v[1] * a + o[1] * b;
        v[2] = v[2] * a + o[2] * b;
        v[0] = m;
    }
    __device__ __forceinline__ static void pass1(State&, const uint4* const (&tiles)[2], int nvec, const float4&,
                                                 float (&part)[4]) {
        // the thread's own maximum first (a pass over shared memory, no exponentials), then the sums at
        // that scale in four independent chains: no branch and no rescaling inside the loop, so the
        // exponentials of several vectors are in flight at once
        float m = -INFINITY;
#pragma unroll 4
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 x = vec(tiles[0], v);
            m = fmaxf(m, fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w)));
        }
        const float mm = m == -INFINITY ? 0.0f : m;   // nothing but -inf: every term below is exp(-inf) = 0
        float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f}, t4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 x = vec(tiles[0], v), g = vec(tiles[1], v);
            const float e0 = __expf(x.x - mm), e1 = __expf(x.y - mm), e2 = __expf(x.z - mm), e3 = __expf(x.w - mm);
            s4[0] += e0; s4[1] += e1; s4[2] += e2; s4[3] += e3;
            t4[0] = fmaf(e0, g.x, t4[0]); t4[1] = fmaf(e1, g.y, t4[1]);
            t4[2] = fmaf(e2, g.z, t4[2]); t4[3] = fmaf(e3, g.w, t4[3]);
        }
        const float s = (s4[0] + s4[1]) + (s4[2] + s4[3]), t = (t4[0] + t4[1]) + (t4[2] + t4[3]);
        part[0] = m; part[1] = s; part[2] = t; part[3] = 0.0f;
    }
    __device__ __forceinline__ static void pass2(State&, const uint4* const (&tiles)[2], int nvec, const float4&,
                                                 const float (&tot)[4], const NormParams& p, int row, int cols, int col0,
                                                 uint32_t) {
        const float m = tot[0];
        const float inv_sum = 1.0f / tot[1];
        const float neg_dot_scaled = -(tot[2] * inv_sum) * inv_sum;
        float4* out = reinterpret_cast<float4*>(static_cast<float*>(p.y) + static_cast<size_t>(row) * cols + col0);
        // p * (g - dot) = e * (g / sum - dot / sum): one fused operation and one product per element
        auto f = [&](float xv, float gv) { return __expf(xv - m) * fmaf(gv, inv_sum, neg_dot_scaled); };
#pragma unroll 4
        for (int v = threadIdx.x; v < nvec; v += THREADS) {
            const float4 x = vec(tiles[0], v), g = vec(tiles[1], v);
            __stcs(out + v, make_float4(f(x.x, g.x), f(x.y, g.y), f(x.z, g.z), f(x.w, g.w)));
        }
    }
};

}  // namespace credit
