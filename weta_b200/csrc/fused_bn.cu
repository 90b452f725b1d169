// BatchNorm2d and the fused conv-block tail (BatchNorm -> ReLU -> MaxPool2d(2)), forward and backward.
//   batch norm 2d    crates/weta-nn/src/functional.rs:144-180  (~9 reductions + ~20 element-wise passes per call)
//   BN + ReLU + pool crates/weta/examples/mnist_cnn.rs:18-20, 22-24; max-pool ties share the gradient
//                    (crates/weta-autograd/src/ops.rs:305-314), ReLU passes it where its input is positive (ops.rs:85)
// These results are tolerance-checked, not bit-checked, so this file is compiled with FMA contraction on;
// the running-statistics update alone keeps the reference's exact rounding sequence (explicit _rn ops).
#include <algorithm>
#include <cmath>

#include <cstdlib>

#include "common.h"

namespace {

constexpr int THREADS = 256;

// ---- per-channel statistics over [N, C, HW] -----------------------------------------------------
// grid (C, S): block (c, s) covers images n = s, s + S, ...  Values are shifted by the channel's
// first element before squaring so the one-pass variance does not cancel.
__global__ void __launch_bounds__(THREADS) bn_stats_kernel(const float* __restrict__ x, int64_t n_img, int c_total, int64_t hw,
                                                            double* __restrict__ part) {
    const int c = blockIdx.x;
    const float pivot = x[static_cast<int64_t>(c) * hw];
    double s1 = 0.0, s2 = 0.0;
    // This block's images [n0, n1); its threads walk the (image, position) pairs of that slab
    // flattened, so every thread is busy whatever the plane size.
    const int64_t per = (n_img + gridDim.y - 1) / gridDim.y;
    const int64_t n0 = min(n_img, static_cast<int64_t>(blockIdx.y) * per), n1 = min(n_img, n0 + per);  // n1 >= n0, empty slab allowed
    const int64_t plane_stride = static_cast<int64_t>(c_total) * hw;
    const float* slab = x + (n0 * c_total + c) * hw;
    if ((hw & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {  // planes are whole float4s and x starts on one
        const uint32_t q = static_cast<uint32_t>(hw >> 2), items = static_cast<uint32_t>(n1 - n0) * q;  // host checks the range
        float a1 = 0.f, a2 = 0.f;
        int flushed = 0;
        for (uint32_t j = threadIdx.x; j < items; j += THREADS) {
            const uint32_t n = j / q, p = j - n * q;
            float4 v = *reinterpret_cast<const float4*>(slab + n * plane_stride + p * 4);
            float d0 = v.x - pivot, d1 = v.y - pivot, d2 = v.z - pivot, d3 = v.w - pivot;
            a1 += (d0 + d1) + (d2 + d3);
            a2 += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
            if (++flushed == 64) { s1 += a1; s2 += a2; a1 = a2 = 0.f; flushed = 0; }  // keep f32 partial sums short
        }
        s1 += a1;
        s2 += a2;
    } else {
        const uint32_t uhw = static_cast<uint32_t>(hw), items = static_cast<uint32_t>(n1 - n0) * uhw;
        float a1 = 0.f, a2 = 0.f;
        int flushed = 0;
        for (uint32_t j = threadIdx.x; j < items; j += THREADS) {
            const uint32_t n = j / uhw, p = j - n * uhw;
            float d = slab[n * plane_stride + p] - pivot;
            a1 += d;
            a2 += d * d;
            if (++flushed == 256) { s1 += a1; s2 += a2; a1 = a2 = 0.f; flushed = 0; }
        }
        s1 += a1;
        s2 += a2;
    }
    __shared__ double r1[THREADS], r2[THREADS];
    r1[threadIdx.x] = s1;
    r2[threadIdx.x] = s2;
    __syncthreads();
    for (int s = THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) { r1[threadIdx.x] += r1[threadIdx.x + s]; r2[threadIdx.x] += r2[threadIdx.x + s]; }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        part[(static_cast<int64_t>(c) * gridDim.y + blockIdx.y) * 2] = r1[0];
        part[(static_cast<int64_t>(c) * gridDim.y + blockIdx.y) * 2 + 1] = r2[0];
    }
}

// mean, biased variance, rstd; running stats as crates/weta-nn/src/functional.rs:163-168.
__global__ void bn_finalize_kernel(const double* __restrict__ part, int splits, const float* __restrict__ x, int c_total, int64_t hw,
                                   int64_t count, float eps, float momentum, float one_minus_momentum, float* __restrict__ mean,
                                   float* __restrict__ rstd,
                                   float* __restrict__ running_mean, float* __restrict__ running_var) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= c_total) return;
    double s1 = 0.0, s2 = 0.0;
    for (int s = 0; s < splits; ++s) {
        s1 += part[(static_cast<int64_t>(c) * splits + s) * 2];
        s2 += part[(static_cast<int64_t>(c) * splits + s) * 2 + 1];
    }
    double pivot = x[static_cast<int64_t>(c) * hw];
    double dm = s1 / static_cast<double>(count);
    double var = s2 / static_cast<double>(count) - dm * dm;
    if (var < 0.0) var = 0.0;
    float m = static_cast<float>(pivot + dm), v = static_cast<float>(var);
    mean[c] = m;
    rstd[c] = 1.f / sqrtf(v + eps);
    if (running_mean) {
        // running = running*(1-m) + batch*m with every product and sum rounded separately (functional.rs:165-167)
        float unbiased = __fadd_rn(__fmul_rn(v, static_cast<float>(static_cast<double>(count) / static_cast<double>((count > 2 ? count : 2) - 1))), 0.f);
        running_mean[c] = __fadd_rn(__fadd_rn(__fmul_rn(running_mean[c], one_minus_momentum), 0.f), __fadd_rn(__fmul_rn(m, momentum), 0.f));
        running_var[c] = __fadd_rn(__fadd_rn(__fmul_rn(running_var[c], one_minus_momentum), 0.f), __fadd_rn(__fmul_rn(unbiased, momentum), 0.f));
    }
}

// Batch statistics from the sums a producer of x accumulated while it wrote x: per channel, in double, the sum and
// the sum of squares of (x - pivot[c]) (pivot null = 0; for a convolution the pivot is its bias, so the sums are those
// of the raw accumulator).  variance = E[d^2] - E[d]^2 loses digits when |E[d]| >> the standard deviation: the
// producer's per-tile partial sums are f32, so E[d^2] carries about 1e-7 of relative error and a channel whose
// variance is below 1e-3 of E[d^2] would keep fewer than four digits of it.  Such channels are recomputed from x
// by the same kernel that finalises the others (bn_stats_from_sums_kernel).
__device__ __forceinline__ bool sums_cancel(double e1, double e2) { return !(e2 - e1 * e1 > 1e-3 * e2) && e2 > 0.0; }

__device__ __forceinline__ void bn_store_stats(int c, double mean_d, double var_d, int64_t count, float eps, float momentum, float one_minus_momentum,
                                               float* __restrict__ mean, float* __restrict__ rstd, float* __restrict__ running_mean,
                                               float* __restrict__ running_var) {
    if (var_d < 0.0) var_d = 0.0;
    float m = static_cast<float>(mean_d), v = static_cast<float>(var_d);
    mean[c] = m;
    rstd[c] = 1.f / sqrtf(v + eps);
    if (running_mean) {
        // running = running*(1-m) + batch*m with every product and sum rounded separately (functional.rs:165-167)
        float unbiased = __fadd_rn(__fmul_rn(v, static_cast<float>(static_cast<double>(count) / static_cast<double>((count > 2 ? count : 2) - 1))), 0.f);
        running_mean[c] = __fadd_rn(__fadd_rn(__fmul_rn(running_mean[c], one_minus_momentum), 0.f), __fadd_rn(__fmul_rn(m, momentum), 0.f));
        running_var[c] = __fadd_rn(__fadd_rn(__fmul_rn(running_var[c], one_minus_momentum), 0.f), __fadd_rn(__fmul_rn(unbiased, momentum), 0.f));
    }
}

// One block per channel.  Normally thread 0 turns the channel's sums into mean / rstd / running statistics and the
// block is done; when the sums cancel (see above) the block reads the channel's n_img planes again and sums
// (x - m0), (x - m0)^2 about m0 = pivot + E[d], which is already within rounding of the mean, so nothing cancels.
__global__ void __launch_bounds__(THREADS) bn_stats_from_sums_kernel(const float* __restrict__ x, const double* __restrict__ sums,
                                                                 const float* __restrict__ pivot, int64_t n_img, int c_total, int64_t hw, float eps,
                                                                 float momentum, float one_minus_momentum, float* __restrict__ mean,
                                                                 float* __restrict__ rstd, float* __restrict__ running_mean,
                                                                 float* __restrict__ running_var) {
    wb_pdl_enter();
    const int c = blockIdx.x;
    const int64_t count = n_img * hw;
    const double e1 = sums[2 * c] / static_cast<double>(count), e2 = sums[2 * c + 1] / static_cast<double>(count);
    if (!sums_cancel(e1, e2)) {
        if (threadIdx.x == 0)
            bn_store_stats(c, (pivot ? static_cast<double>(pivot[c]) : 0.0) + e1, e2 - e1 * e1, count, eps, momentum, one_minus_momentum, mean, rstd,
                           running_mean, running_var);
        return;
    }
    const float m0 = static_cast<float>((pivot ? static_cast<double>(pivot[c]) : 0.0) + e1);
    double s1 = 0.0, s2 = 0.0;
    float a1 = 0.f, a2 = 0.f;
    int run = 0;
    for (int64_t n = 0; n < n_img; ++n) {
        const float* plane = x + (n * c_total + c) * hw;
        for (int64_t p = threadIdx.x; p < hw; p += THREADS) {
            const float d = plane[p] - m0;
            a1 += d;
            a2 += d * d;
            if (++run == 64) { s1 += a1; s2 += a2; a1 = a2 = 0.f; run = 0; }
        }
    }
    s1 += a1;
    s2 += a2;
    __shared__ double r1[THREADS], r2[THREADS];
    r1[threadIdx.x] = s1;
    r2[threadIdx.x] = s2;
    __syncthreads();
    for (int s = THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) { r1[threadIdx.x] += r1[threadIdx.x + s]; r2[threadIdx.x] += r2[threadIdx.x + s]; }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const double dm = r1[0] / static_cast<double>(count);
        bn_store_stats(c, static_cast<double>(m0) + dm, r2[0] / static_cast<double>(count) - dm * dm, count, eps, momentum, one_minus_momentum, mean,
                       rstd, running_mean, running_var);
    }
}

// y = ((x - mean) * rstd) * gamma + beta, optionally ReLU.  One (n, c) plane per blockIdx.y.
__global__ void __launch_bounds__(THREADS) bn_apply_kernel(float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ mean,
                                                            const float* __restrict__ rstd, const float* __restrict__ gamma,
                                                            const float* __restrict__ beta, int c_total, int64_t hw, int relu) {
    int64_t plane = blockIdx.y;
    int c = static_cast<int>(plane % c_total);
    float m = mean[c], r = rstd[c], g = gamma ? gamma[c] : 1.f, b = beta ? beta[c] : 0.f;
    const float* src = x + plane * hw;
    float* dst = y + plane * hw;
    const bool vec = (hw & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) * 4; i < hw; i += static_cast<int64_t>(gridDim.x) * THREADS * 4) {
        if (vec && i + 4 <= hw) {
            float4 v = *reinterpret_cast<const float4*>(src + i);
            float o[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float t = ((o[k] - m) * r) * g + b;
                o[k] = relu ? (t > 0.f ? t : 0.f) : t;
            }
            *reinterpret_cast<float4*>(dst + i) = make_float4(o[0], o[1], o[2], o[3]);
        } else {
            for (int64_t j = i; j < hw && j < i + 4; ++j) {
                float t = ((src[j] - m) * r) * g + b;
                dst[j] = relu ? (t > 0.f ? t : 0.f) : t;
            }
        }
    }
}

// Plain BN backward statistics: sum(dy) and sum(dy * xhat) per channel.  Same grid as bn_stats.
__global__ void __launch_bounds__(THREADS) bn_bwd_stats_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                                const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                int64_t n_img, int c_total, int64_t hw, double* __restrict__ part) {
    const int c = blockIdx.x;
    const float m = mean[c], r = rstd[c];
    double s1 = 0.0, s2 = 0.0;
    {
        const int64_t per = (n_img + gridDim.y - 1) / gridDim.y;
        const int64_t n0 = min(n_img, static_cast<int64_t>(blockIdx.y) * per), n1 = min(n_img, n0 + per);  // n1 >= n0, empty slab allowed
        const int64_t stride = static_cast<int64_t>(c_total) * hw;
        const float* xslab = x + (n0 * c_total + c) * hw;
        const float* gslab = dy + (n0 * c_total + c) * hw;
        float a1 = 0.f, a2 = 0.f;
        int flushed = 0;
        if ((hw & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy)) & 15) == 0) {
            const uint32_t q = static_cast<uint32_t>(hw >> 2), items = static_cast<uint32_t>(n1 - n0) * q;
#pragma unroll 2
            for (uint32_t j = threadIdx.x; j < items; j += THREADS) {
                const uint32_t n = j / q, i = (j - n * q) * 4;
                const float4 g = *reinterpret_cast<const float4*>(gslab + n * stride + i);
                const float4 v = *reinterpret_cast<const float4*>(xslab + n * stride + i);
                a1 += (g.x + g.y) + (g.z + g.w);
                a2 += g.x * ((v.x - m) * r) + g.y * ((v.y - m) * r) + g.z * ((v.z - m) * r) + g.w * ((v.w - m) * r);
                if (++flushed == 64) { s1 += a1; s2 += a2; a1 = a2 = 0.f; flushed = 0; }
            }
        } else {
            const uint32_t uhw = static_cast<uint32_t>(hw), items = static_cast<uint32_t>(n1 - n0) * uhw;
            for (uint32_t j = threadIdx.x; j < items; j += THREADS) {
                const uint32_t n = j / uhw, i = j - n * uhw;
                float g = gslab[n * stride + i];
                a1 += g;
                a2 += g * ((xslab[n * stride + i] - m) * r);
                if (++flushed == 256) { s1 += a1; s2 += a2; a1 = a2 = 0.f; flushed = 0; }
            }
        }
        s1 += a1;
        s2 += a2;
    }
    __shared__ double r1[THREADS], r2[THREADS];
    r1[threadIdx.x] = s1;
    r2[threadIdx.x] = s2;
    __syncthreads();
    for (int s = THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) { r1[threadIdx.x] += r1[threadIdx.x + s]; r2[threadIdx.x] += r2[threadIdx.x + s]; }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        part[(static_cast<int64_t>(c) * gridDim.y + blockIdx.y) * 2] = r1[0];
        part[(static_cast<int64_t>(c) * gridDim.y + blockIdx.y) * 2 + 1] = r2[0];
    }
}

// dbeta = sum dy, dgamma = sum dy*xhat (gradients of the affine parameters).
// One warp per channel: lane l adds the slabs l, l + 32, ... in ascending order and the lanes' sums are combined by a
// fixed shuffle tree (one order, every run).
__global__ void __launch_bounds__(128) bn_bwd_finalize_kernel(const double* __restrict__ part, int splits, int c_total, float* __restrict__ dgamma,
                                                              float* __restrict__ dbeta) {
    wb_pdl_enter();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (c >= c_total) return;
    double s1 = 0.0, s2 = 0.0;
    for (int s = lane; s < splits; s += 32) {
        s1 += part[(static_cast<int64_t>(c) * splits + s) * 2];
        s2 += part[(static_cast<int64_t>(c) * splits + s) * 2 + 1];
    }
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) {
        s1 += __shfl_down_sync(0xffffffffu, s1, sh);
        s2 += __shfl_down_sync(0xffffffffu, s2, sh);
    }
    if (lane == 0) {
        dbeta[c] = static_cast<float>(s1);
        dgamma[c] = static_cast<float>(s2);
    }
}

// dx = gamma * rstd * (dy - dbeta/count - xhat * dgamma/count)
__global__ void __launch_bounds__(THREADS) bn_bwd_dx_kernel(float* __restrict__ dx, const float* __restrict__ x, const float* __restrict__ dy,
                                                             const float* __restrict__ mean, const float* __restrict__ rstd,
                                                             const float* __restrict__ gamma, const float* __restrict__ dgamma,
                                                             const float* __restrict__ dbeta, int c_total, int64_t hw, float inv_count) {
    int64_t plane = blockIdx.y;
    int c = static_cast<int>(plane % c_total);
    float m = mean[c], r = rstd[c], g = gamma ? gamma[c] : 1.f;
    float k1 = dbeta[c] * inv_count, k2 = dgamma[c] * inv_count, gr = g * r;
    const float* xs = x + plane * hw;
    const float* gs = dy + plane * hw;
    float* dst = dx + plane * hw;
    if ((hw & 3) == 0 && ((reinterpret_cast<uintptr_t>(xs) | reinterpret_cast<uintptr_t>(gs) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
        for (int64_t i = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) * 4; i < hw; i += static_cast<int64_t>(gridDim.x) * THREADS * 4) {
            const float4 v = *reinterpret_cast<const float4*>(xs + i);
            const float4 gg = *reinterpret_cast<const float4*>(gs + i);
            float4 o;
            o.x = gr * (gg.x - k1 - ((v.x - m) * r) * k2);
            o.y = gr * (gg.y - k1 - ((v.y - m) * r) * k2);
            o.z = gr * (gg.z - k1 - ((v.z - m) * r) * k2);
            o.w = gr * (gg.w - k1 - ((v.w - m) * r) * k2);
            *reinterpret_cast<float4*>(dst + i) = o;
        }
        return;
    }
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x; i < hw; i += static_cast<int64_t>(gridDim.x) * THREADS) {
        float xh = (xs[i] - m) * r;
        dst[i] = gr * (gs[i] - k1 - xh * k2);
    }
}

// ---- conv block tail: BN -> ReLU -> 2x2 max pool, one pass each way ------------------------------

// Forward, w % 8 == 0: one thread per four pooled values of a row (two float4 loads from each of two input
// rows, one float4 store).  SHIFT also writes the pooled tensor shifted one column right (left[y][x] = y[y][x-1])
// and left (right[y][x] = y[y][x+1]) with zeros shifted in: the three copies an implicit-GEMM convolution of the
// pooled tensor reads.  The neighbour values come from the adjacent lanes, so SHIFT needs rows that do not
// straddle warps: w / 8 must divide 32.
template <bool SHIFT>
__global__ void __launch_bounds__(THREADS) bn_relu_pool_fwd_quad_kernel(float* __restrict__ yp, float* __restrict__ y_left,
                                                                         float* __restrict__ y_right, const float* __restrict__ x,
                                                                         const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                         const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                         int c_total, int h, int w, uint32_t total, FastDiv div_ipp,
                                                                         FastDiv div_owq, FastDiv div_c) {
    wb_pdl_enter();
    const uint32_t owq = static_cast<uint32_t>(w >> 3), ipp = static_cast<uint32_t>(h >> 1) * owq;
    const int64_t plane_elems = static_cast<int64_t>(h) * w;
    const uint32_t stride = gridDim.x * THREADS;
    for (uint32_t base = blockIdx.x * THREADS + (threadIdx.x & ~31u); base < total; base += stride) {
        const uint32_t j = base + (threadIdx.x & 31u);
        const bool valid = j < total;
        float4 out = make_float4(0.f, 0.f, 0.f, 0.f);
        uint32_t oxq = 0;
        if (valid) {
            const uint32_t plane = div_ipp.div(j), i = j - plane * ipp;
            const uint32_t oy = div_owq.div(i);
            oxq = i - oy * owq;
            const uint32_t c = plane - div_c.div(plane) * static_cast<uint32_t>(c_total);
            const float m = __ldg(mean + c), r = __ldg(rstd + c), g = __ldg(gamma + c), b = __ldg(beta + c);
            const float* src = x + static_cast<int64_t>(plane) * plane_elems + static_cast<int64_t>(2 * oy) * w + 8 * oxq;
            const float4 a0 = *reinterpret_cast<const float4*>(src), a1 = *reinterpret_cast<const float4*>(src + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(src + w), b1 = *reinterpret_cast<const float4*>(src + w + 4);
#define WB_BN_ACT(v) fmaf(((v) - m) * r, g, b)
            out.x = fmaxf(fmaxf(fmaxf(WB_BN_ACT(a0.x), WB_BN_ACT(a0.y)), fmaxf(WB_BN_ACT(b0.x), WB_BN_ACT(b0.y))), 0.f);
            out.y = fmaxf(fmaxf(fmaxf(WB_BN_ACT(a0.z), WB_BN_ACT(a0.w)), fmaxf(WB_BN_ACT(b0.z), WB_BN_ACT(b0.w))), 0.f);
            out.z = fmaxf(fmaxf(fmaxf(WB_BN_ACT(a1.x), WB_BN_ACT(a1.y)), fmaxf(WB_BN_ACT(b1.x), WB_BN_ACT(b1.y))), 0.f);
            out.w = fmaxf(fmaxf(fmaxf(WB_BN_ACT(a1.z), WB_BN_ACT(a1.w)), fmaxf(WB_BN_ACT(b1.z), WB_BN_ACT(b1.w))), 0.f);
#undef WB_BN_ACT
            reinterpret_cast<float4*>(yp)[j] = out;
        }
        if (SHIFT) {
            float prev = __shfl_up_sync(0xffffffffu, out.w, 1), next = __shfl_down_sync(0xffffffffu, out.x, 1);
            if (valid) {
                if (oxq == 0) prev = 0.f;
                if (oxq == owq - 1) next = 0.f;
                reinterpret_cast<float4*>(y_left)[j] = make_float4(prev, out.x, out.y, out.z);
                reinterpret_cast<float4*>(y_right)[j] = make_float4(out.y, out.z, out.w, next);
            }
        }
    }
}


// Forward: one thread per pooled element.
__global__ void __launch_bounds__(THREADS) bn_relu_pool_fwd_kernel(float* __restrict__ yp, const float* __restrict__ x,
                                                                    const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                    const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                    int c_total, int h, int w, int64_t total) {
    wb_pdl_enter();
    int64_t i = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (i >= total) return;
    const int ow = w >> 1, oh = h >> 1;
    int ox = static_cast<int>(i % ow);
    int64_t t = i / ow;
    int oy = static_cast<int>(t % oh);
    int64_t plane = t / oh;
    int c = static_cast<int>(plane % c_total);
    float m = mean[c], r = rstd[c], g = gamma[c], b = beta[c];
    const float* src = x + plane * h * w + static_cast<int64_t>(2 * oy) * w + 2 * ox;
    float2 r0 = *reinterpret_cast<const float2*>(src);
    float2 r1 = *reinterpret_cast<const float2*>(src + w);
    float v[4] = {r0.x, r0.y, r1.x, r1.y};
    float best = -INFINITY;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        best = fmaxf(best, fmaxf(fmaf((v[k] - m) * r, g, b), 0.f));
    }
    yp[i] = best;
}

// Backward recompute for one pooled element: the gradient each of the 4 window positions receives
// through max-pool (ties share equally, crates/weta-autograd/src/ops.rs:305-314) and ReLU
// (g * step(pre-activation), ops.rs:85), plus xhat at those positions.
// The pooled maximum is never negative (it follows a ReLU); when it is zero every position is at or
// below the ReLU threshold and receives nothing.  Otherwise the winners are the positions equal to
// the maximum and each gets (1/count) * dy, the reference's mask/count then * g.
__device__ __forceinline__ void pool_window_grads(const float v[4], float m, float r, float g, float b, float dyp, float gout[4], float xh[4]) {
    float act[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        xh[k] = (v[k] - m) * r;
        act[k] = fmaxf(fmaf(xh[k], g, b), 0.f);
    }
    const float best = fmaxf(fmaxf(act[0], act[1]), fmaxf(act[2], act[3]));
    const int cnt = (act[0] == best) + (act[1] == best) + (act[2] == best) + (act[3] == best);
    const float inv = cnt == 1 ? 1.f : (cnt == 2 ? 0.5f : (cnt == 3 ? (1.f / 3.f) : 0.25f));
    const float share = best > 0.f ? inv * dyp : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) gout[k] = act[k] == best ? share : 0.f;
}

// grid (C, S) like bn_stats: sums of the full-resolution gradient and of gradient * xhat.
__global__ void __launch_bounds__(THREADS) bn_relu_pool_bwd_stats_kernel(const float* __restrict__ x, const float* __restrict__ dyp,
                                                                          const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                          const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                          int64_t n_img, int c_total, int h, int w, double* __restrict__ part) {
    wb_pdl_enter();
    const int c = blockIdx.x;
    const float m = mean[c], r = rstd[c], g = gamma[c], b = beta[c];
    const int ow = w >> 1, oh = h >> 1, pooled = ow * oh;
    double s1 = 0.0, s2 = 0.0;
    {
        const int64_t per = (n_img + gridDim.y - 1) / gridDim.y;
        const int64_t n0 = min(n_img, static_cast<int64_t>(blockIdx.y) * per), n1 = min(n_img, n0 + per);  // n1 >= n0, empty slab allowed
        const uint32_t up = static_cast<uint32_t>(pooled), items = static_cast<uint32_t>(n1 - n0) * up;
        const int64_t xstride = static_cast<int64_t>(c_total) * h * w, gstride = static_cast<int64_t>(c_total) * pooled;
        const float* xslab = x + (n0 * c_total + c) * h * w;
        const float* gslab = dyp + (n0 * c_total + c) * pooled;
        float a1 = 0.f, a2 = 0.f;
        int flushed = 0;
        for (uint32_t j = threadIdx.x; j < items; j += THREADS) {
            const uint32_t n = j / up, i = j - n * up;
            const uint32_t oy = i / static_cast<uint32_t>(ow), ox = i - oy * ow;
            const float* src = xslab + n * xstride + 2 * oy * w + 2 * ox;
            float2 r0 = *reinterpret_cast<const float2*>(src);
            float2 r1 = *reinterpret_cast<const float2*>(src + w);
            float v[4] = {r0.x, r0.y, r1.x, r1.y}, go[4], xh[4];
            pool_window_grads(v, m, r, g, b, gslab[n * gstride + i], go, xh);
#pragma unroll
            for (int k = 0; k < 4; ++k) { a1 += go[k]; a2 += go[k] * xh[k]; }
            if (++flushed == 64) { s1 += a1; s2 += a2; a1 = a2 = 0.f; flushed = 0; }
        }
        s1 += a1;
        s2 += a2;
    }
    __shared__ double r1s[THREADS], r2s[THREADS];
    r1s[threadIdx.x] = s1;
    r2s[threadIdx.x] = s2;
    __syncthreads();
    for (int s = THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) { r1s[threadIdx.x] += r1s[threadIdx.x + s]; r2s[threadIdx.x] += r2s[threadIdx.x + s]; }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        part[(static_cast<int64_t>(c) * gridDim.y + blockIdx.y) * 2] = r1s[0];
        part[(static_cast<int64_t>(c) * gridDim.y + blockIdx.y) * 2 + 1] = r2s[0];
    }
}

// dx at full resolution; also per-(channel, split) sums of dx, which is the gradient of the
// convolution bias that feeds this BatchNorm.  grid (C, S), same walk as the stats kernel.
__global__ void __launch_bounds__(THREADS) bn_relu_pool_bwd_dx_kernel(float* __restrict__ dx, const float* __restrict__ x,
                                                                       const float* __restrict__ dyp, const float* __restrict__ mean,
                                                                       const float* __restrict__ rstd, const float* __restrict__ gamma,
                                                                       const float* __restrict__ beta, const float* __restrict__ dgamma,
                                                                       const float* __restrict__ dbeta, int64_t n_img, int c_total, int h,
                                                                       int w, float inv_count, double* __restrict__ bias_part) {
    wb_pdl_enter();
    const int c = blockIdx.x;
    const float m = mean[c], r = rstd[c], g = gamma[c], b = beta[c];
    const float k1 = dbeta[c] * inv_count, k2 = dgamma[c] * inv_count, gr = g * r;
    const int ow = w >> 1, oh = h >> 1, pooled = ow * oh;
    double sb = 0.0;
    {
        const int64_t per = (n_img + gridDim.y - 1) / gridDim.y;
        const int64_t n0 = min(n_img, static_cast<int64_t>(blockIdx.y) * per), n1 = min(n_img, n0 + per);  // n1 >= n0, empty slab allowed
        const uint32_t up = static_cast<uint32_t>(pooled), items = static_cast<uint32_t>(n1 - n0) * up;
        const int64_t xstride = static_cast<int64_t>(c_total) * h * w, gstride = static_cast<int64_t>(c_total) * pooled;
        const float* xslab = x + (n0 * c_total + c) * h * w;
        const float* gslab = dyp + (n0 * c_total + c) * pooled;
        float* dslab = dx + (n0 * c_total + c) * h * w;
        float a = 0.f;
        int flushed = 0;
        for (uint32_t j = threadIdx.x; j < items; j += THREADS) {
            const uint32_t n = j / up, i = j - n * up;
            const uint32_t oy = i / static_cast<uint32_t>(ow), ox = i - oy * ow;
            const int64_t o = n * xstride + static_cast<int64_t>(2 * oy) * w + 2 * ox;
            float2 r0 = *reinterpret_cast<const float2*>(xslab + o);
            float2 r1 = *reinterpret_cast<const float2*>(xslab + o + w);
            float v[4] = {r0.x, r0.y, r1.x, r1.y}, go[4], xh[4], d[4];
            pool_window_grads(v, m, r, g, b, gslab[n * gstride + i], go, xh);
#pragma unroll
            for (int k = 0; k < 4; ++k) { d[k] = gr * (go[k] - k1 - xh[k] * k2); a += d[k]; }
            *reinterpret_cast<float2*>(dslab + o) = make_float2(d[0], d[1]);
            *reinterpret_cast<float2*>(dslab + o + w) = make_float2(d[2], d[3]);
            if (++flushed == 64) { sb += a; a = 0.f; flushed = 0; }
        }
        sb += a;
    }
    __shared__ double rs[THREADS];
    rs[threadIdx.x] = sb;
    __syncthreads();
    for (int s = THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) rs[threadIdx.x] += rs[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0 && bias_part) bias_part[static_cast<int64_t>(c) * gridDim.y + blockIdx.y] = rs[0];
}

// The backward sums of BatchNorm -> ReLU -> MaxPool(2) can be taken from the POOLED tensors alone: a window passes
// gradient only to the positions equal to its maximum, all of which hold the same value, so per window
//     sum(dy)        = g                     if y > 0 else 0        (g: the window's upstream gradient, y: its pooled output)
//     sum(dy * xhat) = g * (y - beta)/gamma  if y > 0 else 0        (y = xhat_w * gamma + beta at the winner)
// which reads a quarter of the activation instead of all of it.  Recovering xhat from y costs |y| * 2^-23 / |gamma| of
// accuracy, so a channel takes this path only when |gamma| >= |beta| / 64 and |gamma| >= 1e-6 (always, for freshly
// initialised and normally trained layers); the other channels are summed from x by the kernel below.
__device__ __forceinline__ bool pooled_sums_ok(float g, float b) { return fabsf(g) * 64.f >= fabsf(b) && fabsf(g) >= 1e-6f; }

// Same (channel, slab) items and the same layout of `part` as bn_relu_pool_bwd_pair_kernel<false, ...>, one WARP per
// item (no block-wide barrier: an item is a few hundred to a few thousand float4s).  Channels that fail the test above
// are summed from x by the same warp, window by window, with the arithmetic of pool_window_grads.
__global__ void __launch_bounds__(THREADS) bn_relu_pool_bwd_sums_pooled_kernel(const float* __restrict__ yp, const float* __restrict__ dyp,
                                                                                const float* __restrict__ x, const float* __restrict__ mean,
                                                                                const float* __restrict__ rstd, const float* __restrict__ gamma,
                                                                                const float* __restrict__ beta, int64_t n_img, int c_total, int h,
                                                                                int w, double* __restrict__ part, int slabs) {
    wb_pdl_enter();
    const int ow = w >> 1, oh = h >> 1, pooled = ow * oh;
    const int64_t per = (n_img + slabs - 1) / slabs;
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * THREADS) >> 5, first = (blockIdx.x * THREADS + threadIdx.x) >> 5;
    const uint32_t q = static_cast<uint32_t>(pooled >> 2);  // pooled % 4 == 0 (checked by the host)
    // Channel fastest: the warps that run side by side read neighbouring planes of the same images, so the 1-4 KB
    // pieces they fetch lie next to one another in memory.
    for (int item = first; item < c_total * slabs; item += warps) {
        const int sl = item / c_total, c = item - sl * c_total;
        const float g = __ldg(gamma + c), b = __ldg(beta + c);
        const int64_t n0 = min(n_img, static_cast<int64_t>(sl) * per), n1 = min(n_img, n0 + per);
        const int64_t stride = static_cast<int64_t>(c_total) * pooled, base = (n0 * c_total + c) * pooled;
        double s1 = 0.0, s2 = 0.0;
        float a1 = 0.f, a2 = 0.f;
        int flushed = 0;
        if (pooled_sums_ok(g, b)) {
            const uint32_t items = static_cast<uint32_t>(n1 - n0) * q;
            // four float4 pairs per lane in flight: all eight loads are issued before any of them is used
            for (uint32_t j0 = lane; j0 < items; j0 += 128) {
                float4 y[4], u[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const uint32_t j = j0 + 32 * t;
                    if (j < items) {
                        const uint32_t n = j / q, i = j - n * q;
                        const int64_t o = base + n * stride + 4 * static_cast<int64_t>(i);
                        y[t] = *reinterpret_cast<const float4*>(yp + o);
                        u[t] = *reinterpret_cast<const float4*>(dyp + o);
                    } else {
                        y[t] = u[t] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float ys[4] = {y[t].x, y[t].y, y[t].z, y[t].w}, us[4] = {u[t].x, u[t].y, u[t].z, u[t].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (ys[k] > 0.f) {
                            a1 += us[k];
                            a2 += us[k] * ((ys[k] - b) / g);
                        }
                }
                if (++flushed == 8) { s1 += a1; s2 += a2; a1 = a2 = 0.f; flushed = 0; }
            }
        } else {
            const float m = __ldg(mean + c), r = __ldg(rstd + c);
            const uint32_t up = static_cast<uint32_t>(pooled), items = static_cast<uint32_t>(n1 - n0) * up;
            const int64_t xstride = static_cast<int64_t>(c_total) * h * w;
            const float* xslab = x + (n0 * c_total + c) * h * w;
            for (uint32_t j = lane; j < items; j += 32) {
                const uint32_t n = j / up, i = j - n * up;
                const uint32_t oy = i / static_cast<uint32_t>(ow), ox = i - oy * ow;
                const float* src = xslab + n * xstride + 2 * oy * w + 2 * ox;
                const float2 r0 = *reinterpret_cast<const float2*>(src), r1 = *reinterpret_cast<const float2*>(src + w);
                float v[4] = {r0.x, r0.y, r1.x, r1.y}, go[4], xh[4];
                pool_window_grads(v, m, r, g, b, dyp[base + n * stride + i], go, xh);
#pragma unroll
                for (int k = 0; k < 4; ++k) { a1 += go[k]; a2 += go[k] * xh[k]; }
                if (++flushed == 32) { s1 += a1; s2 += a2; a1 = a2 = 0.f; flushed = 0; }
            }
        }
        s1 += a1;
        s2 += a2;
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) {
            s1 += __shfl_down_sync(0xffffffffu, s1, sh);
            s2 += __shfl_down_sync(0xffffffffu, s2, sh);
        }
        if (lane == 0) {
            part[(static_cast<int64_t>(c) * slabs + sl) * 2] = s1;
            part[(static_cast<int64_t>(c) * slabs + sl) * 2 + 1] = s2;
        }
    }
}

// Width-multiple-of-4 variants: one thread handles two neighbouring pooled elements, i.e. a 2x4 patch
// of x, with 128-bit loads and stores; same arithmetic as the kernels above.
// SHIFT (with WRITE_DX): also writes dx shifted one column right (dx_left[y][x] = dx[y][x-1]) and left
// (dx_right[y][x] = dx[y][x+1]), zeros shifted in; the neighbour values come from the adjacent lanes, so
// w / 4 must divide 32.
template <bool WRITE_DX, bool SHIFT>
__global__ void __launch_bounds__(THREADS, 5) bn_relu_pool_bwd_pair_kernel(float* __restrict__ dx, float* __restrict__ dx_left,
                                                                            float* __restrict__ dx_right, const float* __restrict__ x,
                                                                            const float* __restrict__ dyp, const float* __restrict__ mean,
                                                                            const float* __restrict__ rstd, const float* __restrict__ gamma,
                                                                            const float* __restrict__ beta, const float* __restrict__ dgamma,
                                                                            const float* __restrict__ dbeta, int64_t n_img, int c_total, int h,
                                                                            int w, float inv_count, double* __restrict__ part, FastDiv div_pairs,
                                                                            FastDiv div_owp, int slabs, int skip_pooled_ok) {
    wb_pdl_enter();
    // Work items are (channel, slab of images) pairs, many more than blocks, walked round-robin: every SM stays
    // equally loaded whatever the channel count.  The two windows a thread owns are computed side by side in
    // packed f32x2 arithmetic (.x = left window, .y = right window).
    const int ow = w >> 1, oh = h >> 1, pooled = ow * oh;
    const uint32_t owp = static_cast<uint32_t>(ow >> 1), pairs = static_cast<uint32_t>(oh) * owp;
    const int64_t per = (n_img + slabs - 1) / slabs;
    const int64_t xstride = static_cast<int64_t>(c_total) * h * w, gstride = static_cast<int64_t>(c_total) * pooled;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ double red[2][THREADS / 32];
    for (int item = blockIdx.x; item < c_total * slabs; item += gridDim.x) {
        // channel fastest: blocks that run side by side read neighbouring planes of the same images (the dx pass of the
        // 128 -> 256 channel block: 0.548 -> 0.537 ms against slab fastest)
        const int sl = item / c_total, c = item - sl * c_total;
        const int64_t slot = static_cast<int64_t>(c) * slabs + sl;
        const float m = __ldg(mean + c), r = __ldg(rstd + c), g = __ldg(gamma + c), b = __ldg(beta + c);
        // sums pass only: this channel's sums were already taken from the pooled tensors (block-uniform)
        if (!WRITE_DX && skip_pooled_ok && pooled_sums_ok(g, b)) continue;
        float k1 = 0.f, k2 = 0.f, gr = 0.f;
        if (WRITE_DX) { k1 = __ldg(dbeta + c) * inv_count; k2 = __ldg(dgamma + c) * inv_count; gr = g * r; }
        const float2 negm2 = make_float2(-m, -m), r2 = make_float2(r, r), g2 = make_float2(g, g), b2 = make_float2(b, b);
        const float2 negk1 = make_float2(-k1, -k1), negk2 = make_float2(-k2, -k2), gr2 = make_float2(gr, gr);
        const int64_t n0 = min(n_img, static_cast<int64_t>(sl) * per), n1 = min(n_img, n0 + per);
        const uint32_t items = static_cast<uint32_t>(n1 - n0) * pairs;
        const int64_t slab_off = (n0 * c_total + c) * h * w;
        const float* xslab = x + slab_off;
        const float* gslab = dyp + (n0 * c_total + c) * pooled;
        double s1 = 0.0, s2 = 0.0;
        float2 acc1 = make_float2(0.f, 0.f), acc2 = make_float2(0.f, 0.f);
        int flushed = 0;
#pragma unroll 2
        for (uint32_t base = threadIdx.x & ~31u; base < items; base += THREADS) {
            const uint32_t j = base + lane;
            const bool valid = j < items;
            float2 d[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) d[k] = make_float2(0.f, 0.f);
            uint32_t oxp = 0;
            int64_t o = 0;
            if (valid) {
                const uint32_t n = div_pairs.div(j), i = j - n * pairs;
                const uint32_t oy = div_owp.div(i);
                oxp = i - oy * owp;
                o = n * xstride + static_cast<int64_t>(2 * oy) * w + 4 * oxp;
                const float4 r0 = *reinterpret_cast<const float4*>(xslab + o);
                const float4 r1 = *reinterpret_cast<const float4*>(xslab + o + w);
                const float2 gy = *reinterpret_cast<const float2*>(gslab + n * gstride + oy * ow + 2 * oxp);
                // window positions k = 0..3: (row 0, col 0), (row 0, col 1), (row 1, col 0), (row 1, col 1)
                const float2 v[4] = {make_float2(r0.x, r0.z), make_float2(r0.y, r0.w), make_float2(r1.x, r1.z), make_float2(r1.y, r1.w)};
                float2 xh[4], act[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    xh[k] = __fmul2_rn(__fadd2_rn(v[k], negm2), r2);
                    const float2 pre = __ffma2_rn(xh[k], g2, b2);
                    act[k] = make_float2(fmaxf(pre.x, 0.f), fmaxf(pre.y, 0.f));
                }
                // Ties share the gradient (1/count each); a window whose maximum is 0 lies at or below the ReLU
                // threshold everywhere and receives nothing.
                const float bx = fmaxf(fmaxf(act[0].x, act[1].x), fmaxf(act[2].x, act[3].x));
                const float by = fmaxf(fmaxf(act[0].y, act[1].y), fmaxf(act[2].y, act[3].y));
                const int cx = (act[0].x == bx) + (act[1].x == bx) + (act[2].x == bx) + (act[3].x == bx);
                const int cy = (act[0].y == by) + (act[1].y == by) + (act[2].y == by) + (act[3].y == by);
                const float ix = cx == 1 ? 1.f : (cx == 2 ? 0.5f : (cx == 3 ? (1.f / 3.f) : 0.25f));
                const float iy = cy == 1 ? 1.f : (cy == 2 ? 0.5f : (cy == 3 ? (1.f / 3.f) : 0.25f));
                const float sx = bx > 0.f ? ix * gy.x : 0.f, sy = by > 0.f ? iy * gy.y : 0.f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 go = make_float2(act[k].x == bx ? sx : 0.f, act[k].y == by ? sy : 0.f);
                    if (WRITE_DX) {
                        d[k] = __fmul2_rn(gr2, __ffma2_rn(xh[k], negk2, __fadd2_rn(go, negk1)));
                        acc1 = __fadd2_rn(acc1, d[k]);
                    } else {
                        acc1 = __fadd2_rn(acc1, go);
                        acc2 = __ffma2_rn(go, xh[k], acc2);
                    }
                }
                if (WRITE_DX) {
                    *reinterpret_cast<float4*>(dx + slab_off + o) = make_float4(d[0].x, d[1].x, d[0].y, d[1].y);
                    *reinterpret_cast<float4*>(dx + slab_off + o + w) = make_float4(d[2].x, d[3].x, d[2].y, d[3].y);
                }
            }
            if (WRITE_DX && SHIFT) {
                float p0 = __shfl_up_sync(0xffffffffu, d[1].y, 1), p1 = __shfl_up_sync(0xffffffffu, d[3].y, 1);
                float q0 = __shfl_down_sync(0xffffffffu, d[0].x, 1), q1 = __shfl_down_sync(0xffffffffu, d[2].x, 1);
                if (valid) {
                    if (oxp == 0) p0 = p1 = 0.f;
                    if (oxp == owp - 1) q0 = q1 = 0.f;
                    const int64_t so = slab_off + o;
                    *reinterpret_cast<float4*>(dx_left + so) = make_float4(p0, d[0].x, d[1].x, d[0].y);
                    *reinterpret_cast<float4*>(dx_left + so + w) = make_float4(p1, d[2].x, d[3].x, d[2].y);
                    *reinterpret_cast<float4*>(dx_right + so) = make_float4(d[1].x, d[0].y, d[1].y, q0);
                    *reinterpret_cast<float4*>(dx_right + so + w) = make_float4(d[3].x, d[2].y, d[3].y, q1);
                }
            }
            if (++flushed == 32) {  // keep the f32 partial sums short
                s1 += static_cast<double>(acc1.x) + static_cast<double>(acc1.y);
                s2 += static_cast<double>(acc2.x) + static_cast<double>(acc2.y);
                acc1 = acc2 = make_float2(0.f, 0.f);
                flushed = 0;
            }
        }
        s1 += static_cast<double>(acc1.x) + static_cast<double>(acc1.y);
        s2 += static_cast<double>(acc2.x) + static_cast<double>(acc2.y);
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) {
            s1 += __shfl_down_sync(0xffffffffu, s1, sh);
            s2 += __shfl_down_sync(0xffffffffu, s2, sh);
        }
        if (lane == 0) { red[0][warp] = s1; red[1][warp] = s2; }
        __syncthreads();
        if (threadIdx.x == 0 && part) {
            double t1 = 0.0, t2 = 0.0;
            for (int q = 0; q < THREADS / 32; ++q) { t1 += red[0][q]; t2 += red[1][q]; }
            if (WRITE_DX) {
                part[slot] = t1;  // sum of dx: the conv bias gradient
            } else {
                part[slot * 2] = t1;
                part[slot * 2 + 1] = t2;
            }
        }
        __syncthreads();
    }
}

// One warp per channel, as bn_bwd_finalize_kernel.
__global__ void __launch_bounds__(128) sum_parts_kernel(const double* __restrict__ part, int splits, int c_total, float* __restrict__ out) {
    wb_pdl_enter();
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (c >= c_total) return;
    double s = 0.0;
    for (int k = lane; k < splits; k += 32) s += part[static_cast<int64_t>(c) * splits + k];
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) s += __shfl_down_sync(0xffffffffu, s, sh);
    if (lane == 0) out[c] = static_cast<float>(s);
}

// Number of image slabs per channel for the per-channel reductions (grid = channels x slabs).  The grid
// is sized to ONE resident wave of the kernel (occupancy x SM count): these kernels stream for the
// whole launch, so a second, partly filled wave would cost as much as the first.  Also few enough
// images per slab that the kernels' 32-bit item counters cannot overflow.
template <class Kernel>
int stat_splits(WbBackend* be, Kernel kernel, int c, int64_t n_img, int64_t items_per_image) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, THREADS, 0) != cudaSuccess || per_sm < 1) {
        (void)cudaGetLastError();
        per_sm = 4;
    }
    int64_t want = std::max<int64_t>(1, static_cast<int64_t>(per_sm) * be->sm_count / c);
    int64_t need = (n_img * items_per_image + (int64_t(1) << 30) - 1) / (int64_t(1) << 30);
    int64_t splits = std::max<int64_t>(1, std::min<int64_t>(std::max(want, need), n_img));
    int64_t per = (n_img + splits - 1) / splits;
    return static_cast<int>((n_img + per - 1) / per);  // no slab is empty
}

}  // namespace

extern "C" int wb_bn2d_stats(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t hw, double eps, double momentum, float* mean,
                             float* rstd, float* running_mean, float* running_var) {
    WB_REQUIRE(b && x && mean && rstd, WB_ERR_INVALID, "wb_bn2d_stats: null pointer");
    WB_REQUIRE(n > 0 && c > 0 && hw > 0, WB_ERR_INVALID, "wb_bn2d_stats: empty input");
    WbProfileScope ps(b, "bn2d_stats");
    int splits = stat_splits(b, bn_stats_kernel, static_cast<int>(c), n, hw);
    void* s = nullptr;
    WB_TRY(wb_scratch(b, static_cast<size_t>(c) * splits * 2 * sizeof(double), &s));
    bn_stats_kernel<<<dim3(static_cast<unsigned>(c), splits), THREADS, 0, b->stream>>>(x, n, static_cast<int>(c), hw, static_cast<double*>(s));
    WB_LAUNCH_OK(b);
    bn_finalize_kernel<<<static_cast<unsigned>((c + 127) / 128), 128, 0, b->stream>>>(static_cast<double*>(s), splits, x, static_cast<int>(c), hw,
                                                                                    n * hw, static_cast<float>(eps), static_cast<float>(momentum),
                                                                                    static_cast<float>(1.0 - momentum), mean, rstd, running_mean,
                                                                                    running_var);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

// ---- batch statistics without any allocation ----------------------------------------------------
// Some hosts of this library may not allocate device memory at the time they need batch statistics:
// code running inside a framework's memory-pool callback or an allocator hook, a real-time loop that
// has frozen its memory map, or a process whose device memory is fully budgeted to another component.
// For them the per-(channel, slab) partial sums live in this fixed array, which every GPU that loads
// the library carries from load to exit (WB_NOALLOC_SCRATCH_DOUBLES * 8 bytes = 512 KiB).
#define WB_NOALLOC_SCRATCH_DOUBLES 65536
static __device__ __align__(256) double g_noalloc_scratch[WB_NOALLOC_SCRATCH_DOUBLES];

namespace {
// In host code `g_noalloc_scratch` is only a stand-in for the device array; a kernel must be given the
// address cudaGetSymbolAddress reports for the device that is current, looked up once per device.
constexpr int MAX_DEVICES = 64;
double* g_noalloc_ptr[MAX_DEVICES] = {};
}  // namespace

// Same result as wb_bn2d_stats (batch mean, rstd = 1/sqrt(biased var + eps), running statistics), on the
// CURRENT device and the given stream, using only the fixed scratch array above: no cudaMalloc, no
// cudaFree, no backend handle.  It fits c channels when 2*c <= WB_NOALLOC_SCRATCH_DOUBLES (c <= 32768);
// larger inputs are rejected with WB_ERR_INVALID.  The first call on each device looks up the array's
// address (cudaGetSymbolAddress) and, with CUDA's lazy module loading, may be the call that loads this
// library's device code, which itself takes device memory: make one warm-up call per device at start-up,
// outside the context that must not allocate and before starting any stream capture.  Two host threads
// that make the first call at once both store the same address into the per-device slot, which is
// harmless.  x may start at any float (an unaligned start takes the scalar loads).  All calls on a
// device share the one array: every slot a call reads is written by that call first, so nothing needs
// clearing, but two calls that overlap on the GPU (different streams, or different host threads on
// different streams) would overwrite each other's partial sums; run them on one stream or order them.
extern "C" int wb_bn2d_stats_noalloc(void* cuda_stream, const float* x, int64_t n, int64_t c, int64_t hw, double eps, double momentum,
                                     float* mean, float* rstd, float* running_mean, float* running_var) {
    WB_REQUIRE(x && mean && rstd, WB_ERR_INVALID, "wb_bn2d_stats_noalloc: null pointer");
    WB_REQUIRE(n > 0 && c > 0 && hw > 0, WB_ERR_INVALID, "wb_bn2d_stats_noalloc: empty input");
    WB_REQUIRE(2 * c <= WB_NOALLOC_SCRATCH_DOUBLES, WB_ERR_INVALID,
               "wb_bn2d_stats_noalloc: %lld channels need %lld scratch doubles, the fixed array holds %d (at most %d channels)", (long long)c,
               (long long)(2 * c), WB_NOALLOC_SCRATCH_DOUBLES, WB_NOALLOC_SCRATCH_DOUBLES / 2);
    int dev = -1;
    WB_CHECK_CUDA(cudaGetDevice(&dev));
    WB_REQUIRE(dev >= 0 && dev < MAX_DEVICES, WB_ERR_UNSUPPORTED, "wb_bn2d_stats_noalloc: device ordinal %d out of range", dev);
    if (!g_noalloc_ptr[dev]) {
        double* p = nullptr;
        WB_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch));
        WB_REQUIRE(p != nullptr, WB_ERR_CUDA, "wb_bn2d_stats_noalloc: the scratch array has no device address");
        g_noalloc_ptr[dev] = p;
    }
    double* scratch = g_noalloc_ptr[dev];
    int sm_count = 0;
    WB_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
    // As many image slabs per channel as fill the GPU once, capped by what the array holds and by n;
    // slabs are sized so that none is empty and the kernel's 32-bit item counter cannot overflow.
    int64_t splits = std::max<int64_t>(1, 8LL * sm_count / c);
    splits = std::min<int64_t>(splits, WB_NOALLOC_SCRATCH_DOUBLES / (2 * c));
    const int64_t need = (n * hw + (int64_t(1) << 30) - 1) / (int64_t(1) << 30);
    splits = std::min<int64_t>(std::max(splits, need), n);
    WB_REQUIRE(2 * c * splits <= WB_NOALLOC_SCRATCH_DOUBLES, WB_ERR_INVALID,
               "wb_bn2d_stats_noalloc: input of %lld x %lld x %lld elements does not fit the fixed scratch array", (long long)n, (long long)c,
               (long long)hw);
    const int64_t per = (n + splits - 1) / splits;
    splits = (n + per - 1) / per;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    bn_stats_kernel<<<dim3(static_cast<unsigned>(c), static_cast<unsigned>(splits)), THREADS, 0, stream>>>(x, n, static_cast<int>(c), hw, scratch);
    WB_CHECK_CUDA(cudaPeekAtLastError());
    bn_finalize_kernel<<<static_cast<unsigned>((c + 127) / 128), 128, 0, stream>>>(scratch, static_cast<int>(splits), x, static_cast<int>(c), hw, n * hw,
                                                                                 static_cast<float>(eps), static_cast<float>(momentum),
                                                                                 static_cast<float>(1.0 - momentum), mean, rstd, running_mean,
                                                                                 running_var);
    WB_CHECK_CUDA(cudaPeekAtLastError());
    return WB_OK;
}

extern "C" int wb_bn2d_apply(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t hw, const float* mean, const float* rstd,
                             const float* gamma, const float* beta, int relu, float* y) {
    WB_REQUIRE(b && x && y && mean && rstd, WB_ERR_INVALID, "wb_bn2d_apply: null pointer");
    WbProfileScope ps(b, "bn2d_apply");
    unsigned gx = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((hw / 4 + THREADS - 1) / THREADS, 64)));
    WB_REQUIRE(c <= 65535, WB_ERR_UNSUPPORTED, "wb_bn2d_apply: too many channels");
    // gridDim.y is limited to 65535: launch whole images' worth of planes at a time.
    for (int64_t p0 = 0; p0 < n * c; p0 += 65535 / c * c) {
        int64_t cnt = std::min<int64_t>(65535 / c * c, n * c - p0);
        bn_apply_kernel<<<dim3(gx, static_cast<unsigned>(cnt)), THREADS, 0, b->stream>>>(y + p0 * hw, x + p0 * hw, mean, rstd, gamma, beta,
                                                                                         static_cast<int>(c), hw, relu);
        WB_LAUNCH_OK(b);
    }
    return WB_OK;
}

extern "C" int wb_bn2d_fwd(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t hw, const float* gamma, const float* beta,
                           float* running_mean, float* running_var, double momentum, double eps, float* y, float* save_mean,
                           float* save_rstd) {
    WB_TRY(wb_bn2d_stats(b, x, n, c, hw, eps, momentum, save_mean, save_rstd, running_mean, running_var));
    return wb_bn2d_apply(b, x, n, c, hw, save_mean, save_rstd, gamma, beta, 0, y);
}

extern "C" int wb_bn2d_bwd(WbBackend* b, const float* x, const float* dy, int64_t n, int64_t c, int64_t hw, const float* gamma,
                           const float* save_mean, const float* save_rstd, float* dx, float* dgamma, float* dbeta) {
    WB_REQUIRE(b && x && dy && dx && dgamma && dbeta && save_mean && save_rstd, WB_ERR_INVALID, "wb_bn2d_bwd: null pointer");
    WbProfileScope ps(b, "bn2d_bwd");
    int splits = stat_splits(b, bn_bwd_stats_kernel, static_cast<int>(c), n, hw);
    void* s = nullptr;
    WB_TRY(wb_scratch(b, static_cast<size_t>(c) * splits * 2 * sizeof(double), &s));
    bn_bwd_stats_kernel<<<dim3(static_cast<unsigned>(c), splits), THREADS, 0, b->stream>>>(x, dy, save_mean, save_rstd, n, static_cast<int>(c), hw,
                                                                                          static_cast<double*>(s));
    WB_LAUNCH_OK(b);
    wb_launch_pdl(bn_bwd_finalize_kernel, dim3(static_cast<unsigned>((c + 3) / 4)), dim3(128), 0, b->stream, static_cast<double*>(s), splits, static_cast<int>(c), dgamma, dbeta);
    WB_LAUNCH_OK(b);
    unsigned gx = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((hw / 4 + THREADS - 1) / THREADS, 64)));
    for (int64_t p0 = 0; p0 < n * c; p0 += 65535 / c * c) {
        int64_t cnt = std::min<int64_t>(65535 / c * c, n * c - p0);
        bn_bwd_dx_kernel<<<dim3(gx, static_cast<unsigned>(cnt)), THREADS, 0, b->stream>>>(dx + p0 * hw, x + p0 * hw, dy + p0 * hw, save_mean, save_rstd,
                                                                                          gamma, dgamma, dbeta, static_cast<int>(c), hw,
                                                                                          static_cast<float>(1.0 / static_cast<double>(n * hw)));
        WB_LAUNCH_OK(b);
    }
    return WB_OK;
}

// BatchNorm2d (training statistics) -> ReLU -> MaxPool2d(2); y_left / y_right (both or neither) also receive the
// pooled tensor shifted one column right / left, zeros shifted in (needs w / 8 in {1, 2, 4, ..., 32}, aligned buffers).
// channel_sums (optional): per channel (sum d, sum d^2) in double with d = x - sums_pivot[channel] (pivot null = 0), when
// the producer of x already has them.
int wb_bn_relu_pool_fwd_shifted(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t h, int64_t w, const float* gamma, const float* beta,
                                float* running_mean, float* running_var, double momentum, double eps, float* y_pooled, float* save_mean,
                                float* save_rstd, float* y_left, float* y_right, const double* channel_sums, const float* sums_pivot) {
    WB_REQUIRE(b && x && gamma && beta && y_pooled, WB_ERR_INVALID, "wb_bn_relu_pool_fwd: null pointer");
    WB_REQUIRE(h % 2 == 0 && w % 2 == 0, WB_ERR_UNSUPPORTED, "wb_bn_relu_pool_fwd: height and width must be even");
    WB_REQUIRE((y_left == nullptr) == (y_right == nullptr), WB_ERR_INVALID, "wb_bn_relu_pool_fwd: give both shifted outputs or neither");
    if (channel_sums) {
        // (sum, sum of squares) per channel already accumulated by the kernel that wrote x
        WB_REQUIRE(n * h * w > 0, WB_ERR_INVALID, "wb_bn_relu_pool_fwd: empty input");
        // One block per channel: statistics straight from the sums, or recomputed from x where the sums cancel.
        wb_launch_pdl(bn_stats_from_sums_kernel, dim3(static_cast<unsigned>(c)), dim3(THREADS), 0, b->stream, x, channel_sums, sums_pivot, n, static_cast<int>(c), h * w,
                                                                                  static_cast<float>(eps), static_cast<float>(momentum),
                                                                                  static_cast<float>(1.0 - momentum), save_mean, save_rstd, running_mean,
                                                                                  running_var);
        WB_LAUNCH_OK(b);
    } else {
        WB_TRY(wb_bn2d_stats(b, x, n, c, h * w, eps, momentum, save_mean, save_rstd, running_mean, running_var));
    }
    WbProfileScope ps(b, "bn_relu_pool_fwd");
    const int64_t total = n * c * (h / 2) * (w / 2);
    if (total == 0) return WB_OK;
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y_pooled) | reinterpret_cast<uintptr_t>(y_left) |
                           reinterpret_cast<uintptr_t>(y_right)) & 15) == 0;
    const bool quads = w % 8 == 0 && aligned && total / 4 < (int64_t(1) << 31) && n * c < (int64_t(1) << 31);
    WB_REQUIRE(!y_left || (quads && 32 % (w / 8) == 0), WB_ERR_UNSUPPORTED,
               "wb_bn_relu_pool_fwd: shifted outputs need w / 8 in {1, 2, 4, 8, 16, 32} and 16-byte aligned buffers");
    if (quads) {
        const uint32_t items = static_cast<uint32_t>(total / 4);
        const FastDiv div_ipp(static_cast<uint32_t>((h / 2) * (w / 8))), div_owq(static_cast<uint32_t>(w / 8)), div_c(static_cast<uint32_t>(c));
        const unsigned grid = static_cast<unsigned>(std::min<int64_t>((items + THREADS - 1) / THREADS, static_cast<int64_t>(b->sm_count) * 8));
        if (y_left)
            wb_launch_pdl(bn_relu_pool_fwd_quad_kernel<true>, dim3(grid), dim3(THREADS), 0, b->stream, y_pooled, y_left, y_right, x, save_mean, save_rstd, gamma, beta,
                                                                               static_cast<int>(c), static_cast<int>(h), static_cast<int>(w),
                                                                               items, div_ipp, div_owq, div_c);
        else
            wb_launch_pdl(bn_relu_pool_fwd_quad_kernel<false>, dim3(grid), dim3(THREADS), 0, b->stream, y_pooled, nullptr, nullptr, x, save_mean, save_rstd, gamma, beta,
                                                                                static_cast<int>(c), static_cast<int>(h), static_cast<int>(w),
                                                                                items, div_ipp, div_owq, div_c);
    } else {
        wb_launch_pdl(bn_relu_pool_fwd_kernel, dim3(static_cast<unsigned>((total + THREADS - 1) / THREADS)), dim3(THREADS), 0, b->stream, 
            y_pooled, x, save_mean, save_rstd, gamma, beta, static_cast<int>(c), static_cast<int>(h), static_cast<int>(w), total);
    }
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_bn_relu_pool_fwd(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t h, int64_t w, const float* gamma,
                                   const float* beta, float* running_mean, float* running_var, double momentum, double eps, float* y_pooled,
                                   float* save_mean, float* save_rstd) {
    return wb_bn_relu_pool_fwd_shifted(b, x, n, c, h, w, gamma, beta, running_mean, running_var, momentum, eps, y_pooled, save_mean, save_rstd,
                                       nullptr, nullptr, nullptr, nullptr);
}

// Backward of BatchNorm2d -> ReLU -> MaxPool2d(2); dx_left / dx_right (both or neither) also receive dx shifted one
// column right / left, zeros shifted in (needs w / 4 in {1, 2, 4, ..., 32} and 16-byte aligned buffers).
// dx == nullptr: only dgamma and dbeta are computed (the caller produces dx itself, see conv1_bwd_fused.cu).
int wb_bn_relu_pool_bwd_shifted(WbBackend* b, const float* x, const float* dy_pooled, int64_t n, int64_t c, int64_t h, int64_t w,
                                const float* gamma, const float* beta, const float* save_mean, const float* save_rstd, float* dx,
                                float* dgamma, float* dbeta, float* dbias_conv, float* dx_left, float* dx_right, const float* y_pooled) {
    WB_REQUIRE(b && x && dy_pooled && dgamma && dbeta, WB_ERR_INVALID, "wb_bn_relu_pool_bwd: null pointer");
    WB_REQUIRE(h % 2 == 0 && w % 2 == 0, WB_ERR_UNSUPPORTED, "wb_bn_relu_pool_bwd: height and width must be even");
    WB_REQUIRE(dx || (!dx_left && !dbias_conv), WB_ERR_INVALID, "wb_bn_relu_pool_bwd: outputs of the dx pass asked for without dx");
    WB_REQUIRE((dx_left == nullptr) == (dx_right == nullptr), WB_ERR_INVALID, "wb_bn_relu_pool_bwd: give both shifted outputs or neither");
    WbProfileScope ps(b, "bn_relu_pool_bwd");
    const bool pairs = w % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dx_left) |
                                        reinterpret_cast<uintptr_t>(dx_right)) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(dy_pooled) & 7) == 0;
    WB_REQUIRE(!dx_left || (pairs && 32 % (w / 4) == 0), WB_ERR_UNSUPPORTED,
               "wb_bn_relu_pool_bwd: shifted outputs need w / 4 in {1, 2, 4, 8, 16, 32} and 16-byte aligned buffers");
    // Paired kernels: a flat grid of one resident wave whose blocks walk (channel, slab) items, about eight per block.
    // Scalar kernels: grid (channels, slabs), one slab per block.
    int splits = stat_splits(b, bn_relu_pool_bwd_pair_kernel<true, false>, static_cast<int>(c), n, h * w);
    int flat_blocks = 0;
    if (pairs) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, bn_relu_pool_bwd_pair_kernel<true, true>, THREADS, 0) != cudaSuccess || per_sm < 1) {
            (void)cudaGetLastError();
            per_sm = 3;
        }
        flat_blocks = per_sm * b->sm_count;
        const int64_t want = (8 * static_cast<int64_t>(flat_blocks) + c - 1) / c;
        int64_t slabs = std::max<int64_t>(splits, std::min<int64_t>(want, n));
        const int64_t per = (n + slabs - 1) / slabs;
        splits = static_cast<int>((n + per - 1) / per);  // no slab is empty
        flat_blocks = static_cast<int>(std::min<int64_t>(flat_blocks, c * splits));
    }
    void* s = nullptr;
    WB_TRY(wb_scratch(b, static_cast<size_t>(c) * splits * 3 * sizeof(double), &s));
    double* part = static_cast<double*>(s);
    double* bias_part = part + static_cast<size_t>(c) * splits * 2;
    dim3 grid(static_cast<unsigned>(c), splits);
    const float inv_count = static_cast<float>(1.0 / static_cast<double>(n * h * w));
    const FastDiv div_pairs(static_cast<uint32_t>(std::max<int64_t>(1, (h / 2) * (w / 4)))), div_owp(static_cast<uint32_t>(std::max<int64_t>(1, w / 4)));
    // y_pooled (the forward's output, when the caller still has it): channels with a usable gamma take their sums from
    // the pooled tensors, a quarter of the bytes; the same kernel sums the other channels (normally none) from x.
    const int64_t pooled = (h / 2) * (w / 2);
    static const bool sums_from_x = [] { const char* e = std::getenv("WETA_B200_BN_SUMS_FROM_X"); return e && e[0] == '1'; }();  // diagnostic switch
    const bool from_pooled = !sums_from_x && pairs && y_pooled && pooled % 4 == 0 && pooled < (int64_t(1) << 30) &&
                             ((reinterpret_cast<uintptr_t>(y_pooled) | reinterpret_cast<uintptr_t>(dy_pooled)) & 15) == 0;
    if (from_pooled) {
        const int64_t warps_needed = static_cast<int64_t>(c) * splits;
        const unsigned grid = static_cast<unsigned>(std::min<int64_t>((warps_needed + THREADS / 32 - 1) / (THREADS / 32), 8LL * b->sm_count));
        wb_launch_pdl(bn_relu_pool_bwd_sums_pooled_kernel, dim3(grid), dim3(THREADS), 0, b->stream, y_pooled, dy_pooled, x, save_mean, save_rstd, gamma, beta, n,
                                                                            static_cast<int>(c), static_cast<int>(h), static_cast<int>(w), part, splits);
    } else if (pairs)
        wb_launch_pdl(bn_relu_pool_bwd_pair_kernel<false, false>, dim3(flat_blocks), dim3(THREADS), 0, b->stream, 
            nullptr, nullptr, nullptr, x, dy_pooled, save_mean, save_rstd, gamma, beta, nullptr, nullptr, n, static_cast<int>(c), static_cast<int>(h),
            static_cast<int>(w), inv_count, part, div_pairs, div_owp, splits, 0);
    else
        wb_launch_pdl(bn_relu_pool_bwd_stats_kernel, dim3(grid), dim3(THREADS), 0, b->stream, x, dy_pooled, save_mean, save_rstd, gamma, beta, n, static_cast<int>(c),
                                                                      static_cast<int>(h), static_cast<int>(w), part);
    WB_LAUNCH_OK(b);
    wb_launch_pdl(bn_bwd_finalize_kernel, dim3(static_cast<unsigned>((c + 3) / 4)), dim3(128), 0, b->stream, part, splits, static_cast<int>(c), dgamma, dbeta);
    WB_LAUNCH_OK(b);
    if (!dx) return WB_OK;
    if (pairs && dx_left)
        wb_launch_pdl(bn_relu_pool_bwd_pair_kernel<true, true>, dim3(flat_blocks), dim3(THREADS), 0, b->stream, 
            dx, dx_left, dx_right, x, dy_pooled, save_mean, save_rstd, gamma, beta, dgamma, dbeta, n, static_cast<int>(c), static_cast<int>(h),
            static_cast<int>(w), inv_count, dbias_conv ? bias_part : nullptr, div_pairs, div_owp, splits, 0);
    else if (pairs)
        wb_launch_pdl(bn_relu_pool_bwd_pair_kernel<true, false>, dim3(flat_blocks), dim3(THREADS), 0, b->stream, 
            dx, nullptr, nullptr, x, dy_pooled, save_mean, save_rstd, gamma, beta, dgamma, dbeta, n, static_cast<int>(c), static_cast<int>(h),
            static_cast<int>(w), inv_count, dbias_conv ? bias_part : nullptr, div_pairs, div_owp, splits, 0);
    else
        wb_launch_pdl(bn_relu_pool_bwd_dx_kernel, dim3(grid), dim3(THREADS), 0, b->stream, dx, x, dy_pooled, save_mean, save_rstd, gamma, beta, dgamma, dbeta, n,
                                                                   static_cast<int>(c), static_cast<int>(h), static_cast<int>(w), inv_count,
                                                                   dbias_conv ? bias_part : nullptr);
    WB_LAUNCH_OK(b);
    if (dbias_conv) {
        wb_launch_pdl(sum_parts_kernel, dim3(static_cast<unsigned>((c + 3) / 4)), dim3(128), 0, b->stream, bias_part, splits, static_cast<int>(c), dbias_conv);
        WB_LAUNCH_OK(b);
    }
    return WB_OK;
}

extern "C" int wb_bn_relu_pool_bwd(WbBackend* b, const float* x, const float* dy_pooled, int64_t n, int64_t c, int64_t h, int64_t w,
                                   const float* gamma, const float* beta, const float* save_mean, const float* save_rstd, float* dx,
                                   float* dgamma, float* dbeta, float* dbias_conv) {
    WB_REQUIRE(dx, WB_ERR_INVALID, "wb_bn_relu_pool_bwd: null pointer");
    return wb_bn_relu_pool_bwd_shifted(b, x, dy_pooled, n, c, h, w, gamma, beta, save_mean, save_rstd, dx, dgamma, dbeta, dbias_conv, nullptr,
                                       nullptr, nullptr);
}

