// Fused extension ops: each replaces a chain of primitive calls the reference issues for one layer.
//   dropout            crates/weta-nn/src/functional.rs:64-74       (random, gt_scalar, mul_scalar, mul)
//   softmax-cross-ent. crates/weta-autograd/src/ops.rs:444-519      (~20 calls and two one-hot uploads)
//   batch norm 2d      crates/weta-nn/src/functional.rs:144-180     (~9 reductions + ~20 element-wise passes)
//   BN+ReLU+maxpool    the conv block of crates/weta/examples/mnist_cnn.rs:16-32 as one pass each way
//   Adam               crates/weta-optim/src/lib.rs:210-239         (13 calls per parameter tensor)
// Compiled with -fmad=false: where an op is a fixed sequence of f32 roundings in the reference
// (dropout mask, Adam), the same sequence is performed here so results are bit-identical.
#include <algorithm>
#include <cmath>

#include "common.h"

namespace {

constexpr int THREADS = 256;

__device__ __forceinline__ uint64_t splitmix64(uint64_t seed, uint64_t i) {
    uint64_t z = seed + (i + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// rand_f32 element i for Uniform{0,1}: (f32)((z >> 11) * 2^-53), see random.cu.
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t i) {
    return __ull2float_rn(splitmix64(seed, i) >> 11) * 1.1102230246251565e-16f;
}

// ---- dropout ------------------------------------------------------------------------------------
// mask = ((u > f32(p)) ? 1 : 0) * f32(1/(1-p)) + 0;  y = x * mask.  With relu_src != null the
// incoming value is additionally multiplied by step(relu_src) (ReLU backward folded in).
__global__ void __launch_bounds__(THREADS) dropout_kernel(float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ relu_src,
                                                           int64_t n, float p, float scale, uint64_t seed) {
    int64_t i = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) * 4;
    if (i >= n) return;
    if (i + 4 <= n) {
        float4 v = *reinterpret_cast<const float4*>(x + i);
        float in[4] = {v.x, v.y, v.z, v.w}, out[4];
        float rs[4] = {1.f, 1.f, 1.f, 1.f};
        if (relu_src) {
            float4 r = *reinterpret_cast<const float4*>(relu_src + i);
            rs[0] = r.x; rs[1] = r.y; rs[2] = r.z; rs[3] = r.w;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float mask = p > 0.f ? (uniform01(seed, static_cast<uint64_t>(i + k)) > p ? 1.f : 0.f) * scale + 0.f : 1.f;
            float g = in[k] * mask;
            out[k] = relu_src ? g * (rs[k] > 0.f ? 1.f : 0.f) : g;
        }
        *reinterpret_cast<float4*>(y + i) = make_float4(out[0], out[1], out[2], out[3]);
    } else {
        for (int64_t j = i; j < n; ++j) {
            float mask = p > 0.f ? (uniform01(seed, static_cast<uint64_t>(j)) > p ? 1.f : 0.f) * scale + 0.f : 1.f;
            float g = x[j] * mask;
            y[j] = relu_src ? g * (relu_src[j] > 0.f ? 1.f : 0.f) : g;
        }
    }
}

__global__ void __launch_bounds__(THREADS) dropout_mask_kernel(float* __restrict__ m, int64_t n, float p, float scale, uint64_t seed) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (i < n) m[i] = (uniform01(seed, static_cast<uint64_t>(i)) > p ? 1.f : 0.f) * scale + 0.f;
}

// ---- softmax cross-entropy ----------------------------------------------------------------------
// One warp per row.  loss_row = -(z[y] - max - log(sum exp(z - max))); p = exp(z - lse);
// dz = (p - onehot) * gscale, with gscale = upstream_grad / N for the mean reduction.
__global__ void __launch_bounds__(THREADS) softmax_ce_kernel(const float* __restrict__ z, const int64_t* __restrict__ labels, int64_t rows,
                                                              int cols, float* __restrict__ probs, float* __restrict__ dz,
                                                              float* __restrict__ row_loss, float gscale) {
    int64_t row = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* zr = z + row * cols;
    float mx = -INFINITY;
    for (int c = lane; c < cols; c += 32) mx = fmaxf(mx, zr[c]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float s = 0.f;
    for (int c = lane; c < cols; c += 32) s += expf(zr[c] - mx);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    float lse = logf(s) + mx;
    int64_t y = labels[row];
    for (int c = lane; c < cols; c += 32) {
        float p = expf(zr[c] - lse);
        if (probs) probs[row * cols + c] = p;
        if (dz) dz[row * cols + c] = (p - (c == y ? 1.f : 0.f)) * gscale;
    }
    if (lane == 0 && row_loss) row_loss[row] = (y >= 0 && y < cols) ? -(zr[y] - lse) : 0.f;
}

// mean of row_loss in a fixed order (one block; rows is a batch size).
__global__ void __launch_bounds__(THREADS) mean_kernel(const float* __restrict__ v, int64_t n, float* __restrict__ out) {
    __shared__ double part[THREADS];
    double acc = 0.0;
    for (int64_t i = threadIdx.x; i < n; i += THREADS) acc += v[i];
    part[threadIdx.x] = acc;
    __syncthreads();
    for (int s = THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) part[threadIdx.x] += part[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) *out = static_cast<float>(part[0] / static_cast<double>(n));
}

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
    if ((hw & 3) == 0) {
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
        float unbiased = v * static_cast<float>(static_cast<double>(count) / static_cast<double>((count > 2 ? count : 2) - 1)) + 0.f;
        running_mean[c] = (running_mean[c] * one_minus_momentum + 0.f) + (m * momentum + 0.f);
        running_var[c] = (running_var[c] * one_minus_momentum + 0.f) + (unbiased * momentum + 0.f);
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
    for (int64_t i = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) * 4; i < hw; i += static_cast<int64_t>(gridDim.x) * THREADS * 4) {
        if (i + 4 <= hw && (hw & 3) == 0) {
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
        const uint32_t uhw = static_cast<uint32_t>(hw), items = static_cast<uint32_t>(n1 - n0) * uhw;
        const int64_t stride = static_cast<int64_t>(c_total) * hw;
        const float* xslab = x + (n0 * c_total + c) * hw;
        const float* gslab = dy + (n0 * c_total + c) * hw;
        float a1 = 0.f, a2 = 0.f;
        int flushed = 0;
        for (uint32_t j = threadIdx.x; j < items; j += THREADS) {
            const uint32_t n = j / uhw, i = j - n * uhw;
            float g = gslab[n * stride + i];
            a1 += g;
            a2 += g * ((xslab[n * stride + i] - m) * r);
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

// dbeta = sum dy, dgamma = sum dy*xhat (gradients of the affine parameters).
__global__ void bn_bwd_finalize_kernel(const double* __restrict__ part, int splits, int c_total, float* __restrict__ dgamma,
                                       float* __restrict__ dbeta) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= c_total) return;
    double s1 = 0.0, s2 = 0.0;
    for (int s = 0; s < splits; ++s) {
        s1 += part[(static_cast<int64_t>(c) * splits + s) * 2];
        s2 += part[(static_cast<int64_t>(c) * splits + s) * 2 + 1];
    }
    dbeta[c] = static_cast<float>(s1);
    dgamma[c] = static_cast<float>(s2);
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
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x; i < hw; i += static_cast<int64_t>(gridDim.x) * THREADS) {
        float xh = (xs[i] - m) * r;
        dst[i] = gr * (gs[i] - k1 - xh * k2);
    }
}

// ---- conv block tail: BN -> ReLU -> 2x2 max pool, one pass each way ------------------------------
// Forward: one thread per pooled element.
__global__ void __launch_bounds__(THREADS) bn_relu_pool_fwd_kernel(float* __restrict__ yp, const float* __restrict__ x,
                                                                    const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                    const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                    int c_total, int h, int w, int64_t total) {
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
        float tv = ((v[k] - m) * r) * g + b;
        tv = tv > 0.f ? tv : 0.f;
        best = (best >= tv || best != best) ? best : tv;  // acc.max(v), crates/weta-core/src/dtype.rs:136-142
    }
    yp[i] = best;
}

// Backward recompute for one pooled element: the gradient each of the 4 window positions receives
// through max-pool (ties share equally, crates/weta-autograd/src/ops.rs:305-314) and ReLU
// (g * step(pre-activation), ops.rs:85), plus xhat at those positions.
__device__ __forceinline__ void pool_window_grads(const float v[4], float m, float r, float g, float b, float dyp, float gout[4], float xh[4]) {
    float act[4];
    float best = -INFINITY;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        xh[k] = (v[k] - m) * r;
        float tv = xh[k] * g + b;
        act[k] = tv > 0.f ? tv : 0.f;
        best = (best >= act[k] || best != best) ? best : act[k];
    }
    float cnt = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) cnt += (act[k] == best) ? 1.f : 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float share = ((act[k] == best) ? 1.f : 0.f) / cnt * dyp;
        gout[k] = share * (act[k] > 0.f ? 1.f : 0.f);  // step of the ReLU input == step of its output
    }
}

// grid (C, S) like bn_stats: sums of the full-resolution gradient and of gradient * xhat.
__global__ void __launch_bounds__(THREADS) bn_relu_pool_bwd_stats_kernel(const float* __restrict__ x, const float* __restrict__ dyp,
                                                                          const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                          const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                          int64_t n_img, int c_total, int h, int w, double* __restrict__ part) {
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

// Width-multiple-of-4 variants: one thread handles two neighbouring pooled elements, i.e. a 2x4 patch
// of x, with 128-bit loads and stores; same arithmetic as the kernels above.
template <bool WRITE_DX>
__global__ void __launch_bounds__(THREADS) bn_relu_pool_bwd_pair_kernel(float* __restrict__ dx, const float* __restrict__ x,
                                                                         const float* __restrict__ dyp, const float* __restrict__ mean,
                                                                         const float* __restrict__ rstd, const float* __restrict__ gamma,
                                                                         const float* __restrict__ beta, const float* __restrict__ dgamma,
                                                                         const float* __restrict__ dbeta, int64_t n_img, int c_total, int h,
                                                                         int w, float inv_count, double* __restrict__ part) {
    const int c = blockIdx.x;
    const float m = mean[c], r = rstd[c], g = gamma[c], b = beta[c];
    float k1 = 0.f, k2 = 0.f, gr = 0.f;
    if (WRITE_DX) { k1 = dbeta[c] * inv_count; k2 = dgamma[c] * inv_count; gr = g * r; }
    const int ow = w >> 1, oh = h >> 1, pooled = ow * oh;
    const uint32_t owp = static_cast<uint32_t>(ow >> 1), pairs = static_cast<uint32_t>(oh) * owp;
    const int64_t per = (n_img + gridDim.y - 1) / gridDim.y;
    const int64_t n0 = min(n_img, static_cast<int64_t>(blockIdx.y) * per), n1 = min(n_img, n0 + per);
    const uint32_t items = static_cast<uint32_t>(n1 - n0) * pairs;
    const int64_t xstride = static_cast<int64_t>(c_total) * h * w, gstride = static_cast<int64_t>(c_total) * pooled;
    const float* xslab = x + (n0 * c_total + c) * h * w;
    const float* gslab = dyp + (n0 * c_total + c) * pooled;
    float* dslab = WRITE_DX ? dx + (n0 * c_total + c) * h * w : nullptr;
    double s1 = 0.0, s2 = 0.0;
    float a1 = 0.f, a2 = 0.f;
    int flushed = 0;
#pragma unroll 2
    for (uint32_t j = threadIdx.x; j < items; j += THREADS) {
        const uint32_t n = j / pairs, i = j - n * pairs;
        const uint32_t oy = i / owp, oxp = i - oy * owp;
        const int64_t o = n * xstride + static_cast<int64_t>(2 * oy) * w + 4 * oxp;
        const float4 r0 = *reinterpret_cast<const float4*>(xslab + o);
        const float4 r1 = *reinterpret_cast<const float4*>(xslab + o + w);
        const float2 gy = *reinterpret_cast<const float2*>(gslab + n * gstride + oy * ow + 2 * oxp);
        const float va[4] = {r0.x, r0.y, r1.x, r1.y}, vb[4] = {r0.z, r0.w, r1.z, r1.w};
        float ga[4], gb[4], xa[4], xb[4];
        pool_window_grads(va, m, r, g, b, gy.x, ga, xa);
        pool_window_grads(vb, m, r, g, b, gy.y, gb, xb);
        if (WRITE_DX) {
            float da[4], db[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                da[k] = gr * (ga[k] - k1 - xa[k] * k2);
                db[k] = gr * (gb[k] - k1 - xb[k] * k2);
                a1 += da[k] + db[k];
            }
            *reinterpret_cast<float4*>(dslab + o) = make_float4(da[0], da[1], db[0], db[1]);
            *reinterpret_cast<float4*>(dslab + o + w) = make_float4(da[2], da[3], db[2], db[3]);
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                a1 += ga[k] + gb[k];
                a2 += ga[k] * xa[k] + gb[k] * xb[k];
            }
        }
        if (++flushed == 32) { s1 += a1; s2 += a2; a1 = a2 = 0.f; flushed = 0; }
    }
    s1 += a1;
    s2 += a2;
    __shared__ double r1s[THREADS], r2s[THREADS];
    r1s[threadIdx.x] = s1;
    r2s[threadIdx.x] = s2;
    __syncthreads();
    for (int s = THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) { r1s[threadIdx.x] += r1s[threadIdx.x + s]; r2s[threadIdx.x] += r2s[threadIdx.x + s]; }
        __syncthreads();
    }
    if (threadIdx.x == 0 && part) {
        if (WRITE_DX) {
            part[static_cast<int64_t>(c) * gridDim.y + blockIdx.y] = r1s[0];  // sum of dx: the conv bias gradient
        } else {
            part[(static_cast<int64_t>(c) * gridDim.y + blockIdx.y) * 2] = r1s[0];
            part[(static_cast<int64_t>(c) * gridDim.y + blockIdx.y) * 2 + 1] = r2s[0];
        }
    }
}

__global__ void sum_parts_kernel(const double* __restrict__ part, int splits, int c_total, float* __restrict__ out) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= c_total) return;
    double s = 0.0;
    for (int k = 0; k < splits; ++k) s += part[static_cast<int64_t>(c) * splits + k];
    out[c] = static_cast<float>(s);
}

// ---- Adam ---------------------------------------------------------------------------------------
// crates/weta-optim/src/lib.rs:210-239 as one pass; every f32 rounding of the primitive chain is kept
// (each `mul_scalar` is x*s + 0, `add_scalar(eps)` is x*1 + eps).
struct AdamK {
    float b1, omb1, b2, omb2, inv_sqrt_bc2, eps, step_size, wd, decay_mul, gscale;
    int first, decoupled, has_wd, scale_grad;
};

__global__ void __launch_bounds__(THREADS) adam_kernel(float* __restrict__ theta, const float* __restrict__ grad, float* __restrict__ m,
                                                        float* __restrict__ v, int64_t n, AdamK k) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (i >= n) return;
    float g = grad[i], th = theta[i];
    if (k.scale_grad) g = g * k.gscale;
    if (k.has_wd) {
        if (k.decoupled) th = th * k.decay_mul + 0.f;
        else g = g + (th * k.wd + 0.f);
    }
    float gm = g * k.omb1 + 0.f;
    float gv = (g * g) * k.omb2 + 0.f;
    float mn = k.first ? gm : (m[i] * k.b1 + 0.f) + gm;
    float vn = k.first ? gv : (v[i] * k.b2 + 0.f) + gv;
    float den = (sqrtf(vn) * k.inv_sqrt_bc2 + 0.f) * 1.f + k.eps;
    th = th - ((mn / den) * k.step_size + 0.f);
    theta[i] = th;
    m[i] = mn;
    v[i] = vn;
}

double powi(double a, int n) {  // f64::powi (compiler-rt __powidf2)
    double r = 1.0;
    int b = n;
    while (true) {
        if (b & 1) r *= a;
        b /= 2;
        if (b == 0) break;
        a *= a;
    }
    return r;
}

// Number of image slabs per channel for the per-channel reductions: about 8 blocks per SM in total,
// and few enough images per slab that the kernels' 32-bit item counters cannot overflow.
int stat_splits(WbBackend* be, int c, int64_t n_img, int64_t items_per_image) {
    int64_t want = (8LL * be->sm_count + c - 1) / c;
    int64_t need = (n_img * items_per_image + (int64_t(1) << 30) - 1) / (int64_t(1) << 30);
    int64_t splits = std::max<int64_t>(1, std::min<int64_t>(std::max(want, need), n_img));
    int64_t per = (n_img + splits - 1) / splits;
    return static_cast<int>((n_img + per - 1) / per);  // no slab is empty
}

}  // namespace

// ---- entry points -------------------------------------------------------------------------------
extern "C" int wb_dropout_fwd(WbBackend* b, const float* x, float* y, int64_t n, double p, uint64_t seed) {
    WB_REQUIRE(b && x && y, WB_ERR_INVALID, "wb_dropout_fwd: null pointer");
    WB_REQUIRE(p >= 0.0 && p < 1.0, WB_ERR_INVALID, "dropout probability has to be in [0, 1), got %g", p);
    if (n == 0) return WB_OK;
    WbProfileScope ps(b, "dropout");
    int64_t threads = (n + 3) / 4;
    bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    WB_REQUIRE(aligned, WB_ERR_INVALID, "wb_dropout_fwd: buffers must be 16-byte aligned");
    dropout_kernel<<<static_cast<unsigned>((threads + THREADS - 1) / THREADS), THREADS, 0, b->stream>>>(
        y, x, nullptr, n, static_cast<float>(p), static_cast<float>(1.0 / (1.0 - p)), seed);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_dropout_relu_bwd(WbBackend* b, const float* dy, const float* relu_out, float* dx, int64_t n, double p, uint64_t seed) {
    WB_REQUIRE(b && dy && dx, WB_ERR_INVALID, "wb_dropout_relu_bwd: null pointer");
    if (n == 0) return WB_OK;
    WbProfileScope ps(b, "dropout_bwd");
    int64_t threads = (n + 3) / 4;
    dropout_kernel<<<static_cast<unsigned>((threads + THREADS - 1) / THREADS), THREADS, 0, b->stream>>>(
        dx, dy, relu_out, n, static_cast<float>(p), static_cast<float>(1.0 / (1.0 - p)), seed);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_dropout_mask(WbBackend* b, float* mask, int64_t n, double p, uint64_t seed) {
    WB_REQUIRE(b && mask, WB_ERR_INVALID, "wb_dropout_mask: null pointer");
    if (n == 0) return WB_OK;
    WbProfileScope ps(b, "dropout_mask");
    dropout_mask_kernel<<<static_cast<unsigned>((n + THREADS - 1) / THREADS), THREADS, 0, b->stream>>>(
        mask, n, static_cast<float>(p), static_cast<float>(1.0 / (1.0 - p)), seed);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_softmax_ce(WbBackend* b, const float* logits, const int64_t* labels, int64_t rows, int64_t cols, float* probs,
                             float* dlogits, float* row_loss, float* mean_loss, double upstream) {
    WB_REQUIRE(b && logits && labels, WB_ERR_INVALID, "wb_softmax_ce: null pointer");
    WB_REQUIRE(cols > 0 && cols < (int64_t(1) << 31), WB_ERR_INVALID, "wb_softmax_ce: bad class count");
    if (rows == 0) return WB_OK;
    WbProfileScope ps(b, "softmax_ce");
    float* rl = row_loss;
    if (mean_loss && !rl) {
        void* s = nullptr;
        WB_TRY(wb_scratch(b, static_cast<size_t>(rows) * sizeof(float), &s));
        rl = static_cast<float*>(s);
    }
    int64_t threads = rows * 32;
    softmax_ce_kernel<<<static_cast<unsigned>((threads + THREADS - 1) / THREADS), THREADS, 0, b->stream>>>(
        logits, labels, rows, static_cast<int>(cols), probs, dlogits, rl, static_cast<float>(upstream * (1.0 / static_cast<double>(rows))));
    WB_LAUNCH_OK(b);
    if (mean_loss) {
        mean_kernel<<<1, THREADS, 0, b->stream>>>(rl, rows, mean_loss);
        WB_LAUNCH_OK(b);
    }
    return WB_OK;
}

extern "C" int wb_bn2d_stats(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t hw, double eps, double momentum, float* mean,
                             float* rstd, float* running_mean, float* running_var) {
    WB_REQUIRE(b && x && mean && rstd, WB_ERR_INVALID, "wb_bn2d_stats: null pointer");
    WB_REQUIRE(n > 0 && c > 0 && hw > 0, WB_ERR_INVALID, "wb_bn2d_stats: empty input");
    WbProfileScope ps(b, "bn2d_stats");
    int splits = stat_splits(b, static_cast<int>(c), n, hw);
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
    int splits = stat_splits(b, static_cast<int>(c), n, hw);
    void* s = nullptr;
    WB_TRY(wb_scratch(b, static_cast<size_t>(c) * splits * 2 * sizeof(double), &s));
    bn_bwd_stats_kernel<<<dim3(static_cast<unsigned>(c), splits), THREADS, 0, b->stream>>>(x, dy, save_mean, save_rstd, n, static_cast<int>(c), hw,
                                                                                          static_cast<double*>(s));
    WB_LAUNCH_OK(b);
    bn_bwd_finalize_kernel<<<static_cast<unsigned>((c + 127) / 128), 128, 0, b->stream>>>(static_cast<double*>(s), splits, static_cast<int>(c), dgamma, dbeta);
    WB_LAUNCH_OK(b);
    unsigned gx = static_cast<unsigned>(std::max<int64_t>(1, std::min<int64_t>((hw + THREADS - 1) / THREADS, 64)));
    for (int64_t p0 = 0; p0 < n * c; p0 += 65535 / c * c) {
        int64_t cnt = std::min<int64_t>(65535 / c * c, n * c - p0);
        bn_bwd_dx_kernel<<<dim3(gx, static_cast<unsigned>(cnt)), THREADS, 0, b->stream>>>(dx + p0 * hw, x + p0 * hw, dy + p0 * hw, save_mean, save_rstd,
                                                                                          gamma, dgamma, dbeta, static_cast<int>(c), hw,
                                                                                          static_cast<float>(1.0 / static_cast<double>(n * hw)));
        WB_LAUNCH_OK(b);
    }
    return WB_OK;
}

extern "C" int wb_bn_relu_pool_fwd(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t h, int64_t w, const float* gamma,
                                   const float* beta, float* running_mean, float* running_var, double momentum, double eps, float* y_pooled,
                                   float* save_mean, float* save_rstd) {
    WB_REQUIRE(b && x && gamma && beta && y_pooled, WB_ERR_INVALID, "wb_bn_relu_pool_fwd: null pointer");
    WB_REQUIRE(h % 2 == 0 && w % 2 == 0, WB_ERR_UNSUPPORTED, "wb_bn_relu_pool_fwd: height and width must be even");
    WB_TRY(wb_bn2d_stats(b, x, n, c, h * w, eps, momentum, save_mean, save_rstd, running_mean, running_var));
    WbProfileScope ps(b, "bn_relu_pool_fwd");
    int64_t total = n * c * (h / 2) * (w / 2);
    bn_relu_pool_fwd_kernel<<<static_cast<unsigned>((total + THREADS - 1) / THREADS), THREADS, 0, b->stream>>>(
        y_pooled, x, save_mean, save_rstd, gamma, beta, static_cast<int>(c), static_cast<int>(h), static_cast<int>(w), total);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_bn_relu_pool_bwd(WbBackend* b, const float* x, const float* dy_pooled, int64_t n, int64_t c, int64_t h, int64_t w,
                                   const float* gamma, const float* beta, const float* save_mean, const float* save_rstd, float* dx,
                                   float* dgamma, float* dbeta, float* dbias_conv) {
    WB_REQUIRE(b && x && dy_pooled && dx && dgamma && dbeta, WB_ERR_INVALID, "wb_bn_relu_pool_bwd: null pointer");
    WB_REQUIRE(h % 2 == 0 && w % 2 == 0, WB_ERR_UNSUPPORTED, "wb_bn_relu_pool_bwd: height and width must be even");
    WbProfileScope ps(b, "bn_relu_pool_bwd");
    int splits = stat_splits(b, static_cast<int>(c), n, h * w);
    void* s = nullptr;
    WB_TRY(wb_scratch(b, static_cast<size_t>(c) * splits * 3 * sizeof(double), &s));
    double* part = static_cast<double*>(s);
    double* bias_part = part + static_cast<size_t>(c) * splits * 2;
    dim3 grid(static_cast<unsigned>(c), splits);
    const bool pairs = w % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx)) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(dy_pooled) & 7) == 0;
    const float inv_count = static_cast<float>(1.0 / static_cast<double>(n * h * w));
    if (pairs)
        bn_relu_pool_bwd_pair_kernel<false><<<grid, THREADS, 0, b->stream>>>(nullptr, x, dy_pooled, save_mean, save_rstd, gamma, beta, nullptr,
                                                                            nullptr, n, static_cast<int>(c), static_cast<int>(h),
                                                                            static_cast<int>(w), inv_count, part);
    else
        bn_relu_pool_bwd_stats_kernel<<<grid, THREADS, 0, b->stream>>>(x, dy_pooled, save_mean, save_rstd, gamma, beta, n, static_cast<int>(c),
                                                                      static_cast<int>(h), static_cast<int>(w), part);
    WB_LAUNCH_OK(b);
    bn_bwd_finalize_kernel<<<static_cast<unsigned>((c + 127) / 128), 128, 0, b->stream>>>(part, splits, static_cast<int>(c), dgamma, dbeta);
    WB_LAUNCH_OK(b);
    if (pairs)
        bn_relu_pool_bwd_pair_kernel<true><<<grid, THREADS, 0, b->stream>>>(dx, x, dy_pooled, save_mean, save_rstd, gamma, beta, dgamma, dbeta, n,
                                                                           static_cast<int>(c), static_cast<int>(h), static_cast<int>(w),
                                                                           inv_count, dbias_conv ? bias_part : nullptr);
    else
        bn_relu_pool_bwd_dx_kernel<<<grid, THREADS, 0, b->stream>>>(dx, x, dy_pooled, save_mean, save_rstd, gamma, beta, dgamma, dbeta, n,
                                                                   static_cast<int>(c), static_cast<int>(h), static_cast<int>(w), inv_count,
                                                                   dbias_conv ? bias_part : nullptr);
    WB_LAUNCH_OK(b);
    if (dbias_conv) {
        sum_parts_kernel<<<static_cast<unsigned>((c + 127) / 128), 128, 0, b->stream>>>(bias_part, splits, static_cast<int>(c), dbias_conv);
        WB_LAUNCH_OK(b);
    }
    return WB_OK;
}

extern "C" int wb_adam_step(WbBackend* b, float* theta, const float* grad, float* m, float* v, int64_t n, int64_t t, double lr,
                            double beta1, double beta2, double eps, double weight_decay, int decoupled, double grad_scale) {
    WB_REQUIRE(b && theta && grad && m && v, WB_ERR_INVALID, "wb_adam_step: null pointer");
    WB_REQUIRE(t >= 1, WB_ERR_INVALID, "wb_adam_step: step counts from 1");
    if (n == 0) return WB_OK;
    WbProfileScope ps(b, "adam_step");
    double bc1 = 1.0 - powi(beta1, static_cast<int>(t)), bc2 = 1.0 - powi(beta2, static_cast<int>(t));
    AdamK k;
    k.b1 = static_cast<float>(beta1);
    k.omb1 = static_cast<float>(1.0 - beta1);
    k.b2 = static_cast<float>(beta2);
    k.omb2 = static_cast<float>(1.0 - beta2);
    k.inv_sqrt_bc2 = static_cast<float>(1.0 / std::sqrt(bc2));
    k.eps = static_cast<float>(eps);
    k.step_size = static_cast<float>(lr / bc1);
    k.wd = static_cast<float>(weight_decay);
    k.decay_mul = static_cast<float>(1.0 - lr * weight_decay);
    k.gscale = static_cast<float>(grad_scale);
    k.first = t == 1;
    k.decoupled = decoupled;
    k.has_wd = weight_decay != 0.0;
    k.scale_grad = grad_scale != 1.0;
    adam_kernel<<<static_cast<unsigned>((n + THREADS - 1) / THREADS), THREADS, 0, b->stream>>>(theta, grad, m, v, n, k);
    WB_LAUNCH_OK(b);
    return WB_OK;
}
