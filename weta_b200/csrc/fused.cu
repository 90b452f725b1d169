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

#include "adam.cuh"
#include "common.h"

namespace {

constexpr int THREADS = 256;

__device__ __forceinline__ uint64_t splitmix64(uint64_t seed, uint64_t i) {
    uint64_t z = seed + (i + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// The 53-bit integer k behind rand_f32 element i: u = (f32)(k * 2^-53) (crates/weta-core/src/ops.rs:172-174).
// `u > f32(p)` is monotone in k, so the host turns the float comparison into `k >= kmin` once
// (dropout_threshold below) and the kernels never convert k to floating point: same mask, bit for bit.
__device__ __forceinline__ uint64_t mix_tail(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return (z ^ (z >> 31)) >> 11;
}

constexpr uint64_t GOLDEN = 0x9E3779B97F4A7C15ull;

// ---- dropout ------------------------------------------------------------------------------------
// mask = ((u > f32(p)) ? 1 : 0) * f32(1/(1-p)) + 0 = (k >= kmin) ? scale : 0;  y = x * mask.  With
// relu_src != null the incoming value is additionally multiplied by step(relu_src) (ReLU backward folded in).
__global__ void __launch_bounds__(THREADS) dropout_kernel(float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ relu_src,
                                                           int64_t n, uint64_t kmin, float scale, uint64_t seed, int vec) {
    wb_pdl_enter();
    int64_t i = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) * 4;
    if (i >= n) return;
    uint64_t z = seed + (static_cast<uint64_t>(i) + 1) * GOLDEN;
    if (vec && i + 4 <= n) {  // vec: every buffer is 16-byte aligned (checked by the host)
        float4 v = *reinterpret_cast<const float4*>(x + i);
        float in[4] = {v.x, v.y, v.z, v.w}, out[4];
        float rs[4] = {1.f, 1.f, 1.f, 1.f};
        if (relu_src) {
            float4 r = *reinterpret_cast<const float4*>(relu_src + i);
            rs[0] = r.x; rs[1] = r.y; rs[2] = r.z; rs[3] = r.w;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float mask = mix_tail(z) >= kmin ? scale : 0.f;
            z += GOLDEN;
            float g = in[k] * mask;
            out[k] = relu_src ? g * (rs[k] > 0.f ? 1.f : 0.f) : g;
        }
        *reinterpret_cast<float4*>(y + i) = make_float4(out[0], out[1], out[2], out[3]);
    } else {
        for (int64_t j = i; j < n && j < i + 4; ++j) {
            float mask = mix_tail(z) >= kmin ? scale : 0.f;
            z += GOLDEN;
            float g = x[j] * mask;
            y[j] = relu_src ? g * (relu_src[j] > 0.f ? 1.f : 0.f) : g;
        }
    }
}

__global__ void __launch_bounds__(THREADS) dropout_mask_kernel(float* __restrict__ m, int64_t n, uint64_t kmin, float scale, uint64_t seed) {
    int64_t i = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) * 4;
    if (i >= n) return;
    uint64_t z = seed + (static_cast<uint64_t>(i) + 1) * GOLDEN;
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        v[k] = mix_tail(z) >= kmin ? scale : 0.f;
        z += GOLDEN;
    }
    if (i + 4 <= n && (reinterpret_cast<uintptr_t>(m) & 15) == 0) {
        *reinterpret_cast<float4*>(m + i) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        for (int k = 0; k < 4 && i + k < n; ++k) m[i + k] = v[k];
    }
}

// ---- softmax cross-entropy ----------------------------------------------------------------------
// One warp per row.  loss_row = -(z[y] - max - log(sum exp(z - max))); p = exp(z - lse) (the 128-bit kernels take
// p = exp(z - max) / sum, see softmax_ce_reg4_row); dz = (p - onehot) * gscale, with gscale = upstream_grad / N for
// the mean reduction.
__device__ __forceinline__ void softmax_ce_rows(const float* __restrict__ z, const int64_t* __restrict__ labels, int64_t rows,
                                                              int cols, float* __restrict__ probs, float* __restrict__ dz, int dz_pitch,
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
        if (dz) dz[row * dz_pitch + c] = (p - (c == y ? 1.f : 0.f)) * gscale;
    }
    if (dz) for (int c = cols + lane; c < dz_pitch; c += 32) dz[row * dz_pitch + c] = 0.f;  // padding columns of a pitched gradient
    if (lane == 0 && row_loss) row_loss[row] = (y >= 0 && y < cols) ? -(zr[y] - lse) : 0.f;
}

// Same, for rows of at most 32*PER_LANE classes: the row lives in registers, so the logits are read once.
template <int PER_LANE>
__device__ __forceinline__ void softmax_ce_reg_rows(const float* __restrict__ z, const int64_t* __restrict__ labels, int64_t rows,
                                                                  int cols, float* __restrict__ probs, float* __restrict__ dz, int dz_pitch,
                                                                  float* __restrict__ row_loss, float gscale) {
    int64_t row = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* zr = z + row * cols;
    float v[PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
        int c = lane + 32 * k;
        v[k] = c < cols ? zr[c] : -INFINITY;
        mx = fmaxf(mx, v[k]);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k)
        if (lane + 32 * k < cols) s += expf(v[k] - mx);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    const float lse = logf(s) + mx;
    const int64_t y = labels[row];
#pragma unroll
    for (int k = 0; k < PER_LANE; ++k) {
        int c = lane + 32 * k;
        if (c < cols) {
            float p = expf(v[k] - lse);
            if (probs) probs[row * cols + c] = p;
            if (dz) dz[row * dz_pitch + c] = (p - (c == y ? 1.f : 0.f)) * gscale;
            if (row_loss && c == y) row_loss[row] = -(v[k] - lse);
        }
    }
    if (row_loss && lane == 0 && (y < 0 || y >= cols)) row_loss[row] = 0.f;
    if (dz) for (int c = cols + lane; c < dz_pitch; c += 32) dz[row * dz_pitch + c] = 0.f;
}

// The same with 128-bit accesses: cols a multiple of 4 (so is dz_pitch), rows 16-byte aligned; lane l holds the
// float4 groups l, l + 32, ... of its row (Q of them).
template <int Q>
__device__ __forceinline__ void softmax_ce_reg4_load(const float* __restrict__ z, int64_t row, int cols, int lane, float4 (&v)[Q]) {
    const float4* zr = reinterpret_cast<const float4*>(z + row * cols);
    const int groups = cols >> 2;
#pragma unroll
    for (int k = 0; k < Q; ++k) {
        const int q = lane + 32 * k;
        v[k] = q < groups ? zr[q] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
}

// One row from its logits in registers (label y).  The exponentials taken for the sum are kept and
// p = exp(z - max) * (1 / sum): one exponential per element instead of the two of p = exp(z - lse), which made this
// kernel issue-bound (20.6 us on [8192, 1000]; 16.8 us this way; fetching the next row ahead, through registers or
// cp.async, changed neither).  The two forms differ by a few units in the last place.
template <int Q>
__device__ __forceinline__ void softmax_ce_reg4_row(float4 (&v)[Q], int64_t row, int64_t y, int lane, int cols, float* __restrict__ probs,
                                                    float* __restrict__ dz, int dz_pitch, float* __restrict__ row_loss, float gscale) {
    const int groups = cols >> 2;
    const int yq = (y >= 0 && y < cols) ? static_cast<int>(y >> 2) : -1, yj = static_cast<int>(y & 3);
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < Q; ++k) mx = fmaxf(fmaxf(mx, fmaxf(v[k].x, v[k].y)), fmaxf(v[k].z, v[k].w));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    float s = 0.f, zy = 0.f;
#pragma unroll
    for (int k = 0; k < Q; ++k) {
        const int q = lane + 32 * k;
        if (q < groups) {
            if (q == yq) zy = yj == 0 ? v[k].x : (yj == 1 ? v[k].y : (yj == 2 ? v[k].z : v[k].w));
            const float4 e = make_float4(expf(v[k].x - mx), expf(v[k].y - mx), expf(v[k].z - mx), expf(v[k].w - mx));
            s += (e.x + e.y) + (e.z + e.w);
            v[k] = e;
        }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
    const float lse = logf(s) + mx, inv = 1.f / s;
#pragma unroll
    for (int k = 0; k < Q; ++k) {
        const int q = lane + 32 * k;
        if (q < groups) {
            const float4 p = make_float4(v[k].x * inv, v[k].y * inv, v[k].z * inv, v[k].w * inv);
            if (probs) reinterpret_cast<float4*>(probs + row * cols)[q] = p;
            if (dz) {
                float4 d4 = make_float4(p.x * gscale, p.y * gscale, p.z * gscale, p.w * gscale);  // (p - 0) * gscale
                if (q == yq) {
                    if (yj == 0) d4.x = (p.x - 1.f) * gscale;
                    else if (yj == 1) d4.y = (p.y - 1.f) * gscale;
                    else if (yj == 2) d4.z = (p.z - 1.f) * gscale;
                    else d4.w = (p.w - 1.f) * gscale;
                }
                reinterpret_cast<float4*>(dz + row * dz_pitch)[q] = d4;
            }
            if (row_loss && q == yq) row_loss[row] = -(zy - lse);
        }
    }
    if (row_loss && lane == 0 && yq < 0) row_loss[row] = 0.f;
    if (dz) for (int c = cols + lane; c < dz_pitch; c += 32) dz[row * dz_pitch + c] = 0.f;
}

template <int Q>
__device__ __forceinline__ void softmax_ce_reg4_rows(const float* __restrict__ z, const int64_t* __restrict__ labels, int64_t rows,
                                                                   int cols, float* __restrict__ probs, float* __restrict__ dz, int dz_pitch,
                                                                   float* __restrict__ row_loss, float gscale) {
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    float4 v[Q];
    softmax_ce_reg4_load<Q>(z, row, cols, lane, v);
    softmax_ce_reg4_row<Q>(v, row, labels[row], lane, cols, probs, dz, dz_pitch, row_loss, gscale);
}

// The mean of row_loss in a fixed order, by the last block of the launch to finish (one launch instead of two; every
// block's row losses are fenced before its arrival is counted).  `counter` is zero before and after.
__device__ __forceinline__ void mean_by_last_block(const float* __restrict__ v, int64_t n, float* __restrict__ out, unsigned int* __restrict__ counter) {
    __shared__ double part[THREADS];
    __shared__ unsigned int last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(counter, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    // This block runs alone at the end of the launch: sixteen row losses per thread are in flight at a time.
    double acc = 0.0;
    int64_t done = 0;
    if ((reinterpret_cast<uintptr_t>(v) & 15) == 0) {
        const float4* v4 = reinterpret_cast<const float4*>(v);
        const int64_t n4 = n >> 2;
        for (int64_t i0 = threadIdx.x; i0 < n4; i0 += 4 * THREADS) {
            float4 t[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int64_t i = i0 + u * THREADS;
                t[u] = i < n4 ? __ldcg(v4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) acc += (static_cast<double>(t[u].x) + t[u].y) + (static_cast<double>(t[u].z) + t[u].w);
        }
        done = n4 << 2;
    }
    for (int64_t i = done + threadIdx.x; i < n; i += THREADS) acc += __ldcg(v + i);
    part[threadIdx.x] = acc;
    __syncthreads();
    for (int s = THREADS / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) part[threadIdx.x] += part[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        *out = static_cast<float>(part[0] / static_cast<double>(n));
        *counter = 0;
    }
}

__global__ void __launch_bounds__(THREADS) softmax_ce_kernel(const float* __restrict__ z, const int64_t* __restrict__ labels, int64_t rows, int cols,
                                                              float* __restrict__ probs, float* __restrict__ dz, int dz_pitch,
                                                              float* __restrict__ row_loss, float gscale, float* __restrict__ mean_out,
                                                              unsigned int* __restrict__ counter) {
    wb_pdl_enter();
    softmax_ce_rows(z, labels, rows, cols, probs, dz, dz_pitch, row_loss, gscale);
    if (mean_out) mean_by_last_block(row_loss, rows, mean_out, counter);
}
template <int PER_LANE>
__global__ void __launch_bounds__(THREADS) softmax_ce_reg_kernel(const float* __restrict__ z, const int64_t* __restrict__ labels, int64_t rows,
                                                                  int cols, float* __restrict__ probs, float* __restrict__ dz, int dz_pitch,
                                                                  float* __restrict__ row_loss, float gscale, float* __restrict__ mean_out,
                                                                  unsigned int* __restrict__ counter) {
    wb_pdl_enter();
    softmax_ce_reg_rows<PER_LANE>(z, labels, rows, cols, probs, dz, dz_pitch, row_loss, gscale);
    if (mean_out) mean_by_last_block(row_loss, rows, mean_out, counter);
}
template <int PER4>
__global__ void __launch_bounds__(THREADS) softmax_ce_reg4_kernel(const float* __restrict__ z, const int64_t* __restrict__ labels, int64_t rows,
                                                                   int cols, float* __restrict__ probs, float* __restrict__ dz, int dz_pitch,
                                                                   float* __restrict__ row_loss, float gscale, float* __restrict__ mean_out,
                                                                   unsigned int* __restrict__ counter) {
    wb_pdl_enter();
    softmax_ce_reg4_rows<PER4>(z, labels, rows, cols, probs, dz, dz_pitch, row_loss, gscale);
    if (mean_out) mean_by_last_block(row_loss, rows, mean_out, counter);
}

// ---- Adam ---------------------------------------------------------------------------------------
// crates/weta-optim/src/lib.rs:210-239 as one pass: AdamK and adam_one in adam.cuh.
// One thread per four elements (128-bit accesses); the last, partial group is done element by element.
__global__ void __launch_bounds__(THREADS) adam_kernel(float* __restrict__ theta, const float* __restrict__ grad, float* __restrict__ m,
                                                        float* __restrict__ v, int64_t n, AdamK k, int vec) {
    wb_pdl_enter();
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) * 4;
    if (i >= n) return;
    if (vec && i + 4 <= n) {
        float4 th = *reinterpret_cast<const float4*>(theta + i);
        const float4 g = *reinterpret_cast<const float4*>(grad + i);
        float4 mi = k.first ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(m + i);
        float4 vi = k.first ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(v + i);
        adam_one(th.x, g.x, mi.x, vi.x, k);
        adam_one(th.y, g.y, mi.y, vi.y, k);
        adam_one(th.z, g.z, mi.z, vi.z, k);
        adam_one(th.w, g.w, mi.w, vi.w, k);
        *reinterpret_cast<float4*>(theta + i) = th;
        *reinterpret_cast<float4*>(m + i) = mi;
        *reinterpret_cast<float4*>(v + i) = vi;
    } else {
        for (int64_t j = i; j < n && j < i + 4; ++j) {
            float th = theta[j], mi = k.first ? 0.f : m[j], vi = k.first ? 0.f : v[j];
            adam_one(th, grad[j], mi, vi, k);
            theta[j] = th;
            m[j] = mi;
            v[j] = vi;
        }
    }
}

// Smallest 53-bit k whose uniform value (f32)((double)k * 2^-53) exceeds f32(p); 2^53 if none does.
// p <= 0 keeps everything (the reference returns x unchanged for p = 0); p = 1 keeps nothing (the reference
// returns x * 0, crates/weta-nn/src/functional.rs:66-71).
uint64_t dropout_threshold(double p) {
    if (p <= 0.0) return 0;
    if (p >= 1.0) return 1ull << 53;
    const float pf = static_cast<float>(p);
    uint64_t lo = 0, hi = 1ull << 53;  // invariant: u(lo - 1) <= pf (or lo == 0), u(hi) > pf (or hi == 2^53)
    while (lo < hi) {
        uint64_t mid = lo + (hi - lo) / 2;
        float u = static_cast<float>(static_cast<double>(mid) * (1.0 / 9007199254740992.0));
        if (u > pf) hi = mid;
        else lo = mid + 1;
    }
    return lo;
}


}  // namespace

// ---- entry points -------------------------------------------------------------------------------
extern "C" int wb_dropout_fwd(WbBackend* b, const float* x, float* y, int64_t n, double p, uint64_t seed) {
    WB_REQUIRE(b && x && y, WB_ERR_INVALID, "wb_dropout_fwd: null pointer");
    WB_REQUIRE(p >= 0.0 && p <= 1.0, WB_ERR_INVALID, "dropout probability has to be in [0, 1], got %g", p);
    if (n == 0) return WB_OK;
    WbProfileScope ps(b, "dropout");
    int64_t threads = (n + 3) / 4;
    const int vec = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
    wb_launch_pdl(dropout_kernel, dim3(static_cast<unsigned>((threads + THREADS - 1) / THREADS)), dim3(THREADS), 0, b->stream, 
        y, x, nullptr, n, dropout_threshold(p), p < 1.0 ? static_cast<float>(1.0 / (1.0 - p)) : 0.f, seed, vec);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_dropout_relu_bwd(WbBackend* b, const float* dy, const float* relu_out, float* dx, int64_t n, double p, uint64_t seed) {
    WB_REQUIRE(b && dy && dx, WB_ERR_INVALID, "wb_dropout_relu_bwd: null pointer");
    WB_REQUIRE(p >= 0.0 && p <= 1.0, WB_ERR_INVALID, "dropout probability has to be in [0, 1], got %g", p);
    if (n == 0) return WB_OK;
    WbProfileScope ps(b, "dropout_bwd");
    int64_t threads = (n + 3) / 4;
    const int vec = ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(relu_out)) & 15) == 0;
    wb_launch_pdl(dropout_kernel, dim3(static_cast<unsigned>((threads + THREADS - 1) / THREADS)), dim3(THREADS), 0, b->stream, 
        dx, dy, relu_out, n, dropout_threshold(p), p < 1.0 ? static_cast<float>(1.0 / (1.0 - p)) : 0.f, seed, vec);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_dropout_mask(WbBackend* b, float* mask, int64_t n, double p, uint64_t seed) {
    WB_REQUIRE(b && mask, WB_ERR_INVALID, "wb_dropout_mask: null pointer");
    WB_REQUIRE(p >= 0.0 && p <= 1.0, WB_ERR_INVALID, "dropout probability has to be in [0, 1], got %g", p);
    if (n == 0) return WB_OK;
    WbProfileScope ps(b, "dropout_mask");
    dropout_mask_kernel<<<static_cast<unsigned>(((n + 3) / 4 + THREADS - 1) / THREADS), THREADS, 0, b->stream>>>(
        mask, n, dropout_threshold(p), p < 1.0 ? static_cast<float>(1.0 / (1.0 - p)) : 0.f, seed);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

// dlogits rows may be padded to `dz_pitch` floats (>= cols, padding zero-filled) so that a following
// tensor-core contraction can read them through TMA even when cols is not a multiple of 4.
int wb_softmax_ce_pitched(WbBackend* b, const float* logits, const int64_t* labels, int64_t rows, int64_t cols, float* probs, float* dlogits,
                          int64_t dz_pitch, float* row_loss, float* mean_loss, double upstream) {
    WB_REQUIRE(b && logits && labels, WB_ERR_INVALID, "wb_softmax_ce: null pointer");
    WB_REQUIRE(cols > 0 && cols < (int64_t(1) << 31) && dz_pitch >= cols, WB_ERR_INVALID, "wb_softmax_ce: bad class count");
    if (rows == 0) return WB_OK;
    WbProfileScope ps(b, "softmax_ce");
    float* rl = row_loss;
    if (mean_loss && !rl) {
        void* s = nullptr;
        WB_TRY(wb_scratch(b, static_cast<size_t>(rows) * sizeof(float), &s));
        rl = static_cast<float*>(s);
    }
    int64_t threads = rows * 32;
    const unsigned grid = static_cast<unsigned>((threads + THREADS - 1) / THREADS);
    const float gscale = static_cast<float>(upstream * (1.0 / static_cast<double>(rows)));
    const int ic = static_cast<int>(cols), ip = static_cast<int>(dz_pitch);
    const bool v4 = cols % 4 == 0 && dz_pitch % 4 == 0 &&
                    ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(probs) | reinterpret_cast<uintptr_t>(dlogits)) & 15) == 0;
    unsigned int* counter = nullptr;
    if (mean_loss) WB_TRY(wb_block_counters(b, &counter));
    float* mo = mean_loss;
    if (v4 && cols > 32 && cols <= 128) wb_launch_pdl(softmax_ce_reg4_kernel<1>, dim3(grid), dim3(THREADS), 0, b->stream, logits, labels, rows, ic, probs, dlogits, ip, rl, gscale, mo, counter);
    else if (v4 && cols > 128 && cols <= 1024) wb_launch_pdl(softmax_ce_reg4_kernel<8>, dim3(grid), dim3(THREADS), 0, b->stream, logits, labels, rows, ic, probs, dlogits, ip, rl, gscale, mo, counter);
    else if (cols <= 32) wb_launch_pdl(softmax_ce_reg_kernel<1>, dim3(grid), dim3(THREADS), 0, b->stream, logits, labels, rows, ic, probs, dlogits, ip, rl, gscale, mo, counter);
    else if (cols <= 128) wb_launch_pdl(softmax_ce_reg_kernel<4>, dim3(grid), dim3(THREADS), 0, b->stream, logits, labels, rows, ic, probs, dlogits, ip, rl, gscale, mo, counter);
    else if (cols <= 1024) wb_launch_pdl(softmax_ce_reg_kernel<32>, dim3(grid), dim3(THREADS), 0, b->stream, logits, labels, rows, ic, probs, dlogits, ip, rl, gscale, mo, counter);
    else wb_launch_pdl(softmax_ce_kernel, dim3(grid), dim3(THREADS), 0, b->stream, logits, labels, rows, ic, probs, dlogits, ip, rl, gscale, mo, counter);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_softmax_ce(WbBackend* b, const float* logits, const int64_t* labels, int64_t rows, int64_t cols, float* probs,
                             float* dlogits, float* row_loss, float* mean_loss, double upstream) {
    return wb_softmax_ce_pitched(b, logits, labels, rows, cols, probs, dlogits, cols, row_loss, mean_loss, upstream);
}

// Addresses and argument positions of the two kernels whose arguments change from step to step (the dropout seed, the
// Adam scalars): a captured training step (trainer.cu) finds their nodes by these and rewrites those arguments.
const void* wb_dropout_kernel_func() { return reinterpret_cast<const void*>(&dropout_kernel); }  // arguments: y, x, relu_src, n, kmin, scale, seed, vec
const void* wb_adam_kernel_func() { return reinterpret_cast<const void*>(&adam_kernel); }        // arguments: theta, grad, m, v, n, AdamK, vec

extern "C" int wb_adam_step(WbBackend* b, float* theta, const float* grad, float* m, float* v, int64_t n, int64_t t, double lr,
                            double beta1, double beta2, double eps, double weight_decay, int decoupled, double grad_scale) {
    WB_REQUIRE(b && theta && grad && m && v, WB_ERR_INVALID, "wb_adam_step: null pointer");
    WB_REQUIRE(t >= 1, WB_ERR_INVALID, "wb_adam_step: step counts from 1");
    if (n == 0) return WB_OK;
    WbProfileScope ps(b, "adam_step");
    const AdamK k = wb_adam_constants(t, lr, beta1, beta2, eps, weight_decay, decoupled, grad_scale);
    const int vec = ((reinterpret_cast<uintptr_t>(theta) | reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(m) |
                      reinterpret_cast<uintptr_t>(v)) & 15) == 0;
    const int64_t groups = (n + 3) / 4;
    wb_launch_pdl(adam_kernel, dim3(static_cast<unsigned>((groups + THREADS - 1) / THREADS)), dim3(THREADS), 0, b->stream, theta, grad, m, v, n, k, vec);
    WB_LAUNCH_OK(b);
    return WB_OK;
}
