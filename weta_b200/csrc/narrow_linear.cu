// Linear layers with very few outputs (the logits layer: 10 classes), forward and backward, on CUDA cores.
//
// F::linear and MatmulBw (crates/weta-nn/src/functional.rs:54-60, crates/weta-autograd/src/ops.rs:821-827) for
// out <= 16.  The tensor-core kernel needs ~10-20 us for such a product whatever its size (a 128-wide tile, a
// pipeline of K blocks walked by four CTAs, a split-K pass): at small batches the three products of a 1024 -> 10
// layer cost more than its 20 MFLOP deserve.  Here each is one short launch (the callers use the two gradient kernels;
// the forward kernel measured slower than the tensor-core path and is kept for layers TMA cannot read):
//   forward   y[b][s]  = sum_k x[b][k] w[s][k] (+ bias[s])   one warp per sample, lanes stride over k
//   dweight   dw[s][j] = sum_b dy[b][s] x[b][j]             slabs of samples in parallel, the last block adds the
//                                                           slabs in ascending order (deterministic, one launch)
//   dx        dx[b][j] = sum_s dy[b][s] w[s][j]             one thread per four inputs j
// In TF32 mode both operands lose their low 13 mantissa bits first, the way the tensor core reads them, so the layer
// keeps the arithmetic of the mode it runs in (a product of two such values is exact in f32); FP32 and 3xTF32 modes
// use the operands as they are.
#include "common.h"

namespace {

constexpr int MAX_OUT = 16;

__device__ __forceinline__ float operand(float v, int tf32) { return tf32 ? __uint_as_float(__float_as_uint(v) & 0xFFFFE000u) : v; }

template <int S>
__global__ void __launch_bounds__(256) narrow_fwd_kernel(float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ w,
                                                          const float* __restrict__ bias, int n, int in, int out, int relu, int tf32) {
    const int row = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (row >= n) return;
    float acc[S];
#pragma unroll
    for (int s = 0; s < S; ++s) acc[s] = 0.f;
    const float4* xr = reinterpret_cast<const float4*>(x + static_cast<int64_t>(row) * in);  // in % 4 == 0, 16-byte aligned rows
    const int q = in >> 2;
    for (int k = lane; k < q; k += 32) {
        const float4 xv = xr[k];
        const float x0 = operand(xv.x, tf32), x1 = operand(xv.y, tf32), x2 = operand(xv.z, tf32), x3 = operand(xv.w, tf32);
        float4 wv[S];
#pragma unroll
        for (int s = 0; s < S; ++s)
            wv[s] = s < out ? __ldg(reinterpret_cast<const float4*>(w + static_cast<int64_t>(s) * in) + k) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < S; ++s) {
            acc[s] += x0 * operand(wv[s].x, tf32);
            acc[s] += x1 * operand(wv[s].y, tf32);
            acc[s] += x2 * operand(wv[s].z, tf32);
            acc[s] += x3 * operand(wv[s].w, tf32);
        }
    }
#pragma unroll
    for (int s = 0; s < S; ++s)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[s] += __shfl_xor_sync(0xffffffffu, acc[s], o);
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < S; ++s)
            if (s < out) {
                float v = acc[s] + (bias ? bias[s] : 0.f);
                y[static_cast<int64_t>(row) * out + s] = relu ? fmaxf(v, 0.f) : v;
            }
    }
}

// grid (ceil(in / 256), slabs): block (jb, sl) adds samples [sl * per, ...) for inputs j of its 256-wide strip.
template <int S>
__global__ void __launch_bounds__(256) narrow_wgrad_kernel(float* __restrict__ dw, float* __restrict__ part, unsigned int* __restrict__ counter,
                                                            const float* __restrict__ dy, int64_t dy_pitch, const float* __restrict__ x, int n, int in,
                                                            int out, int per, int tf32) {
    const int j = blockIdx.x * 256 + threadIdx.x;
    const int b0 = blockIdx.y * per, b1 = min(n, b0 + per);
    __shared__ float g[64][S];
    float acc[S];
#pragma unroll
    for (int s = 0; s < S; ++s) acc[s] = 0.f;
    for (int base = b0; base < b1; base += 64) {
        const int cnt = min(64, b1 - base);
        __syncthreads();
        for (int t = threadIdx.x; t < cnt * S; t += 256) {
            const int bb = t / S, s = t - bb * S;
            g[bb][s] = s < out ? operand(dy[static_cast<int64_t>(base + bb) * dy_pitch + s], tf32) : 0.f;
        }
        __syncthreads();
        if (j < in) {
            for (int bb = 0; bb < cnt; ++bb) {
                const float xv = operand(x[static_cast<int64_t>(base + bb) * in + j], tf32);
#pragma unroll
                for (int s = 0; s < S; ++s) acc[s] += g[bb][s] * xv;
            }
        }
    }
    const int slabs = gridDim.y;
    if (j < in)
        for (int s = 0; s < out; ++s) part[(static_cast<int64_t>(blockIdx.y) * out + s) * in + j] = acc[s];
    // the last block of this strip to finish adds the slabs in ascending order
    __threadfence();
    __syncthreads();
    __shared__ unsigned int last;
    if (threadIdx.x == 0) last = atomicAdd(&counter[blockIdx.x], 1u) == static_cast<unsigned>(slabs - 1);
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (j < in) {
        float t[S];
#pragma unroll
        for (int s = 0; s < S; ++s) t[s] = 0.f;
        for (int sl = 0; sl < slabs; ++sl)
#pragma unroll
            for (int s = 0; s < S; ++s)
                if (s < out) t[s] += __ldcg(&part[(static_cast<int64_t>(sl) * out + s) * in + j]);
#pragma unroll
        for (int s = 0; s < S; ++s)
            if (s < out) dw[static_cast<int64_t>(s) * in + j] = t[s];
    }
    if (threadIdx.x == 0) counter[blockIdx.x] = 0;  // ready for the next launch
}

template <int S>
__global__ void __launch_bounds__(256) narrow_dgrad_kernel(float* __restrict__ dx, const float* __restrict__ dy, int64_t dy_pitch,
                                                            const float* __restrict__ w, int n, int in, int out, int tf32) {
    const int64_t t = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    const int q = in >> 2;  // in % 4 == 0
    if (t >= static_cast<int64_t>(n) * q) return;
    const int row = static_cast<int>(t / q), j = static_cast<int>(t - static_cast<int64_t>(row) * q) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < S; ++s)
        if (s < out) {
            const float gv = operand(dy[static_cast<int64_t>(row) * dy_pitch + s], tf32);
            const float4 wv = *reinterpret_cast<const float4*>(w + static_cast<int64_t>(s) * in + j);
            acc.x += gv * operand(wv.x, tf32);
            acc.y += gv * operand(wv.y, tf32);
            acc.z += gv * operand(wv.z, tf32);
            acc.w += gv * operand(wv.w, tf32);
        }
    *reinterpret_cast<float4*>(dx + static_cast<int64_t>(row) * in + j) = acc;
}

}  // namespace

bool wb_narrow_linear_ok(int64_t n, int64_t in, int64_t out, const float* x, const float* w) {
    return out >= 1 && out <= MAX_OUT && in % 4 == 0 && in >= 32 && n >= 1 && n < (1 << 24) && in < (1 << 24) &&
           ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0;
}

int wb_narrow_linear_fwd(WbBackend* b, int mode, const float* x, const float* w, const float* bias, int n, int in, int out, int relu, float* y) {
    const int tf32 = mode == WB_MM_TF32;
    const unsigned grid = static_cast<unsigned>((static_cast<int64_t>(n) * 32 + 255) / 256);
    if (out <= 10) narrow_fwd_kernel<10><<<grid, 256, 0, b->stream>>>(y, x, w, bias, n, in, out, relu, tf32);
    else narrow_fwd_kernel<16><<<grid, 256, 0, b->stream>>>(y, x, w, bias, n, in, out, relu, tf32);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

// scratch: slabs * out * in floats of partial sums followed by one counter per 256-input strip (zero between launches).
int wb_narrow_linear_wgrad(WbBackend* b, int mode, const float* dy, int64_t dy_pitch, const float* x, int n, int in, int out, float* dw) {
    const int tf32 = mode == WB_MM_TF32;
    const int strips = (in + 255) / 256;
    int slabs = std::max(1, std::min(std::min(n / 64, 16), (2 * b->sm_count + strips - 1) / strips));
    const int per = ((n + slabs - 1) / slabs + 63) / 64 * 64;
    slabs = (n + per - 1) / per;
    const size_t part_bytes = static_cast<size_t>(slabs) * out * in * sizeof(float);
    // The counters live in their own small allocation of the backend (zeroed once, restored to zero by every launch).
    if (!b->narrow_counters) {
        WB_CHECK_CUDA(cudaMalloc(&b->narrow_counters, 4096 * sizeof(unsigned int)));
        WB_CHECK_CUDA(cudaMemsetAsync(b->narrow_counters, 0, 4096 * sizeof(unsigned int), b->stream));
    }
    WB_REQUIRE(strips <= 4096, WB_ERR_UNSUPPORTED, "narrow linear layer: too many inputs");
    void* part = nullptr;
    WB_TRY(wb_scratch(b, part_bytes, &part));
    const dim3 grid(static_cast<unsigned>(strips), static_cast<unsigned>(slabs));
    if (out <= 10)
        narrow_wgrad_kernel<10><<<grid, 256, 0, b->stream>>>(dw, static_cast<float*>(part), static_cast<unsigned int*>(b->narrow_counters), dy, dy_pitch, x,
                                                             n, in, out, per, tf32);
    else
        narrow_wgrad_kernel<16><<<grid, 256, 0, b->stream>>>(dw, static_cast<float*>(part), static_cast<unsigned int*>(b->narrow_counters), dy, dy_pitch, x,
                                                             n, in, out, per, tf32);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

int wb_narrow_linear_dgrad(WbBackend* b, int mode, const float* dy, int64_t dy_pitch, const float* w, int n, int in, int out, float* dx) {
    const int tf32 = mode == WB_MM_TF32;
    const int64_t threads = static_cast<int64_t>(n) * (in / 4);
    const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
    if (out <= 10) narrow_dgrad_kernel<10><<<grid, 256, 0, b->stream>>>(dx, dy, dy_pitch, w, n, in, out, tf32);
    else narrow_dgrad_kernel<16><<<grid, 256, 0, b->stream>>>(dx, dy, dy_pitch, w, n, in, out, tf32);
    WB_LAUNCH_OK(b);
    return WB_OK;
}
