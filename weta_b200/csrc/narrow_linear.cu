// Linear layers with very few outputs (the logits layer: 10 classes): the two gradient products on CUDA cores.
//
// MatmulBw (crates/weta-autograd/src/ops.rs:821-827) for out <= 16.  The tensor-core kernel needs ~10-20 us for such a
// product whatever its size (a 128-wide tile, a pipeline of K blocks walked by four CTAs, a split-K pass): at small
// batches the gradients of a 1024 -> 10 layer cost more than their 20 MFLOP deserve.  Here each is one short launch:
//   dweight   dw[s][j] = sum_b dy[b][s] x[b][j]             one block per 32 inputs j walks the whole batch
//   dx        dx[b][j] = sum_s dy[b][s] w[s][j]             one thread per four inputs j
// (The forward product stays on the tensor cores: a warp per sample on CUDA cores measured slower.)
// In TF32 mode both operands lose their low 13 mantissa bits first, the way the tensor core reads them, so the layer
// keeps the arithmetic of the mode it runs in (a product of two such values is exact in f32); FP32 and 3xTF32 modes
// use the operands as they are.
#include "common.h"

namespace {

constexpr int MAX_OUT = 16;

__device__ __forceinline__ float operand(float v, int tf32) { return tf32 ? __uint_as_float(__float_as_uint(v) & 0xFFFFE000u) : v; }

// One block per 32 inputs, 16 warps: warp w adds the samples [w * per, (w + 1) * per) for input strip * 32 + lane in
// ascending order; the warps' sums are then added in ascending warp order.  No partial sums leave the block, so the
// result is the same every run.  A warp first copies the dy rows of 32 samples into shared memory with one round of
// independent loads (read in place, every sample's row would cost the in-order pipeline a trip to L2), then keeps
// eight samples' x loads in flight at a time.
template <int S>
__global__ void __launch_bounds__(512) narrow_wgrad_kernel(float* __restrict__ dw, const float* __restrict__ dy, int64_t dy_pitch,
                                                            const float* __restrict__ x, int n, int in, int out, int tf32) {
    wb_pdl_enter();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int j = blockIdx.x * 32 + lane;
    const int per = (n + 15) / 16, b0 = min(n, warp * per), b1 = min(n, b0 + per);
    __shared__ float sh[16 * S * 33];       // first the warps' dy tiles [16][32][S], then the warps' sums [16][S][33]
    float* gsh = sh + warp * 32 * S;
    float acc[S];
#pragma unroll
    for (int s = 0; s < S; ++s) acc[s] = 0.f;
    for (int c0 = b0; c0 < b1; c0 += 32) {
        const int cnt = min(32, b1 - c0);
        __syncwarp();
        for (int t = lane; t < cnt * S; t += 32) {
            const int i = t / S, s = t - i * S;
            gsh[t] = s < out ? operand(dy[static_cast<int64_t>(c0 + i) * dy_pitch + s], tf32) : 0.f;
        }
        __syncwarp();
        if (j < in) {
            for (int bb = 0; bb < cnt; bb += 8) {
                float xv[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) xv[u] = bb + u < cnt ? operand(x[static_cast<int64_t>(c0 + bb + u) * in + j], tf32) : 0.f;
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (bb + u < cnt) {
#pragma unroll
                        for (int s = 0; s < S; ++s) acc[s] += gsh[(bb + u) * S + s] * xv[u];
                    }
            }
        }
    }
    __syncthreads();  // every warp is done with its dy tile: the array now takes the warps' sums
#pragma unroll
    for (int s = 0; s < S; ++s) sh[(warp * S + s) * 33 + lane] = acc[s];
    __syncthreads();
    for (int t = threadIdx.x; t < S * 32; t += 512) {
        const int s = t >> 5, l = t & 31, col = blockIdx.x * 32 + l;
        if (s < out && col < in) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 16; ++w) v += sh[(w * S + s) * 33 + l];
            dw[static_cast<int64_t>(s) * in + col] = v;
        }
    }
}

template <int S>
__global__ void __launch_bounds__(256) narrow_dgrad_kernel(float* __restrict__ dx, const float* __restrict__ dy, int64_t dy_pitch,
                                                            const float* __restrict__ w, int n, int in, int out, int tf32) {
    wb_pdl_enter();
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

int wb_narrow_linear_wgrad(WbBackend* b, int mode, const float* dy, int64_t dy_pitch, const float* x, int n, int in, int out, float* dw) {
    const int tf32 = mode == WB_MM_TF32;
    const unsigned grid = static_cast<unsigned>((in + 31) / 32);
    if (out <= 10) wb_launch_pdl(narrow_wgrad_kernel<10>, dim3(grid), dim3(512), 0, b->stream, dw, dy, dy_pitch, x, n, in, out, tf32);
    else wb_launch_pdl(narrow_wgrad_kernel<16>, dim3(grid), dim3(512), 0, b->stream, dw, dy, dy_pitch, x, n, in, out, tf32);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

int wb_narrow_linear_dgrad(WbBackend* b, int mode, const float* dy, int64_t dy_pitch, const float* w, int n, int in, int out, float* dx) {
    const int tf32 = mode == WB_MM_TF32;
    const int64_t threads = static_cast<int64_t>(n) * (in / 4);
    const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
    if (out <= 10) wb_launch_pdl(narrow_dgrad_kernel<10>, dim3(grid), dim3(256), 0, b->stream, dx, dy, dy_pitch, w, n, in, out, tf32);
    else wb_launch_pdl(narrow_dgrad_kernel<16>, dim3(grid), dim3(256), 0, b->stream, dx, dy, dy_pitch, w, n, in, out, tf32);
    WB_LAUNCH_OK(b);
    return WB_OK;
}
