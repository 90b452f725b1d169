// Fused extension entry points around the contraction and the pooling of the named models:
//   linear forward / backward   crates/weta-nn/src/functional.rs:54-60, crates/weta-autograd/src/ops.rs:821-827, 46-58
//   max-pool forward / backward functional.rs:121-130, ops.rs:305-314 (ties share the gradient)
//   ReLU backward               ops.rs:85
// plus the dispatcher the fused trainer shares with them: tensor cores first, CUDA-core tiles when TMA cannot
// read an operand or the backend is in FP32 mode.
#include <algorithm>
#include <cmath>

#include "common.h"
#include "gemm.h"

// D[batch][m][n] = A x B (+ epilogue) in the given matmul mode.  *used_tc (optional) tells whether the tensor-core
// kernel ran (only it honours Epilogue::row_stats).
int wb_gemm_dispatch(WbBackend* be, int mode, WbGemmOperand A, WbGemmOperand B, int64_t batch, int m, int n, int k, tc::Epilogue ep,
                     int64_t span_batch, bool* used_tc) {
    if (used_tc) *used_tc = false;
    if (mode != WB_MM_FP32 && static_cast<int64_t>(m) * n * k >= (1 << 15)) {
        int s = wb_tc_gemm(be, A, B, batch, m, n, k, ep, mode, 0, span_batch);
        if (s != WB_ERR_UNSUPPORTED) {
            if (used_tc) *used_tc = true;
            return s;
        }
    }
    WB_REQUIRE(span_batch == 0 && !ep.accumulate, WB_ERR_UNSUPPORTED, "no CUDA-core path for this contraction");
    // CUDA-core path: describe the operands as [B, M, K] x [B, K, N] views.
    WbView a{}, b{};
    a.data = const_cast<float*>(A.ptr); a.dtype = WB_F32; a.ndim = 3; a.offset = 0;
    a.shape[0] = batch; a.shape[1] = m; a.shape[2] = k;
    a.stride[0] = A.batch_stride; a.stride[1] = A.mn_major ? 1 : A.ld; a.stride[2] = A.mn_major ? A.ld : 1;
    b.data = const_cast<float*>(B.ptr); b.dtype = WB_F32; b.ndim = 3; b.offset = 0;
    b.shape[0] = batch; b.shape[1] = k; b.shape[2] = n;
    b.stride[0] = B.batch_stride; b.stride[1] = B.mn_major ? B.ld : 1; b.stride[2] = B.mn_major ? 1 : B.ld;
    WB_REQUIRE(ep.ldd == n && (batch == 1 || ep.batch_stride_d == static_cast<int64_t>(m) * n), WB_ERR_UNSUPPORTED,
               "the CUDA-core contraction needs a dense output");
    WB_TRY(wb_matmul_simt(be, &a, &b, ep.out));
    if (ep.bias_n || ep.bias_m || ep.relu) {
        // bias / ReLU as one broadcast add (+ relu) over the dense result
        WbView o{}, bias{};
        o.data = ep.out; o.dtype = WB_F32; o.ndim = 3; o.shape[0] = batch; o.shape[1] = m; o.shape[2] = n;
        o.stride[0] = static_cast<int64_t>(m) * n; o.stride[1] = n; o.stride[2] = 1;
        if (ep.bias_n || ep.bias_m) {
            bias = o;
            bias.data = const_cast<float*>(ep.bias_n ? ep.bias_n : ep.bias_m);
            bias.stride[0] = 0; bias.stride[1] = ep.bias_m ? 1 : 0; bias.stride[2] = ep.bias_n ? 1 : 0;
            WB_TRY(wb_binary_into(be, WB_ADD, &o, &bias, ep.out));
        }
        if (ep.relu) WB_TRY(wb_unary_into(be, WB_RELU, 0.0, 0.0, &o, ep.out));
    }
    return WB_OK;
}

extern "C" int wb_linear_fwd(WbBackend* b, const float* x, const float* weight, const float* bias, int64_t n, int64_t in, int64_t out, int relu,
                             float* y) {
    WB_REQUIRE(b && x && weight && y && n > 0 && in > 0 && out > 0, WB_ERR_INVALID, "wb_linear_fwd: bad arguments");
    WB_REQUIRE(n < (1 << 30) && in < (1 << 30) && out < (1 << 30), WB_ERR_INVALID, "wb_linear_fwd: dimension too large");
    WbProfileScope ps(b, "linear_fwd");
    WbGemmOperand Ax{x, n, in, in, 0, false};
    WbGemmOperand Bw{weight, out, in, in, 0, false};
    tc::Epilogue ep{y, out, 0, bias, nullptr, relu ? 1 : 0, 0};
    return wb_gemm_dispatch(b, b->matmul_mode, Ax, Bw, 1, static_cast<int>(n), static_cast<int>(out), static_cast<int>(in), ep, 0, nullptr);
}

extern "C" int wb_linear_bwd(WbBackend* b, const float* x, const float* weight, const float* dy, int64_t n, int64_t in, int64_t out, float* dx,
                             float* dweight, float* dbias) {
    WB_REQUIRE(b && x && weight && dy && n > 0 && in > 0 && out > 0, WB_ERR_INVALID, "wb_linear_bwd: bad arguments");
    WB_REQUIRE(n < (1 << 30) && in < (1 << 30) && out < (1 << 30), WB_ERR_INVALID, "wb_linear_bwd: dimension too large");
    WbProfileScope ps(b, "linear_bwd");
    const bool narrow = wb_narrow_linear_ok(n, in, out, x, weight);
    // at most 16 outputs: CUDA-core kernels (narrow_linear.cu), the weight gradient only for small batches
    if (narrow && dweight && n <= 1024) {
        WB_TRY(wb_narrow_linear_wgrad(b, b->matmul_mode, dy, out, x, static_cast<int>(n), static_cast<int>(in), static_cast<int>(out), dweight));
        dweight = nullptr;
    }
    if (narrow && dx) {
        WB_TRY(wb_narrow_linear_dgrad(b, b->matmul_mode, dy, out, weight, static_cast<int>(n), static_cast<int>(in), static_cast<int>(out), dx));
        dx = nullptr;
    }
    if (dweight) {  // dW[out, in] = dY^T X
        WbGemmOperand Az{dy, out, n, out, 0, true};
        WbGemmOperand Bx{x, in, n, in, 0, true};
        tc::Epilogue ep{dweight, in, 0, nullptr, nullptr, 0, 0};
        WB_TRY(wb_gemm_dispatch(b, b->matmul_mode, Az, Bx, 1, static_cast<int>(out), static_cast<int>(in), static_cast<int>(n), ep, 0, nullptr));
    }
    if (dbias) {  // sum over the batch
        WbView v{};
        v.data = const_cast<float*>(dy); v.dtype = WB_F32; v.ndim = 2;
        v.shape[0] = n; v.shape[1] = out; v.stride[0] = out; v.stride[1] = 1;
        WB_TRY(wb_reduce_into(b, WB_SUM, &v, 0, dbias));
    }
    if (dx) {  // dX[n, in] = dY W
        WbGemmOperand Ad{dy, n, out, out, 0, false};
        WbGemmOperand Bw{weight, in, out, in, 0, true};
        tc::Epilogue ep{dx, in, 0, nullptr, nullptr, 0, 0};
        WB_TRY(wb_gemm_dispatch(b, b->matmul_mode, Ad, Bw, 1, static_cast<int>(n), static_cast<int>(in), static_cast<int>(out), ep, 0, nullptr));
    }
    return WB_OK;
}

namespace {

// weta's max: (a >= b || isnan(a)) ? a : b, folded from -inf (crates/weta-core/src/dtype.rs:136-149).
__device__ __forceinline__ float wmax(float a, float b) { return (a >= b || isnan(a)) ? a : b; }

__global__ void __launch_bounds__(256) maxpool_fwd_kernel(float* __restrict__ y, const float* __restrict__ x, int h, int w, int oh, int ow, int k,
                                                          int s, int64_t total) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total) return;
    const int ox = static_cast<int>(i % ow), oy = static_cast<int>(i / ow % oh);
    const int64_t plane = i / (static_cast<int64_t>(ow) * oh);
    const float* src = x + plane * h * w + static_cast<int64_t>(oy) * s * w + ox * s;
    float best = -INFINITY;
    for (int ki = 0; ki < k; ++ki)
        for (int kj = 0; kj < k; ++kj) best = wmax(best, src[ki * w + kj]);
    y[i] = best;
}

// One thread per input element: the sum, over the windows that contain it, of (x == window max) / (number of
// window positions equal to the max) * dy.  A window whose max is NaN has no position equal to it: 0/0, as in the
// reference's mask / sum(mask).
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(float* __restrict__ dx, const float* __restrict__ x, const float* __restrict__ dy, int h,
                                                          int w, int oh, int ow, int k, int s, int64_t total) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total) return;
    const int px = static_cast<int>(i % w), py = static_cast<int>(i / w % h);
    const int64_t plane = i / (static_cast<int64_t>(w) * h);
    const float* src = x + plane * h * w;
    const float* g = dy + plane * oh * ow;
    const float v = src[py * w + px];
    // windows (oy, ox) with oy*s <= py < oy*s + k, in ascending (ki, kj) order of the position inside the window
    float acc = 0.f;
    for (int ki = 0; ki < k; ++ki) {
        const int ty = py - ki;
        if (ty < 0 || ty % s != 0 || ty / s >= oh) continue;
        for (int kj = 0; kj < k; ++kj) {
            const int tx = px - kj;
            if (tx < 0 || tx % s != 0 || tx / s >= ow) continue;
            const int oy = ty / s, ox = tx / s;
            const float* win = src + static_cast<int64_t>(oy) * s * w + ox * s;
            float best = -INFINITY;
            for (int a = 0; a < k; ++a)
                for (int c = 0; c < k; ++c) best = wmax(best, win[a * w + c]);
            float cnt = 0.f;
            for (int a = 0; a < k; ++a)
                for (int c = 0; c < k; ++c) cnt += win[a * w + c] == best ? 1.f : 0.f;
            acc += ((v == best ? 1.f : 0.f) / cnt) * g[oy * ow + ox];
        }
    }
    dx[i] = acc;
}

}  // namespace

extern "C" int wb_maxpool2d_fwd(WbBackend* b, const float* x, int64_t planes, int64_t h, int64_t w, int64_t kernel, int64_t stride, float* y) {
    WB_REQUIRE(b && x && y, WB_ERR_INVALID, "wb_maxpool2d_fwd: null pointer");
    WB_REQUIRE(kernel > 0 && stride > 0 && h >= kernel && w >= kernel && planes >= 0, WB_ERR_INVALID, "wb_maxpool2d_fwd: bad geometry");
    const int64_t oh = (h - kernel) / stride + 1, ow = (w - kernel) / stride + 1, total = planes * oh * ow;
    if (total == 0) return WB_OK;
    WbProfileScope ps(b, "maxpool2d_fwd");
    maxpool_fwd_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, b->stream>>>(y, x, static_cast<int>(h), static_cast<int>(w),
                                                                                          static_cast<int>(oh), static_cast<int>(ow),
                                                                                          static_cast<int>(kernel), static_cast<int>(stride), total);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_maxpool2d_bwd(WbBackend* b, const float* x, const float* dy, int64_t planes, int64_t h, int64_t w, int64_t kernel, int64_t stride,
                                float* dx) {
    WB_REQUIRE(b && x && dy && dx, WB_ERR_INVALID, "wb_maxpool2d_bwd: null pointer");
    WB_REQUIRE(kernel > 0 && stride > 0 && h >= kernel && w >= kernel && planes >= 0, WB_ERR_INVALID, "wb_maxpool2d_bwd: bad geometry");
    const int64_t oh = (h - kernel) / stride + 1, ow = (w - kernel) / stride + 1, total = planes * h * w;
    if (total == 0) return WB_OK;
    WbProfileScope ps(b, "maxpool2d_bwd");
    maxpool_bwd_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, b->stream>>>(dx, x, dy, static_cast<int>(h), static_cast<int>(w),
                                                                                          static_cast<int>(oh), static_cast<int>(ow),
                                                                                          static_cast<int>(kernel), static_cast<int>(stride), total);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_relu_bwd(WbBackend* b, const float* dy, const float* y, float* dx, int64_t n) {
    // dx = dy * step(y): UnaryBw for ReLU; y may be the ReLU's input or its output (same sign test)
    WB_REQUIRE(y, WB_ERR_INVALID, "wb_relu_bwd: y (the ReLU's input or output) is null");
    return wb_dropout_relu_bwd(b, dy, y, dx, n, 0.0, 0);
}
