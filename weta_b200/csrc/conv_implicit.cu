// 3x3 / stride 1 / padding 1 convolution as an implicit GEMM on the tensor cores: forward, weight gradient
// and input gradient without materialising the im2col matrix.  It computes what the reference's chain
// im2col -> matmul -> add (crates/weta-nn/src/functional.rs:84-106) and that chain's backward
// (crates/weta-autograd/src/ops.rs:821-827, 865-868) compute, with TF32 operands and f32 accumulation.
#include <algorithm>

#include "common.h"
#include "gemm.h"

// The tensor-core kernel fetches a tap's window as the image's own pixel run moved by whole rows; the
// move by one column cannot be a TMA start address (4-byte granularity), so the image is kept in three
// copies: itself, shifted right (left[y][x] = image[y][x-1]) and shifted left (right[y][x] = image[y][x+1]),
// zeros shifted in.  (The input gradient of layers that pass wb_conv3_dgrad_needs_no_copies applies the column
// move to its result instead and reads dY alone.)
namespace {

__global__ void __launch_bounds__(256) shift_copies_kernel(const float* __restrict__ in, float* __restrict__ left, float* __restrict__ right,
                                                           int64_t groups, int w4) {
    wb_pdl_enter();
    // one thread per 4 consecutive pixels of a row (w is a multiple of 4)
    for (int64_t gi = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; gi < groups; gi += static_cast<int64_t>(gridDim.x) * 256) {
        const int xg = static_cast<int>(gi % w4);
        const float4 v = reinterpret_cast<const float4*>(in)[gi];
        const float prev = xg > 0 ? in[gi * 4 - 1] : 0.f;
        const float next = xg + 1 < w4 ? in[gi * 4 + 4] : 0.f;
        reinterpret_cast<float4*>(left)[gi] = make_float4(prev, v.x, v.y, v.z);
        reinterpret_cast<float4*>(right)[gi] = make_float4(v.y, v.z, v.w, next);
    }
}

// kind 0: dst[o][tap][c] = src[o][c][tap]        (forward operand)
// kind 1: dst[c][tap][o] = src[o][c][8 - tap]    (input-gradient operand: transposed channels, flipped taps)
// kind 2: dst[o][c][tap] = src[tap][c][o]        (weight gradient back to the parameter's element order)
// kind 3: kinds 0 and 1 in one launch, into dst and dst2 (both operands of a step from the same parameters)
__global__ void __launch_bounds__(256) weight_reorder_kernel(const float* __restrict__ src, float* __restrict__ dst, float* __restrict__ dst2,
                                                             int o_n, int c_n, int kind) {
    wb_pdl_enter();
    const int64_t total = static_cast<int64_t>(o_n) * c_n * 9;
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total) return;
    if (kind == 0 || kind == 3) {
        const int c = static_cast<int>(i % c_n), tap = static_cast<int>(i / c_n % 9), o = static_cast<int>(i / (9 * c_n));
        dst[i] = src[(static_cast<int64_t>(o) * c_n + c) * 9 + tap];
    }
    if (kind == 1 || kind == 3) {
        const int o = static_cast<int>(i % o_n), tap = static_cast<int>(i / o_n % 9), c = static_cast<int>(i / (9 * o_n));
        (kind == 3 ? dst2 : dst)[i] = src[(static_cast<int64_t>(o) * c_n + c) * 9 + (8 - tap)];
    }
    if (kind == 2) {
        const int tap = static_cast<int>(i % 9), c = static_cast<int>(i / 9 % c_n), o = static_cast<int>(i / (9 * c_n));
        dst[i] = src[(static_cast<int64_t>(tap) * c_n + c) * o_n + o];
    }
}

}  // namespace

int wb_conv3_shift_copies(WbBackend* b, const float* in, int64_t rows, int w, float* left, float* right) {
    WB_REQUIRE(w % 4 == 0 && !(reinterpret_cast<uintptr_t>(in) & 15) && !(reinterpret_cast<uintptr_t>(left) & 15) &&
                   !(reinterpret_cast<uintptr_t>(right) & 15),
               WB_ERR_INVALID, "conv3 shift copies: width must be a multiple of 4 and the buffers 16-byte aligned");
    const int64_t groups = rows * (w / 4);
    if (groups == 0) return WB_OK;
    const int64_t blocks = std::min<int64_t>((groups + 255) / 256, static_cast<int64_t>(b->sm_count) * 16);
    wb_launch_pdl(shift_copies_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, b->stream, in, left, right, groups, w / 4);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

int wb_conv3_weight_reorder(WbBackend* b, int kind, const float* src, float* dst, int o_n, int c_n, float* dst2) {
    const int64_t total = static_cast<int64_t>(o_n) * c_n * 9;
    if (total == 0) return WB_OK;
    wb_launch_pdl(weight_reorder_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, b->stream, src, dst, dst2, o_n, c_n, kind);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

bool wb_conv3_eligible(const WbConv3& g) {
    return g.w % 4 == 0 && g.c % 128 == 0 && g.o % 32 == 0 && g.n > 0 && g.h > 0 && g.h * g.w < (int64_t(1) << 30) && g.o < (1 << 30) &&
           9 * g.c < (1 << 30);
}

// y[n][o][h][w] = conv(x, weight) + bias[o];  wr = weight as [o][tap][c] (wb_conv3_weight_reorder kind 0).
// channel_sums (optional, zeroed by the caller): receives per output channel (sum y, sum y^2) over the batch.
int wb_conv3_fwd(WbBackend* b, const WbConv3& g, const float* const x3[3], const float* wr, const float* bias, float* y, double* channel_sums) {
    const int64_t hw = g.h * g.w;
    tc::Epilogue ep{y, hw, g.o * hw, nullptr, bias, 0, 0};
    ep.row_stats = channel_sums;
    // (Applying the horizontal moves to the result, as the input gradient does, measured no faster here: 600 against
    // 611 TFLOP/s on 128 -> 256 channels, whose contraction per kernel column is only 12 K blocks long.)
    return wb_tc_conv_gemm(b, 1, wr, x3, g.n, g.c, g.h, g.w, static_cast<int>(g.o), ep);
}

// dweight[o][c][3][3] = sum over images and pixels of dy * window(x);  dwr: scratch of o*9*c floats.
int wb_conv3_wgrad(WbBackend* b, const WbConv3& g, const float* dy, const float* const x3[3], float* dwr, float* dweight) {
    tc::Epilogue ep{dwr, g.o, 0, nullptr, nullptr, 0, 0};
    WB_TRY(wb_tc_conv_gemm(b, 2, dy, x3, g.n, g.c, g.h, g.w, static_cast<int>(g.o), ep));
    return wb_conv3_weight_reorder(b, 2, dwr, dweight, static_cast<int>(g.o), static_cast<int>(g.c));
}

// dx[n][c][h][w] = transposed convolution of dy;  wt = weight as [c][flipped tap][o] (kind 1), dy3 = dy and its shifted
// copies, or dy alone (dy3[0] = dy3[2] = nullptr) for layers that pass wb_conv3_dgrad_needs_no_copies.
bool wb_conv3_dgrad_needs_no_copies(const WbConv3& g) { return wb_tc_conv_mode3_ok(g.o, g.h, g.w, g.c); }

int wb_conv3_dgrad(WbBackend* b, const WbConv3& g, const float* const dy3[3], const float* wt, float* dx) {
    const int64_t hw = g.h * g.w;
    tc::Epilogue ep{dx, hw, g.c * hw, nullptr, nullptr, 0, 0};
    const int mode = (dy3[0] == nullptr && dy3[2] == nullptr) ? 3 : 1;
    return wb_tc_conv_gemm(b, mode, wt, dy3, g.n, g.o, g.h, g.w, static_cast<int>(g.c), ep);
}

namespace {

struct Scratch {
    WbBackend* b;
    void* p[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t klass[4] = {0, 0, 0, 0};
    int used = 0;
    explicit Scratch(WbBackend* be) : b(be) {}
    ~Scratch() {
        for (int i = 0; i < used; ++i) wb_arena_free(b, p[i], klass[i]);
    }
    int get(int64_t floats, float** out) {
        WB_TRY(wb_arena_alloc(b, static_cast<size_t>(floats) * sizeof(float), &p[used], &klass[used]));
        *out = static_cast<float*>(p[used++]);
        return WB_OK;
    }
};

int check_args(const char* what, WbBackend* b, int64_t n, int64_t c, int64_t h, int64_t w, int64_t o, WbConv3* g) {
    WB_REQUIRE(b && n > 0 && c > 0 && h > 0 && w > 0 && o > 0, WB_ERR_INVALID, "%s: bad arguments", what);
    *g = WbConv3{n, c, h, w, o};
    if (!wb_conv3_eligible(*g)) {
        wb_set_error("%s: needs W %% 4 == 0, C %% 128 == 0 and O %% 32 == 0 (got C %lld, W %lld, O %lld); use im2col + matmul", what, (long long)c,
                     (long long)w, (long long)o);
        return WB_ERR_UNSUPPORTED;
    }
    return WB_OK;
}

}  // namespace

extern "C" int wb_conv3x3_fwd(WbBackend* b, const float* x, const float* weight, const float* bias, int64_t n, int64_t c, int64_t h, int64_t w,
                              int64_t o, float* y) {
    WbConv3 g;
    WB_TRY(check_args("wb_conv3x3_fwd", b, n, c, h, w, o, &g));
    WB_REQUIRE(x && weight && y, WB_ERR_INVALID, "wb_conv3x3_fwd: null pointer");
    WbProfileScope ps(b, "conv3x3_fwd");
    Scratch sc(b);
    float *left, *right, *wr;
    WB_TRY(sc.get(n * c * h * w, &left));
    WB_TRY(sc.get(n * c * h * w, &right));
    WB_TRY(sc.get(o * c * 9, &wr));
    WB_TRY(wb_conv3_shift_copies(b, x, n * c * h, static_cast<int>(w), left, right));
    WB_TRY(wb_conv3_weight_reorder(b, 0, weight, wr, static_cast<int>(o), static_cast<int>(c)));
    const float* x3[3] = {left, x, right};
    return wb_conv3_fwd(b, g, x3, wr, bias, y, nullptr);
}

extern "C" int wb_conv3x3_bwd(WbBackend* b, const float* x, const float* weight, const float* dy, int64_t n, int64_t c, int64_t h, int64_t w,
                              int64_t o, float* dx, float* dweight) {
    WbConv3 g;
    WB_TRY(check_args("wb_conv3x3_bwd", b, n, c, h, w, o, &g));
    WB_REQUIRE(x && weight && dy, WB_ERR_INVALID, "wb_conv3x3_bwd: null pointer");
    WbProfileScope ps(b, "conv3x3_bwd");
    if (dweight) {
        Scratch sc(b);
        float *left, *right, *dwr;
        WB_TRY(sc.get(n * c * h * w, &left));
        WB_TRY(sc.get(n * c * h * w, &right));
        WB_TRY(sc.get(o * c * 9, &dwr));
        WB_TRY(wb_conv3_shift_copies(b, x, n * c * h, static_cast<int>(w), left, right));
        const float* x3[3] = {left, x, right};
        WB_TRY(wb_conv3_wgrad(b, g, dy, x3, dwr, dweight));
    }
    if (dx) {
        Scratch sc(b);
        float *left = nullptr, *right = nullptr, *wt;
        WB_TRY(sc.get(o * c * 9, &wt));
        WB_TRY(wb_conv3_weight_reorder(b, 1, weight, wt, static_cast<int>(o), static_cast<int>(c)));
        if (!wb_conv3_dgrad_needs_no_copies(g)) {
            WB_TRY(sc.get(n * o * h * w, &left));
            WB_TRY(sc.get(n * o * h * w, &right));
            WB_TRY(wb_conv3_shift_copies(b, dy, n * o * h, static_cast<int>(w), left, right));
        }
        const float* d3[3] = {left, dy, right};
        WB_TRY(wb_conv3_dgrad(b, g, d3, wt, dx));
    }
    return WB_OK;
}
