// Backend::im2col and Backend::col2im (crates/weta-core/src/backend.rs:89-91).
//
// im2col is a pure gather: out[n][c*kh*kw + ki*kw + kj][oy*OW + ox] = x[n][c][oy*s - p + ki*d][ox*s - p + kj*d]
// or 0 outside the image (crates/weta-cpu/src/lib.rs:367-408), so results are bit-exact.  Threads run
// along the output's inner (oy, ox) index, which makes the stores coalesced and, for unit stride,
// the loads too.
// col2im is its adjoint.  The CPU loops (ki, kj) outermost and adds into the image
// (crates/weta-cpu/src/lib.rs:410-446); for one pixel that is a sum over (ki, kj) ascending, which the
// gather form below reproduces without atomics: same order, same roundings.
#include "common.h"

namespace {

constexpr int THREADS = 256;

struct GP {
    int64_t n, c, h, w, kh, kw, sh, sw, ph, pw, dh, dw, oh, ow;
    int64_t xs0, xs1, xs2, xs3, xoff;  // input strides (elements)
};

template <class T>
__global__ void __launch_bounds__(THREADS) im2col_kernel(T* __restrict__ out, const T* __restrict__ x, GP p, int64_t total) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (i >= total) return;
    int64_t l = p.oh * p.ow;
    int64_t col = i % l;
    int64_t r = i / l;
    int64_t kk = p.kh * p.kw;
    int64_t kidx = r % kk;
    int64_t nc = r / kk;
    int64_t ci = nc % p.c, n = nc / p.c;
    int64_t ki = kidx / p.kw, kj = kidx % p.kw;
    int64_t oy = col / p.ow, ox = col % p.ow;
    int64_t iy = oy * p.sh + ki * p.dh - p.ph;
    int64_t ix = ox * p.sw + kj * p.dw - p.pw;
    T v = T(0);
    if (iy >= 0 && iy < p.h && ix >= 0 && ix < p.w) v = x[p.xoff + n * p.xs0 + ci * p.xs1 + iy * p.xs2 + ix * p.xs3];
    out[i] = v;
}

// cols: contiguous [N, C*kh*kw, OH*OW] or strided (cs0, cs1, cs2).
template <class T>
__global__ void __launch_bounds__(THREADS) col2im_kernel(T* __restrict__ out, const T* __restrict__ cols, GP p, int64_t cs0,
                                                          int64_t cs1, int64_t cs2, int64_t coff, int64_t total) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (i >= total) return;
    int64_t ix = i % p.w;
    int64_t t = i / p.w;
    int64_t iy = t % p.h;
    t /= p.h;
    int64_t ci = t % p.c, n = t / p.c;
    T acc = T(0);
    const T* base = cols + coff + n * cs0 + ci * p.kh * p.kw * cs1;
    for (int64_t ki = 0; ki < p.kh; ++ki) {
        int64_t ny = iy + p.ph - ki * p.dh;
        if (ny < 0 || ny % p.sh != 0) continue;
        int64_t oy = ny / p.sh;
        if (oy >= p.oh) continue;
        for (int64_t kj = 0; kj < p.kw; ++kj) {
            int64_t nx = ix + p.pw - kj * p.dw;
            if (nx < 0 || nx % p.sw != 0) continue;
            int64_t ox = nx / p.sw;
            if (ox >= p.ow) continue;
            acc = acc + base[(ki * p.kw + kj) * cs1 + (oy * p.ow + ox) * cs2];
        }
    }
    out[i] = acc;
}

// ---- 3x3, stride 1, padding 1, dilation 1 on contiguous f32 images (every convolution of the named models) ----
// Same gather, V consecutive output columns per thread (V = 4, 2 or 1: the largest that divides the width) and 32-bit
// index arithmetic by multiply and shift: one vector store per thread, the nine shifted reads of each pixel come
// from L1/L2.  (MNIST's 14-wide second layer ran the generic 64-bit kernels at 31 us per call; with V = 2 the gather
// takes 8 us and its adjoint 5.5 us.)
template <int V>
struct VecOf;
template <> struct VecOf<4> { using type = float4; };
template <> struct VecOf<2> { using type = float2; };
template <> struct VecOf<1> { using type = float; };

template <int V>
__global__ void __launch_bounds__(THREADS) im2col3_kernel(float* __restrict__ out, const float* __restrict__ x, int h, int w,
                                                           uint32_t groups, FastDiv div_wq, FastDiv div_h, FastDiv div_9) {
    wb_pdl_enter();
    using Vec = typename VecOf<V>::type;
    uint32_t i = blockIdx.x * THREADS + threadIdx.x;
    if (i >= groups) return;
    const uint32_t wq = static_cast<uint32_t>(w) / V;
    uint32_t t = div_wq.div(i);
    const uint32_t xq = i - t * wq;
    const uint32_t t2 = div_h.div(t);
    const uint32_t y = t - t2 * static_cast<uint32_t>(h);
    t = t2;
    const uint32_t nc = div_9.div(t), k9 = t - nc * 9u;
    int ki = static_cast<int>(k9 / 3u), kj = static_cast<int>(k9 % 3u);
    int iy = static_cast<int>(y) + ki - 1;
    int ix0 = static_cast<int>(xq * V) + kj - 1;
    float v[V];
#pragma unroll
    for (int k = 0; k < V; ++k) v[k] = 0.f;
    if (iy >= 0 && iy < h) {
        const float* row = x + (static_cast<int64_t>(nc) * h + iy) * w;
        if (V > 1 && kj == 1) {  // the unshifted tap: one aligned vector load
            const Vec q = *reinterpret_cast<const Vec*>(row + ix0);
            const float* qf = reinterpret_cast<const float*>(&q);
#pragma unroll
            for (int k = 0; k < V; ++k) v[k] = qf[k];
        } else {
#pragma unroll
            for (int k = 0; k < V; ++k) {
                int ix = ix0 + k;
                if (ix >= 0 && ix < w) v[k] = row[ix];
            }
        }
    }
    Vec r;
    float* rf = reinterpret_cast<float*>(&r);
#pragma unroll
    for (int k = 0; k < V; ++k) rf[k] = v[k];
    *reinterpret_cast<Vec*>(out + static_cast<int64_t>(i) * V) = r;
}

// Adjoint: each thread owns V consecutive pixels of one (n, c) plane and adds its (up to) nine
// column entries in (ki, kj) order, the order the CPU backend's scatter reaches them.
template <int V>
__global__ void __launch_bounds__(THREADS) col2im3_kernel(float* __restrict__ out, const float* __restrict__ cols, int h, int w,
                                                           uint32_t groups, FastDiv div_wq, FastDiv div_h) {
    wb_pdl_enter();
    using Vec = typename VecOf<V>::type;
    uint32_t i = blockIdx.x * THREADS + threadIdx.x;
    if (i >= groups) return;
    const uint32_t wq = static_cast<uint32_t>(w) / V;
    uint32_t t = div_wq.div(i);
    const uint32_t xq = i - t * wq;
    const uint32_t nc = div_h.div(t), y = t - nc * static_cast<uint32_t>(h);
    const int64_t l = static_cast<int64_t>(h) * w;
    const float* base = cols + static_cast<int64_t>(nc) * 9 * l;
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = 0.f;
#pragma unroll
    for (int ki = 0; ki < 3; ++ki) {
        int oy = static_cast<int>(y) + 1 - ki;
        if (oy < 0 || oy >= h) continue;
#pragma unroll
        for (int kj = 0; kj < 3; ++kj) {
            const float* row = base + (ki * 3 + kj) * l + static_cast<int64_t>(oy) * w;
            int ox0 = static_cast<int>(xq * V) + 1 - kj;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                int ox = ox0 + k;
                if (ox >= 0 && ox < w) acc[k] = acc[k] + row[ox];
            }
        }
    }
    Vec r;
    float* rf = reinterpret_cast<float*>(&r);
#pragma unroll
    for (int k = 0; k < V; ++k) rf[k] = acc[k];
    *reinterpret_cast<Vec*>(out + static_cast<int64_t>(i) * V) = r;
}

inline bool same_conv3(const WbConvParams& p) {
    return p.kh == 3 && p.kw == 3 && p.sh == 1 && p.sw == 1 && p.ph == 1 && p.pw == 1 && p.dh == 1 && p.dw == 1;
}

inline int64_t out_size1(int64_t x, int64_t k, int64_t s, int64_t p, int64_t d) {  // crates/weta-core/src/ops.rs:136-149
    int64_t span = d * (k - 1) + 1;
    if (x + 2 * p < span) return 0;
    return (x + 2 * p - span) / s + 1;
}

GP make_gp(const WbConvParams& cp, int64_t n, int64_t c, int64_t h, int64_t w) {
    GP p{};
    p.n = n; p.c = c; p.h = h; p.w = w;
    p.kh = cp.kh; p.kw = cp.kw; p.sh = cp.sh; p.sw = cp.sw; p.ph = cp.ph; p.pw = cp.pw; p.dh = cp.dh; p.dw = cp.dw;
    p.oh = out_size1(h, cp.kh, cp.sh, cp.ph, cp.dh);
    p.ow = out_size1(w, cp.kw, cp.sw, cp.pw, cp.dw);
    return p;
}

bool params_ok(const WbConvParams* p) { return p && p->kh > 0 && p->kw > 0 && p->sh > 0 && p->sw > 0 && p->dh > 0 && p->dw > 0 && p->ph >= 0 && p->pw >= 0; }

}  // namespace

extern "C" int wb_im2col_into(WbBackend* b, const WbView* x, const WbConvParams* cp, void* out) {
    WB_REQUIRE(b && x && out, WB_ERR_INVALID, "wb_im2col: null pointer");
    WB_REQUIRE(params_ok(cp), WB_ERR_INVALID, "im2col: kernel, stride and dilation must be positive");
    WB_REQUIRE(x->ndim == 4, WB_ERR_INVALID, "im2col: expected [N, C, H, W], got %d dims", x->ndim);
    GP p = make_gp(*cp, x->shape[0], x->shape[1], x->shape[2], x->shape[3]);
    p.xs0 = x->stride[0]; p.xs1 = x->stride[1]; p.xs2 = x->stride[2]; p.xs3 = x->stride[3]; p.xoff = x->offset;
    int64_t total = p.n * p.c * p.kh * p.kw * p.oh * p.ow;
    if (total == 0) return WB_OK;
    WbProfileScope ps(b, "im2col");
    if (same_conv3(*cp) && x->dtype == WB_F32 && wb_is_contiguous(*x) && total < (int64_t(1) << 31)) {
        const float* xp = static_cast<const float*>(x->data) + x->offset;
        const uintptr_t bits = reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(xp);
        const int v = (p.w % 4 == 0 && (bits & 15) == 0) ? 4 : ((p.w % 2 == 0 && (bits & 7) == 0) ? 2 : 1);
        const int64_t groups = total / v;
        const unsigned grid3 = static_cast<unsigned>((groups + THREADS - 1) / THREADS);
        const FastDiv dwq(static_cast<uint32_t>(p.w / v)), dh(static_cast<uint32_t>(p.h)), d9(9u);
        float* op = static_cast<float*>(out);
        if (v == 4) wb_launch_pdl(im2col3_kernel<4>, dim3(grid3), dim3(THREADS), 0, b->stream, op, xp, static_cast<int>(p.h), static_cast<int>(p.w), static_cast<uint32_t>(groups), dwq, dh, d9);
        else if (v == 2) wb_launch_pdl(im2col3_kernel<2>, dim3(grid3), dim3(THREADS), 0, b->stream, op, xp, static_cast<int>(p.h), static_cast<int>(p.w), static_cast<uint32_t>(groups), dwq, dh, d9);
        else wb_launch_pdl(im2col3_kernel<1>, dim3(grid3), dim3(THREADS), 0, b->stream, op, xp, static_cast<int>(p.h), static_cast<int>(p.w), static_cast<uint32_t>(groups), dwq, dh, d9);
        WB_LAUNCH_OK(b);
        return WB_OK;
    }
    unsigned grid = static_cast<unsigned>((total + THREADS - 1) / THREADS);
    switch (x->dtype) {
        case WB_F32: im2col_kernel<float><<<grid, THREADS, 0, b->stream>>>(static_cast<float*>(out), static_cast<const float*>(x->data), p, total); break;
        case WB_F64: im2col_kernel<double><<<grid, THREADS, 0, b->stream>>>(static_cast<double*>(out), static_cast<const double*>(x->data), p, total); break;
        case WB_I64: im2col_kernel<int64_t><<<grid, THREADS, 0, b->stream>>>(static_cast<int64_t*>(out), static_cast<const int64_t*>(x->data), p, total); break;
        default: wb_set_error("im2col: unknown dtype %d", x->dtype); return WB_ERR_INVALID;
    }
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_im2col(WbBackend* b, const WbView* x, const WbConvParams* cp, WbStorage** out) {
    WB_REQUIRE(b && x && out && params_ok(cp), WB_ERR_INVALID, "wb_im2col: bad arguments");
    WB_REQUIRE(x->ndim == 4, WB_ERR_INVALID, "im2col: expected [N, C, H, W], got %d dims", x->ndim);
    GP p = make_gp(*cp, x->shape[0], x->shape[1], x->shape[2], x->shape[3]);
    WB_TRY(wb_new_storage(b, p.n * p.c * p.kh * p.kw * p.oh * p.ow, x->dtype, out));
    int s = wb_im2col_into(b, x, cp, (*out)->ptr);
    if (s != WB_OK) { wb_free(b, *out); *out = nullptr; }
    return s;
}

extern "C" int wb_col2im_into(WbBackend* b, const WbView* cols, const WbConvParams* cp, int64_t c, int64_t h, int64_t w, void* out) {
    WB_REQUIRE(b && cols && out, WB_ERR_INVALID, "wb_col2im: null pointer");
    WB_REQUIRE(params_ok(cp), WB_ERR_INVALID, "col2im: kernel, stride and dilation must be positive");
    WB_REQUIRE(cols->ndim == 3, WB_ERR_INVALID, "col2im: expected [N, C*kh*kw, L], got %d dims", cols->ndim);
    WB_REQUIRE(cols->dtype != WB_I64, WB_ERR_UNSUPPORTED, "col2im: unsupported dtype i64");
    GP p = make_gp(*cp, cols->shape[0], c, h, w);
    WB_REQUIRE(cols->shape[1] == c * p.kh * p.kw && cols->shape[2] == p.oh * p.ow, WB_ERR_INVALID,
               "col2im: columns [%lld, %lld] do not match image [%lld, %lld, %lld]", (long long)cols->shape[1],
               (long long)cols->shape[2], (long long)c, (long long)h, (long long)w);
    int64_t total = p.n * c * h * w;
    if (total == 0) return WB_OK;
    WbProfileScope ps(b, "col2im");
    if (same_conv3(*cp) && cols->dtype == WB_F32 && wb_is_contiguous(*cols) && total < (int64_t(1) << 31) && total * 9 < (int64_t(1) << 40)) {
        const int v = (w % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) ? 4 : ((w % 2 == 0 && (reinterpret_cast<uintptr_t>(out) & 7) == 0) ? 2 : 1);
        const int64_t groups = total / v;
        const unsigned grid3 = static_cast<unsigned>((groups + THREADS - 1) / THREADS);
        const FastDiv dwq(static_cast<uint32_t>(w / v)), dh(static_cast<uint32_t>(h));
        float* op = static_cast<float*>(out);
        const float* cp3 = static_cast<const float*>(cols->data) + cols->offset;
        if (v == 4) wb_launch_pdl(col2im3_kernel<4>, dim3(grid3), dim3(THREADS), 0, b->stream, op, cp3, static_cast<int>(h), static_cast<int>(w), static_cast<uint32_t>(groups), dwq, dh);
        else if (v == 2) wb_launch_pdl(col2im3_kernel<2>, dim3(grid3), dim3(THREADS), 0, b->stream, op, cp3, static_cast<int>(h), static_cast<int>(w), static_cast<uint32_t>(groups), dwq, dh);
        else wb_launch_pdl(col2im3_kernel<1>, dim3(grid3), dim3(THREADS), 0, b->stream, op, cp3, static_cast<int>(h), static_cast<int>(w), static_cast<uint32_t>(groups), dwq, dh);
        WB_LAUNCH_OK(b);
        return WB_OK;
    }
    unsigned grid = static_cast<unsigned>((total + THREADS - 1) / THREADS);
    if (cols->dtype == WB_F32)
        col2im_kernel<float><<<grid, THREADS, 0, b->stream>>>(static_cast<float*>(out), static_cast<const float*>(cols->data), p,
                                                             cols->stride[0], cols->stride[1], cols->stride[2], cols->offset, total);
    else
        col2im_kernel<double><<<grid, THREADS, 0, b->stream>>>(static_cast<double*>(out), static_cast<const double*>(cols->data), p,
                                                              cols->stride[0], cols->stride[1], cols->stride[2], cols->offset, total);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

extern "C" int wb_col2im(WbBackend* b, const WbView* cols, const WbConvParams* cp, int64_t c, int64_t h, int64_t w, WbStorage** out) {
    WB_REQUIRE(b && cols && out, WB_ERR_INVALID, "wb_col2im: null pointer");
    WB_REQUIRE(cols->ndim == 3, WB_ERR_INVALID, "col2im: expected [N, C*kh*kw, L], got %d dims", cols->ndim);
    WB_TRY(wb_new_storage(b, cols->shape[0] * c * h * w, cols->dtype, out));
    int s = wb_col2im_into(b, cols, cp, c, h, w, (*out)->ptr);
    if (s != WB_OK) { wb_free(b, *out); *out = nullptr; }
    return s;
}
