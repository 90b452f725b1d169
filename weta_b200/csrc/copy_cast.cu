// Backend::cast and Backend::copy_strided (crates/weta-core/src/backend.rs:79, 92).
// cast with equal dtypes is `contiguous()` (crates/weta-cuda/src/lib.rs:325-327).  copy_strided
// writes into a strided destination: slice assignment, cat, in-place updates
// (crates/weta-tensor/src/tensor.rs:766-777).
#include "elementwise.cuh"

namespace {

// Rust `as` casts (crates/weta-cpu/src/lib.rs:552-565): float -> i64 truncates, saturates, NaN -> 0.
template <class TI, class TO> struct Cast {
    __device__ TO operator()(TI v) const {
        if constexpr (std::is_same<TO, int64_t>::value && !std::is_same<TI, int64_t>::value) {
            if (v != v) return 0;
            if (v >= TI(9223372036854775808.0)) return INT64_MAX;
            if (v <= TI(-9223372036854775808.0)) return INT64_MIN;
            return static_cast<int64_t>(v);
        } else {
            return static_cast<TO>(v);
        }
    }
};

template <class TI, class TO>
int cast_typed(WbBackend* be, const WbView* x, void* out) {
    const WbView* ops[1] = {x};
    WbIterPlan plan;
    wb_make_plan(ops, 1, &plan);
    return ew::launch<TI, TO, 1>(be, static_cast<TO*>(out), static_cast<const TI*>(x->data),
                                 static_cast<const TI*>(nullptr), plan, Cast<TI, TO>{});
}

// dst[dst_off(i)] = src[src_off(i)] for every row-major index i of the shared shape.
template <class T, class IdxT>
__global__ void __launch_bounds__(256) copy_strided_kernel(T* __restrict__ dst, const T* __restrict__ src, ew::Plan p) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= p.n) return;
    int64_t os = p.off[0], od = p.off[1];
    IdxT rem = static_cast<IdxT>(i);
#pragma unroll 1
    for (int d = p.nd - 1; d >= 0; --d) {
        IdxT sz = static_cast<IdxT>(p.size[d]);
        IdxT q = rem / sz;
        IdxT c = rem - q * sz;
        rem = q;
        os += static_cast<int64_t>(c) * p.st[0][d];
        od += static_cast<int64_t>(c) * p.st[1][d];
    }
    dst[od] = src[os];
}

template <class T>
int copy_typed(WbBackend* be, const WbView* src, const WbView* dst) {
    const WbView* ops[2] = {src, dst};
    WbIterPlan wp;
    wb_make_plan(ops, 2, &wp);
    if (wp.n == 0) return WB_OK;
    // Contiguous destination: the element-wise machinery (vector / tile paths) applies directly.
    if (wb_is_contiguous(*dst)) {
        WbIterPlan sp;
        const WbView* one[1] = {src};
        wb_make_plan(one, 1, &sp);
        return ew::launch<T, T, 1>(be, static_cast<T*>(dst->data) + dst->offset, static_cast<const T*>(src->data),
                                   static_cast<const T*>(nullptr), sp, Cast<T, T>{});
    }
    ew::Plan p;
    p.nd = wp.nd;
    p.n = wp.n;
    for (int d = 0; d < WB_MAX_DIMS; ++d) {
        p.size[d] = wp.size[d];
        for (int o = 0; o < WB_PLAN_MAX_OPS; ++o) p.st[o][d] = wp.st[o][d];
    }
    for (int o = 0; o < WB_PLAN_MAX_OPS; ++o) p.off[o] = wp.off[o];
    unsigned grid = static_cast<unsigned>((wp.n + 255) / 256);
    if (wp.n < (int64_t(1) << 31))
        copy_strided_kernel<T, uint32_t><<<grid, 256, 0, be->stream>>>(static_cast<T*>(dst->data), static_cast<const T*>(src->data), p);
    else
        copy_strided_kernel<T, int64_t><<<grid, 256, 0, be->stream>>>(static_cast<T*>(dst->data), static_cast<const T*>(src->data), p);
    WB_LAUNCH_OK(be);
    return WB_OK;
}

}  // namespace

extern "C" int wb_cast_into(WbBackend* b, const WbView* x, int dtype, void* out) {
    WB_REQUIRE(b && x && out, WB_ERR_INVALID, "wb_cast: null pointer");
    WB_REQUIRE(dtype >= 0 && dtype <= 2 && x->dtype >= 0 && x->dtype <= 2, WB_ERR_INVALID, "wb_cast: unknown dtype");
    WbProfileScope ps(b, "cast");
    switch (x->dtype * 3 + dtype) {
        case 0: return cast_typed<float, float>(b, x, out);
        case 1: return cast_typed<float, double>(b, x, out);
        case 2: return cast_typed<float, int64_t>(b, x, out);
        case 3: return cast_typed<double, float>(b, x, out);
        case 4: return cast_typed<double, double>(b, x, out);
        case 5: return cast_typed<double, int64_t>(b, x, out);
        case 6: return cast_typed<int64_t, float>(b, x, out);
        case 7: return cast_typed<int64_t, double>(b, x, out);
        case 8: return cast_typed<int64_t, int64_t>(b, x, out);
    }
    return WB_ERR_INVALID;
}

extern "C" int wb_cast(WbBackend* b, const WbView* x, int dtype, WbStorage** out) {
    WB_REQUIRE(b && x && out, WB_ERR_INVALID, "wb_cast: null pointer");
    WB_TRY(wb_new_storage(b, wb_numel(*x), dtype, out));
    int s = wb_cast_into(b, x, dtype, (*out)->ptr);
    if (s != WB_OK) { wb_free(b, *out); *out = nullptr; }
    return s;
}

extern "C" int wb_copy_strided(WbBackend* b, const WbView* src, const WbView* dst) {
    WB_REQUIRE(b && src && dst, WB_ERR_INVALID, "wb_copy_strided: null pointer");
    WB_REQUIRE(src->dtype == dst->dtype, WB_ERR_INVALID, "copy: dtype mismatch %d -> %d", src->dtype, dst->dtype);
    WB_REQUIRE(src->ndim == dst->ndim, WB_ERR_INVALID, "copy: source and destination must share one shape");
    for (int i = 0; i < src->ndim; ++i)
        WB_REQUIRE(src->shape[i] == dst->shape[i], WB_ERR_INVALID, "copy: source and destination must share one shape");
    WbProfileScope ps(b, "copy_strided");
    switch (src->dtype) {
        case WB_F32: return copy_typed<float>(b, src, dst);
        case WB_F64: return copy_typed<double>(b, src, dst);
        case WB_I64: return copy_typed<int64_t>(b, src, dst);
    }
    return WB_ERR_INVALID;
}
