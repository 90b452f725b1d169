// Backend::binary for f32 / f64 / i64 (crates/weta-core/src/backend.rs:83).
// Operands arrive already broadcast to one shape, with stride 0 on stretched dims
// (crates/weta-tensor/src/tensor.rs:396-406).  Semantics follow crates/weta-cpu/src/lib.rs:205-241:
// comparisons give 1/0 in the input dtype, max/min let a NaN on the left win, i64 Div is Euclidean.
#include "elementwise.cuh"

namespace {

template <class T> struct Add { __device__ T operator()(T x, T y) const { return x + y; } };
template <class T> struct Sub { __device__ T operator()(T x, T y) const { return x - y; } };
template <class T> struct Mul { __device__ T operator()(T x, T y) const { return x * y; } };
template <class T> struct Div { __device__ T operator()(T x, T y) const { return x / y; } };
template <class T> struct Pow { __device__ T operator()(T x, T y) const { return pow(x, y); } };
template <class T> struct Maximum { __device__ T operator()(T x, T y) const { return (x >= y || x != x) ? x : y; } };
template <class T> struct Minimum { __device__ T operator()(T x, T y) const { return (x <= y || x != x) ? x : y; } };
template <class T> struct Eq { __device__ T operator()(T x, T y) const { return x == y ? T(1) : T(0); } };
template <class T> struct Ne { __device__ T operator()(T x, T y) const { return x != y ? T(1) : T(0); } };
template <class T> struct Lt { __device__ T operator()(T x, T y) const { return x < y ? T(1) : T(0); } };
template <class T> struct Le { __device__ T operator()(T x, T y) const { return x <= y ? T(1) : T(0); } };
template <class T> struct Gt { __device__ T operator()(T x, T y) const { return x > y ? T(1) : T(0); } };
template <class T> struct Ge { __device__ T operator()(T x, T y) const { return x >= y ? T(1) : T(0); } };

using I = int64_t;
using U = uint64_t;
struct IAdd { __device__ I operator()(I x, I y) const { return static_cast<I>(U(x) + U(y)); } };
struct ISub { __device__ I operator()(I x, I y) const { return static_cast<I>(U(x) - U(y)); } };
struct IMul { __device__ I operator()(I x, I y) const { return static_cast<I>(U(x) * U(y)); } };
struct IDiv {  // i64::div_euclid; the reference panics on a zero divisor, here the result is 0
    __device__ I operator()(I x, I y) const {
        if (y == 0) return 0;
        if (y == -1) return static_cast<I>(0ull - U(x));
        I q = x / y;
        if (x % y < 0) return y > 0 ? q - 1 : q + 1;
        return q;
    }
};
struct IPow {  // i64::pow(y as u32), wrapping
    __device__ I operator()(I x, I y) const {
        uint32_t e = static_cast<uint32_t>(y);
        U base = U(x), acc = 1;
        while (e) {
            if (e & 1) acc *= base;
            base *= base;
            e >>= 1;
        }
        return static_cast<I>(acc);
    }
};
struct IMaximum { __device__ I operator()(I x, I y) const { return x > y ? x : y; } };
struct IMinimum { __device__ I operator()(I x, I y) const { return x < y ? x : y; } };

template <class T>
int binary_any(WbBackend* be, int op, const WbView* a, const WbView* b, T* out) {
    const WbView* ops[2] = {a, b};
    WbIterPlan plan;
    wb_make_plan(ops, 2, &plan);
    const T* pa = static_cast<const T*>(a->data);
    const T* pb = static_cast<const T*>(b->data);
    constexpr bool is_int = std::is_same<T, int64_t>::value;
#define GO(F) return ew::launch<T, T, 2>(be, out, pa, pb, plan, F)
    if constexpr (is_int) {
        switch (op) {
            case WB_ADD: GO(IAdd{});
            case WB_SUB: GO(ISub{});
            case WB_MUL: GO(IMul{});
            case WB_DIV: GO(IDiv{});
            case WB_POW: GO(IPow{});
            case WB_MAXIMUM: GO(IMaximum{});
            case WB_MINIMUM: GO(IMinimum{});
        }
    } else {
        switch (op) {
            case WB_ADD: GO(Add<T>{});
            case WB_SUB: GO(Sub<T>{});
            case WB_MUL: GO(Mul<T>{});
            case WB_DIV: GO(Div<T>{});
            case WB_POW: GO(Pow<T>{});
            case WB_MAXIMUM: GO(Maximum<T>{});
            case WB_MINIMUM: GO(Minimum<T>{});
        }
    }
    switch (op) {
        case WB_EQ: GO(Eq<T>{});
        case WB_NE: GO(Ne<T>{});
        case WB_LT: GO(Lt<T>{});
        case WB_LE: GO(Le<T>{});
        case WB_GT: GO(Gt<T>{});
        case WB_GE: GO(Ge<T>{});
    }
#undef GO
    wb_set_error("binary: unknown op code %d", op);
    return WB_ERR_INVALID;
}

}  // namespace

extern "C" int wb_binary_into(WbBackend* b, int op, const WbView* a, const WbView* bb, void* out) {
    WB_REQUIRE(b && a && bb && out, WB_ERR_INVALID, "wb_binary: null pointer");
    WB_REQUIRE(a->dtype == bb->dtype, WB_ERR_INVALID, "binary: dtype mismatch %d and %d", a->dtype, bb->dtype);
    WB_REQUIRE(a->ndim == bb->ndim && a->ndim <= WB_MAX_DIMS, WB_ERR_INVALID, "binary: operands must share one shape");
    for (int i = 0; i < a->ndim; ++i)
        WB_REQUIRE(a->shape[i] == bb->shape[i], WB_ERR_INVALID, "binary: operands must share one shape");
    WbProfileScope ps(b, "binary");
    switch (a->dtype) {
        case WB_F32: return binary_any<float>(b, op, a, bb, static_cast<float*>(out));
        case WB_F64: return binary_any<double>(b, op, a, bb, static_cast<double*>(out));
        case WB_I64: return binary_any<int64_t>(b, op, a, bb, static_cast<int64_t*>(out));
    }
    wb_set_error("wb_binary: unknown dtype %d", a->dtype);
    return WB_ERR_INVALID;
}

extern "C" int wb_binary(WbBackend* b, int op, const WbView* a, const WbView* bb, WbStorage** out) {
    WB_REQUIRE(b && a && bb && out, WB_ERR_INVALID, "wb_binary: null pointer");
    WB_TRY(wb_new_storage(b, wb_numel(*a), a->dtype, out));
    int s = wb_binary_into(b, op, a, bb, (*out)->ptr);
    if (s != WB_OK) { wb_free(b, *out); *out = nullptr; }
    return s;
}
