// Backend::unary for f32 / f64 / i64 (crates/weta-core/src/backend.rs:81).
// Semantics follow the CPU backend op by op (crates/weta-cpu/src/lib.rs:133-203): scalar
// parameters are rounded to the tensor dtype once, `x*m + a` is two roundings (this file is
// compiled with -fmad=false), max/min let a NaN in the tensor win (crates/weta-core/src/dtype.rs:136-149).
#include "elementwise.cuh"

namespace {

template <class T> struct Neg { __device__ T operator()(T v) const { return -v; } };
template <class T> struct Exp { __device__ T operator()(T v) const { return exp(v); } };
template <class T> struct Log { __device__ T operator()(T v) const { return log(v); } };
template <class T> struct Sqrt { __device__ T operator()(T v) const { return sqrt(v); } };
template <class T> struct Abs { __device__ T operator()(T v) const { return fabs(v); } };
template <class T> struct Sign { __device__ T operator()(T v) const { return v > T(0) ? T(1) : (v < T(0) ? T(-1) : T(0)); } };
template <class T> struct Relu { __device__ T operator()(T v) const { return v > T(0) ? v : T(0); } };
template <class T> struct Step { __device__ T operator()(T v) const { return v > T(0) ? T(1) : T(0); } };
template <class T> struct Tanh { __device__ T operator()(T v) const { return tanh(v); } };
template <class T> struct Sigmoid {
    __device__ T operator()(T v) const {
        if (v >= T(0)) return T(1) / (T(1) + exp(-v));
        T e = exp(v);
        return e / (T(1) + e);
    }
};
template <class T> struct Erf { __device__ T operator()(T v) const { return erf(v); } };
template <class T> struct Sin { __device__ T operator()(T v) const { return sin(v); } };
template <class T> struct Cos { __device__ T operator()(T v) const { return cos(v); } };
template <class T> struct Recip { __device__ T operator()(T v) const { return T(1) / v; } };
template <class T> struct Affine { T m, a; __device__ T operator()(T v) const { return v * m + a; } };
template <class T> struct Powf { T e; __device__ T operator()(T v) const { return pow(v, e); } };
template <class T> struct GtScalar { T s; __device__ T operator()(T v) const { return v > s ? T(1) : T(0); } };
template <class T> struct MaxScalar { T s; __device__ T operator()(T v) const { return (v >= s || v != v) ? v : s; } };
template <class T> struct MinScalar { T s; __device__ T operator()(T v) const { return (v <= s || v != v) ? v : s; } };

// Rust `as i64` from f64: truncate, saturate, NaN -> 0.
__host__ __device__ inline int64_t f64_to_i64(double v) {
    if (v != v) return 0;
    if (v >= 9223372036854775808.0) return INT64_MAX;
    if (v <= -9223372036854775808.0) return INT64_MIN;
    return static_cast<int64_t>(v);
}

using I = int64_t;
struct INeg { __device__ I operator()(I v) const { return static_cast<I>(0ull - static_cast<uint64_t>(v)); } };
struct IAbs { __device__ I operator()(I v) const { return v < 0 ? static_cast<I>(0ull - static_cast<uint64_t>(v)) : v; } };
struct ISign { __device__ I operator()(I v) const { return static_cast<I>((v > 0) - (v < 0)); } };
struct IRelu { __device__ I operator()(I v) const { return v > 0 ? v : 0; } };
struct IStep { __device__ I operator()(I v) const { return v > 0 ? 1 : 0; } };
struct IAffine { double m, a; __device__ I operator()(I v) const { return f64_to_i64(static_cast<double>(v) * m + a); } };
struct IGt { double s; __device__ I operator()(I v) const { return static_cast<double>(v) > s ? 1 : 0; } };
struct IMax { I s; __device__ I operator()(I v) const { return v > s ? v : s; } };
struct IMin { I s; __device__ I operator()(I v) const { return v < s ? v : s; } };

template <class T>
int unary_float(WbBackend* be, int op, double p1, double p2, const WbView* x, T* out) {
    const WbView* ops[1] = {x};
    WbIterPlan plan;
    wb_make_plan(ops, 1, &plan);
    const T* in = static_cast<const T*>(x->data);
#define GO(F) return ew::launch<T, T, 1>(be, out, in, static_cast<const T*>(nullptr), plan, F)
    switch (op) {
        case WB_NEG: GO(Neg<T>{});
        case WB_EXP: GO(Exp<T>{});
        case WB_LOG: GO(Log<T>{});
        case WB_SQRT: GO(Sqrt<T>{});
        case WB_ABS: GO(Abs<T>{});
        case WB_SIGN: GO(Sign<T>{});
        case WB_RELU: GO(Relu<T>{});
        case WB_STEP: GO(Step<T>{});
        case WB_TANH: GO(Tanh<T>{});
        case WB_SIGMOID: GO(Sigmoid<T>{});
        case WB_ERF: GO(Erf<T>{});
        case WB_SIN: GO(Sin<T>{});
        case WB_COS: GO(Cos<T>{});
        case WB_RECIP: GO(Recip<T>{});
        case WB_AFFINE: GO((Affine<T>{static_cast<T>(p1), static_cast<T>(p2)}));
        case WB_POWF: GO((Powf<T>{static_cast<T>(p1)}));
        case WB_GT_SCALAR: GO((GtScalar<T>{static_cast<T>(p1)}));
        case WB_MAX_SCALAR: GO((MaxScalar<T>{static_cast<T>(p1)}));
        case WB_MIN_SCALAR: GO((MinScalar<T>{static_cast<T>(p1)}));
    }
#undef GO
    wb_set_error("unary: unknown op code %d", op);
    return WB_ERR_INVALID;
}

int unary_int(WbBackend* be, int op, double p1, double p2, const WbView* x, I* out) {
    const WbView* ops[1] = {x};
    WbIterPlan plan;
    wb_make_plan(ops, 1, &plan);
    const I* in = static_cast<const I*>(x->data);
#define GO(F) return ew::launch<I, I, 1>(be, out, in, static_cast<const I*>(nullptr), plan, F)
    switch (op) {
        case WB_NEG: GO(INeg{});
        case WB_ABS: GO(IAbs{});
        case WB_SIGN: GO(ISign{});
        case WB_RELU: GO(IRelu{});
        case WB_STEP: GO(IStep{});
        case WB_AFFINE: GO((IAffine{p1, p2}));
        case WB_GT_SCALAR: GO((IGt{p1}));
        case WB_MAX_SCALAR: GO((IMax{f64_to_i64(p1)}));
        case WB_MIN_SCALAR: GO((IMin{f64_to_i64(p1)}));
    }
#undef GO
    static const char* names[] = {"neg", "exp", "log", "sqrt", "abs", "sign", "relu", "step", "tanh", "sigmoid", "erf",
                                  "sin", "cos", "reciprocal", "affine", "pow", "gt", "clamp_min", "clamp_max"};
    if (op >= 0 && op <= 18) {
        wb_set_error("%s: not supported for i64 tensors", names[op]);  // crates/weta-cpu/src/lib.rs:201
        return WB_ERR_UNSUPPORTED;
    }
    wb_set_error("unary: unknown op code %d", op);
    return WB_ERR_INVALID;
}

}  // namespace

extern "C" int wb_unary_into(WbBackend* b, int op, double p1, double p2, const WbView* x, void* out) {
    WB_REQUIRE(b && x && out, WB_ERR_INVALID, "wb_unary: null pointer");
    WB_REQUIRE(x->ndim >= 0 && x->ndim <= WB_MAX_DIMS, WB_ERR_INVALID, "wb_unary: at most 8 dims are supported");
    WbProfileScope ps(b, "unary");
    switch (x->dtype) {
        case WB_F32: return unary_float<float>(b, op, p1, p2, x, static_cast<float*>(out));
        case WB_F64: return unary_float<double>(b, op, p1, p2, x, static_cast<double*>(out));
        case WB_I64: return unary_int(b, op, p1, p2, x, static_cast<int64_t*>(out));
    }
    wb_set_error("wb_unary: unknown dtype %d", x->dtype);
    return WB_ERR_INVALID;
}

extern "C" int wb_unary(WbBackend* b, int op, double p1, double p2, const WbView* x, WbStorage** out) {
    WB_REQUIRE(b && x && out, WB_ERR_INVALID, "wb_unary: null pointer");
    WB_TRY(wb_new_storage(b, wb_numel(*x), x->dtype, out));
    int s = wb_unary_into(b, op, p1, p2, x, (*out)->ptr);
    if (s != WB_OK) { wb_free(b, *out); *out = nullptr; }
    return s;
}
