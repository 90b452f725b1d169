// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// A CPU restatement of weta's reference backend (crates/weta-cpu/src/lib.rs) plus the
// counter RNG (crates/weta-core/src/ops.rs:164-189).  It exists so the CUDA backend can be
// checked against the arithmetic weta-cpu performs: same traversal order, same rounding
// points, same tie / NaN rules.  Only the tests, the smoke check and the CPU-baseline leg of
// the benchmark load this library; the product library never does.
//
// Build: g++ -O3 -mavx2 -ffp-contract=off -fopenmp -shared -fPIC (see oracle/Makefile).
// `-ffp-contract=off` matters: Rust never fuses a*b+c into an FMA, GCC does by default.
//
// Parity pin: every known answer in the reference's own unit tests and the PyTorch f64
// fixture (crates/weta/tests/fixtures/reference.safetensors) are replayed against this file
// by tests/test_oracle_*.py.  The RNG streams have no literal vectors in the reference, so
// their bit patterns are pinned only by the algorithm text ("RNG literal parity unpinned").
//
// The GEMM of weta-cpu lives in the third-party crate `gemm` 0.17.1 (not vendored); its
// summation order is unspecified, so matmul here is a plain k-ascending accumulation in the
// storage dtype and matmul parity is tolerance based.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>
#include <algorithm>
#include <omp.h>

extern "C" {

// Same field order as the product's WbView so one ctypes Structure serves both.
struct WoView {
    void* data;
    int32_t dtype;  // 0 = f32, 1 = f64, 2 = i64
    int32_t ndim;
    int64_t shape[8];
    int64_t stride[8];
    int64_t offset;
};

}  // extern "C"

namespace {

constexpr int64_t PAR_MIN = 1 << 15;  // crates/weta-cpu/src/lib.rs:47

inline int64_t numel(const WoView& v) {
    int64_t n = 1;
    for (int i = 0; i < v.ndim; ++i) n *= v.shape[i];
    return n;
}

// crates/weta-core/src/layout.rs:60-69
inline bool is_contiguous(const WoView& v) {
    int64_t expected = 1;
    for (int i = v.ndim - 1; i >= 0; --i) {
        if (v.shape[i] != 1 && v.stride[i] != expected) return false;
        expected *= v.shape[i];
    }
    return true;
}

// Storage index of the element whose row-major linear index is `lin`
// (crates/weta-core/src/layout.rs:226-263 walks the same order with an odometer).
inline int64_t offset_of(const WoView& v, int64_t lin) {
    int64_t off = v.offset;
    for (int i = v.ndim - 1; i >= 0; --i) {
        int64_t d = v.shape[i];
        off += (lin % d) * v.stride[i];
        lin /= d;
    }
    return off;
}

// Row-major odometer over a view, started at linear index `lin`.
struct Odo {
    const WoView& v;
    int64_t idx[8];
    int64_t off;
    Odo(const WoView& view, int64_t lin) : v(view) {
        off = v.offset;
        for (int i = v.ndim - 1; i >= 0; --i) {
            int64_t d = v.shape[i];
            idx[i] = lin % d;
            off += idx[i] * v.stride[i];
            lin /= d;
        }
    }
    inline void next() {
        for (int i = v.ndim - 1; i >= 0; --i) {
            off += v.stride[i];
            if (++idx[i] < v.shape[i]) return;
            off -= idx[i] * v.stride[i];
            idx[i] = 0;
        }
    }
};

// crates/weta-cpu/src/lib.rs:55-72 (`map`): contiguous fast path, else strided walk.
template <class T, class U, class F>
void map1(const WoView& x, U* out, F f) {
    const T* xp = static_cast<const T*>(x.data);
    int64_t n = numel(x);
    if (n == 0) return;
    if (is_contiguous(x)) {
        const T* s = xp + x.offset;
#pragma omp parallel for if (n >= PAR_MIN) schedule(static)
        for (int64_t i = 0; i < n; ++i) out[i] = f(s[i]);
        return;
    }
    int nt = n >= PAR_MIN ? omp_get_max_threads() : 1;
#pragma omp parallel for num_threads(nt) schedule(static)
    for (int t = 0; t < nt; ++t) {
        int64_t lo = n * t / nt, hi = n * (t + 1) / nt;
        if (lo >= hi) continue;
        Odo o(x, lo);
        for (int64_t i = lo; i < hi; ++i) {
            out[i] = f(xp[o.off]);
            o.next();
        }
    }
}

// crates/weta-cpu/src/lib.rs:75-99 (`zip`)
template <class T, class U, class F>
void zip2(const WoView& a, const WoView& b, U* out, F f) {
    const T* ap = static_cast<const T*>(a.data);
    const T* bp = static_cast<const T*>(b.data);
    int64_t n = numel(a);
    if (n == 0) return;
    if (is_contiguous(a) && is_contiguous(b)) {
        const T* sa = ap + a.offset;
        const T* sb = bp + b.offset;
#pragma omp parallel for if (n >= PAR_MIN) schedule(static)
        for (int64_t i = 0; i < n; ++i) out[i] = f(sa[i], sb[i]);
        return;
    }
    int nt = n >= PAR_MIN ? omp_get_max_threads() : 1;
#pragma omp parallel for num_threads(nt) schedule(static)
    for (int t = 0; t < nt; ++t) {
        int64_t lo = n * t / nt, hi = n * (t + 1) / nt;
        if (lo >= hi) continue;
        Odo oa(a, lo), ob(b, lo);
        for (int64_t i = lo; i < hi; ++i) {
            out[i] = f(ap[oa.off], bp[ob.off]);
            oa.next();
            ob.next();
        }
    }
}

// crates/weta-core/src/dtype.rs:136-149: NaN in `self` wins, NaN in `o` loses.
template <class T> inline T fmax_weta(T a, T o) { return (a >= o || std::isnan(a)) ? a : o; }
template <class T> inline T fmin_weta(T a, T o) { return (a <= o || std::isnan(a)) ? a : o; }

// Rust `as i64` from a float: truncates, saturates, NaN -> 0 (crates/weta-cpu/src/lib.rs:557).
template <class T> inline int64_t float_to_i64(T v) {
    if (std::isnan(v)) return 0;
    if (v >= static_cast<T>(9223372036854775808.0)) return std::numeric_limits<int64_t>::max();
    if (v <= static_cast<T>(-9223372036854775808.0)) return std::numeric_limits<int64_t>::min();
    return static_cast<int64_t>(v);
}

inline int64_t div_euclid(int64_t x, int64_t y) {  // Rust i64::div_euclid
    int64_t q = x / y;
    if (x % y < 0) return y > 0 ? q - 1 : q + 1;
    return q;
}

inline int64_t ipow(int64_t x, uint32_t e) {  // Rust i64::pow (wrapping in release builds)
    uint64_t base = static_cast<uint64_t>(x), acc = 1;
    while (e) {
        if (e & 1) acc *= base;
        base *= base;
        e >>= 1;
    }
    return static_cast<int64_t>(acc);
}

// crates/weta-cpu/src/lib.rs:133-188
template <class T>
int unary_float(int op, double p1, double p2, const WoView& x, T* out) {
    const T zero = 0, one = 1;
    switch (op) {
        case 0: map1<T>(x, out, [](T v) { return -v; }); break;
        case 1: map1<T>(x, out, [](T v) { return std::exp(v); }); break;
        case 2: map1<T>(x, out, [](T v) { return std::log(v); }); break;
        case 3: map1<T>(x, out, [](T v) { return std::sqrt(v); }); break;
        case 4: map1<T>(x, out, [](T v) { return std::fabs(v); }); break;
        case 5: map1<T>(x, out, [=](T v) { return v > zero ? one : (v < zero ? -one : zero); }); break;
        case 6: map1<T>(x, out, [=](T v) { return v > zero ? v : zero; }); break;
        case 7: map1<T>(x, out, [=](T v) { return v > zero ? one : zero; }); break;
        case 8: map1<T>(x, out, [](T v) { return std::tanh(v); }); break;
        case 9:
            map1<T>(x, out, [=](T v) {
                if (v >= zero) return one / (one + std::exp(-v));
                T e = std::exp(v);
                return e / (one + e);
            });
            break;
        case 10: map1<T>(x, out, [](T v) { return std::erf(v); }); break;
        case 11: map1<T>(x, out, [](T v) { return std::sin(v); }); break;
        case 12: map1<T>(x, out, [](T v) { return std::cos(v); }); break;
        case 13: map1<T>(x, out, [=](T v) { return one / v; }); break;
        case 14: {
            T m = static_cast<T>(p1), a = static_cast<T>(p2);  // scalars rounded once, :168
            map1<T>(x, out, [=](T v) { return v * m + a; });
            break;
        }
        case 15: {
            T e = static_cast<T>(p1);
            map1<T>(x, out, [=](T v) { return std::pow(v, e); });
            break;
        }
        case 16: {
            T s = static_cast<T>(p1);
            map1<T>(x, out, [=](T v) { return v > s ? one : zero; });
            break;
        }
        case 17: {
            T s = static_cast<T>(p1);
            map1<T>(x, out, [=](T v) { return fmax_weta(v, s); });
            break;
        }
        case 18: {
            T s = static_cast<T>(p1);
            map1<T>(x, out, [=](T v) { return fmin_weta(v, s); });
            break;
        }
        default: return 2;
    }
    return 0;
}

// crates/weta-cpu/src/lib.rs:190-203
int unary_int(int op, double p1, double p2, const WoView& x, int64_t* out) {
    using I = int64_t;
    switch (op) {
        case 0: map1<I>(x, out, [](I v) { return static_cast<I>(0 - static_cast<uint64_t>(v)); }); break;
        case 4: map1<I>(x, out, [](I v) { return v < 0 ? static_cast<I>(0 - static_cast<uint64_t>(v)) : v; }); break;
        case 5: map1<I>(x, out, [](I v) { return static_cast<I>((v > 0) - (v < 0)); }); break;
        case 6: map1<I>(x, out, [](I v) { return v > 0 ? v : I(0); }); break;
        case 7: map1<I>(x, out, [](I v) { return static_cast<I>(v > 0); }); break;
        case 14: map1<I>(x, out, [=](I v) { return float_to_i64(static_cast<double>(v) * p1 + p2); }); break;
        case 16: map1<I>(x, out, [=](I v) { return static_cast<I>(static_cast<double>(v) > p1); }); break;
        case 17: { I s = float_to_i64(p1); map1<I>(x, out, [=](I v) { return std::max(v, s); }); break; }
        case 18: { I s = float_to_i64(p1); map1<I>(x, out, [=](I v) { return std::min(v, s); }); break; }
        default: return 3;  // "not supported for i64 tensors" (panics in the reference)
    }
    return 0;
}

// crates/weta-cpu/src/lib.rs:205-223
template <class T>
int binary_float(int op, const WoView& a, const WoView& b, T* out) {
    const T zero = 0, one = 1;
    switch (op) {
        case 0: zip2<T>(a, b, out, [](T x, T y) { return x + y; }); break;
        case 1: zip2<T>(a, b, out, [](T x, T y) { return x - y; }); break;
        case 2: zip2<T>(a, b, out, [](T x, T y) { return x * y; }); break;
        case 3: zip2<T>(a, b, out, [](T x, T y) { return x / y; }); break;
        case 4: zip2<T>(a, b, out, [](T x, T y) { return std::pow(x, y); }); break;
        case 5: zip2<T>(a, b, out, [](T x, T y) { return fmax_weta(x, y); }); break;
        case 6: zip2<T>(a, b, out, [](T x, T y) { return fmin_weta(x, y); }); break;
        case 7: zip2<T>(a, b, out, [=](T x, T y) { return x == y ? one : zero; }); break;
        case 8: zip2<T>(a, b, out, [=](T x, T y) { return x != y ? one : zero; }); break;
        case 9: zip2<T>(a, b, out, [=](T x, T y) { return x < y ? one : zero; }); break;
        case 10: zip2<T>(a, b, out, [=](T x, T y) { return x <= y ? one : zero; }); break;
        case 11: zip2<T>(a, b, out, [=](T x, T y) { return x > y ? one : zero; }); break;
        case 12: zip2<T>(a, b, out, [=](T x, T y) { return x >= y ? one : zero; }); break;
        default: return 2;
    }
    return 0;
}

// crates/weta-cpu/src/lib.rs:225-241
int binary_int(int op, const WoView& a, const WoView& b, int64_t* out) {
    using I = int64_t;
    using U = uint64_t;
    switch (op) {
        case 0: zip2<I>(a, b, out, [](I x, I y) { return static_cast<I>(U(x) + U(y)); }); break;
        case 1: zip2<I>(a, b, out, [](I x, I y) { return static_cast<I>(U(x) - U(y)); }); break;
        case 2: zip2<I>(a, b, out, [](I x, I y) { return static_cast<I>(U(x) * U(y)); }); break;
        case 3: zip2<I>(a, b, out, [](I x, I y) { return y == 0 ? I(0) : div_euclid(x, y); }); break;
        case 4: zip2<I>(a, b, out, [](I x, I y) { return ipow(x, static_cast<uint32_t>(y)); }); break;
        case 5: zip2<I>(a, b, out, [](I x, I y) { return std::max(x, y); }); break;
        case 6: zip2<I>(a, b, out, [](I x, I y) { return std::min(x, y); }); break;
        case 7: zip2<I>(a, b, out, [](I x, I y) { return I(x == y); }); break;
        case 8: zip2<I>(a, b, out, [](I x, I y) { return I(x != y); }); break;
        case 9: zip2<I>(a, b, out, [](I x, I y) { return I(x < y); }); break;
        case 10: zip2<I>(a, b, out, [](I x, I y) { return I(x <= y); }); break;
        case 11: zip2<I>(a, b, out, [](I x, I y) { return I(x > y); }); break;
        case 12: zip2<I>(a, b, out, [](I x, I y) { return I(x >= y); }); break;
        default: return 2;
    }
    return 0;
}

// crates/weta-cpu/src/lib.rs:245-300.  `f(base, n, stride)` folds one output.
template <class T, class U, class F>
void reduce_generic(const WoView& x, int axis, U* out, F f) {
    WoView outer = x;
    int64_t n = x.shape[axis], stride = x.stride[axis];
    for (int i = axis; i + 1 < x.ndim; ++i) {
        outer.shape[i] = x.shape[i + 1];
        outer.stride[i] = x.stride[i + 1];
    }
    outer.ndim = x.ndim - 1;
    int64_t n_out = numel(outer);
    const T* xp = static_cast<const T*>(x.data);
    bool par = numel(x) >= PAR_MIN;
#pragma omp parallel for if (par) schedule(static)
    for (int64_t o = 0; o < n_out; ++o) out[o] = f(xp + offset_of(outer, o), n, stride);
}

template <class T>
int reduce_any(int op, const WoView& x, int axis, void* out) {
    constexpr bool is_int = std::is_same<T, int64_t>::value;
    switch (op) {
        case 0:  // Sum: sequential, k ascending, in the storage dtype (:284)
            reduce_generic<T>(x, axis, static_cast<T*>(out), [](const T* p, int64_t n, int64_t s) {
                if constexpr (is_int) {
                    uint64_t acc = 0;
                    for (int64_t k = 0; k < n; ++k) acc += static_cast<uint64_t>(p[k * s]);
                    return static_cast<T>(acc);
                } else {
                    T acc = 0;
                    for (int64_t k = 0; k < n; ++k) acc = acc + p[k * s];
                    return acc;
                }
            });
            break;
        case 1:  // Max (:285, :295)
            reduce_generic<T>(x, axis, static_cast<T*>(out), [](const T* p, int64_t n, int64_t s) {
                if constexpr (is_int) {
                    T acc = std::numeric_limits<T>::min();
                    for (int64_t k = 0; k < n; ++k) acc = std::max(acc, p[k * s]);
                    return acc;
                } else {
                    T acc = -std::numeric_limits<T>::infinity();
                    for (int64_t k = 0; k < n; ++k) acc = fmax_weta(acc, p[k * s]);
                    return acc;
                }
            });
            break;
        case 2:  // Min
            reduce_generic<T>(x, axis, static_cast<T*>(out), [](const T* p, int64_t n, int64_t s) {
                if constexpr (is_int) {
                    T acc = std::numeric_limits<T>::max();
                    for (int64_t k = 0; k < n; ++k) acc = std::min(acc, p[k * s]);
                    return acc;
                } else {
                    T acc = std::numeric_limits<T>::infinity();
                    for (int64_t k = 0; k < n; ++k) acc = fmin_weta(acc, p[k * s]);
                    return acc;
                }
            });
            break;
        case 3:  // ArgMax: first strictly-better element wins (:268-277)
        case 4:
            reduce_generic<T>(x, axis, static_cast<int64_t*>(out), [op](const T* p, int64_t n, int64_t s) {
                if (n == 0) return int64_t(0);
                int64_t bi = 0;
                T best = p[0];
                for (int64_t k = 1; k < n; ++k) {
                    T v = p[k * s];
                    bool better = (op == 3) ? (v > best) : (v < best);
                    if (better) { bi = k; best = v; }
                }
                return bi;
            });
            break;
        default: return 2;
    }
    return 0;
}

// crates/weta-cpu/src/lib.rs:319-365.  out[b][i][j] = sum_k a[b][i][k] * b[b][k][j], k ascending,
// accumulated in T.  The i-k-j loop keeps that order per output while letting the inner loop
// vectorise; B is packed to unit column stride first when it is not already.
// Test-only switches for f32 products (default off = the restatement above):
//   g_tf32_operands   both operands are reduced to TF32 (10 mantissa bits) first, the way a TF32 tensor-core
//                     instruction reads an f32 operand (1 = low 13 bits dropped, 2 / 3 = rounded to nearest); a GPU
//                     run in TF32 mode then differs from this oracle by accumulation error only;
//   g_f64_accumulate  the sum over k is kept in double and rounded to f32 once.
int g_tf32_operands = 0;  // 0 off, 1 truncate, 2 round to nearest (ties away from zero), 3 round to nearest even
bool g_f64_accumulate = false;

inline float tf32_trunc(float v) {  // f32 -> the 19-bit TF32 value a tensor core would use, by the selected rule
    uint32_t u;
    std::memcpy(&u, &v, 4);
    if ((u & 0x7F800000u) != 0x7F800000u) {  // finite
        if (g_tf32_operands == 2) u += 0x00001000u;
        else if (g_tf32_operands == 3) u += 0x00000FFFu + ((u >> 13) & 1u);
    }
    u &= 0xFFFFE000u;
    std::memcpy(&v, &u, 4);
    return v;
}

template <class T>
void matmul_float(const WoView& a, const WoView& b, T* out) {
    int64_t bs = a.shape[0], m = a.shape[1], k = a.shape[2], n = b.shape[2];
    if (bs * m * n == 0) return;
    const T* ap = static_cast<const T*>(a.data) + a.offset;
    const T* bp = static_cast<const T*>(b.data) + b.offset;
    const bool special = sizeof(T) == 4 && (g_tf32_operands || g_f64_accumulate);
    std::vector<T> packed;
    for (int64_t batch = 0; batch < bs; ++batch) {
        const T* A = ap + batch * a.stride[0];
        const T* B = bp + batch * b.stride[0];
        int64_t brs = b.stride[1];
        if ((b.stride[2] != 1 && n > 1) || (special && g_tf32_operands)) {
            if (batch == 0 || b.stride[0] != 0) {
                packed.resize(static_cast<size_t>(k * n));
#pragma omp parallel for schedule(static)
                for (int64_t kk = 0; kk < k; ++kk)
                    for (int64_t j = 0; j < n; ++j) {
                        T v = B[kk * b.stride[1] + j * b.stride[2]];
                        if constexpr (sizeof(T) == 4) { if (g_tf32_operands) v = tf32_trunc(v); }
                        packed[kk * n + j] = v;
                    }
            }
            B = packed.data();
            brs = n;
        }
        T* O = out + batch * m * n;
        int64_t as1 = a.stride[1], as2 = a.stride[2];
        if (special) {
#pragma omp parallel
            {
                std::vector<double> acc(static_cast<size_t>(n));
#pragma omp for schedule(static)
                for (int64_t i = 0; i < m; ++i) {
                    T* orow = O + i * n;
                    if (g_f64_accumulate) {
                        std::fill(acc.begin(), acc.end(), 0.0);
                        for (int64_t kk = 0; kk < k; ++kk) {
                            T av = A[i * as1 + kk * as2];
                            if constexpr (sizeof(T) == 4) { if (g_tf32_operands) av = tf32_trunc(av); }
                            const double avd = static_cast<double>(av);
                            const T* brow = B + kk * brs;
                            for (int64_t j = 0; j < n; ++j) acc[j] += avd * static_cast<double>(brow[j]);
                        }
                        for (int64_t j = 0; j < n; ++j) orow[j] = static_cast<T>(acc[j]);
                    } else {
                        for (int64_t j = 0; j < n; ++j) orow[j] = 0;
                        for (int64_t kk = 0; kk < k; ++kk) {
                            T av = A[i * as1 + kk * as2];
                            if constexpr (sizeof(T) == 4) av = tf32_trunc(av);
                            const T* brow = B + kk * brs;
                            for (int64_t j = 0; j < n; ++j) orow[j] = orow[j] + av * brow[j];
                        }
                    }
                }
            }
            continue;
        }
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < m; ++i) {
            T* orow = O + i * n;
            for (int64_t j = 0; j < n; ++j) orow[j] = 0;
            for (int64_t kk = 0; kk < k; ++kk) {
                T av = A[i * as1 + kk * as2];
                const T* brow = B + kk * brs;
                for (int64_t j = 0; j < n; ++j) orow[j] = orow[j] + av * brow[j];
            }
        }
    }
}

struct ConvP {
    int64_t kh, kw, sh, sw, ph, pw, dh, dw;
};

// crates/weta-core/src/ops.rs:136-149
inline int64_t out_size1(int64_t x, int64_t k, int64_t s, int64_t p, int64_t d) {
    int64_t span = d * (k - 1) + 1;
    if (x + 2 * p < span) return 0;
    return (x + 2 * p - span) / s + 1;
}

// crates/weta-cpu/src/lib.rs:367-408
template <class T>
void im2col_generic(const WoView& x, const ConvP& p, T* out) {
    int64_t nb = x.shape[0], c = x.shape[1], h = x.shape[2], w = x.shape[3];
    int64_t oh = out_size1(h, p.kh, p.sh, p.ph, p.dh), ow = out_size1(w, p.kw, p.sw, p.pw, p.dw);
    int64_t chunk = p.kh * p.kw * oh * ow;
    int64_t total = nb * c * chunk;
    if (total == 0) return;
    std::memset(out, 0, sizeof(T) * static_cast<size_t>(total));
    const T* xp = static_cast<const T*>(x.data);
#pragma omp parallel for if (total >= PAR_MIN) schedule(static)
    for (int64_t nc = 0; nc < nb * c; ++nc) {
        int64_t n = nc / c, ci = nc % c;
        int64_t base = x.offset + n * x.stride[0] + ci * x.stride[1];
        T* ch = out + nc * chunk;
        for (int64_t ki = 0; ki < p.kh; ++ki)
            for (int64_t kj = 0; kj < p.kw; ++kj) {
                T* row = ch + (ki * p.kw + kj) * oh * ow;
                for (int64_t y = 0; y < oh; ++y) {
                    int64_t iy = y * p.sh + ki * p.dh - p.ph;
                    if (iy < 0 || iy >= h) continue;
                    for (int64_t xx = 0; xx < ow; ++xx) {
                        int64_t ix = xx * p.sw + kj * p.dw - p.pw;
                        if (ix >= 0 && ix < w) row[y * ow + xx] = xp[base + iy * x.stride[2] + ix * x.stride[3]];
                    }
                }
            }
    }
}

// crates/weta-cpu/src/lib.rs:410-446 (cols are gathered to contiguous first, :546)
template <class T>
void col2im_float(const WoView& cols, const ConvP& p, int64_t c, int64_t h, int64_t w, T* out) {
    int64_t nb = cols.shape[0];
    int64_t oh = out_size1(h, p.kh, p.sh, p.ph, p.dh), ow = out_size1(w, p.kw, p.sw, p.pw, p.dw);
    int64_t total = nb * c * h * w;
    if (total == 0) return;
    std::vector<T> cont(static_cast<size_t>(numel(cols)));
    map1<T>(cols, cont.data(), [](T v) { return v; });
    std::memset(out, 0, sizeof(T) * static_cast<size_t>(total));
    int64_t per = p.kh * p.kw * oh * ow;
#pragma omp parallel for if (total >= PAR_MIN) schedule(static)
    for (int64_t nc = 0; nc < nb * c; ++nc) {
        const T* src = cont.data() + nc * per;
        T* img = out + nc * h * w;
        for (int64_t ki = 0; ki < p.kh; ++ki)
            for (int64_t kj = 0; kj < p.kw; ++kj) {
                const T* row = src + (ki * p.kw + kj) * oh * ow;
                for (int64_t y = 0; y < oh; ++y) {
                    int64_t iy = y * p.sh + ki * p.dh - p.ph;
                    if (iy < 0 || iy >= h) continue;
                    for (int64_t xx = 0; xx < ow; ++xx) {
                        int64_t ix = xx * p.sw + kj * p.dw - p.pw;
                        if (ix >= 0 && ix < w) img[iy * w + ix] = img[iy * w + ix] + row[y * ow + xx];
                    }
                }
            }
    }
}

// crates/weta-cpu/src/lib.rs:448-457
template <class T>
void copy_into(const WoView& src, const WoView& dst) {
    const T* sp = static_cast<const T*>(src.data);
    T* dp = static_cast<T*>(dst.data);
    int64_t n = numel(src);
    if (n == 0) return;
    if (is_contiguous(src) && is_contiguous(dst)) {
        std::memmove(dp + dst.offset, sp + src.offset, sizeof(T) * static_cast<size_t>(n));
        return;
    }
    Odo os(src, 0), od(dst, 0);
    for (int64_t i = 0; i < n; ++i) {
        dp[od.off] = sp[os.off];
        os.next();
        od.next();
    }
}

// crates/weta-core/src/ops.rs:164-169
inline uint64_t splitmix64(uint64_t seed, uint64_t i) {
    uint64_t z = seed + (i + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// crates/weta-core/src/ops.rs:172-174
inline double unit(uint64_t seed, uint64_t i) {
    return static_cast<double>(splitmix64(seed, i) >> 11) * (1.0 / 9007199254740992.0);
}

// crates/weta-core/src/ops.rs:179-188
inline double sample(int dist, double a, double b, uint64_t seed, uint64_t i) {
    if (dist == 0) return a + (b - a) * unit(seed, i);
    double u1 = 1.0 - unit(seed, 2 * i);
    double u2 = unit(seed, 2 * i + 1);
    return a + b * std::sqrt(-2.0 * std::log(u1)) * std::cos(2.0 * M_PI * u2);
}

}  // namespace

extern "C" {

int wo_num_threads() { return omp_get_max_threads(); }
void wo_set_num_threads(int n) { omp_set_num_threads(n); }
// Test-only: TF32-truncated operands and / or double accumulation for f32 matmul (see matmul_float).
void wo_set_matmul_test_mode(int tf32_operands, int f64_accumulate) {
    g_tf32_operands = tf32_operands;
    g_f64_accumulate = f64_accumulate != 0;
}

// crates/weta-cpu/src/lib.rs:510-512
int wo_unary(int op, double p1, double p2, const WoView* x, void* out) {
    switch (x->dtype) {
        case 0: return unary_float<float>(op, p1, p2, *x, static_cast<float*>(out));
        case 1: return unary_float<double>(op, p1, p2, *x, static_cast<double*>(out));
        case 2: return unary_int(op, p1, p2, *x, static_cast<int64_t*>(out));
    }
    return 1;
}

// crates/weta-cpu/src/lib.rs:514-521
int wo_binary(int op, const WoView* a, const WoView* b, void* out) {
    if (a->dtype != b->dtype) return 1;
    switch (a->dtype) {
        case 0: return binary_float<float>(op, *a, *b, static_cast<float*>(out));
        case 1: return binary_float<double>(op, *a, *b, static_cast<double*>(out));
        case 2: return binary_int(op, *a, *b, static_cast<int64_t*>(out));
    }
    return 1;
}

// crates/weta-cpu/src/lib.rs:523-529
int wo_reduce(int op, const WoView* x, int axis, void* out) {
    switch (x->dtype) {
        case 0: return reduce_any<float>(op, *x, axis, out);
        case 1: return reduce_any<double>(op, *x, axis, out);
        case 2: return reduce_any<int64_t>(op, *x, axis, out);
    }
    return 1;
}

// crates/weta-cpu/src/lib.rs:531-537
int wo_matmul(const WoView* a, const WoView* b, void* out) {
    if (a->dtype != b->dtype || a->ndim != 3 || b->ndim != 3) return 1;
    switch (a->dtype) {
        case 0: matmul_float<float>(*a, *b, static_cast<float*>(out)); return 0;
        case 1: matmul_float<double>(*a, *b, static_cast<double*>(out)); return 0;
    }
    return 1;  // i64 matmul panics in the reference
}

// crates/weta-cpu/src/lib.rs:539-541
int wo_im2col(const WoView* x, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
              int64_t dw, void* out) {
    ConvP p{kh, kw, sh, sw, ph, pw, dh, dw};
    if (x->ndim != 4) return 1;
    switch (x->dtype) {
        case 0: im2col_generic<float>(*x, p, static_cast<float*>(out)); return 0;
        case 1: im2col_generic<double>(*x, p, static_cast<double*>(out)); return 0;
        case 2: im2col_generic<int64_t>(*x, p, static_cast<int64_t*>(out)); return 0;
    }
    return 1;
}

// crates/weta-cpu/src/lib.rs:543-550
int wo_col2im(const WoView* cols, int64_t kh, int64_t kw, int64_t sh, int64_t sw, int64_t ph, int64_t pw, int64_t dh,
              int64_t dw, int64_t c, int64_t h, int64_t w, void* out) {
    ConvP p{kh, kw, sh, sw, ph, pw, dh, dw};
    if (cols->ndim != 3) return 1;
    switch (cols->dtype) {
        case 0: col2im_float<float>(*cols, p, c, h, w, static_cast<float*>(out)); return 0;
        case 1: col2im_float<double>(*cols, p, c, h, w, static_cast<double*>(out)); return 0;
    }
    return 1;  // i64 col2im panics in the reference
}

// crates/weta-cpu/src/lib.rs:501-508
int wo_copy_strided(const WoView* src, const WoView* dst) {
    if (src->dtype != dst->dtype) return 1;
    switch (src->dtype) {
        case 0: copy_into<float>(*src, *dst); return 0;
        case 1: copy_into<double>(*src, *dst); return 0;
        case 2: copy_into<int64_t>(*src, *dst); return 0;
    }
    return 1;
}

// crates/weta-cpu/src/lib.rs:552-565
int wo_cast(const WoView* x, int dtype, void* out) {
#define CAST(T, U, expr) map1<T>(*x, static_cast<U*>(out), [](T a) { return expr; }); return 0
    switch (x->dtype * 3 + dtype) {
        case 0: CAST(float, float, a);
        case 1: CAST(float, double, static_cast<double>(a));
        case 2: CAST(float, int64_t, float_to_i64(a));
        case 3: CAST(double, float, static_cast<float>(a));
        case 4: CAST(double, double, a);
        case 5: CAST(double, int64_t, float_to_i64(a));
        case 6: CAST(int64_t, float, static_cast<float>(a));
        case 7: CAST(int64_t, double, static_cast<double>(a));
        case 8: CAST(int64_t, int64_t, a);
    }
#undef CAST
    return 1;
}

// crates/weta-core/src/backend.rs:97-105: sample in f64, then cast to the dtype.
int wo_random(int64_t len, int dtype, int dist, double a, double b, uint64_t seed, void* out) {
    if (dtype == 0) {
        float* o = static_cast<float*>(out);
#pragma omp parallel for if (len >= PAR_MIN) schedule(static)
        for (int64_t i = 0; i < len; ++i) o[i] = static_cast<float>(sample(dist, a, b, seed, static_cast<uint64_t>(i)));
        return 0;
    }
    if (dtype == 1) {
        double* o = static_cast<double*>(out);
#pragma omp parallel for if (len >= PAR_MIN) schedule(static)
        for (int64_t i = 0; i < len; ++i) o[i] = sample(dist, a, b, seed, static_cast<uint64_t>(i));
        return 0;
    }
    return 1;  // "random: expected a float dtype, got i64"
}

uint64_t wo_splitmix64(uint64_t seed, uint64_t i) { return splitmix64(seed, i); }

}  // extern "C"
