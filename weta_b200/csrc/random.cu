// Backend::random (crates/weta-core/src/backend.rs:97-105): element i = Distribution::sample(seed, i)
// evaluated in f64 and cast to the dtype (crates/weta-core/src/ops.rs:164-189).
//
// The counter hash is pure 64-bit integer arithmetic, so uniform fills are bit-identical to the
// CPU backend: `unit = (splitmix64(seed, i) >> 11) * 2^-53` is exact in f64, and for lo = 0,
// hi = 1 the f32 value is that number rounded once, which `__ull2float_rn(k) * 2^-53` also
// produces (one rounding of a 53-bit integer, then an exact power-of-two scale) without touching
// the FP64 pipe.  General bounds take `lo + (hi - lo) * unit` in f64 with two roundings (this file
// is built with -fmad=false).  Normal fills need ln and cos in f64: the device's versions are good to 1 and
// 2 ulp, the CPU backend's libm rounds (almost always) correctly, so normal_dd.h evaluates both in
// double-double and rounds once.  f64 tensors always take that evaluation.  f32 tensors take the device's fast
// log / cos first and fall back to it only when the fast value, with its error bound, straddles an f32 rounding
// boundary (about one element in 2^22), which gives the same f32 bits at the fast path's speed.
#include "common.h"
#include "normal_dd.h"

namespace {

__device__ __forceinline__ uint64_t splitmix64(uint64_t seed, uint64_t i) {
    uint64_t z = seed + (i + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ double unit(uint64_t seed, uint64_t i) {
    return __ull2double_rn(splitmix64(seed, i) >> 11) * (1.0 / 9007199254740992.0);
}

// Distribution::sample in f64 (crates/weta-core/src/ops.rs:176-189), every step rounded as the CPU rounds it.
__device__ __forceinline__ double sample(int dist, double a, double b, uint64_t seed, uint64_t i) {
    if (dist == WB_UNIFORM) return a + (b - a) * unit(seed, i);
    const double u1 = 1.0 - unit(seed, 2 * i);
    const double u2 = unit(seed, 2 * i + 1);
    return wbdd::normal_exact(a, b, u1, u2);
}

// The same sample rounded to f32.  Fast evaluation first: the device's log and cos are within 1 and 2 ulp, the other
// steps within half an ulp each, so the product std * sqrt(..) * cos(..) is within 2^-49 of the exact chain's
// relatively (a generous bound) and the sum within that plus an ulp.  When both ends of that interval round to the
// same f32 the result is settled; otherwise the exact chain decides.
__device__ __forceinline__ float sample_normal_f32(double mean, double std, uint64_t seed, uint64_t i) {
    const double u1 = 1.0 - unit(seed, 2 * i);
    const double u2 = unit(seed, 2 * i + 1);
    const double prod = (std * sqrt(-2.0 * log(u1))) * cos(6.283185307179586 * u2);
    const double v = mean + prod;
    const double err = fabs(prod) * 3.5527136788005009e-15 /* 2^-48 */ + fabs(v) * 4.4408920985006262e-16 /* 2^-51 */;
    const float lo = __double2float_rn(v - err), hi = __double2float_rn(v + err);
    if (lo == hi) return lo;
    return __double2float_rn(wbdd::normal_exact(mean, std, u1, u2));
}

constexpr int THREADS = 256;

// U[0,1) -> f32, four consecutive elements per thread, one 128-bit store.
__global__ void __launch_bounds__(THREADS) uniform01_f32(float* __restrict__ out, int64_t n, uint64_t seed) {
    int64_t i = (static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x) * 4;
    if (i >= n) return;
    float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = __ull2float_rn(splitmix64(seed, static_cast<uint64_t>(i + k)) >> 11) * 1.1102230246251565e-16f;
    if (i + 4 <= n && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        *reinterpret_cast<float4*>(out + i) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        for (int k = 0; k < 4 && i + k < n; ++k) out[i + k] = v[k];
    }
}

template <class T>
__global__ void __launch_bounds__(THREADS) random_general(T* __restrict__ out, int64_t n, int dist, double a, double b, uint64_t seed) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (i >= n) return;
    if constexpr (sizeof(T) == 4) {
        out[i] = dist == WB_NORMAL ? sample_normal_f32(a, b, seed, static_cast<uint64_t>(i)) : __double2float_rn(sample(dist, a, b, seed, static_cast<uint64_t>(i)));
    } else {
        out[i] = sample(dist, a, b, seed, static_cast<uint64_t>(i));
    }
}

}  // namespace

extern "C" int wb_random_into(WbBackend* b, int64_t len, int dtype, int dist, double pa, double pb, uint64_t seed, void* out) {
    WB_REQUIRE(b && (out || len == 0), WB_ERR_INVALID, "wb_random: null pointer");
    WB_REQUIRE(dtype == WB_F32 || dtype == WB_F64, WB_ERR_UNSUPPORTED, "random: expected a float dtype, got i64");
    WB_REQUIRE(dist == WB_UNIFORM || dist == WB_NORMAL, WB_ERR_INVALID, "random: unknown distribution %d", dist);
    if (len == 0) return WB_OK;
    WbProfileScope ps(b, "random");
    if (dtype == WB_F32 && dist == WB_UNIFORM && pa == 0.0 && pb == 1.0) {
        int64_t threads = (len + 3) / 4;
        uniform01_f32<<<static_cast<unsigned>((threads + THREADS - 1) / THREADS), THREADS, 0, b->stream>>>(static_cast<float*>(out), len, seed);
    } else if (dtype == WB_F32) {
        random_general<float><<<static_cast<unsigned>((len + THREADS - 1) / THREADS), THREADS, 0, b->stream>>>(static_cast<float*>(out), len, dist, pa, pb, seed);
    } else {
        random_general<double><<<static_cast<unsigned>((len + THREADS - 1) / THREADS), THREADS, 0, b->stream>>>(static_cast<double*>(out), len, dist, pa, pb, seed);
    }
    WB_LAUNCH_OK(b);
    return WB_OK;
}

// Host evaluation of the functions the Normal fill runs on the device (same source, compiled for the CPU): lets a
// test without a GPU compare them with arbitrary-precision values.
extern "C" double wb_host_log_rn(double x) { return wbdd::log_rn(x); }
extern "C" double wb_host_cos_rn(double t) { return wbdd::cos_rn(t); }
extern "C" double wb_host_normal_sample(uint64_t seed, uint64_t i, double mean, double std) {
    const double u1 = 1.0 - static_cast<double>(wb_splitmix64(seed, 2 * i) >> 11) * (1.0 / 9007199254740992.0);
    const double u2 = static_cast<double>(wb_splitmix64(seed, 2 * i + 1) >> 11) * (1.0 / 9007199254740992.0);
    return wbdd::normal_exact(mean, std, u1, u2);
}

extern "C" int wb_random(WbBackend* b, int64_t len, int dtype, int dist, double pa, double pb, uint64_t seed, WbStorage** out) {
    WB_REQUIRE(b && out, WB_ERR_INVALID, "wb_random: null pointer");
    WB_REQUIRE(dtype == WB_F32 || dtype == WB_F64, WB_ERR_UNSUPPORTED, "random: expected a float dtype, got i64");
    WB_TRY(wb_new_storage(b, len, dtype, out));
    int s = wb_random_into(b, len, dtype, dist, pa, pb, seed, (*out)->ptr);
    if (s != WB_OK) { wb_free(b, *out); *out = nullptr; }
    return s;
}
