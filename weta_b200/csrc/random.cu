// Backend::random (crates/weta-core/src/backend.rs:97-105): element i = Distribution::sample(seed, i)
// evaluated in f64 and cast to the dtype (crates/weta-core/src/ops.rs:164-189).
//
// The counter hash is pure 64-bit integer arithmetic, so uniform fills are bit-identical to the
// CPU backend: `unit = (splitmix64(seed, i) >> 11) * 2^-53` is exact in f64, and for lo = 0,
// hi = 1 the f32 value is that number rounded once, which `__ull2float_rn(k) * 2^-53` also
// produces (one rounding of a 53-bit integer, then an exact power-of-two scale) without touching
// the FP64 pipe.  General bounds take `lo + (hi - lo) * unit` in f64 with two roundings (this file
// is built with -fmad=false).  Normal fills use the device's f64 log / cos, which can differ from
// glibc's in the last place; after the cast to f32 that shows up in at most a few elements per 2^28.
#include "common.h"

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

__device__ __forceinline__ double sample(int dist, double a, double b, uint64_t seed, uint64_t i) {
    if (dist == WB_UNIFORM) return a + (b - a) * unit(seed, i);
    double u1 = 1.0 - unit(seed, 2 * i);
    double u2 = unit(seed, 2 * i + 1);
    return a + b * sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2);
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
    double v = sample(dist, a, b, seed, static_cast<uint64_t>(i));
    if constexpr (sizeof(T) == 4) out[i] = __double2float_rn(v);
    else out[i] = v;
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

extern "C" int wb_random(WbBackend* b, int64_t len, int dtype, int dist, double pa, double pb, uint64_t seed, WbStorage** out) {
    WB_REQUIRE(b && out, WB_ERR_INVALID, "wb_random: null pointer");
    WB_REQUIRE(dtype == WB_F32 || dtype == WB_F64, WB_ERR_UNSUPPORTED, "random: expected a float dtype, got i64");
    WB_TRY(wb_new_storage(b, len, dtype, out));
    int s = wb_random_into(b, len, dtype, dist, pa, pb, seed, (*out)->ptr);
    if (s != WB_OK) { wb_free(b, *out); *out = nullptr; }
    return s;
}
