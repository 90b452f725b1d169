// Backend::reduce (crates/weta-core/src/backend.rs:85): Sum / Max / Min / ArgMax / ArgMin over one axis.
//
// CPU semantics (crates/weta-cpu/src/lib.rs:245-300): sums start at 0 and add elements in axis
// order in the storage dtype; Max/Min fold from -inf/+inf with a NaN-propagating compare
// (crates/weta-core/src/dtype.rs:136-149); ArgMax/ArgMin keep the first strictly-better element.
//
// Four kernels, picked from the collapsed layout of the non-reduced dims:
//   rows_smem   : axis has unit stride and rows are adjacent in memory, len <= ROWS_MAX.  A block
//                 stages a slab of whole rows in shared memory with coalesced loads, then one
//                 thread folds each row front to back (the CPU's order, so sums match bit for bit).
//   cols        : outputs are adjacent in memory along the innermost kept dim (a column reduce, e.g.
//                 a bias gradient).  One thread per output walks the axis in order; a warp reads
//                 32 neighbouring columns per step.  Long axes with few outputs are split across
//                 blockIdx.y into partials held in scratch memory, then folded by a second pass.
//   block       : one block per output for long axes with any stride; warp-shuffle tree.  A single
//                 huge row is split across blocks into scratch partials first.
//   generic     : one thread per output, any strides; short axes.
#include <limits>

#include "common.h"

namespace {

constexpr int THREADS = 256;

struct RPlan {
    int nd;            // collapsed rank of the kept dims (>= 1)
    int64_t n_out;
    int64_t size[WB_MAX_DIMS];
    int64_t st[WB_MAX_DIMS];
    int64_t off;
    int64_t len;       // axis length
    int64_t astride;   // axis stride
};

__device__ __forceinline__ int64_t out_offset(const RPlan& p, int64_t o) {
    int64_t off = p.off;
#pragma unroll 1
    for (int d = p.nd - 1; d >= 0; --d) {
        int64_t q = o / p.size[d];
        off += (o - q * p.size[d]) * p.st[d];
        o = q;
    }
    return off;
}

template <class T> __device__ __forceinline__ T ident(int op) {
    if constexpr (std::is_same<T, int64_t>::value) return op == 0 ? 0 : (op == 1 ? INT64_MIN : INT64_MAX);
    else return op == 0 ? T(0) : (op == 1 ? -INFINITY : INFINITY);
}

// acc <- acc (op) v, with the reference's operand order: acc.max(v).
template <class T, int OP> __device__ __forceinline__ T fold(T acc, T v) {
    if constexpr (OP == 0) {
        if constexpr (std::is_same<T, int64_t>::value) return static_cast<T>(static_cast<uint64_t>(acc) + static_cast<uint64_t>(v));
        else return acc + v;
    } else if constexpr (OP == 1) {
        if constexpr (std::is_same<T, int64_t>::value) return acc > v ? acc : v;
        else return (acc >= v || acc != acc) ? acc : v;
    } else {
        if constexpr (std::is_same<T, int64_t>::value) return acc < v ? acc : v;
        else return (acc <= v || acc != acc) ? acc : v;
    }
}

template <class T> __device__ __forceinline__ T shfl_down(T v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }

// ---- rows_smem ----------------------------------------------------------------------------------
// vec4 (4-byte elements, len % 4 == 0, 16-byte aligned rows): the block's rows are fetched with 128-bit loads, four
// elements of one row each (the three-reduce BatchNorm mean of [256, 64, 56, 56]: 0.085 -> 0.074-0.077 ms).
template <class T, int OP>
__global__ void __launch_bounds__(THREADS) reduce_rows_smem(T* __restrict__ out, const T* __restrict__ x, int64_t n_rows,
                                                            int len, int rows_per_block, int vec4) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* sm = reinterpret_cast<T*>(smem_raw);
    const int pitch = len | 1;  // odd pitch: a warp's 32 rows hit 32 different banks
    int64_t row0 = static_cast<int64_t>(blockIdx.x) * rows_per_block;
    int64_t left = n_rows - row0;
    int rows = left < rows_per_block ? static_cast<int>(left) : rows_per_block;
    const T* src = x + row0 * len;
    int total = rows * len;
    if constexpr (sizeof(T) == 4) {
        if (vec4) {
            const int len4 = len >> 2, total4 = total >> 2;
            int r4 = threadIdx.x / len4, c4 = threadIdx.x - r4 * len4;
            const int dr4 = THREADS / len4, dc4 = THREADS - dr4 * len4;
            for (int i = threadIdx.x; i < total4; i += THREADS) {
                const uint4 v = reinterpret_cast<const uint4*>(src)[i];
                uint32_t* dst = reinterpret_cast<uint32_t*>(sm) + r4 * pitch + 4 * c4;
                dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
                r4 += dr4;
                c4 += dc4;
                if (c4 >= len4) { c4 -= len4; ++r4; }
            }
            total = 0;  // nothing left for the scalar loop
        }
    }
    int r = threadIdx.x / len, c = threadIdx.x - r * len;
    const int dr = THREADS / len, dc = THREADS - dr * len;
    for (int i = threadIdx.x; i < total; i += THREADS) {
        sm[r * pitch + c] = src[i];
        r += dr;
        c += dc;
        if (c >= len) { c -= len; ++r; }
    }
    __syncthreads();
    for (int rr = threadIdx.x; rr < rows; rr += THREADS) {
        T acc = ident<T>(OP);
        const T* row = sm + rr * pitch;
        for (int k = 0; k < len; ++k) acc = fold<T, OP>(acc, row[k]);
        out[row0 + rr] = acc;
    }
}

// ---- cols ---------------------------------------------------------------------------------------
// Output o lives at out_offset(p, o); consecutive o along the innermost kept dim are adjacent.
// blockIdx.y selects a chunk of the axis; with gridDim.y == 1 the result goes straight to `out`.
template <class T, int OP>
__global__ void __launch_bounds__(THREADS) reduce_cols(T* __restrict__ out, const T* __restrict__ x, RPlan p, int64_t chunk) {
    int64_t o = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (o >= p.n_out) return;
    int64_t k0 = static_cast<int64_t>(blockIdx.y) * chunk;
    int64_t k1 = min(k0 + chunk, p.len);
    const T* src = x + out_offset(p, o) + k0 * p.astride;
    T acc = ident<T>(OP);
    for (int64_t k = k0; k < k1; ++k) {
        acc = fold<T, OP>(acc, *src);
        src += p.astride;
    }
    out[static_cast<int64_t>(blockIdx.y) * p.n_out + o] = acc;
}

// ---- block --------------------------------------------------------------------------------------
// grid = (n_out, splits): block (o, s) folds chunk s of row o.
template <class T, int OP>
__global__ void __launch_bounds__(THREADS) reduce_block(T* __restrict__ out, const T* __restrict__ x, RPlan p, int64_t chunk) {
    __shared__ T warp_part[THREADS / 32];
    int64_t o = blockIdx.x;
    int64_t k0 = static_cast<int64_t>(blockIdx.y) * chunk;
    int64_t k1 = min(k0 + chunk, p.len);
    const T* src = x + out_offset(p, o);
    T acc = ident<T>(OP);
    for (int64_t k = k0 + threadIdx.x; k < k1; k += THREADS) acc = fold<T, OP>(acc, src[k * p.astride]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc = fold<T, OP>(acc, shfl_down(acc, d));
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        acc = threadIdx.x < THREADS / 32 ? warp_part[threadIdx.x] : ident<T>(OP);
#pragma unroll
        for (int d = 4; d > 0; d >>= 1) acc = fold<T, OP>(acc, shfl_down(acc, d));
        if (threadIdx.x == 0) out[o * gridDim.y + blockIdx.y] = acc;
    }
}

// ---- generic ------------------------------------------------------------------------------------
template <class T, int OP>
__global__ void __launch_bounds__(THREADS) reduce_generic(T* __restrict__ out, const T* __restrict__ x, RPlan p) {
    int64_t o = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (o >= p.n_out) return;
    const T* src = x + out_offset(p, o);
    T acc = ident<T>(OP);
    for (int64_t k = 0; k < p.len; ++k) acc = fold<T, OP>(acc, src[k * p.astride]);
    out[o] = acc;
}

// ---- arg reductions -----------------------------------------------------------------------------
// Sequential rule: best = x[0]; x[k] replaces it only if strictly better.  A NaN at k > 0 never
// wins; a NaN at k = 0 is never beaten.
template <class T, bool IS_MAX> __device__ __forceinline__ bool better(T v, T best) { return IS_MAX ? v > best : v < best; }

template <class T, bool IS_MAX>
__global__ void __launch_bounds__(THREADS) argreduce_generic(int64_t* __restrict__ out, const T* __restrict__ x, RPlan p) {
    int64_t o = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (o >= p.n_out) return;
    const T* src = x + out_offset(p, o);
    int64_t bi = 0;
    if (p.len > 0) {
        T best = src[0];
        for (int64_t k = 1; k < p.len; ++k) {
            T v = src[k * p.astride];
            if (better<T, IS_MAX>(v, best)) { best = v; bi = k; }
        }
    }
    out[o] = bi;
}

// One block per output.  Each thread keeps (value, index) over its strided subset, seeded with
// "absent" (index = INT64_MAX); partials merge by (strictly better) or (equal and lower index).
template <class T, bool IS_MAX>
__global__ void __launch_bounds__(THREADS) argreduce_block(int64_t* __restrict__ out, const T* __restrict__ x, RPlan p) {
    __shared__ T sv[THREADS / 32];
    __shared__ int64_t si[THREADS / 32];
    int64_t o = blockIdx.x;
    const T* src = x + out_offset(p, o);
    T x0 = src[0];
    T bv = x0;
    int64_t bi = INT64_MAX;
    for (int64_t k = threadIdx.x; k < p.len; k += THREADS) {
        T v = src[k * p.astride];
        if (v != v) continue;  // NaN never wins (k = 0 is handled below)
        if (bi == INT64_MAX || better<T, IS_MAX>(v, bv)) { bv = v; bi = k; }
    }
    auto merge = [](T& av, int64_t& ai, T ov, int64_t oi) {
        if (oi == INT64_MAX) return;
        if (ai == INT64_MAX || better<T, IS_MAX>(ov, av) || (ov == av && oi < ai)) { av = ov; ai = oi; }
    };
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        T ov = shfl_down(bv, d);
        int64_t oi = shfl_down(bi, d);
        merge(bv, bi, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < THREADS / 32; ++w) merge(bv, bi, sv[w], si[w]);
        if (x0 != x0 || bi == INT64_MAX) bi = 0;
        out[o] = bi;
    }
}

template <class T>
__global__ void fill_kernel(T* out, int64_t n, T v) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (i < n) out[i] = v;
}

RPlan make_rplan(const WbView& x, int axis) {
    RPlan p{};
    p.len = x.shape[axis];
    p.astride = x.stride[axis];
    p.off = x.offset;
    int64_t size[WB_MAX_DIMS], st[WB_MAX_DIMS];
    int nd = 0;
    p.n_out = 1;
    for (int d = 0; d < x.ndim; ++d) {
        if (d == axis) continue;
        p.n_out *= x.shape[d];
        if (x.shape[d] == 1) continue;
        if (nd > 0 && st[nd - 1] == x.stride[d] * x.shape[d]) {
            size[nd - 1] *= x.shape[d];
            st[nd - 1] = x.stride[d];
        } else {
            size[nd] = x.shape[d];
            st[nd] = x.stride[d];
            ++nd;
        }
    }
    if (nd == 0) { size[0] = 1; st[0] = 0; nd = 1; }
    p.nd = nd;
    for (int d = 0; d < WB_MAX_DIMS; ++d) {
        p.size[d] = d < nd ? size[d] : 1;
        p.st[d] = d < nd ? st[d] : 0;
    }
    return p;
}

template <class T, int OP>
int reduce_value(WbBackend* be, const WbView& x, int axis, T* out) {
    RPlan p = make_rplan(x, axis);
    if (p.n_out == 0) return WB_OK;
    cudaStream_t st = be->stream;
    const T* xp = static_cast<const T*>(x.data);
    if (p.len == 0) {
        T v;
        if constexpr (std::is_same<T, int64_t>::value) v = OP == 0 ? 0 : (OP == 1 ? INT64_MIN : INT64_MAX);
        else v = OP == 0 ? T(0) : (OP == 1 ? -std::numeric_limits<T>::infinity() : std::numeric_limits<T>::infinity());
        fill_kernel<T><<<static_cast<unsigned>((p.n_out + THREADS - 1) / THREADS), THREADS, 0, st>>>(out, p.n_out, v);
        WB_LAUNCH_OK(be);
        return WB_OK;
    }
    const int64_t rows_max = sizeof(T) == 4 ? 1024 : 512;
    bool rows_adjacent = p.astride == 1 && (p.n_out == 1 || (p.nd == 1 && p.st[0] == p.len));
    // rows_smem: many short adjacent rows
    if (rows_adjacent && p.len <= rows_max && p.n_out >= 64) {
        int len = static_cast<int>(p.len);
        int budget = sizeof(T) == 4 ? 8192 : 4096;  // elements of shared memory per block
        int rpb = std::max(1, std::min(THREADS, budget / (len | 1)));
        size_t smem = static_cast<size_t>(rpb) * (len | 1) * sizeof(T);
        unsigned grid = static_cast<unsigned>((p.n_out + rpb - 1) / rpb);
        const int vec4 = sizeof(T) == 4 && len % 4 == 0 && (reinterpret_cast<uintptr_t>(xp + p.off) & 15) == 0;
        reduce_rows_smem<T, OP><<<grid, THREADS, smem, st>>>(out, xp + p.off, p.n_out, len, rpb, vec4);
        WB_LAUNCH_OK(be);
        return WB_OK;
    }
    // cols: innermost kept dim has unit stride and is wide enough to fill warps
    if (p.st[p.nd - 1] == 1 && p.size[p.nd - 1] >= 16) {
        int64_t col_blocks = (p.n_out + THREADS - 1) / THREADS;
        int64_t splits = 1;
        if (p.len >= 2048 && col_blocks < 2 * be->sm_count) {
            splits = std::min<int64_t>((4 * be->sm_count + col_blocks - 1) / col_blocks, p.len / 256);
            splits = std::max<int64_t>(1, std::min<int64_t>(splits, 1024));
        }
        int64_t chunk = (p.len + splits - 1) / splits;
        splits = (p.len + chunk - 1) / chunk;
        if (splits == 1) {
            reduce_cols<T, OP><<<dim3(static_cast<unsigned>(col_blocks), 1), THREADS, 0, st>>>(out, xp, p, chunk);
            WB_LAUNCH_OK(be);
            return WB_OK;
        }
        void* scratch = nullptr;
        WB_TRY(wb_scratch(be, static_cast<size_t>(splits * p.n_out) * sizeof(T), &scratch));
        T* part = static_cast<T*>(scratch);
        reduce_cols<T, OP><<<dim3(static_cast<unsigned>(col_blocks), static_cast<unsigned>(splits)), THREADS, 0, st>>>(part, xp, p, chunk);
        WB_LAUNCH_OK(be);
        RPlan q{};
        q.nd = 1; q.n_out = p.n_out; q.size[0] = p.n_out; q.st[0] = 1; q.off = 0; q.len = splits; q.astride = p.n_out;
        for (int d = 1; d < WB_MAX_DIMS; ++d) { q.size[d] = 1; q.st[d] = 0; }
        reduce_cols<T, OP><<<dim3(static_cast<unsigned>(col_blocks), 1), THREADS, 0, st>>>(out, part, q, splits);
        WB_LAUNCH_OK(be);
        return WB_OK;
    }
    if (p.len >= 128) {
        int64_t splits = 1;
        if (p.n_out < be->sm_count && p.len >= (int64_t(1) << 16)) {
            splits = std::min<int64_t>((4 * be->sm_count + p.n_out - 1) / p.n_out, p.len / 8192);
            splits = std::max<int64_t>(1, std::min<int64_t>(splits, 4096));
        }
        int64_t chunk = (p.len + splits - 1) / splits;
        splits = (p.len + chunk - 1) / chunk;
        WB_REQUIRE(p.n_out < (int64_t(1) << 31), WB_ERR_UNSUPPORTED, "reduce: too many outputs for one launch");
        if (splits == 1) {
            reduce_block<T, OP><<<dim3(static_cast<unsigned>(p.n_out), 1), THREADS, 0, st>>>(out, xp, p, chunk);
            WB_LAUNCH_OK(be);
            return WB_OK;
        }
        void* scratch = nullptr;
        WB_TRY(wb_scratch(be, static_cast<size_t>(splits * p.n_out) * sizeof(T), &scratch));
        T* part = static_cast<T*>(scratch);
        reduce_block<T, OP><<<dim3(static_cast<unsigned>(p.n_out), static_cast<unsigned>(splits)), THREADS, 0, st>>>(part, xp, p, chunk);
        WB_LAUNCH_OK(be);
        RPlan q{};
        q.nd = 1; q.n_out = p.n_out; q.size[0] = p.n_out; q.st[0] = splits; q.off = 0; q.len = splits; q.astride = 1;
        for (int d = 1; d < WB_MAX_DIMS; ++d) { q.size[d] = 1; q.st[d] = 0; }
        reduce_block<T, OP><<<dim3(static_cast<unsigned>(p.n_out), 1), THREADS, 0, st>>>(out, part, q, splits);
        WB_LAUNCH_OK(be);
        return WB_OK;
    }
    reduce_generic<T, OP><<<static_cast<unsigned>((p.n_out + THREADS - 1) / THREADS), THREADS, 0, st>>>(out, xp, p);
    WB_LAUNCH_OK(be);
    return WB_OK;
}

template <class T, bool IS_MAX>
int reduce_arg(WbBackend* be, const WbView& x, int axis, int64_t* out) {
    RPlan p = make_rplan(x, axis);
    if (p.n_out == 0) return WB_OK;
    cudaStream_t st = be->stream;
    const T* xp = static_cast<const T*>(x.data);
    if (p.len >= 512 && p.n_out < (int64_t(1) << 31) && !(p.st[p.nd - 1] == 1 && p.n_out >= 4096)) {
        argreduce_block<T, IS_MAX><<<static_cast<unsigned>(p.n_out), THREADS, 0, st>>>(out, xp, p);
    } else {
        argreduce_generic<T, IS_MAX><<<static_cast<unsigned>((p.n_out + THREADS - 1) / THREADS), THREADS, 0, st>>>(out, xp, p);
    }
    WB_LAUNCH_OK(be);
    return WB_OK;
}

template <class T>
int reduce_typed(WbBackend* be, int op, const WbView& x, int axis, void* out) {
    switch (op) {
        case WB_SUM: return reduce_value<T, 0>(be, x, axis, static_cast<T*>(out));
        case WB_MAX: return reduce_value<T, 1>(be, x, axis, static_cast<T*>(out));
        case WB_MIN: return reduce_value<T, 2>(be, x, axis, static_cast<T*>(out));
        case WB_ARGMAX: return reduce_arg<T, true>(be, x, axis, static_cast<int64_t*>(out));
        case WB_ARGMIN: return reduce_arg<T, false>(be, x, axis, static_cast<int64_t*>(out));
    }
    wb_set_error("reduce: unknown op code %d", op);
    return WB_ERR_INVALID;
}

}  // namespace

extern "C" int wb_reduce_into(WbBackend* b, int op, const WbView* x, int axis, void* out) {
    WB_REQUIRE(b && x && out, WB_ERR_INVALID, "wb_reduce: null pointer");
    WB_REQUIRE(axis >= 0 && axis < x->ndim && x->ndim <= WB_MAX_DIMS, WB_ERR_INVALID, "reduce: axis %d out of range for %d dims", axis, x->ndim);
    WbProfileScope ps(b, "reduce");
    switch (x->dtype) {
        case WB_F32: return reduce_typed<float>(b, op, *x, axis, out);
        case WB_F64: return reduce_typed<double>(b, op, *x, axis, out);
        case WB_I64: return reduce_typed<int64_t>(b, op, *x, axis, out);
    }
    wb_set_error("wb_reduce: unknown dtype %d", x->dtype);
    return WB_ERR_INVALID;
}

extern "C" int wb_reduce(WbBackend* b, int op, const WbView* x, int axis, WbStorage** out) {
    WB_REQUIRE(b && x && out, WB_ERR_INVALID, "wb_reduce: null pointer");
    WB_REQUIRE(axis >= 0 && axis < x->ndim, WB_ERR_INVALID, "reduce: axis %d out of range for %d dims", axis, x->ndim);
    int64_t n_out = 1;
    for (int d = 0; d < x->ndim; ++d)
        if (d != axis) n_out *= x->shape[d];
    int dt = (op == WB_ARGMAX || op == WB_ARGMIN) ? WB_I64 : x->dtype;
    WB_TRY(wb_new_storage(b, n_out, dt, out));
    int s = wb_reduce_into(b, op, x, axis, (*out)->ptr);
    if (s != WB_OK) { wb_free(b, *out); *out = nullptr; }
    return s;
}
