// Element-wise kernel templates shared by unary / binary / cast / copy.
//
// Three kernels cover every layout the trait can hand over:
//   ew_flat   : every operand is one contiguous (or stride-0) run          -> 128-bit loads/stores
//   ew_strided: collapsed rank <= 8, arbitrary strides; VEC consecutive outputs per thread share
//               one index decomposition; an operand with unit inner stride is read with one
//               128-bit load, a stride-0 operand with one scalar load
//   ew_tile   : an operand whose unit-stride dim is not the output's inner dim (a transposed
//               view) is staged through a 32x33 shared-memory tile so both its reads and the
//               output's writes are coalesced
// All arithmetic is done by a functor, so each op compiles to straight-line code.
#pragma once

#include <atomic>
#include "common.h"

namespace ew {

constexpr int THREADS = 256;

template <class T> struct VecOf;
template <> struct VecOf<float> { using type = float4; static constexpr int N = 4; };
template <> struct VecOf<double> { using type = double2; static constexpr int N = 2; };
template <> struct VecOf<int64_t> { using type = longlong2; static constexpr int N = 2; };

template <class T, int N> struct alignas(sizeof(T) * N) Pack { T v[N]; };

struct Plan {
    int nd;
    int64_t n;
    int64_t size[WB_MAX_DIMS];
    int64_t st[WB_PLAN_MAX_OPS][WB_MAX_DIMS];
    int64_t off[WB_PLAN_MAX_OPS];
    int mode[WB_PLAN_MAX_OPS];  // 0 scalar loads, 1 vector load (unit inner stride, aligned), 2 inner broadcast
    FastDiv fd[WB_MAX_DIMS];    // division by size[d] as a multiply and a shift (32-bit index space only)
};

// ---- flat ---------------------------------------------------------------------------------------
// Each block covers THREADS*VEC*UNROLL consecutive outputs.  bcast[o] != 0: operand o is a scalar.
template <class TI, class TO, int NOPS, int VEC, int UNROLL, class F>
__global__ void __launch_bounds__(THREADS) ew_flat(TO* __restrict__ out, const TI* __restrict__ a, const TI* __restrict__ b,
                                                    int64_t n, int bcast_a, int bcast_b, F f) {
    int64_t base = static_cast<int64_t>(blockIdx.x) * (THREADS * VEC * UNROLL) + threadIdx.x * VEC;
    Pack<TI, VEC> va[UNROLL], vb[UNROLL];
    TI sa = bcast_a ? a[0] : TI(0);
    TI sb = (NOPS > 1 && bcast_b) ? b[0] : TI(0);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        int64_t i = base + static_cast<int64_t>(u) * THREADS * VEC;
        if (i + VEC <= n) {
            if (!bcast_a) va[u] = *reinterpret_cast<const Pack<TI, VEC>*>(a + i);
            if (NOPS > 1 && !bcast_b) vb[u] = *reinterpret_cast<const Pack<TI, VEC>*>(b + i);
        }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        int64_t i = base + static_cast<int64_t>(u) * THREADS * VEC;
        if (i + VEC <= n) {
            Pack<TO, VEC> r;
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                TI x = bcast_a ? sa : va[u].v[k];
                if constexpr (NOPS > 1) {
                    TI y = bcast_b ? sb : vb[u].v[k];
                    r.v[k] = f(x, y);
                } else {
                    r.v[k] = f(x);
                }
            }
            *reinterpret_cast<Pack<TO, VEC>*>(out + i) = r;
        } else {
            for (int64_t j = i; j < n; ++j) {  // ragged tail
                TI x = bcast_a ? sa : a[j];
                if constexpr (NOPS > 1) {
                    TI y = bcast_b ? sb : b[j];
                    out[j] = f(x, y);
                } else {
                    out[j] = f(x);
                }
            }
        }
    }
}

// ---- strided ------------------------------------------------------------------------------------
template <class TI, class TO, int NOPS, int VEC, class IdxT, class F>
__global__ void __launch_bounds__(THREADS) ew_strided(TO* __restrict__ out, const TI* __restrict__ a,
                                                       const TI* __restrict__ b, Plan p, F f) {
    int64_t groups = p.n / VEC;
    int64_t g = static_cast<int64_t>(blockIdx.x) * THREADS + threadIdx.x;
    if (g >= groups) return;
    int64_t e0 = g * VEC;
    int64_t oa = p.off[0], ob = p.off[1];
    IdxT rem = static_cast<IdxT>(e0);
#pragma unroll 1
    for (int d = p.nd - 1; d >= 0; --d) {
        IdxT sz = static_cast<IdxT>(p.size[d]);
        IdxT q;
        if constexpr (sizeof(IdxT) == 4) q = p.fd[d].div(rem);
        else q = rem / sz;
        IdxT c = rem - q * sz;
        rem = q;
        oa += static_cast<int64_t>(c) * p.st[0][d];
        if (NOPS > 1) ob += static_cast<int64_t>(c) * p.st[1][d];
    }
    Pack<TI, VEC> va, vb;
    int64_t ia = p.st[0][p.nd - 1], ib = p.st[1][p.nd - 1];
    if (p.mode[0] == 1) va = *reinterpret_cast<const Pack<TI, VEC>*>(a + oa);
    else {
#pragma unroll
        for (int k = 0; k < VEC; ++k) va.v[k] = a[oa + k * ia];
    }
    if constexpr (NOPS > 1) {
        if (p.mode[1] == 1) vb = *reinterpret_cast<const Pack<TI, VEC>*>(b + ob);
        else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) vb.v[k] = b[ob + k * ib];
        }
    }
    Pack<TO, VEC> r;
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
        if constexpr (NOPS > 1) r.v[k] = f(va.v[k], vb.v[k]);
        else r.v[k] = f(va.v[k]);
    }
    *reinterpret_cast<Pack<TO, VEC>*>(out + e0) = r;
}

// ---- tile ---------------------------------------------------------------------------------------
// Output viewed as [..outer.., P, ..mid.., L] (collapsed dims).  `pd` is the dim along which the
// transposed operand(s) have unit stride; L is the output's inner dim.  A block owns a TILE(P) x
// TILE(L) tile for one setting of all other dims: transposed operands are read with threads running
// along P (coalesced), parked in shared memory, and consumed with threads running along L, so the
// output (and any operand that is already L-contiguous) is written/read coalesced as well.
// tmode[o]: 1 = operand o is read along P through shared memory, 0 = it is read along L directly.
constexpr int TILE = 64;
constexpr int TILE_THREADS = 256;
constexpr int TILE_ROWS = TILE_THREADS / TILE;  // 4 rows of the tile per pass, 16 passes

template <class TI, class TO, int NOPS, class F>
__global__ void __launch_bounds__(TILE_THREADS) ew_tile(TO* __restrict__ out, const TI* __restrict__ a, const TI* __restrict__ b, Plan p,
                                                        int pd, int tmode_a, int tmode_b, uint32_t tiles_p, uint32_t tiles_l, F f) {
    extern __shared__ __align__(16) unsigned char tile_raw[];
    TI(*sm)[TILE][TILE + 1] = reinterpret_cast<TI(*)[TILE][TILE + 1]>(tile_raw);
    const int L = p.nd - 1;
    uint32_t bid = blockIdx.x;
    const uint32_t tl = bid % tiles_l;
    bid /= tiles_l;
    const uint32_t tp = bid % tiles_p;
    bid /= tiles_p;
    // Remaining dims (all but pd and L), innermost first; `s` is the output stride of dim d.
    int64_t oa = p.off[0], ob = p.off[1], oo = 0, s = p.size[L], ostride_p = 0;
    for (int d = L - 1; d >= 0; --d) {
        const uint32_t sz = static_cast<uint32_t>(p.size[d]);
        if (d == pd) {
            ostride_p = s;
        } else {
            const uint32_t q = bid / sz, c = bid - q * sz;
            bid = q;
            oa += c * p.st[0][d];
            if (NOPS > 1) ob += c * p.st[1][d];
            oo += c * s;
        }
        s *= sz;
    }
    const int64_t p0 = static_cast<int64_t>(tp) * TILE, l0 = static_cast<int64_t>(tl) * TILE;
    const int tx = threadIdx.x % TILE, ty = threadIdx.x / TILE;
    const int64_t szp = p.size[pd], szl = p.size[L];
    const int64_t sap = p.st[0][pd], sal = p.st[0][L], sbp = p.st[1][pd], sbl = p.st[1][L];
    // Stage transposed operands: threads run along P (their unit-stride dim).
    if (tmode_a) {
        const int64_t pi = p0 + tx;
#pragma unroll 4
        for (int j = ty; j < TILE; j += TILE_ROWS) {
            const int64_t li = l0 + j;
            if (pi < szp && li < szl) sm[0][j][tx] = a[oa + pi * sap + li * sal];
        }
    }
    if constexpr (NOPS > 1) {
        if (tmode_b) {
            const int64_t pi = p0 + tx;
#pragma unroll 4
            for (int j = ty; j < TILE; j += TILE_ROWS) {
                const int64_t li = l0 + j;
                if (pi < szp && li < szl) sm[1][j][tx] = b[ob + pi * sbp + li * sbl];
            }
        }
    }
    __syncthreads();
    // Compute: threads run along L (the output's unit-stride dim).
    const int64_t li = l0 + tx;
    if (li < szl) {
#pragma unroll 4
        for (int j = ty; j < TILE; j += TILE_ROWS) {
            const int64_t pi = p0 + j;
            if (pi >= szp) break;
            TI x = tmode_a ? sm[0][tx][j] : a[oa + pi * sap + li * sal];
            TO r;
            if constexpr (NOPS > 1) {
                TI y = tmode_b ? sm[1][tx][j] : b[ob + pi * sbp + li * sbl];
                r = f(x, y);
            } else {
                r = f(x);
            }
            out[oo + pi * ostride_p + li] = r;
        }
    }
}

// Four-wide variant of ew_tile for 4-byte element types: 128-bit global loads along P for the transposed operands
// and 128-bit global loads / stores along L for everything else.  The tile sits in shared memory as sm[p][64] with
// the 16-byte group g = l / 4 of row p stored at group g ^ ((p / 4) & 7): the scalar stores of the staging phase (a
// warp covers 8 float4 columns of P by 4 rows of L) and the 128-bit loads of the compute phase are both free of bank
// conflicts.  Needs every size, stride and offset involved to be a multiple of 4 elements and 16-byte aligned base
// pointers (checked by the launcher).
template <class TI, class TO, int NOPS, int DEPTH, class F>
__global__ void __launch_bounds__(TILE_THREADS) ew_tile4(TO* __restrict__ out, const TI* __restrict__ a, const TI* __restrict__ b, Plan p,
                                                         int pd, int tmode_a, int tmode_b, uint32_t tiles_p, uint32_t tiles_l, int dd, F f) {
    constexpr int depth = DEPTH;
    static_assert(sizeof(TI) == 4 && sizeof(TO) == 4, "ew_tile4 is for 4-byte elements");
    static_assert(TILE == 64 && TILE_THREADS == 256, "the lane mappings below assume a 64 x 64 tile and 8 warps");
    extern __shared__ __align__(16) unsigned char tile_raw[];
    TI(*sm)[TILE][TILE] = reinterpret_cast<TI(*)[TILE][TILE]>(tile_raw);  // sm[o * depth + slice][p][swizzled l]
    const int L = p.nd - 1;
    uint32_t bid = blockIdx.x;
    const uint32_t tl = bid % tiles_l;
    bid /= tiles_l;
    const uint32_t tp = bid % tiles_p;
    bid /= tiles_p;
    // A block owns `depth` consecutive positions ("slices") of dim dd, the dim next to L: all their loads are issued
    // before any of their stores, so a transposed operand whose dd stride continues its P runs is read in runs `depth`
    // times as long, and the output (dd is its second-innermost dim) is written in runs `depth` tiles long.
    int64_t oa = p.off[0], ob = p.off[1], oo = 0, s = p.size[L], ostride_p = 0, ostride_d = 0;
    int slices = 1;
    for (int d = L - 1; d >= 0; --d) {
        const uint32_t sz = static_cast<uint32_t>(p.size[d]);
        if (d == pd) {
            ostride_p = s;
        } else {
            const uint32_t szb = d == dd ? (sz + depth - 1) / depth : sz;
            const uint32_t q = bid / szb;
            uint32_t c = bid - q * szb;
            bid = q;
            if (d == dd) {
                c *= depth;
                slices = min(depth, static_cast<int>(sz - c));
                ostride_d = s;
            }
            oa += c * p.st[0][d];
            if (NOPS > 1) ob += c * p.st[1][d];
            oo += c * s;
        }
        s *= sz;
    }
    const int64_t sad = dd >= 0 ? p.st[0][dd] : 0, sbd = dd >= 0 ? p.st[1][dd] : 0;
    const int64_t p0 = static_cast<int64_t>(tp) * TILE, l0 = static_cast<int64_t>(tl) * TILE;
    const int64_t szp = p.size[pd], szl = p.size[L];
    const int64_t sap = p.st[0][pd], sal = p.st[0][L], sbp = p.st[1][pd], sbl = p.st[1][L];
    using V4 = Pack<TI, 4>;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // Stage transposed operands: a thread loads 4 consecutive P positions of one L row (the operand's unit-stride dim is P).
    auto stage = [&](const TI* __restrict__ src, int64_t base, int64_t sl, int o) {  // o: index of the shared-memory tile
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int u = k * 8 + warp;                                   // 32 units of 4 L rows x 8 float4 columns
            const int lj = 4 * (u >> 1) + (lane >> 3), p4 = 8 * (u & 1) + (lane & 7);
            const int64_t pi = p0 + 4 * p4, li = l0 + lj;
            if (pi < szp && li < szl) {
                const V4 v = *reinterpret_cast<const V4*>(src + base + pi + li * sl);
                const int col = 4 * ((lj >> 2) ^ (p4 & 7)) + (lj & 3);    // (p / 4) & 7 == p4 & 7 for p = 4 * p4 + i
#pragma unroll
                for (int i = 0; i < 4; ++i) sm[o][4 * p4 + i][col] = v.v[i];
            }
        }
    };
    auto stage_slice = [&](int sl) {
        if (tmode_a) stage(a, oa + sl * sad, sal, sl);
        if constexpr (NOPS > 1) {
            if (tmode_b) stage(b, ob + sl * sbd, sbl, depth + sl);
        }
    };
    if constexpr (DEPTH == 1) {
        stage_slice(0);
    } else {
        // one slice after the other (measured: unrolling the slices into one batch of loads is slower, 0.62 against 0.83)
#pragma unroll 1
        for (int sl = 0; sl < slices; ++sl) stage_slice(sl);
    }
    __syncthreads();
    // Compute: a thread produces 4 consecutive L positions of one P row.
    auto compute_slice = [&](int sl) {
        const int64_t oas = oa + sl * sad, obs = ob + sl * sbd, oos = oo + sl * ostride_d;
#pragma unroll
        for (int k = 0; k < (TILE * TILE / 4) / TILE_THREADS; ++k) {
            const int idx = threadIdx.x + k * TILE_THREADS;
            const int pj = idx / (TILE / 4), l4 = idx % (TILE / 4);
            const int64_t pi = p0 + pj, li = l0 + 4 * l4;
            if (pi >= szp || li >= szl) continue;
            const int col = 4 * (l4 ^ ((pj >> 2) & 7));
            V4 x, y;
            if (tmode_a) {
                x = *reinterpret_cast<const V4*>(&sm[sl][pj][col]);
            } else if (sal == 1) {
                x = *reinterpret_cast<const V4*>(a + oas + pi * sap + li);
            } else {  // broadcast along L
                const TI v = a[oas + pi * sap];
                x.v[0] = x.v[1] = x.v[2] = x.v[3] = v;
            }
            Pack<TO, 4> r;
            if constexpr (NOPS > 1) {
                if (tmode_b) {
                    y = *reinterpret_cast<const V4*>(&sm[depth + sl][pj][col]);
                } else if (sbl == 1) {
                    y = *reinterpret_cast<const V4*>(b + obs + pi * sbp + li);
                } else {
                    const TI v = b[obs + pi * sbp];
                    y.v[0] = y.v[1] = y.v[2] = y.v[3] = v;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) r.v[i] = f(x.v[i], y.v[i]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) r.v[i] = f(x.v[i]);
            }
            *reinterpret_cast<Pack<TO, 4>*>(out + oos + pi * ostride_p + li) = r;
        }
    };
    if constexpr (DEPTH == 1) {
        compute_slice(0);
    } else {
#pragma unroll 1
        for (int sl = 0; sl < slices; ++sl) compute_slice(sl);
    }
}

// ---- host-side launcher -------------------------------------------------------------------------
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Launches f over the operands described by `plan` (built by wb_make_plan over NOPS views).
template <class TI, class TO, int NOPS, class F>
int launch(WbBackend* be, TO* out, const TI* a, const TI* b, const WbIterPlan& wp, F f) {
    if (wp.n == 0) return WB_OK;
    // Vector width: 16 bytes of the wider of the two element types.
    constexpr int VEC = 16 / (sizeof(TI) > sizeof(TO) ? sizeof(TI) : sizeof(TO));
    const int L = wp.nd - 1;
    cudaStream_t st = be->stream;
    // flat: one collapsed dim whose stride is 1 or 0 for every operand
    bool flat = wp.nd == 1;
    for (int o = 0; o < NOPS && flat; ++o) flat = wp.st[o][0] == 1 || wp.st[o][0] == 0 || wp.n == 1;
    if (flat) {
        const TI* pa = a + wp.off[0];
        const TI* pb = NOPS > 1 ? b + wp.off[1] : nullptr;
        int ba = wp.st[0][0] != 1 && wp.n > 1, bb = NOPS > 1 && wp.st[1][0] != 1 && wp.n > 1;
        if (wp.n == 1) { ba = 0; bb = 0; }
        bool vec_ok = aligned16(out) && (ba || aligned16(pa)) && (NOPS == 1 || bb || aligned16(pb));
        if (vec_ok) {
            constexpr int UNROLL = 4;
            int64_t per_block = THREADS * VEC * UNROLL;
            unsigned grid = static_cast<unsigned>((wp.n + per_block - 1) / per_block);
            ew_flat<TI, TO, NOPS, VEC, UNROLL, F><<<grid, THREADS, 0, st>>>(out, pa, pb, wp.n, ba, bb, f);
        } else {
            constexpr int UNROLL = 4;
            int64_t per_block = THREADS * UNROLL;
            unsigned grid = static_cast<unsigned>((wp.n + per_block - 1) / per_block);
            ew_flat<TI, TO, NOPS, 1, UNROLL, F><<<grid, THREADS, 0, st>>>(out, pa, pb, wp.n, ba, bb, f);
        }
        WB_LAUNCH_OK(be);
        return WB_OK;
    }
    Plan p;
    p.nd = wp.nd;
    p.n = wp.n;
    for (int d = 0; d < WB_MAX_DIMS; ++d) {
        p.size[d] = wp.size[d];
        for (int o = 0; o < WB_PLAN_MAX_OPS; ++o) p.st[o][d] = wp.st[o][d];
    }
    for (int o = 0; o < WB_PLAN_MAX_OPS; ++o) p.off[o] = wp.off[o];
    for (int d = 0; d < wp.nd; ++d)
        if (wp.size[d] >= 1 && wp.size[d] < (int64_t(1) << 32)) p.fd[d] = FastDiv(static_cast<uint32_t>(wp.size[d]));
    // tile: some operand has a non-unit, non-zero inner stride but unit stride along another dim
    // that is reasonably long; the other operands must be readable along L (inner stride 1 or 0)
    // or share that unit-stride dim.
    int pd = -1;
    bool tile_ok = wp.size[L] >= 8;
    int tmode[WB_PLAN_MAX_OPS] = {0, 0, 0};
    for (int o = 0; o < NOPS && tile_ok; ++o) {
        int64_t is = wp.st[o][L];
        if (is == 1 || is == 0) continue;
        int found = -1;
        for (int d = 0; d < L; ++d)
            if (wp.st[o][d] == 1 && wp.size[d] >= 8) found = d;
        if (found < 0 || (pd >= 0 && pd != found)) tile_ok = false;
        else { pd = found; tmode[o] = 1; }
    }
    if (tile_ok && pd >= 0) {
        int64_t tiles_p = (wp.size[pd] + TILE - 1) / TILE, tiles_l = (wp.size[L] + TILE - 1) / TILE;
        int64_t rest = wp.n / (wp.size[pd] * wp.size[L]);
        int64_t blocks = tiles_p * tiles_l * rest;
        if (blocks < (int64_t(1) << 31)) {
            constexpr size_t tile_smem = sizeof(TI) * NOPS * TILE * (TILE + 1);
            auto kern = ew_tile<TI, TO, NOPS, F>;
            if (tile_smem > 48 * 1024) {
                static std::atomic<uint64_t> attr_done{0};  // one flag per instantiation and device ordinal
                const uint64_t bit = uint64_t(1) << (be->ordinal & 63);
                if (!(attr_done.load(std::memory_order_acquire) & bit)) {
                    WB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(tile_smem)));
                    attr_done.fetch_or(bit, std::memory_order_release);
                }
            }
            // 128-bit variant: 4-byte elements, every size / stride / offset a multiple of 4 where a vector is formed
            bool v4 = false;
            if constexpr (sizeof(TI) == 4 && sizeof(TO) == 4) {
                v4 = wp.size[pd] % 4 == 0 && wp.size[L] % 4 == 0 && aligned16(out);
                const TI* ptrs[2] = {a, b};
                for (int o = 0; o < NOPS && v4; ++o) {
                    v4 = aligned16(ptrs[o]) && wp.off[o] % 4 == 0;
                    for (int d = 0; d <= L && v4; ++d) {
                        const int64_t sd = wp.st[o][d];
                        // the dim the vector runs along has stride 1 (or 0 for a broadcast read along L); all others step by multiples of 4
                        const bool vec_dim = tmode[o] ? d == pd : d == L;
                        if (vec_dim) v4 = sd == 1 || (!tmode[o] && sd == 0);
                        else v4 = sd % 4 == 0;
                    }
                }
            }
            if (v4) {
                if constexpr (sizeof(TI) == 4 && sizeof(TO) == 4) {
                    // Two positions of the dim next to L per block (see the kernel) for unary ops and for binary ops whose
                    // operands are both transposed: transpose(1, 3) of [256, 64, 56, 56] went from 0.76 to 0.85 (ReLU) and
                    // from 0.60 to 0.79 (add, mul) of the copy bandwidth.  Four positions measured slower (0.78 for ReLU),
                    // and with one transposed and one inner-contiguous operand two are slower than one.
                    const int dd = (L >= 1 && L - 1 != pd) ? L - 1 : -1;
                    const bool deep = (NOPS == 1 || (tmode[0] && tmode[1])) && dd >= 0 && wp.size[dd] >= 2;
                    const int depth = deep ? 2 : 1;
                    const size_t smem4 = sizeof(TI) * NOPS * depth * TILE * TILE;
                    const int64_t blocks4 = deep ? blocks / wp.size[dd] * ((wp.size[dd] + depth - 1) / depth) : blocks;
                    if (deep && smem4 > 48 * 1024) {
                        static std::atomic<uint64_t> attr4_done{0};
                        const uint64_t bit = uint64_t(1) << (be->ordinal & 63);
                        if (!(attr4_done.load(std::memory_order_acquire) & bit)) {
                            WB_CHECK_CUDA(cudaFuncSetAttribute(ew_tile4<TI, TO, NOPS, 2, F>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem4)));
                            attr4_done.fetch_or(bit, std::memory_order_release);
                        }
                    }
                    if (deep)
                        ew_tile4<TI, TO, NOPS, 2, F><<<static_cast<unsigned>(blocks4), TILE_THREADS, smem4, st>>>(
                            out, a, b, p, pd, tmode[0], tmode[1], static_cast<uint32_t>(tiles_p), static_cast<uint32_t>(tiles_l), dd, f);
                    else
                        ew_tile4<TI, TO, NOPS, 1, F><<<static_cast<unsigned>(blocks4), TILE_THREADS, smem4, st>>>(
                            out, a, b, p, pd, tmode[0], tmode[1], static_cast<uint32_t>(tiles_p), static_cast<uint32_t>(tiles_l), -1, f);
                }
            } else {
                kern<<<static_cast<unsigned>(blocks), TILE_THREADS, tile_smem, st>>>(out, a, b, p, pd, tmode[0], tmode[1],
                                                                                     static_cast<uint32_t>(tiles_p), static_cast<uint32_t>(tiles_l), f);
            }
            WB_LAUNCH_OK(be);
            return WB_OK;
        }
    }
    // strided
    bool vec = wp.size[L] % VEC == 0 && aligned16(out);
    const TI* ptrs[2] = {a, b};
    for (int o = 0; o < NOPS; ++o) {
        int64_t is = wp.st[o][L];
        p.mode[o] = 0;
        if (is == 1 && vec) {
            bool ok = aligned16(ptrs[o]) && wp.off[o] % VEC == 0;
            for (int d = 0; d < L; ++d) ok = ok && wp.st[o][d] % VEC == 0;
            p.mode[o] = ok ? 1 : 0;
        }
    }
    bool small = wp.n < (int64_t(1) << 31);
    if (vec) {
        int64_t groups = wp.n / VEC;
        unsigned grid = static_cast<unsigned>((groups + THREADS - 1) / THREADS);
        if (small) ew_strided<TI, TO, NOPS, VEC, uint32_t, F><<<grid, THREADS, 0, st>>>(out, a, b, p, f);
        else ew_strided<TI, TO, NOPS, VEC, int64_t, F><<<grid, THREADS, 0, st>>>(out, a, b, p, f);
    } else {
        p.mode[0] = p.mode[1] = 0;
        unsigned grid = static_cast<unsigned>((wp.n + THREADS - 1) / THREADS);
        if (small) ew_strided<TI, TO, NOPS, 1, uint32_t, F><<<grid, THREADS, 0, st>>>(out, a, b, p, f);
        else ew_strided<TI, TO, NOPS, 1, int64_t, F><<<grid, THREADS, 0, st>>>(out, a, b, p, f);
    }
    WB_LAUNCH_OK(be);
    return WB_OK;
}

}  // namespace ew
