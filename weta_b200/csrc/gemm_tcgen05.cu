// Backend::matmul (crates/weta-core/src/backend.rs:87) and the internal GEMM service used by the
// fused Linear / conv2d entry points.
//
// The reference hands every f32/f64 product to cuBLAS after classifying each operand as
// "readable in place" or "copy first" (crates/weta-cuda/src/lib.rs:331-349, 603-628).  Here the
// same classification picks between the tcgen05 TF32 kernel (tc_gemm.cuh), which reads row-major,
// transposed and batch-broadcast operands in place through TMA, and the CUDA-core tiles
// (matmul_simt.cu) for f64, tiny problems and layouts TMA cannot describe.
#include <cuda.h>

#include <atomic>

#include "tc_gemm.cuh"
#include "gemm.h"

int wb_matmul_simt(WbBackend* be, const WbView* a, const WbView* b, void* out);

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct GemmState {
    EncodeFn encode = nullptr;
    int* error_flag = nullptr;       // device
    int* error_host = nullptr;       // pinned
    bool attrs_set = false;
};

int get_state(WbBackend* b, GemmState** out) {
    if (!b->gemm_state) {
        GemmState* st = new GemmState();
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
            delete st;
            (void)cudaGetLastError();
            wb_set_error("cuTensorMapEncodeTiled is not available from this driver");
            return WB_ERR_CUDA;
        }
        st->encode = reinterpret_cast<EncodeFn>(fn);
        WB_CHECK_CUDA(cudaMalloc(&st->error_flag, sizeof(int)));
        WB_CHECK_CUDA(cudaMemsetAsync(st->error_flag, 0, sizeof(int), b->stream));
        WB_CHECK_CUDA(cudaMallocHost(&st->error_host, sizeof(int)));
        *st->error_host = 0;
        b->gemm_state = st;
    }
    *out = static_cast<GemmState*>(b->gemm_state);
    return WB_OK;
}

}  // namespace

void wb_gemm_state_destroy(WbBackend* b) {
    if (!b->gemm_state) return;
    GemmState* st = static_cast<GemmState*>(b->gemm_state);
    if (st->error_flag) cudaFree(st->error_flag);
    if (st->error_host) cudaFreeHost(st->error_host);
    delete st;
    b->gemm_state = nullptr;
}


namespace {

bool operand_ok(const WbGemmOperand& o, int64_t batch) {
    if ((reinterpret_cast<uintptr_t>(o.ptr) & 15) != 0) return false;
    int64_t outer = o.mn_major ? o.k : o.rows;
    if (outer > 1 && o.ld % 4 != 0) return false;
    int64_t inner = o.mn_major ? o.rows : o.k;
    if (o.ld < inner && outer > 1) return false;
    if (batch > 1 && o.batch_stride != 0 && o.batch_stride % 4 != 0) return false;
    return true;
}

int make_map(GemmState* st, const WbGemmOperand& o, int64_t batch, int box_rows, CUtensorMap* map) {
    const int64_t inner = o.mn_major ? o.rows : o.k;
    const int64_t outer = o.mn_major ? o.k : o.rows;
    const int64_t nb = (o.batch_stride != 0) ? batch : 1;
    int64_t ld = o.ld;
    if (outer <= 1) ld = (inner + 3) / 4 * 4;  // pitch is irrelevant for a single row, but must be 16-byte granular
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer), static_cast<cuuint64_t>(nb)};
    int64_t bstride = nb > 1 ? o.batch_stride : outer * ld;
    if (bstride % 4 != 0 || bstride <= 0) bstride = (outer * ld + 3) / 4 * 4;
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 4, static_cast<cuuint64_t>(bstride) * 4};
    cuuint32_t box[3] = {32u, static_cast<cuuint32_t>(o.mn_major ? tc::BK : box_rows), 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = st->encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(o.ptr), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, o.mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        wb_set_error("cuTensorMapEncodeTiled failed with %d (inner %lld, outer %lld, ld %lld, batch %lld)", static_cast<int>(r),
                     (long long)inner, (long long)outer, (long long)ld, (long long)nb);
        return WB_ERR_CUDA;
    }
    return WB_OK;
}

// Split-K finish: out = epilogue(sum over splits of partial).
__global__ void __launch_bounds__(256) splitk_reduce(const float* __restrict__ part, int splits, int64_t split_stride, int64_t total,
                                                     int m, int n, tc::Epilogue ep) {
    wb_pdl_enter();
    int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total) return;
    int64_t per = static_cast<int64_t>(m) * n;
    int64_t batch = i / per, r = i % per;
    int row = static_cast<int>(r / n), col = static_cast<int>(r % n);
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += part[s * split_stride + i];
    if (ep.bias_m) acc += ep.bias_m[row];
    if (ep.bias_n) acc += ep.bias_n[col];
    if (ep.relu) acc = fmaxf(acc, 0.f);
    float* dst = ep.out + batch * ep.batch_stride_d + static_cast<int64_t>(row) * ep.ldd + col;
    *dst = ep.accumulate ? *dst + acc : acc;
}

// The same for many splits over a small output: one warp per output element, lanes over the splits (each lane adds its
// splits in ascending order, the lanes' sums are combined by a fixed shuffle tree: one order, every run).
__global__ void __launch_bounds__(256) splitk_reduce_warp(const float* __restrict__ part, int splits, int64_t split_stride, int64_t total,
                                                          int m, int n, tc::Epilogue ep) {
    wb_pdl_enter();
    const int64_t i = (static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (i >= total) return;
    float acc = 0.f;
    for (int s = lane; s < splits; s += 32) acc += part[s * split_stride + i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if (lane != 0) return;
    const int64_t per = static_cast<int64_t>(m) * n;
    const int64_t batch = i / per, r = i % per;
    const int row = static_cast<int>(r / n), col = static_cast<int>(r % n);
    if (ep.bias_m) acc += ep.bias_m[row];
    if (ep.bias_n) acc += ep.bias_n[col];
    if (ep.relu) acc = fmaxf(acc, 0.f);
    float* dst = ep.out + batch * ep.batch_stride_d + static_cast<int64_t>(row) * ep.ldd + col;
    *dst = ep.accumulate ? *dst + acc : acc;
}

// hi = x with the 13 low mantissa bits cleared (exactly a tf32 value), lo = x - hi (exact in f32).
__global__ void __launch_bounds__(256) split_hi_lo(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo,
                                                   int64_t nb, int64_t outer, int64_t inner, int64_t bs, int64_t ld, int64_t inner_p) {
    wb_pdl_enter();
    int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    int64_t total = nb * outer * inner_p;
    if (i >= total) return;
    int64_t c = i % inner_p, t = i / inner_p;
    int64_t r = t % outer, bz = t / outer;
    float v = c < inner ? x[bz * bs + r * ld + c] : 0.f;
    float h = __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    hi[i] = h;
    lo[i] = v - h;
}

template <int BN, int STAGES, bool A_MN, bool B_MN, int CTAS, int EPW = 8, int MT = 1, int HALO = 0, int CSPLIT = 0>
int launch_tc(WbBackend* be, GemmState* st, const tc::Args& args, dim3 grid) {
    using SS = tc::SharedStorage<BN, STAGES, CTAS, EPW, MT, HALO>;
    constexpr size_t smem = sizeof(SS) + 1024;
    static_assert(smem <= 227 * 1024, "shared-memory ring does not fit");
    auto kern = tc::gemm_tf32_kernel<BN, STAGES, A_MN, B_MN, CTAS, EPW, MT, HALO, CSPLIT>;
    // The attribute belongs to the device's context: one flag per device ordinal and instantiation.
    static std::atomic<uint64_t> attr_done{0};
    const uint64_t bit = uint64_t(1) << (be->ordinal & 63);
    if (!(attr_done.load(std::memory_order_acquire) & bit)) {
        WB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attr_done.fetch_or(bit, std::memory_order_release);
    }
    // Every launch is a programmatic dependent of the kernel before it in the stream (the kernel waits with
    // griddepcontrol.wait after its preamble, see tc_gemm.cuh); CTA pairs and cluster split-K add the cluster size
    // (2; args.splits).
    const bool no_pdl = !wb_pdl_allowed();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(tc::threads_for(EPW));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = be->stream;
    cudaLaunchAttribute attrs[2]{};
    unsigned na = 0;
    if (CTAS == 2 || CSPLIT != 0) {
        attrs[na].id = cudaLaunchAttributeClusterDimension;
        attrs[na].val.clusterDim.x = CSPLIT ? static_cast<unsigned>(args.splits) : 2u;  // grid.x is a multiple of it
        attrs[na].val.clusterDim.y = 1;
        attrs[na].val.clusterDim.z = 1;
        ++na;
    }
    if (!no_pdl) {
        attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = na;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        wb_set_error("launch of the tensor-core GEMM failed: %s", cudaGetErrorString(e));
        return WB_ERR_CUDA;
    }
    WB_LAUNCH_OK(be);
    return WB_OK;
}

// Two CTAs per 256 x 256 tile when the output has more than one 128-row block: a third fewer operand bytes per
// flop through L2, which is what bounds these contractions.  WETA_B200_NO_PAIRS=1 keeps single-CTA tiles.
bool pair_mode(int m, int BN) {
    static const bool off = [] { const char* e = std::getenv("WETA_B200_NO_PAIRS"); return e && e[0] == '1'; }();
    return !off && BN == 256 && m > tc::BM;
}

// How many clusters of `c` CTAs of the cluster split-K kernel the GPU holds at once (every instantiation has the same
// block size and shared memory, so one of them is asked); looked up once per cluster size.
int max_clusters_128(WbBackend* be, int c) {
    static std::atomic<int> cached[9] = {};
    int v = cached[c].load(std::memory_order_acquire);
    if (v) return v - 1;
    using SS = tc::SharedStorage<128, 5, 1, 8, 1, 0>;
    auto kern = tc::gemm_tf32_kernel<128, 5, false, false, 1, 8, 1, 0, 1>;
    int n = 0;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(c));
    cfg.blockDim = dim3(tc::threads_for(8));
    cfg.dynamicSmemBytes = sizeof(SS) + 1024;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = static_cast<unsigned>(c);
    attr.val.clusterDim.y = attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(cfg.dynamicSmemBytes)) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        n = 0;
    }
    cached[c].store(n + 1, std::memory_order_release);
    (void)be;
    return n;
}

// Common tail of every tensor-core contraction: tile count, split-K decision and workspace, launch of
// the persistent kernel, split-K finish.  `args` arrives with its tensor maps, k_blocks and mode fields set.
int run_tiles(WbBackend* be, GemmState* st, tc::Args& args, int m, int n, int64_t grid_batch, int BN, bool pair, bool amn, bool bmn,
              const tc::Epilogue& ep, int force_splits, bool two_blocks = false, bool shared_taps = false, bool three_blocks = false) {
    args.m = m;
    args.n = n;
    args.error_flag = st->error_flag;
    // pair: CTA pairs on 256-row tiles; the caller sized the B tensor map's box for it (BN / 2 rows per CTA).
    // two_blocks: a single CTA owns two 128-row blocks that share every B box (256-wide tiles, long contractions).
    two_blocks = two_blocks && !pair && BN == 256;
    const int tile_m = (pair || two_blocks) ? 2 * tc::BM : tc::BM;
    const int workers = pair ? be->sm_count / 2 : be->sm_count;  // CTAs or CTA pairs that walk the tile list
    const int tiles_m = (m + tile_m - 1) / tile_m, tiles_n = (n + BN - 1) / BN;
    const int64_t tiles = static_cast<int64_t>(tiles_m) * tiles_n * grid_batch;
    int splits = 1;
    if (ep.row_stats) force_splits = 1;  // row statistics come from finished values, not split-K partials
    // Split-K inside a cluster (see tc_gemm.cuh) for plain 128 x 128 tiles that leave most SMs idle: the largest of
    // 8, 4, 2 CTAs per tile that the GPU can hold at once, with at least two K blocks each, for contractions of at most
    // 64 (K block, segment) iterations; longer ones are faster split more than 8 ways with the separate reduction
    // (the 422k-parameter CNN's step went from 232 to 316 us when they took this path too).  Measured: 512^3 TF32
    // 12.4 / 10.7 / 14.5 -> 10.4 us (3xTF32 32.9 / 28.8 / 39.1 -> 22.7 / 20.6 / 22.7), the MLP's captured step 136 -> 131 us.
    // WETA_B200_NO_CLUSTER_SPLITK=1 keeps the two-launch form.
    static const bool cluster_off = [] { const char* e = std::getenv("WETA_B200_NO_CLUSTER_SPLITK"); return e && e[0] == '1'; }();
    int cluster_splits = 0;
    if (!cluster_off && force_splits <= 0 && BN == 128 && !pair && !two_blocks && !shared_taps && !three_blocks && tiles * 2 <= workers &&
        static_cast<int64_t>(args.k_blocks) * args.num_segments <= 64) {
        for (int c = 8; c >= 2 && !cluster_splits; c /= 2)
            if (tiles * c <= workers && tiles <= max_clusters_128(be, c) && args.k_blocks >= 2 * c) cluster_splits = c;
    }
    if (cluster_splits) splits = cluster_splits;
    else if (force_splits > 0) splits = force_splits;
    else if (tiles * 2 <= workers && args.k_blocks >= 16) {
        // A rough cost in microseconds per candidate: pipeline fill + this split's share of the (K block, segment)
        // iterations + a reduction pass that reads every split's partial result.  Measured anchors: a 25-block TF32
        // product (the MLP's first layer) is faster unsplit, its 3xTF32 form (75 iterations) and the 128-block logits
        // weight gradient are faster split 4-16 ways.
        const int64_t max_s = std::min<int64_t>(workers / tiles, args.k_blocks / 4);
        const double iters = static_cast<double>(args.k_blocks) * args.num_segments;
        const double out_mb = static_cast<double>(grid_batch) * m * n * 4.0 / 1e6;
        const double t_iter = two_blocks ? 0.55 : (BN == 256 ? 0.28 : 0.13);  // one iteration of a 2 x 128 x 256, a 256-wide and a 128 x 128 tile
        double best = 3.0 + iters * t_iter;
        for (int64_t c = 2; c <= max_s; ++c) {
            const double cost = 3.0 + iters / c * t_iter + 3.0 + c * out_mb * 0.5;
            if (cost < best) { best = cost; splits = static_cast<int>(c); }
        }
    }
    splits = std::max(1, std::min(splits, args.k_blocks));
    if (!cluster_splits) {
        // Make every split non-empty.
        int per = (args.k_blocks + splits - 1) / splits;
        splits = (args.k_blocks + per - 1) / per;
    }
    args.splits = splits;
    int status = WB_OK;
    void* part = nullptr;
    size_t kp = 0;
    if (splits > 1 && !cluster_splits) {
        const int64_t per_split = grid_batch * static_cast<int64_t>(m) * n;
        status = wb_arena_alloc(be, static_cast<size_t>(per_split) * splits * sizeof(float), &part, &kp);
        if (status == WB_OK) {
            args.ep = tc::Epilogue{static_cast<float*>(part), n, static_cast<int64_t>(m) * n, nullptr, nullptr, 0, 0};
            args.split_stride_d = per_split;
        }
    } else {
        args.ep = ep;
        args.split_stride_d = 0;
    }
    if (status == WB_OK) {
        args.tiles_m = tiles_m;
        args.tiles_n = tiles_n;
        args.div_tiles_m = FastDiv(static_cast<uint32_t>(tiles_m));
        args.div_tiles_n = FastDiv(static_cast<uint32_t>(tiles_n));
        args.div_splits = FastDiv(static_cast<uint32_t>(splits));
        const int64_t total_tiles = tiles * splits;
        if (total_tiles >= (int64_t(1) << 31)) {
            wb_set_error("gemm: too many tiles");
            status = WB_ERR_UNSUPPORTED;
        }
        args.total_tiles = static_cast<int>(total_tiles);
        dim3 grid(static_cast<unsigned>(std::min<int64_t>(total_tiles, workers) * (pair ? 2 : 1)));  // cluster split-K: total_tiles <= workers
        // Shared memory: a 192 KB ring (6 x 32 KB per CTA of a pair, 4 x 48 KB for BN = 256, 5 x 32 KB for BN = 128)
        // + 32 KB epilogue staging; one persistent CTA per SM.
        if (status != WB_OK) {
        } else if (three_blocks) {
            // conv_mode 3: three row blocks (kernel columns) per 128 x 128 tile, 3 x 64 KB ring
            status = launch_tc<128, 3, false, true, 1, 8, 3>(be, st, args, grid);
        } else if (shared_taps && !pair && splits == 1 && BN == 256 && !amn && bmn) {
            // Implicit convolution on 16-pixel-wide images, 128-row tiles: the taps of a kernel column share their pixel
            // copies (a fifth fewer operand bytes through L2; the input gradient of the 128 -> 256 channel layer went
            // from 511 to 618 TFLOP/s).  The ring slots grow by one 4 KB chunk and the staging shrinks to four warps'.
            // CTA pairs gain nothing from it (607 against 610 TFLOP/s on that layer's forward, with 5 slots for 6).
            status = launch_tc<256, 4, false, true, 1, 4, 1, 1>(be, st, args, grid);
        } else if (pair) {
            if (!amn && !bmn) status = launch_tc<256, 6, false, false, 2>(be, st, args, grid);
            else if (!amn && bmn) status = launch_tc<256, 6, false, true, 2>(be, st, args, grid);
            else if (amn && !bmn) status = launch_tc<256, 6, true, false, 2>(be, st, args, grid);
            else status = launch_tc<256, 6, true, true, 2>(be, st, args, grid);
        } else if (two_blocks) {
            // 3 x 64 KB ring: two A row blocks and one 256-row B box per K block.
            if (!amn && !bmn) status = launch_tc<256, 3, false, false, 1, 8, 2>(be, st, args, grid);
            else if (!amn && bmn) status = launch_tc<256, 3, false, true, 1, 8, 2>(be, st, args, grid);
            else if (amn && !bmn) status = launch_tc<256, 3, true, false, 1, 8, 2>(be, st, args, grid);
            else status = launch_tc<256, 3, true, true, 1, 8, 2>(be, st, args, grid);
        } else if (BN == 256 && args.k_blocks * args.num_segments <= 2 && !amn) {
            // One or two K blocks per tile: the epilogue is the whole cost, so it gets 16 warps; a ring of three slots
            // (conv1 forward at batch 4096: 0.524 ms with two, 0.496 ms with three).  Compiling the common case of the
            // epilogue (no column bias, no ReLU, vector stores) without its per-value tests made it slower
            // (0.570 ms: more spills at this variant's 96 registers), so there is one general form.
            if (!bmn) status = launch_tc<256, 3, false, false, 1, 16>(be, st, args, grid);
            else status = launch_tc<256, 3, false, true, 1, 16>(be, st, args, grid);
        } else if (BN == 256) {
            if (!amn && !bmn) status = launch_tc<256, 4, false, false, 1>(be, st, args, grid);
            else if (!amn && bmn) status = launch_tc<256, 4, false, true, 1>(be, st, args, grid);
            else if (amn && !bmn) status = launch_tc<256, 4, true, false, 1>(be, st, args, grid);
            else status = launch_tc<256, 4, true, true, 1>(be, st, args, grid);
        } else if (cluster_splits) {
            if (!amn && !bmn) status = launch_tc<128, 5, false, false, 1, 8, 1, 0, 1>(be, st, args, grid);
            else if (!amn && bmn) status = launch_tc<128, 5, false, true, 1, 8, 1, 0, 1>(be, st, args, grid);
            else if (amn && !bmn) status = launch_tc<128, 5, true, false, 1, 8, 1, 0, 1>(be, st, args, grid);
            else status = launch_tc<128, 5, true, true, 1, 8, 1, 0, 1>(be, st, args, grid);
        } else {
            if (!amn && !bmn) status = launch_tc<128, 5, false, false, 1>(be, st, args, grid);
            else if (!amn && bmn) status = launch_tc<128, 5, false, true, 1>(be, st, args, grid);
            else if (amn && !bmn) status = launch_tc<128, 5, true, false, 1>(be, st, args, grid);
            else status = launch_tc<128, 5, true, true, 1>(be, st, args, grid);
        }
    }
    if (status == WB_OK && splits > 1 && !cluster_splits) {
        const int64_t total = grid_batch * static_cast<int64_t>(m) * n;
        if (splits >= 32 && total <= (1 << 16))
            wb_launch_pdl(splitk_reduce_warp, dim3(static_cast<unsigned>((total * 32 + 255) / 256)), dim3(256), 0, be->stream, static_cast<const float*>(part), splits,
                                                                                                      total, total, m, n, ep);
        else
            wb_launch_pdl(splitk_reduce, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, be->stream, static_cast<const float*>(part), splits, total,
                                                                                            total, m, n, ep);
        cudaError_t e = cudaPeekAtLastError();
        if (e != cudaSuccess) { wb_set_error("split-K reduce launch failed: %s", cudaGetErrorString(e)); status = WB_ERR_CUDA; }
        else be->launches++;
    }
    if (part) wb_arena_free(be, part, kp);
    return status;
}

}  // namespace

// A 3-D tensor map of f32 elements for kernels outside this file (conv1_bwd_fused.cu): dims / box innermost first,
// strides in bytes for dimensions 1 and 2; 128-byte swizzle (K-major operand tiles) or none.
int wb_tc_encode(WbBackend* be, const float* ptr, const uint64_t dims[3], const uint64_t strides[2], const uint32_t box[3], bool swizzle128,
                 CUtensorMap* map) {
    GemmState* st = nullptr;
    WB_TRY(get_state(be, &st));
    cuuint64_t d[3] = {dims[0], dims[1], dims[2]};
    cuuint64_t sb[2] = {strides[0], strides[1]};
    cuuint32_t bx[3] = {box[0], box[1], box[2]};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = st->encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), d, sb, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        wb_set_error("cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
        return WB_ERR_CUDA;
    }
    return WB_OK;
}

// The device flag the tensor-core kernels raise when a bounded wait runs out (read by wb_gemm_check).
int wb_tc_error_flag(WbBackend* be, int** flag) {
    GemmState* st = nullptr;
    WB_TRY(get_state(be, &st));
    *flag = st->error_flag;
    return WB_OK;
}

// Runs D = A x B (+ epilogue) on the tensor cores.  mode: WB_MM_TF32 or WB_MM_TF32X3.
// Returns WB_ERR_UNSUPPORTED (without setting an error message) if an operand cannot be read by TMA.
// span_batch > 0: A and B are batched K-major operands of `span_batch` images and the contraction
// runs over (image, k) pairs, giving one un-batched [m, n] result (a convolution's weight gradient).
int wb_tc_gemm(WbBackend* be, WbGemmOperand A, WbGemmOperand B, int64_t batch_in, int m, int n, int k, tc::Epilogue ep, int mode,
               int force_splits, int64_t span_batch) {
    const int64_t batch = span_batch > 0 ? span_batch : batch_in;  // images the tensor maps cover
    const int64_t grid_batch = span_batch > 0 ? 1 : batch_in;      // independent outputs
    if (span_batch > 0 && (A.mn_major || B.mn_major || A.batch_stride == 0 || B.batch_stride == 0)) return WB_ERR_UNSUPPORTED;
    if (!operand_ok(A, batch) || !operand_ok(B, batch)) return WB_ERR_UNSUPPORTED;
    GemmState* st = nullptr;
    WB_TRY(get_state(be, &st));
    // 128 x 256 tiles when the output is wide enough: half the A traffic and twice the MMA work per pipeline
    // stage; 128 x 128 otherwise.  (128-wide tiles for one-K-block contractions, with four accumulators in
    // flight, measured slower than 256-wide ones.)
    int BN = n > 128 ? 256 : 128;
    {
        // Small outputs: with 256-wide tiles a 512^3 product keeps 16 SMs busy; 128-wide tiles keep four times as many
        // (16.0 -> 19.7 TFLOP/s, cuBLAS: 23).  WETA_B200_WIDE_TILES=1 keeps the wide tiles (diagnostic).
        static const bool wide = [] { const char* e = std::getenv("WETA_B200_WIDE_TILES"); return e && e[0] == '1'; }();
        const int64_t tiles256 = static_cast<int64_t>((m + 255) / 256) * ((n + 255) / 256) * grid_batch;
        // (short contractions only: with a long K the 256-wide pair tiles and split-K win, fc1 forward at batch 512:
        // 47 against 57 us)
        if (!wide && BN == 256 && tiles256 * 8 <= be->sm_count && (k + tc::BK - 1) / tc::BK <= 64 && span_batch <= 0) BN = 128;
    }
    // 256 x 256 tiles come in two forms: a CTA pair, or one CTA with two row blocks (better sustained rate: 641 /
    // 681 / 532 against 583 / 645 / 475 TFLOP/s on 4096^3 NN / NT / TN; but its epilogue does not overlap the next
    // tile).  The single-CTA form is taken when the contraction is long and there are enough tiles to fill the GPU
    // without split-K.
    const int64_t kb_total = (static_cast<int64_t>(k) + tc::BK - 1) / tc::BK * (span_batch > 0 ? span_batch : 1);
    const int64_t big_tiles = static_cast<int64_t>((m + 255) / 256) * ((n + 255) / 256) * grid_batch;
    const bool two_blocks = pair_mode(m, BN) && kb_total >= 64 && big_tiles >= be->sm_count;
    const bool pair = pair_mode(m, BN) && !two_blocks;
    const int b_box = pair ? BN / 2 : BN;  // B rows one CTA loads per K block
    tc::Args args{};
    void *hi_a = nullptr, *hi_b = nullptr;
    size_t ka = 0, kb = 0;
    WbGemmOperand Ah = A, Al = A, Bh = B, Bl = B;
    if (mode == WB_MM_TF32X3) {
        auto split = [&](const WbGemmOperand& o, WbGemmOperand& oh, WbGemmOperand& ol, void** buf, size_t* klass) -> int {
            int64_t inner = o.mn_major ? o.rows : o.k, outer = o.mn_major ? o.k : o.rows;
            int64_t nb = o.batch_stride != 0 ? batch : 1;
            int64_t inner_p = (inner + 3) / 4 * 4;
            int64_t count = nb * outer * inner_p;
            WB_TRY(wb_arena_alloc(be, static_cast<size_t>(2 * count) * sizeof(float), buf, klass));
            float* h = static_cast<float*>(*buf);
            float* l = h + count;
            wb_launch_pdl(split_hi_lo, dim3(static_cast<unsigned>((count + 255) / 256)), dim3(256), 0, be->stream, o.ptr, h, l, nb, outer, inner, o.batch_stride,
                                                                                          o.ld, inner_p);
            WB_LAUNCH_OK(be);
            oh = o; ol = o;
            oh.ptr = h; ol.ptr = l;
            oh.ld = ol.ld = inner_p;
            oh.batch_stride = ol.batch_stride = (o.batch_stride != 0) ? outer * inner_p : 0;
            return WB_OK;
        };
        WB_TRY(split(A, Ah, Al, &hi_a, &ka));
        int s2 = split(B, Bh, Bl, &hi_b, &kb);
        if (s2 != WB_OK) { wb_arena_free(be, hi_a, ka); return s2; }
        args.num_segments = 3;
        int s = make_map(st, Ah, batch, tc::BM, &args.seg[0].a);
        if (s == WB_OK) s = make_map(st, Bh, batch, b_box, &args.seg[0].b);
        if (s == WB_OK) s = make_map(st, Ah, batch, tc::BM, &args.seg[1].a);
        if (s == WB_OK) s = make_map(st, Bl, batch, b_box, &args.seg[1].b);
        if (s == WB_OK) s = make_map(st, Al, batch, tc::BM, &args.seg[2].a);
        if (s == WB_OK) s = make_map(st, Bh, batch, b_box, &args.seg[2].b);
        if (s != WB_OK) { wb_arena_free(be, hi_a, ka); wb_arena_free(be, hi_b, kb); return s; }
    } else {
        args.num_segments = 1;
        WB_TRY(make_map(st, A, batch, tc::BM, &args.seg[0].a));
        WB_TRY(make_map(st, B, batch, b_box, &args.seg[0].b));
    }
    args.k_blocks = (k + tc::BK - 1) / tc::BK;
    args.kpb = 0;
    if (span_batch > 0) {
        args.kpb = args.k_blocks;
        WB_REQUIRE(span_batch * args.kpb < (int64_t(1) << 31), WB_ERR_UNSUPPORTED, "gemm: contraction too long");
        args.k_blocks = static_cast<int>(span_batch * args.kpb);
    }
    args.batched_a = A.batch_stride != 0;
    args.batched_b = B.batch_stride != 0;
    int status = run_tiles(be, st, args, m, n, grid_batch, BN, pair, A.mn_major, B.mn_major, ep, force_splits, two_blocks);
    if (hi_a) wb_arena_free(be, hi_a, ka);
    if (hi_b) wb_arena_free(be, hi_b, kb);
    return status;
}

// Implicit-GEMM 3x3 / stride 1 / padding 1 convolution pieces over NCHW tensors (see tc::Args::conv_mode).
// img[kx] is the image tensor [batch][ch][h][w] shifted horizontally by kx-1 with zeros shifted in
// (img[kx][y][x] = image[y][x+kx-1]; img[1] is the tensor itself).
//   mode 1: D[batch][m][h*w] = Wr[m][tap][ch] (x) windows(img) (+ epilogue).  Forward with Wr = weights as [O][tap][C];
//           input gradient with img = dY and Wr = weights as [C][flipped tap][O].
//   mode 2: D[tap][ch][m] = sum over images and pixels of window_tap(img)[ch][px] * a[img][m][px]  (the weight gradient, a = dY).
//   mode 3: mode 1's result from img[1] alone (img[0], img[2] unused): the input gradient without shifted copies of dY.
// Requirements (else WB_ERR_UNSUPPORTED, no message): w and h*w multiples of 4, ch a multiple of 32 (mode 1)
// or of 128 (mode 2), 16-byte aligned pointers.
// conv_mode 3 needs image rows that tile the accumulator's 32-column chunks and 128-pixel tiles that end on row ends.
bool wb_tc_conv_mode3_ok(int64_t ch, int64_t h, int64_t w, int64_t m) {
    static const bool off = [] { const char* e = std::getenv("WETA_B200_SHIFTED_DGRAD"); return e && e[0] == '1'; }();
    return !off && (w == 4 || w == 8 || w == 16 || w == 32) && (h * w) % 128 == 0 && ch % 32 == 0 && m > 0;
}

int wb_tc_conv_gemm(WbBackend* be, int mode, const float* a, const float* const img[3], int64_t batch, int64_t ch, int64_t h, int64_t w, int m,
                    tc::Epilogue ep) {
    const int64_t hw = h * w;
    if (w % 4 != 0 || hw % 4 != 0 || hw >= (int64_t(1) << 30)) return WB_ERR_UNSUPPORTED;
    if (mode == 2 ? ch % 128 != 0 : ch % 32 != 0) return WB_ERR_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(img[1]) & 15)) return WB_ERR_UNSUPPORTED;
    if (mode != 3 && ((reinterpret_cast<uintptr_t>(img[0]) & 15) || (reinterpret_cast<uintptr_t>(img[2]) & 15))) return WB_ERR_UNSUPPORTED;
    GemmState* st = nullptr;
    WB_TRY(get_state(be, &st));
    tc::Args args{};
    args.num_segments = 1;
    args.conv_mode = mode;
    args.conv_w = static_cast<int>(w);
    if (mode == 3) {
        // Input gradient from the unshifted gradient tensor alone (img[1]); see tc::Args::conv_mode.
        if (!wb_tc_conv_mode3_ok(ch, h, w, m) || ep.bias_m || ep.bias_n || ep.row_stats || ep.relu || ep.accumulate) return WB_ERR_UNSUPPORTED;
        const int64_t k = 9 * ch;
        WbGemmOperand A{a, m, k, k, 0, false};
        WB_TRY(make_map(st, A, 1, tc::BM, &args.seg[0].a));
        WbGemmOperand B{img[1], hw, ch, hw, ch * hw, true};
        WB_TRY(make_map(st, B, batch, 128, &args.seg[0].b));
        args.k_blocks = static_cast<int>(3 * (ch / 32));
        args.conv_cb = static_cast<int>(ch / 32);
        args.batched_a = 0;
        args.batched_b = 1;
        return run_tiles(be, st, args, m, static_cast<int>(hw), batch, 128, false, false, true, ep, 1, false, false, true);
    }
    if (mode == 1) {
        const int BN = hw > 128 ? 256 : 128;
        const int64_t k = 9 * ch;
        WbGemmOperand A{a, m, k, k, 0, false};
        WB_TRY(make_map(st, A, 1, tc::BM, &args.seg[0].a));
        for (int kx = 0; kx < 3; ++kx) {
            WbGemmOperand B{img[kx], hw, ch, hw, ch * hw, true};
            WB_TRY(make_map(st, B, batch, BN, &args.seg[kx].b));
        }
        args.k_blocks = static_cast<int>(k / tc::BK);
        args.conv_cb = static_cast<int>(ch / 32);
        args.batched_a = 0;
        args.batched_b = 1;
        static const bool no_shared_taps = [] { const char* e = std::getenv("WETA_B200_NO_SHARED_TAPS"); return e && e[0] == '1'; }();
        return run_tiles(be, st, args, m, static_cast<int>(hw), batch, BN, pair_mode(m, BN), false, true, ep, 1, false, w == 16 && !no_shared_taps);
    }
    const int BN = m > 128 ? 256 : 128;
    for (int kx = 0; kx < 3; ++kx) {
        WbGemmOperand A{img[kx], ch, hw, hw, ch * hw, false};
        WB_TRY(make_map(st, A, batch, tc::BM, &args.seg[kx].a));
    }
    args.kpb = static_cast<int>((hw + tc::BK - 1) / tc::BK);
    WB_REQUIRE(batch * args.kpb < (int64_t(1) << 31), WB_ERR_UNSUPPORTED, "conv weight gradient: contraction too long");
    args.k_blocks = static_cast<int>(batch * args.kpb);
    args.conv_cb = static_cast<int>(ch / tc::BM);
    args.batched_a = 1;
    args.batched_b = 1;
    // Rows come in blocks of BM = 128 (tap, channel block).  One CTA takes two blocks per tile, sharing every dY box
    // between them (the last tile of an odd block count - 9 blocks for 128 channels - holds one block and skips
    // the second block's loads and MMAs).  Measured on the 128 -> 256 channel layer at batch 4096: 0.97 ms, against
    // 1.22 ms for one block per CTA and 1.40 ms for CTA pairs (whose odd block idles half a tile for the whole
    // contraction; handing the odd block to a second launch re-reads all of dY for a ninth of the work).
    const int blocks = static_cast<int>(9 * ch / tc::BM);
    const bool pair = false;
    WbGemmOperand B{a, m, hw, hw, static_cast<int64_t>(m) * hw, false};
    WB_TRY(make_map(st, B, batch, pair ? BN / 2 : BN, &args.seg[0].b));
    return run_tiles(be, st, args, blocks * tc::BM, m, 1, BN, pair, false, false, ep, 0, /*two_blocks=*/pair_mode(blocks * tc::BM, BN));
}

// One thread waits, with the GEMM kernels' own bounded mbar_wait, on a shared-memory barrier that nothing ever
// arrives at (no copy or MMA is in flight), gives up after `polls` polls and raises the error flag the way the
// GEMM kernels do.
__global__ void mbar_timeout_selftest_kernel(int* error_flag, uint32_t polls) {
    __shared__ alignas(8) uint64_t bar;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!tc::mbar_wait(&bar, 0, polls)) atomicExch(error_flag, 1);
    }
}

// Test hook of the bounded pipeline waits: after this call wb_gemm_check reports WB_ERR_TIMEOUT (and clears the flag),
// exactly as it would after a tensor-core kernel had given up on a barrier; the context stays usable.
extern "C" int wb_gemm_selftest_timeout(WbBackend* b, int polls) {
    WB_REQUIRE(b && polls > 0 && polls <= (1 << 20), WB_ERR_INVALID, "wb_gemm_selftest_timeout: polls must be 1..2^20");
    GemmState* st = nullptr;
    WB_TRY(get_state(b, &st));
    mbar_timeout_selftest_kernel<<<1, 32, 0, b->stream>>>(st->error_flag, static_cast<uint32_t>(polls));
    WB_LAUNCH_OK(b);
    return WB_OK;
}

// Reads the device-side error flag the GEMM kernels raise when a bounded wait runs out.
// Synchronises the stream; meant for tests and for wb_synchronize-style checkpoints.
extern "C" int wb_gemm_check(WbBackend* b) {
    if (!b->gemm_state) return WB_OK;
    GemmState* st = static_cast<GemmState*>(b->gemm_state);
    WB_CHECK_CUDA(cudaMemcpyAsync(st->error_host, st->error_flag, sizeof(int), cudaMemcpyDeviceToHost, b->stream));
    WB_CHECK_CUDA(cudaStreamSynchronize(b->stream));
    if (*st->error_host != 0) {
        cudaMemsetAsync(st->error_flag, 0, sizeof(int), b->stream);
        wb_set_error("a tensor-core GEMM gave up waiting on a pipeline barrier");
        return WB_ERR_TIMEOUT;
    }
    return WB_OK;
}

extern "C" int wb_matmul_into(WbBackend* b, const WbView* a, const WbView* bb, void* out) {
    WB_REQUIRE(b && a && bb && out, WB_ERR_INVALID, "wb_matmul: null pointer");
    WB_REQUIRE(a->ndim == 3 && bb->ndim == 3, WB_ERR_INVALID, "matmul: expected [B,M,K] x [B,K,N] views");
    WB_REQUIRE(a->dtype == bb->dtype, WB_ERR_INVALID, "matmul: dtype mismatch");
    WB_REQUIRE(a->dtype == WB_F32 || a->dtype == WB_F64, WB_ERR_UNSUPPORTED, "matmul: unsupported dtype i64");
    WB_REQUIRE(a->shape[0] == bb->shape[0] && a->shape[2] == bb->shape[1], WB_ERR_INVALID,
               "matmul: [%lld,%lld,%lld] x [%lld,%lld,%lld] do not contract", (long long)a->shape[0], (long long)a->shape[1],
               (long long)a->shape[2], (long long)bb->shape[0], (long long)bb->shape[1], (long long)bb->shape[2]);
    WbProfileScope ps(b, "matmul");
    const int64_t bs = a->shape[0], m = a->shape[1], k = a->shape[2], n = bb->shape[2];
    if (bs * m * n == 0) return WB_OK;
    const bool big = m * n * k >= (int64_t(1) << 18) && k >= 16 && m < (int64_t(1) << 31) && n < (int64_t(1) << 31) && k < (int64_t(1) << 31);
    if (a->dtype == WB_F32 && b->matmul_mode != WB_MM_FP32 && big) {
        // Operand classification, as gemm_operand does for cuBLAS (crates/weta-cuda/src/lib.rs:331-349).
        WbGemmOperand A{static_cast<const float*>(a->data) + a->offset, m, k, 0, a->stride[0], false};
        WbGemmOperand B{static_cast<const float*>(bb->data) + bb->offset, n, k, 0, bb->stride[0], false};
        bool ok = true;
        if (a->stride[2] == 1 || k == 1) { A.mn_major = false; A.ld = a->stride[1]; }
        else if (a->stride[1] == 1 || m == 1) { A.mn_major = true; A.ld = a->stride[2]; }
        else ok = false;
        if (bb->stride[1] == 1 || k == 1) { B.mn_major = false; B.ld = bb->stride[2]; }
        else if (bb->stride[2] == 1 || n == 1) { B.mn_major = true; B.ld = bb->stride[1]; }
        else ok = false;
        if (bs == 1) { A.batch_stride = 0; B.batch_stride = 0; }
        if (ok) {
            tc::Epilogue ep{static_cast<float*>(out), n, m * n, nullptr, nullptr, 0, 0};
            int s = wb_tc_gemm(b, A, B, bs, static_cast<int>(m), static_cast<int>(n), static_cast<int>(k), ep, b->matmul_mode, 0, 0);
            if (s != WB_ERR_UNSUPPORTED) return s;
        }
    }
    return wb_matmul_simt(b, a, bb, out);
}

extern "C" int wb_matmul(WbBackend* b, const WbView* a, const WbView* bb, WbStorage** out) {
    WB_REQUIRE(b && a && bb && out, WB_ERR_INVALID, "wb_matmul: null pointer");
    WB_REQUIRE(a->ndim == 3 && bb->ndim == 3, WB_ERR_INVALID, "matmul: expected [B,M,K] x [B,K,N] views");
    WB_TRY(wb_new_storage(b, a->shape[0] * a->shape[1] * bb->shape[2], a->dtype, out));
    int s = wb_matmul_into(b, a, bb, (*out)->ptr);
    if (s != WB_OK) { wb_free(b, *out); *out = nullptr; }
    return s;
}
