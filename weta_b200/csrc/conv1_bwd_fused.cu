// Backward of the first convolution block without its 2 GB gradient tensor.
//
// For the block conv -> BatchNorm -> ReLU -> MaxPool(2) that opens a network, the gradient of the convolution's output
// (dconv = the BatchNorm+ReLU+pool backward's dx) has two consumers only: the convolution's weight gradient
//     dW[o][k] = sum over images and pixels of dconv[o][px] * cols[k][px]      (MatmulBw, crates/weta-autograd/src/ops.rs:821-827)
// and its bias gradient, the sum of dconv over images and pixels (ops.rs:46-58); there is no input gradient to
// compute.  With 3 input channels the contraction of the forward pass is 27 values long, so both passes over that
// tensor are pure HBM traffic: the stand-alone kernels write it (one activation's worth) and the GEMM reads it back.
// This kernel produces each 128-channel x 64-pixel piece of dconv in shared memory, in the layout the tensor core
// reads, and multiplies it with the matching piece of the im2col matrix at once:
//
//   warp 0      TMA: per step (one image, two image rows = 64 pixels) the conv output x [128][64], the pooled
//               gradient [128][16] and two im2col boxes [32][32] into a ring of three slots
//   warps 2-17  the BatchNorm+ReLU+pool backward of wb_bn_relu_pool_bwd (fused_bn.cu), same arithmetic, one 2x2 window
//               per thread and round, from the slot into two K-major 128 x 32 operand tiles (128-byte swizzle, written
//               with the same chunk permutation TMA gave the x boxes), then a proxy fence and an mbarrier arrival
//   warp 1      tcgen05.mma kind::tf32, M = 128 channels, N = 32 im2col rows (27 used), K = 32 pixels per tile, into
//               one 32-column TMEM accumulator that lives for the whole launch (the contraction runs over all of a
//               CTA's steps); its commits hand the slots back
// Each CTA walks a contiguous range of steps and leaves a partial dW [128][32] and partial bias sums; a second
// kernel adds the CTAs' partials in a fixed order.  Every mbarrier wait is bounded (tc::mbar_wait): on expiry the role
// raises the GEMM error flag and leaves, the other roles run out the same way, TMEM is released.
#include <cuda.h>

#include <atomic>

#include "gemm.h"

namespace {

constexpr int TW = 16;                      // transform warps: eight channels each
constexpr int THREADS = 64 + 32 * TW;
constexpr int RAW = 3, AST = 2;             // ring depths: loaded slots, operand-tile slots
constexpr int CH = 128, PXT = 32, NK = 32;  // channels (M), pixels per operand tile (K), im2col rows per tile (N)

struct Smem {
    alignas(1024) float x[RAW][2][CH * PXT];    // two boxes per step: image rows 2r and 2r + 1, [channel][32 px], 128-byte swizzle
    alignas(1024) float cols[RAW][2][NK * PXT];  // [im2col row][32 px] of the same two image rows
    alignas(1024) float a[AST][2][CH * PXT];     // dconv tiles of the two image rows
    alignas(128) float g[RAW][CH * 16];          // pooled gradient [channel][16 windows]
    float consts[CH][8];                         // mean, rstd, gamma, beta, -dbeta/count, -dgamma/count, gamma*rstd
    alignas(8) uint64_t raw_full[RAW];
    uint64_t raw_empty[RAW], a_full[AST], a_empty[AST], acc_full;
    uint32_t tmem_base;
};

struct Args {
    CUtensorMap map_x, map_g, map_cols;
    const float *mean, *rstd, *gamma, *beta, *dgamma, *dbeta;
    float inv_count;
    int n_img, pairs_per_img;     // image-row pairs per image (h / 2)
    int64_t steps;                // n_img * pairs_per_img
    float* part;                  // [gridDim.x][128][32] partial dW
    double* bias_part;            // [gridDim.x][128] partial sums of dconv
    int* error_flag;
};

__global__ void __launch_bounds__(THREADS, 1) conv1_bwd_fused_kernel(const __grid_constant__ Args args) {
    wb_pdl_enter();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    Smem& ss = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t per = (args.steps + gridDim.x - 1) / gridDim.x;
    const int64_t s0 = min(args.steps, static_cast<int64_t>(blockIdx.x) * per), s1 = min(args.steps, s0 + per);
    const int my_steps = static_cast<int>(s1 - s0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < RAW; ++s) {
            tc::mbar_init(&ss.raw_full[s], 1);
            tc::mbar_init(&ss.raw_empty[s], TW + 1);  // the transform warps (x, g) and the MMA's commit (cols)
        }
        for (int a = 0; a < AST; ++a) {
            tc::mbar_init(&ss.a_full[a], TW);
            tc::mbar_init(&ss.a_empty[a], 1);
        }
        tc::mbar_init(&ss.acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < CH) {
        const int c = threadIdx.x;
        const float m = args.mean[c], r = args.rstd[c], g = args.gamma[c], b = args.beta[c];
        ss.consts[c][0] = m;
        ss.consts[c][1] = r;
        ss.consts[c][2] = g;
        ss.consts[c][3] = b;
        ss.consts[c][4] = -(args.dbeta[c] * args.inv_count);
        ss.consts[c][5] = -(args.dgamma[c] * args.inv_count);
        ss.consts[c][6] = g * r;
        ss.consts[c][7] = 0.f;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc::smem_u32(&ss.tmem_base)), "r"(32) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = ss.tmem_base;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ------------------------------------------------------------------------------
            for (int it = 0; it < my_steps; ++it) {
                const int s = it % RAW;
                if (!tc::mbar_wait(&ss.raw_empty[s], ((it / RAW) & 1) ^ 1)) { ok = false; break; }
                const int64_t step = s0 + it;
                const int img = static_cast<int>(step / args.pairs_per_img), rp = static_cast<int>(step - static_cast<int64_t>(img) * args.pairs_per_img);
                tc::mbar_expect_tx(&ss.raw_full[s], static_cast<uint32_t>((2 * CH * PXT + 2 * NK * PXT + CH * 16) * sizeof(float)));
                for (int j = 0; j < 2; ++j) {
                    tc::tma_load_3d(&ss.x[s][j][0], &args.map_x, &ss.raw_full[s], rp * 64 + j * 32, 0, img);
                    tc::tma_load_3d(&ss.cols[s][j][0], &args.map_cols, &ss.raw_full[s], rp * 64 + j * 32, 0, img);
                }
                tc::tma_load_3d(&ss.g[s][0], &args.map_g, &ss.raw_full[s], rp * 16, 0, img);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- MMA issuer ----------------------------------------------------------------------------------
            constexpr uint32_t idesc = tc::make_idesc(CH, NK, 0, 0);
            for (int it = 0; it < my_steps; ++it) {
                const int s = it % RAW, a = it % AST;
                if (!tc::mbar_wait(&ss.raw_full[s], (it / RAW) & 1)) { ok = false; break; }
                if (!tc::mbar_wait(&ss.a_full[a], (it / AST) & 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t a_base = tc::smem_u32(&ss.a[a][j][0]), b_base = tc::smem_u32(&ss.cols[s][j][0]);
#pragma unroll
                    for (int ks = 0; ks < PXT / tc::UMMA_K; ++ks)
                        tc::umma_tf32(tmem_base, tc::make_smem_desc(a_base + ks * 32, 16, 1024, 2), tc::make_smem_desc(b_base + ks * 32, 16, 1024, 2),
                                      idesc, (it > 0 || j > 0 || ks > 0) ? 1u : 0u);
                }
                tc::umma_commit(&ss.a_empty[a]);
                tc::umma_commit(&ss.raw_empty[s]);
            }
            if (ok) tc::umma_commit(&ss.acc_full);
        }
    } else {
        // ---- transform warps: dconv of the step's 128 x 64 piece into the operand tiles ---------------------
        const int tw = warp - 2;
        const int l = lane & 15, hi = lane >> 4;
        constexpr int IT = CH / (2 * TW);  // rounds per step: two channels per warp and round
        // this thread's channels never change: their constants live in registers
        float cm[IT], cr[IT], cg[IT], cb[IT], cnk1[IT], cnk2[IT], cgr[IT];
        float bias_acc[IT];
        double bias_sum[IT];
#pragma unroll
        for (int i = 0; i < IT; ++i) {
            const int c = 2 * IT * tw + 2 * i + hi;
            cm[i] = ss.consts[c][0]; cr[i] = ss.consts[c][1]; cg[i] = ss.consts[c][2]; cb[i] = ss.consts[c][3];
            cnk1[i] = ss.consts[c][4]; cnk2[i] = ss.consts[c][5]; cgr[i] = ss.consts[c][6];
            bias_acc[i] = 0.f;
            bias_sum[i] = 0.0;
        }
        for (int it = 0; it < my_steps && ok; ++it) {
            const int s = it % RAW, a = it % AST;
            if (!tc::mbar_wait(&ss.raw_full[s], (it / RAW) & 1)) { ok = false; break; }
            if (!tc::mbar_wait(&ss.a_empty[a], ((it / AST) & 1) ^ 1)) { ok = false; break; }
            const float* x0 = &ss.x[s][0][0];
            const float* x1 = &ss.x[s][1][0];
            const float* gs = &ss.g[s][0];
            float* a0 = &ss.a[a][0][0];
            float* a1 = &ss.a[a][1][0];
#pragma unroll
            for (int i = 0; i < IT; ++i) {
                const int c = 2 * IT * tw + 2 * i + hi;
                // pixels 2l, 2l + 1 of the channel's 128-byte row: 16-byte chunk l / 2 sits at chunk (l / 2) ^ (c & 7)
                const int off = c * PXT + ((((l >> 1) ^ (c & 7)) << 2) | ((l & 1) << 1));
                const float2 r0 = *reinterpret_cast<const float2*>(x0 + off);
                const float2 r1 = *reinterpret_cast<const float2*>(x1 + off);
                const float gy = gs[c * 16 + l];
                const float m = cm[i], r = cr[i], g = cg[i], b = cb[i], negk1 = cnk1[i], negk2 = cnk2[i], gr = cgr[i];
                const float v[4] = {r0.x, r0.y, r1.x, r1.y};
                float xh[4], act[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    xh[k] = __fmul_rn(__fadd_rn(v[k], -m), r);
                    act[k] = fmaxf(__fmaf_rn(xh[k], g, b), 0.f);
                }
                // Ties share the gradient; a window whose maximum is 0 receives nothing (as bn_relu_pool_bwd_pair_kernel).
                const float bx = fmaxf(fmaxf(act[0], act[1]), fmaxf(act[2], act[3]));
                const int cnt = (act[0] == bx) + (act[1] == bx) + (act[2] == bx) + (act[3] == bx);
                const float inv = cnt == 1 ? 1.f : (cnt == 2 ? 0.5f : (cnt == 3 ? (1.f / 3.f) : 0.25f));
                const float sh = bx > 0.f ? __fmul_rn(inv, gy) : 0.f;
                float d[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float go = act[k] == bx ? sh : 0.f;
                    d[k] = __fmul_rn(gr, __fmaf_rn(xh[k], negk2, __fadd_rn(go, negk1)));
                    bias_acc[i] = __fadd_rn(bias_acc[i], d[k]);
                }
                *reinterpret_cast<float2*>(a0 + off) = make_float2(d[0], d[1]);
                *reinterpret_cast<float2*>(a1 + off) = make_float2(d[2], d[3]);
            }
            if ((it & 31) == 31) {  // keep the f32 partial sums short
#pragma unroll
                for (int i = 0; i < IT; ++i) { bias_sum[i] += static_cast<double>(bias_acc[i]); bias_acc[i] = 0.f; }
            }
            // the tiles were written through the generic proxy; the tensor core reads them through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                tc::mbar_arrive(&ss.a_full[a]);
                tc::mbar_arrive(&ss.raw_empty[s]);
            }
        }
        // bias partials: the 16 lanes of a half-warp hold the 16 windows of one channel's row pair
#pragma unroll
        for (int i = 0; i < IT; ++i) {
            double t = bias_sum[i] + static_cast<double>(bias_acc[i]);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) t += __shfl_down_sync(0xffffffffu, t, o, 16);
            if (l == 0) args.bias_part[static_cast<int64_t>(blockIdx.x) * CH + 2 * IT * tw + 2 * i + hi] = t;
        }
        // ---- the accumulator: four of the warps read 32 lanes each ------------------------------------------
        if (tw < 4) {
            const int lg = warp & 3;  // the TMEM lanes this warp may read
            float* dst = args.part + (static_cast<int64_t>(blockIdx.x) * CH + lg * 32 + lane) * NK;
            uint32_t raw[32];
            bool have = false;
            if (my_steps > 0 && ok) {
                if (tc::mbar_wait(&ss.acc_full, 0)) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    tc::tmem_ld32_issue(tmem_base + (static_cast<uint32_t>(lg * 32) << 16), raw);
                    tc::tmem_ld_wait();
                    have = true;
                } else {
                    ok = false;
                }
            }
#pragma unroll
            for (int q = 0; q < 8; ++q)
                reinterpret_cast<float4*>(dst)[q] = have ? make_float4(__uint_as_float(raw[4 * q]), __uint_as_float(raw[4 * q + 1]),
                                                                       __uint_as_float(raw[4 * q + 2]), __uint_as_float(raw[4 * q + 3]))
                                                         : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    if (!ok) {
        atomicExch(args.error_flag, 1);
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000) {}  // copies and MMAs still in flight finish before the CTA retires
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32) : "memory");
}

// dW[o][k] and the bias gradient from the CTAs' partials: one warp per output, lanes over the CTAs in ascending
// order, a fixed shuffle tree.
__global__ void __launch_bounds__(256) conv1_bwd_reduce_kernel(const float* __restrict__ part, const double* __restrict__ bias_part, int ctas, int ck,
                                                               float* __restrict__ dweight, float* __restrict__ dbias) {
    wb_pdl_enter();
    const int item = (blockIdx.x * 256 + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (item < CH * ck) {
        const int o = item / ck, k = item - o * ck;
        float acc = 0.f;
        for (int s = lane; s < ctas; s += 32) acc += part[(static_cast<int64_t>(s) * CH + o) * NK + k];
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, sh);
        if (lane == 0) dweight[item] = acc;
    } else if (item < CH * ck + CH && dbias) {
        const int o = item - CH * ck;
        double acc = 0.0;
        for (int s = lane; s < ctas; s += 32) acc += bias_part[static_cast<int64_t>(s) * CH + o];
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, sh);
        if (lane == 0) dbias[o] = static_cast<float>(acc);
    }
}

}  // namespace

// The shapes the kernel is written for: 128 output channels, image rows of 32 pixels (one operand tile per row), an
// even height, at most 32 im2col rows; 16-byte aligned tensors.
bool wb_conv1_bwd_fused_ok(int64_t n, int64_t cout, int64_t h, int64_t w, int64_t ck, const float* x, const float* dy_pooled, const float* cols) {
    const char* e = std::getenv("WETA_B200_NO_FUSED_CONV1_BWD");  // read at every call: a test compares both paths in one process
    const bool off = e && e[0] == '1';
    return !off && cout == CH && w == PXT && h % 2 == 0 && h >= 2 && ck >= 1 && ck <= NK && n >= 1 && n * (h / 2) < (int64_t(1) << 40) &&
           ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy_pooled) | reinterpret_cast<uintptr_t>(cols)) & 15) == 0;
}

int wb_conv1_bwd_fused(WbBackend* b, const float* x, const float* dy_pooled, const float* cols, int64_t n, int64_t h, int64_t w, int64_t ck,
                       const float* gamma, const float* beta, const float* save_mean, const float* save_rstd, const float* dgamma,
                       const float* dbeta, float* dweight, float* dbias_conv) {
    WB_REQUIRE(wb_conv1_bwd_fused_ok(n, CH, h, w, ck, x, dy_pooled, cols), WB_ERR_UNSUPPORTED, "wb_conv1_bwd_fused: unsupported shape");
    Args args{};
    const uint64_t hw = static_cast<uint64_t>(h * w), pooled = hw / 4;
    {
        const uint64_t dims[3] = {hw, CH, static_cast<uint64_t>(n)}, strides[2] = {hw * 4, hw * CH * 4};
        const uint32_t box[3] = {PXT, CH, 1};
        WB_TRY(wb_tc_encode(b, x, dims, strides, box, true, &args.map_x));
    }
    {
        const uint64_t dims[3] = {pooled, CH, static_cast<uint64_t>(n)}, strides[2] = {pooled * 4, pooled * CH * 4};
        const uint32_t box[3] = {16, CH, 1};
        WB_TRY(wb_tc_encode(b, dy_pooled, dims, strides, box, false, &args.map_g));
    }
    {
        const uint64_t dims[3] = {hw, static_cast<uint64_t>(ck), static_cast<uint64_t>(n)}, strides[2] = {hw * 4, hw * static_cast<uint64_t>(ck) * 4};
        const uint32_t box[3] = {PXT, NK, 1};
        WB_TRY(wb_tc_encode(b, cols, dims, strides, box, true, &args.map_cols));
    }
    args.mean = save_mean; args.rstd = save_rstd; args.gamma = gamma; args.beta = beta; args.dgamma = dgamma; args.dbeta = dbeta;
    args.inv_count = static_cast<float>(1.0 / static_cast<double>(n * h * w));
    args.n_img = static_cast<int>(n);
    args.pairs_per_img = static_cast<int>(h / 2);
    args.steps = n * (h / 2);
    const int ctas = static_cast<int>(std::min<int64_t>(b->sm_count, args.steps));
    void* scratch = nullptr;
    const size_t part_bytes = static_cast<size_t>(ctas) * CH * NK * sizeof(float);
    WB_TRY(wb_scratch(b, part_bytes + static_cast<size_t>(ctas) * CH * sizeof(double), &scratch));
    args.part = static_cast<float*>(scratch);
    args.bias_part = reinterpret_cast<double*>(static_cast<char*>(scratch) + part_bytes);
    WB_TRY(wb_tc_error_flag(b, &args.error_flag));
    constexpr size_t smem = sizeof(Smem) + 1024;
    static_assert(smem <= 227 * 1024, "shared-memory rings do not fit");
    static std::atomic<uint64_t> attr_done{0};
    const uint64_t bit = uint64_t(1) << (b->ordinal & 63);
    if (!(attr_done.load(std::memory_order_acquire) & bit)) {
        WB_CHECK_CUDA(cudaFuncSetAttribute(conv1_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        attr_done.fetch_or(bit, std::memory_order_release);
    }
    wb_launch_pdl(conv1_bwd_fused_kernel, dim3(ctas), dim3(THREADS), smem, b->stream, args);
    WB_LAUNCH_OK(b);
    const int items = static_cast<int>(CH * ck + CH);
    wb_launch_pdl(conv1_bwd_reduce_kernel, dim3((items * 32 + 255) / 256), dim3(256), 0, b->stream, args.part, args.bias_part, ctas, static_cast<int>(ck), dweight, dbias_conv);
    WB_LAUNCH_OK(b);
    return WB_OK;
}
