// Fused training-step runner for the named models (the MLP of crates/weta/examples/mnist_mlp.rs and
// the conv-BN CNN of crates/weta/examples/mnist_cnn.rs, at any width).
//
// Where the reference's step is ~400 primitive calls driven by its autograd graph
// (crates/weta-autograd/src/graph.rs:227-276), this runner issues a few dozen kernels in a fixed
// order: for each layer the forward op, then the hand-ordered backward, then one Adam pass over a
// flat parameter arena.  Arithmetic follows the reference's definitions (functional.rs, ops.rs,
// optim lib.rs as cited at each step); parameters, gradients and optimizer state keep the
// reference's tensor shapes and [out, in] / [O, C, kh, kw] element order.
//
// The arena holds the layers in REVERSE order, so the ranges whose gradients are finished first
// in backward are contiguous at the front; after each layer's gradients are written the optional
// callback fires with that range, which is where a data-parallel caller starts its all-reduce
// while earlier layers are still being differentiated.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <string>
#include <vector>

#include "common.h"
#include "adam.cuh"
#include "gemm.h"

int wb_bn_relu_pool_fwd_shifted(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t h, int64_t w, const float* gamma, const float* beta,
                                float* running_mean, float* running_var, double momentum, double eps, float* y_pooled, float* save_mean,
                                float* save_rstd, float* y_left, float* y_right, const double* channel_sums, const float* sums_pivot);
int wb_bn_relu_pool_bwd_shifted(WbBackend* b, const float* x, const float* dy_pooled, int64_t n, int64_t c, int64_t h, int64_t w,
                                const float* gamma, const float* beta, const float* save_mean, const float* save_rstd, float* dx,
                                float* dgamma, float* dbeta, float* dbias_conv, float* dx_left, float* dx_right, const float* y_pooled);
int wb_softmax_ce_pitched(WbBackend* b, const float* logits, const int64_t* labels, int64_t rows, int64_t cols, float* probs, float* dlogits,
                          int64_t dz_pitch, float* row_loss, float* mean_loss, double upstream);

namespace {

enum { L_CONV = 0, L_LINEAR = 1, L_DROPOUT = 2 };

struct Layer {
    int kind;
    // conv block: conv3x3(pad 1) -> BatchNorm2d -> ReLU -> MaxPool2d(2)
    int cin = 0, cout = 0, h = 0, w = 0;
    // linear
    int in = 0, out = 0, relu = 0;
    // dropout
    double p = 0.0;
    // offsets into the flat arena (elements); -1 when absent
    int64_t off_w = -1, off_b = -1, off_gamma = -1, off_beta = -1;
    int64_t range_begin = 0, range_len = 0;
    // buffers
    float* running_mean = nullptr;
    float* running_var = nullptr;
    float* save_mean = nullptr;
    float* save_rstd = nullptr;
    float* cols = nullptr;      // [B, cin*9, h*w]
    float* conv_out = nullptr;  // [B, cout, h, w]
    float* w_pad = nullptr;     // [cout, round_up(cin*9, 32)]: zero-padded copy of the weight when cin*9 is not a multiple of 4 (TMA needs a 16-byte pitch)
    // Implicit-GEMM path (no cols / dcols): the input shifted one column right / left, the weight as
    // [O][tap][C] and [C][flipped tap][O], and the weight gradient as the kernel writes it ([tap][C][O]).
    bool implicit = false;
    bool x_shift_fused = false;   // the previous block's BN/ReLU/pool pass writes x_shift
    bool dy_shift_fused = false;  // this block's BN/ReLU/pool backward writes the trainer's dy_shift
    bool dgrad_plain = false;     // the input gradient reads dY alone (no shifted copies are made)
    float* x_shift[2] = {nullptr, nullptr};
    float *w_fwd = nullptr, *w_dgrad = nullptr, *dw_taps = nullptr;
    double* stat_sums = nullptr;  // [cout][2]: sum and sum of squares of conv_out, accumulated by the convolution's epilogue
    float* out_act = nullptr;   // layer output
    int64_t out_elems = 0;      // per-sample size of the layer output
    bool relu_bwd_done = false;
};

}  // namespace

struct WbTrainer {
    WbBackend* be = nullptr;
    int64_t batch = 0;
    int64_t in_elems = 0;  // per-sample input size
    std::vector<Layer> layers;
    int64_t n_params = 0;
    float *theta = nullptr, *grad = nullptr, *m = nullptr, *v = nullptr;
    float* x_in = nullptr;       // staged input  [B, in_elems]: the trainer's own buffer unless wb_trainer_set_input replaced it
    int64_t* y_in = nullptr;     // staged labels [B]
    float* own_x_in = nullptr;
    int64_t* own_y_in = nullptr;
    float* dlogits = nullptr;    // [B, dl_pitch]: rows padded to a multiple of 4 floats for TMA
    int64_t dl_pitch = 0;
    float* loss_dev = nullptr;
    float* loss_pinned = nullptr;
    float* gbuf[2] = {nullptr, nullptr};  // ping-pong gradient-of-activation buffers
    float* dcols = nullptr;
    float* dy_shift[2] = {nullptr, nullptr};  // shifted copies of a conv block's output gradient (implicit input gradient; only for layers that need them)
    int64_t max_act = 0;
    int64_t t = 0;
    WbAdamConfig adam{};
    int matmul_mode = WB_MM_TF32;
    int classes = 0;
    wb_bucket_callback cb = nullptr;
    void* cb_user = nullptr;
    std::vector<void*> owned;
    // reference-order parameter table: (offset, len)
    std::vector<std::pair<int64_t, int64_t>> param_table;
    // optional per-op device timing: event pairs recorded around each op, read after the fact
    bool timing = false;
    std::vector<std::string> labels;
    struct TimeRec { int label; cudaEvent_t e0, e1; };
    std::vector<TimeRec> recs;
    std::vector<cudaEvent_t> event_pool;
    std::string timing_text;
    // captured whole step (wb_trainer_use_graph / wb_trainer_step)
    bool graph_on = false, graph_failed = false;
    int eager_steps = 0;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t gexec = nullptr;
    const float* g_x = nullptr;      // what the capture baked in: the staged batch and the backend's scratch block
    const int64_t* g_y = nullptr;
    const void* g_scratch = nullptr;
    struct DropNode { cudaGraphNode_t node; cudaKernelNodeParams p; int ordinal; float* y; const float* x; const float* relu_src; int64_t n; uint64_t kmin; float scale; int vec; };
    struct AdamNode { cudaGraphNode_t node; cudaKernelNodeParams p; float* theta; const float* grad; float *m, *v; int64_t n; int vec; };
    std::vector<DropNode> g_drops;
    std::vector<AdamNode> g_adams;
};

namespace {

int dev_alloc(WbTrainer* t, size_t bytes, void** out) {
    cudaError_t e = cudaMalloc(out, bytes ? bytes : 4);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        wb_set_error("trainer: allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        return e == cudaErrorMemoryAllocation ? WB_ERR_OOM : WB_ERR_CUDA;
    }
    t->owned.push_back(*out);
    return WB_OK;
}

template <class T>
int dev_alloc_t(WbTrainer* t, int64_t n, T** out) {
    void* p = nullptr;
    WB_TRY(dev_alloc(t, static_cast<size_t>(n) * sizeof(T), &p));
    *out = static_cast<T*>(p);
    return WB_OK;
}

cudaEvent_t get_event(WbTrainer* t) {
    if (!t->event_pool.empty()) {
        cudaEvent_t e = t->event_pool.back();
        t->event_pool.pop_back();
        return e;
    }
    cudaEvent_t e;
    cudaEventCreate(&e);
    return e;
}

// Records an event pair around one op when timing is on; costs a branch otherwise.  No waits here:
// the elapsed times are read by wb_trainer_timing_report after the stream has drained.
struct OpTimer {
    WbTrainer* t;
    int label = -1;
    cudaEvent_t e0 = nullptr;
    OpTimer(WbTrainer* tr, int layer, const char* what) : t(tr) {
        if (!t->timing) return;
        char name[64];
        snprintf(name, sizeof name, "L%d.%s", layer, what);
        for (size_t i = 0; i < t->labels.size(); ++i)
            if (t->labels[i] == name) label = static_cast<int>(i);
        if (label < 0) { t->labels.push_back(name); label = static_cast<int>(t->labels.size()) - 1; }
        e0 = get_event(t);
        cudaEventRecord(e0, t->be->stream);
    }
    ~OpTimer() {
        if (!e0) return;
        cudaEvent_t e1 = get_event(t);
        cudaEventRecord(e1, t->be->stream);
        t->recs.push_back({label, e0, e1});
    }
};

// D[batch][m][n] = A x B through the tensor cores, or the CUDA-core tiles when TMA cannot read an operand.
int gemm(WbTrainer* t, WbGemmOperand A, WbGemmOperand B, int64_t batch, int m, int n, int k, tc::Epilogue ep, int64_t span_batch = 0,
         bool* used_tc = nullptr) {
    return wb_gemm_dispatch(t->be, t->matmul_mode, A, B, batch, m, n, k, ep, span_batch, used_tc);
}

// Column sums in two fixed-order stages inside one launch: part[slab][j] over a slab of rows (a warp reads 32 adjacent
// columns of one row, eight rows in flight per block); the last block of a column strip to finish then adds the
// strip's slabs in ascending order.
__global__ void __launch_bounds__(256) column_sum_kernel(const float* __restrict__ src, int64_t rows, int64_t cols, int64_t pitch, int64_t per,
                                                         float* __restrict__ part, unsigned int* __restrict__ counter, float* __restrict__ dst) {
    wb_pdl_enter();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t col = static_cast<int64_t>(blockIdx.x) * 32 + lane;
    const int64_t r0 = static_cast<int64_t>(blockIdx.y) * per, r1 = min(rows, r0 + per);
    float acc = 0.f;
    if (col < cols)
        for (int64_t r = r0 + warp; r < r1; r += 8) acc += src[r * pitch + col];
    __shared__ float red[8][33];
    red[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && col < cols) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w][lane];
        part[static_cast<int64_t>(blockIdx.y) * cols + col] = t;
    }
    __threadfence();
    __syncthreads();
    __shared__ unsigned int last;
    if (threadIdx.x == 0) last = atomicAdd(&counter[blockIdx.x], 1u) == gridDim.y - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (warp == 0 && col < cols) {
        float t = 0.f;
        for (unsigned int s = 0; s < gridDim.y; ++s) t += __ldcg(&part[static_cast<int64_t>(s) * cols + col]);
        dst[col] = t;
    }
    if (threadIdx.x == 0) counter[blockIdx.x] = 0;  // ready for the next launch
}

// dst[j] = sum_i src[i][j] over a dense [rows, cols] matrix (a bias gradient, crates/weta-autograd/src/ops.rs:46-58).
// Very small matrices go through Backend::reduce (the reference's summation order); the others are split over row
// slabs (same result every run, order differs from the sequential sum by rounding only): the trait's column walk is one
// thread per column over all rows, 10 us for a 128 x 512 gradient where this kernel takes 3.
int column_sum(WbTrainer* t, const float* src, int64_t rows, int64_t cols, int64_t pitch, float* dst) {
    if (rows < 32 || cols <= 0 || cols > 32 * 4096) {
        WbView v{};
        v.data = const_cast<float*>(src); v.dtype = WB_F32; v.ndim = 2;
        v.shape[0] = rows; v.shape[1] = cols; v.stride[0] = pitch; v.stride[1] = 1;
        return wb_reduce_into(t->be, WB_SUM, &v, 0, dst);
    }
    WbBackend* b = t->be;
    const int64_t col_blocks = (cols + 31) / 32;
    int64_t slabs = std::max<int64_t>(1, std::min<int64_t>(rows / 64, (4 * static_cast<int64_t>(b->sm_count) + col_blocks - 1) / col_blocks));
    slabs = std::min<int64_t>(slabs, 1024);
    const int64_t per = (rows + slabs - 1) / slabs;
    slabs = (rows + per - 1) / per;
    void* scratch = nullptr;
    WB_TRY(wb_scratch(b, static_cast<size_t>(slabs) * cols * sizeof(float), &scratch));
    unsigned int* counters = nullptr;
    WB_TRY(wb_block_counters(b, &counters));
    wb_launch_pdl(column_sum_kernel, dim3(dim3(static_cast<unsigned>(col_blocks), static_cast<unsigned>(slabs))), dim3(256), 0, b->stream, src, rows, cols, pitch, per,
                                                                                                                      static_cast<float*>(scratch), counters, dst);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

int relu_bwd_inplace(WbTrainer* t, float* g, const float* y, int64_t n) {
    // g *= step(y): UnaryBw for ReLU (crates/weta-autograd/src/ops.rs:85), p = 0 dropout = identity mask
    return wb_dropout_relu_bwd(t->be, g, y, g, n, 0.0, 0);
}

}  // namespace

extern "C" int wb_trainer_create(WbBackend* b, const WbLayerSpec* specs, int n_layers, int64_t batch, int64_t in_c, int64_t in_h,
                                 int64_t in_w, const WbAdamConfig* adam, int matmul_mode, WbTrainer** out) {
    WB_REQUIRE(b && specs && out && adam && n_layers > 0 && batch > 0, WB_ERR_INVALID, "wb_trainer_create: bad arguments");
    WB_CHECK_CUDA(cudaSetDevice(b->ordinal));
    WbTrainer* t = new WbTrainer();
    t->be = b;
    t->batch = batch;
    t->adam = *adam;
    t->matmul_mode = matmul_mode;
    t->in_elems = in_c * in_h * in_w;
    int64_t c = in_c, h = in_h, w = in_w, flat = t->in_elems;
    bool spatial = in_h > 0 && in_w > 0 && !(in_h == 1 && in_w == 1 && false);
    for (int i = 0; i < n_layers; ++i) {
        Layer L;
        L.kind = specs[i].kind;
        if (L.kind == L_CONV) {
            if (!spatial || specs[i].a != c || h % 2 || w % 2) {
                delete t;
                wb_set_error("trainer: conv block %d expects %d input channels on an even-sized image, got %lld x %lld x %lld", i, specs[i].a,
                             (long long)c, (long long)h, (long long)w);
                return WB_ERR_INVALID;
            }
            L.cin = static_cast<int>(c); L.cout = specs[i].b; L.h = static_cast<int>(h); L.w = static_cast<int>(w);
            c = L.cout; h /= 2; w /= 2;
            flat = c * h * w;
            L.out_elems = flat;
        } else if (L.kind == L_LINEAR) {
            if (specs[i].a != flat) {
                delete t;
                wb_set_error("trainer: linear layer %d expects %d inputs, the previous layer gives %lld", i, specs[i].a, (long long)flat);
                return WB_ERR_INVALID;
            }
            spatial = false;
            L.in = specs[i].a; L.out = specs[i].b; L.relu = specs[i].c;
            flat = L.out;
            L.out_elems = flat;
        } else if (L.kind == L_DROPOUT) {
            L.p = specs[i].p;
            L.out_elems = flat;
            if (!(L.p >= 0.0 && L.p <= 1.0)) { delete t; wb_set_error("trainer: dropout probability must be in [0, 1]"); return WB_ERR_INVALID; }
        } else {
            delete t;
            wb_set_error("trainer: unknown layer kind %d", L.kind);
            return WB_ERR_INVALID;
        }
        t->layers.push_back(L);
    }
    WB_REQUIRE(t->layers.back().kind == L_LINEAR, WB_ERR_INVALID, "trainer: the last layer must be linear (the logits)");
    t->classes = t->layers.back().out;
    // Arena layout: last layer first.  Each tensor is padded to 32 elements: every tensor starts on a 128-byte
    // boundary (TMA operands need 16), and any run of whole tensors splits into 2, 4 or 8 equal shards that are
    // themselves 16-byte aligned (the data-parallel step gives each rank one shard of every bucket).
    auto pad4 = [](int64_t n) { return (n + 31) / 32 * 32; };
    int64_t off = 0;
    for (int i = n_layers - 1; i >= 0; --i) {
        Layer& L = t->layers[i];
        L.range_begin = off;
        if (L.kind == L_CONV) {
            L.off_w = off; off += pad4(static_cast<int64_t>(L.cout) * L.cin * 9);
            L.off_b = off; off += pad4(L.cout);
            L.off_gamma = off; off += pad4(L.cout);
            L.off_beta = off; off += pad4(L.cout);
        } else if (L.kind == L_LINEAR) {
            L.off_w = off; off += pad4(static_cast<int64_t>(L.out) * L.in);
            L.off_b = off; off += pad4(L.out);
        }
        L.range_len = off - L.range_begin;
    }
    t->n_params = off;
    for (const Layer& L : t->layers) {  // reference order: layer by layer, weight, bias, (bn weight, bn bias)
        if (L.kind == L_CONV) {
            t->param_table.push_back({L.off_w, static_cast<int64_t>(L.cout) * L.cin * 9});
            t->param_table.push_back({L.off_b, L.cout});
            t->param_table.push_back({L.off_gamma, L.cout});
            t->param_table.push_back({L.off_beta, L.cout});
        } else if (L.kind == L_LINEAR) {
            t->param_table.push_back({L.off_w, static_cast<int64_t>(L.out) * L.in});
            t->param_table.push_back({L.off_b, L.out});
        }
    }
    int s = WB_OK;
    auto A = [&](int st) { if (s == WB_OK) s = st; };
    A(dev_alloc_t(t, t->n_params, &t->theta));
    A(dev_alloc_t(t, t->n_params, &t->grad));
    A(dev_alloc_t(t, t->n_params, &t->m));
    A(dev_alloc_t(t, t->n_params, &t->v));
    A(dev_alloc_t(t, batch * t->in_elems, &t->x_in));
    A(dev_alloc_t(t, batch, &t->y_in));
    t->own_x_in = t->x_in;
    t->own_y_in = t->y_in;
    t->dl_pitch = (t->classes + 3) / 4 * 4;
    A(dev_alloc_t(t, batch * t->dl_pitch, &t->dlogits));
    A(dev_alloc_t(t, 4, &t->loss_dev));
    int64_t max_act = batch * t->in_elems, max_dcols = 0, max_dy_shift = 0;
    bool first_conv = true;
    for (Layer& L : t->layers) {
        if (L.kind == L_CONV) {
            int64_t hw = static_cast<int64_t>(L.h) * L.w;
            // The tensor-core implicit GEMM replaces im2col / col2im where its shape rules hold; TF32 mode only
            // (the 3xTF32 and FP32 modes keep the explicit chain).
            // WETA_B200_EXPLICIT_CONV=1 in the environment keeps every block on the explicit chain.
            const char* force_explicit = std::getenv("WETA_B200_EXPLICIT_CONV");
            L.implicit = matmul_mode == WB_MM_TF32 && wb_conv3_eligible(WbConv3{batch, L.cin, L.h, L.w, L.cout}) &&
                         !(force_explicit && force_explicit[0] == '1');
            if (L.implicit) {
                const int64_t wn = static_cast<int64_t>(L.cout) * L.cin * 9;
                A(dev_alloc_t(t, batch * L.cin * hw, &L.x_shift[0]));
                A(dev_alloc_t(t, batch * L.cin * hw, &L.x_shift[1]));
                A(dev_alloc_t(t, wn, &L.w_fwd));
                A(dev_alloc_t(t, wn, &L.dw_taps));
                L.dgrad_plain = !first_conv && wb_conv3_dgrad_needs_no_copies(WbConv3{batch, L.cin, L.h, L.w, L.cout});
                L.dy_shift_fused = !first_conv && !L.dgrad_plain && L.w % 4 == 0 && 32 % (L.w / 4) == 0;
                {
                    // input = the pooled output of a conv block directly before this one, whose width is 2 * L.w
                    const size_t li = static_cast<size_t>(&L - t->layers.data());
                    L.x_shift_fused = li > 0 && t->layers[li - 1].kind == L_CONV && (2 * L.w) % 8 == 0 && 32 % (2 * L.w / 8) == 0;
                }
                if (!first_conv) {
                    A(dev_alloc_t(t, wn, &L.w_dgrad));
                    if (!L.dgrad_plain) max_dy_shift = std::max(max_dy_shift, batch * L.cout * hw);
                }
            } else {
                A(dev_alloc_t(t, batch * L.cin * 9 * hw, &L.cols));
                if ((L.cin * 9) % 4 != 0) {
                    // rows padded with zeros to a whole number of 32-float K blocks: TMA then never fetches a partial row
                    const int64_t padded = static_cast<int64_t>(L.cout) * ((L.cin * 9 + 31) / 32 * 32);
                    A(dev_alloc_t(t, padded, &L.w_pad));
                    if (s == WB_OK && cudaMemsetAsync(L.w_pad, 0, padded * sizeof(float), b->stream) != cudaSuccess) s = WB_ERR_CUDA;
                }
                if (!first_conv) max_dcols = std::max(max_dcols, batch * L.cin * 9 * hw);
            }
            A(dev_alloc_t(t, batch * L.cout * hw, &L.conv_out));
            A(dev_alloc_t(t, 2 * static_cast<int64_t>(L.cout), &L.stat_sums));
            A(dev_alloc_t(t, batch * L.out_elems, &L.out_act));
            A(dev_alloc_t(t, L.cout, &L.running_mean));
            A(dev_alloc_t(t, L.cout, &L.running_var));
            A(dev_alloc_t(t, L.cout, &L.save_mean));
            A(dev_alloc_t(t, L.cout, &L.save_rstd));
            max_act = std::max(max_act, batch * L.cout * hw);
            first_conv = false;
        } else {
            A(dev_alloc_t(t, batch * L.out_elems, &L.out_act));
            max_act = std::max(max_act, batch * L.out_elems);
        }
    }
    if (max_dy_shift > 0) {
        A(dev_alloc_t(t, max_dy_shift, &t->dy_shift[0]));
        A(dev_alloc_t(t, max_dy_shift, &t->dy_shift[1]));
    }
    t->max_act = max_act;
    A(dev_alloc_t(t, max_act, &t->gbuf[0]));
    A(dev_alloc_t(t, max_act, &t->gbuf[1]));
    if (max_dcols > 0) A(dev_alloc_t(t, max_dcols, &t->dcols));
    if (s == WB_OK) {
        cudaError_t e = cudaMallocHost(&t->loss_pinned, 16);
        if (e != cudaSuccess) { (void)cudaGetLastError(); wb_set_error("trainer: pinned allocation failed"); s = WB_ERR_CUDA; }
    }
    if (s == WB_OK) {
        cudaMemsetAsync(t->theta, 0, t->n_params * sizeof(float), b->stream);
        cudaMemsetAsync(t->grad, 0, t->n_params * sizeof(float), b->stream);
        cudaMemsetAsync(t->m, 0, t->n_params * sizeof(float), b->stream);
        cudaMemsetAsync(t->v, 0, t->n_params * sizeof(float), b->stream);
    }
    if (s != WB_OK) {
        for (void* p : t->owned) cudaFree(p);
        delete t;
        return s;
    }
    *out = t;
    return WB_OK;
}

extern "C" int wb_trainer_destroy(WbTrainer* t) {
    if (!t) return WB_OK;
    cudaStreamSynchronize(t->be->stream);
    if (t->gexec) cudaGraphExecDestroy(t->gexec);
    if (t->graph) cudaGraphDestroy(t->graph);
    for (void* p : t->owned) cudaFree(p);
    if (t->loss_pinned) cudaFreeHost(t->loss_pinned);
    delete t;
    return WB_OK;
}

// Default initialisation (crates/weta-nn/src/layers.rs:19-26): weight then bias of every Linear /
// Conv2d from U(-1/sqrt(fan_in), 1/sqrt(fan_in)), one seed each in creation order; BatchNorm
// weight 1, bias 0, running mean 0, running variance 1 (layers.rs:235-247).
extern "C" int wb_trainer_init(WbTrainer* t, const uint64_t* seeds, int n_seeds) {
    WB_REQUIRE(t && seeds, WB_ERR_INVALID, "wb_trainer_init: null pointer");
    int need = 0;
    for (const Layer& L : t->layers) need += (L.kind == L_CONV || L.kind == L_LINEAR) ? 2 : 0;
    WB_REQUIRE(n_seeds == need, WB_ERR_INVALID, "wb_trainer_init: expected %d seeds, got %d", need, n_seeds);
    WbBackend* b = t->be;
    WB_CHECK_CUDA(cudaMemsetAsync(t->theta, 0, t->n_params * sizeof(float), b->stream));
    WB_CHECK_CUDA(cudaMemsetAsync(t->m, 0, t->n_params * sizeof(float), b->stream));
    WB_CHECK_CUDA(cudaMemsetAsync(t->v, 0, t->n_params * sizeof(float), b->stream));
    t->t = 0;
    int si = 0;
    std::vector<float> ones;
    for (Layer& L : t->layers) {
        if (L.kind == L_DROPOUT) continue;
        int64_t fan_in = L.kind == L_CONV ? static_cast<int64_t>(L.cin) * 9 : L.in;
        int64_t wn = L.kind == L_CONV ? static_cast<int64_t>(L.cout) * L.cin * 9 : static_cast<int64_t>(L.out) * L.in;
        int64_t bn = L.kind == L_CONV ? L.cout : L.out;
        double bound = 1.0 / std::sqrt(static_cast<double>(fan_in));
        WB_TRY(wb_random_into(b, wn, WB_F32, WB_UNIFORM, -bound, bound, seeds[si++], t->theta + L.off_w));
        WB_TRY(wb_random_into(b, bn, WB_F32, WB_UNIFORM, -bound, bound, seeds[si++], t->theta + L.off_b));
        if (L.kind == L_CONV) {
            ones.assign(L.cout, 1.0f);
            WB_CHECK_CUDA(cudaMemcpyAsync(t->theta + L.off_gamma, ones.data(), L.cout * sizeof(float), cudaMemcpyHostToDevice, b->stream));
            WB_CHECK_CUDA(cudaMemcpyAsync(L.running_var, ones.data(), L.cout * sizeof(float), cudaMemcpyHostToDevice, b->stream));
            WB_CHECK_CUDA(cudaMemsetAsync(L.running_mean, 0, L.cout * sizeof(float), b->stream));
            WB_CHECK_CUDA(cudaStreamSynchronize(b->stream));  // `ones` is pageable host memory
        }
    }
    return WB_OK;
}

extern "C" int64_t wb_trainer_arena_len(const WbTrainer* t) { return t->n_params; }
extern "C" float* wb_trainer_params(WbTrainer* t) { return t->theta; }
extern "C" float* wb_trainer_grads(WbTrainer* t) { return t->grad; }
extern "C" float* wb_trainer_exp_avg(WbTrainer* t) { return t->m; }
extern "C" float* wb_trainer_exp_avg_sq(WbTrainer* t) { return t->v; }
extern "C" float* wb_trainer_input(WbTrainer* t) { return t->x_in; }
extern "C" int64_t* wb_trainer_labels(WbTrainer* t) { return t->y_in; }
// Makes the next steps read their batch from caller-owned device buffers ([B, in_elems] f32 and [B] i64), e.g. the
// slots of a double-buffered upload pipeline; null pointers restore the trainer's own staging buffers.
extern "C" int wb_trainer_set_input(WbTrainer* t, float* x, int64_t* y) {
    WB_REQUIRE(t && ((x == nullptr) == (y == nullptr)), WB_ERR_INVALID, "wb_trainer_set_input: give both buffers or neither");
    WB_REQUIRE(!x || (reinterpret_cast<uintptr_t>(x) & 15) == 0, WB_ERR_INVALID, "wb_trainer_set_input: the image buffer must be 16-byte aligned");
    t->x_in = x ? x : t->own_x_in;
    t->y_in = y ? y : t->own_y_in;
    return WB_OK;
}
extern "C" float* wb_trainer_loss_ptr(WbTrainer* t) { return t->loss_dev; }
extern "C" int wb_trainer_num_tensors(const WbTrainer* t) { return static_cast<int>(t->param_table.size()); }

extern "C" int wb_trainer_tensor_range(const WbTrainer* t, int index, int64_t* offset, int64_t* len) {
    WB_REQUIRE(t && index >= 0 && index < static_cast<int>(t->param_table.size()), WB_ERR_INVALID, "trainer: no parameter tensor %d", index);
    *offset = t->param_table[index].first;
    *len = t->param_table[index].second;
    return WB_OK;
}

extern "C" int wb_trainer_bn_buffers(WbTrainer* t, int conv_index, float** running_mean, float** running_var, int64_t* channels) {
    int k = 0;
    for (Layer& L : t->layers) {
        if (L.kind != L_CONV) continue;
        if (k++ == conv_index) {
            *running_mean = L.running_mean;
            *running_var = L.running_var;
            *channels = L.cout;
            return WB_OK;
        }
    }
    wb_set_error("trainer: no conv block %d", conv_index);
    return WB_ERR_INVALID;
}

// Internal (dp.cu): the trainer's backend, batch geometry and per-layer arena ranges in arena order (last layer first).
// conv_follows[k]: after range k has been reported, backward still has a conv block to go (so a "quiet point"
// notification, see wb_bucket_callback, will follow).
int wb_trainer_internal_info(WbTrainer* t, WbBackend** be, int64_t* batch, int64_t* in_elems, std::vector<std::pair<int64_t, int64_t>>* ranges,
                             std::vector<int>* conv_follows) {
    if (be) *be = t->be;
    if (batch) *batch = t->batch;
    if (in_elems) *in_elems = t->in_elems;
    if (ranges) {
        ranges->clear();
        if (conv_follows) conv_follows->clear();
        for (int i = static_cast<int>(t->layers.size()) - 1; i >= 0; --i) {
            if (t->layers[i].range_len <= 0) continue;
            ranges->push_back({t->layers[i].range_begin, t->layers[i].range_len});
            bool follows = false;
            for (int j = 0; j < i; ++j) follows = follows || t->layers[j].kind == L_CONV;
            if (conv_follows) conv_follows->push_back(follows ? 1 : 0);
        }
    }
    return WB_OK;
}

const WbAdamConfig* wb_trainer_adam_config(const WbTrainer* t) { return &t->adam; }

extern "C" int wb_trainer_set_bucket_callback(WbTrainer* t, wb_bucket_callback cb, void* user) {
    t->cb = cb;
    t->cb_user = user;
    return WB_OK;
}

// Forward + loss + backward over the staged batch (wb_trainer_input / wb_trainer_labels).
// dropout_seeds: one per dropout layer, in forward order (the reference draws them from the global
// generator in that order, crates/weta-tensor/src/random.rs:95-98).
extern "C" int wb_trainer_forward_backward(WbTrainer* t, const uint64_t* dropout_seeds, int n_seeds) {
    WB_REQUIRE(t, WB_ERR_INVALID, "wb_trainer_forward_backward: null trainer");
    WbBackend* b = t->be;
    const int64_t B = t->batch;
    int n_drop = 0;
    // The reference draws a seed only when a mask is needed: F::dropout returns before Tensor::rand for p = 0 and
    // p = 1 (crates/weta-nn/src/functional.rs:66-71), so those layers consume none.
    for (const Layer& L : t->layers) n_drop += L.kind == L_DROPOUT && L.p > 0.0 && L.p < 1.0;
    WB_REQUIRE(n_seeds == n_drop && (n_drop == 0 || dropout_seeds), WB_ERR_INVALID, "trainer: expected %d dropout seeds, got %d", n_drop, n_seeds);
    const int nl = static_cast<int>(t->layers.size());
    // ---- forward ----------------------------------------------------------------------------
    const float* act = t->x_in;
    int di = 0;
    std::vector<uint64_t> seed_of(nl, 0);
    for (int i = 0; i < nl; ++i) {
        Layer& L = t->layers[i];
        L.relu_bwd_done = false;
        if (L.kind == L_CONV) {
            // F::conv2d_ext (crates/weta-nn/src/functional.rs:84-106): im2col, W[O, C*9] x cols[n], + bias[O,1]
            const int64_t hw = static_cast<int64_t>(L.h) * L.w, ck = static_cast<int64_t>(L.cin) * 9;
            bool have_sums = false;  // the tensor-core epilogue filled L.stat_sums
            if (L.implicit) {
                const WbConv3 geo{B, L.cin, L.h, L.w, L.cout};
                if (!L.x_shift_fused) {
                    OpTimer tm(t, i, "conv_shift_x");
                    WB_TRY(wb_conv3_shift_copies(b, act, B * L.cin * L.h, L.w, L.x_shift[0], L.x_shift[1]));
                }
                // the forward operand and, when this block has an input gradient, its operand too: the parameters do not
                // change between this block's forward and its backward
                WB_TRY(wb_conv3_weight_reorder(b, L.w_dgrad ? 3 : 0, t->theta + L.off_w, L.w_fwd, L.cout, L.cin, L.w_dgrad));
                const float* x3[3] = {L.x_shift[0], act, L.x_shift[1]};
                WB_CHECK_CUDA(cudaMemsetAsync(L.stat_sums, 0, 2 * sizeof(double) * L.cout, b->stream));
                { OpTimer tm(t, i, "conv_fwd_gemm"); WB_TRY(wb_conv3_fwd(b, geo, x3, L.w_fwd, t->theta + L.off_b, L.conv_out, L.stat_sums)); }
                have_sums = true;
            } else {
            WbView xv{};
            xv.data = const_cast<float*>(act); xv.dtype = WB_F32; xv.ndim = 4;
            xv.shape[0] = B; xv.shape[1] = L.cin; xv.shape[2] = L.h; xv.shape[3] = L.w;
            xv.stride[0] = L.cin * hw; xv.stride[1] = hw; xv.stride[2] = L.w; xv.stride[3] = 1;
            WbConvParams cp{3, 3, 1, 1, 1, 1, 1, 1};
            { OpTimer tm(t, i, "im2col"); WB_TRY(wb_im2col_into(b, &xv, &cp, L.cols)); }
            WbGemmOperand Aw{t->theta + L.off_w, L.cout, ck, ck, 0, false};
            if (L.w_pad) {
                // TMA needs a 16-byte row pitch: copy the [O, C*9] weight into zero-padded rows of round_up(C*9, 32) floats.
                const int64_t ckp = (ck + 31) / 32 * 32;
                WB_CHECK_CUDA(cudaMemcpy2DAsync(L.w_pad, ckp * sizeof(float), t->theta + L.off_w, ck * sizeof(float), ck * sizeof(float), L.cout,
                                                cudaMemcpyDeviceToDevice, b->stream));
                Aw.ptr = L.w_pad;
                Aw.ld = ckp;
                Aw.k = ckp;  // the padding columns are zeros; B's rows past C*9 are zero-filled by TMA
            }
            WbGemmOperand Bc{L.cols, hw, ck, hw, ck * hw, true};
            tc::Epilogue ep{L.conv_out, hw, L.cout * hw, nullptr, t->theta + L.off_b, 0, 0};
            ep.row_stats = L.stat_sums;  // rows are output channels: the batch-norm sums come with the store
            WB_CHECK_CUDA(cudaMemsetAsync(L.stat_sums, 0, 2 * sizeof(double) * L.cout, b->stream));
            { OpTimer tm(t, i, "conv_fwd_gemm"); WB_TRY(gemm(t, Aw, Bc, B, L.cout, static_cast<int>(hw), static_cast<int>(ck), ep, 0, &have_sums)); }
            }
            // BatchNorm2d (train) -> ReLU -> MaxPool2d(2)
            {
                OpTimer tm(t, i, "bn_relu_pool_fwd");
                // The block that follows reads its input in three column-shifted copies when it is an implicit GEMM:
                // write the two extra copies from here instead of re-reading the pooled tensor.
                Layer* next = (i + 1 < nl && t->layers[i + 1].kind == L_CONV && t->layers[i + 1].x_shift_fused) ? &t->layers[i + 1] : nullptr;
                WB_TRY(wb_bn_relu_pool_fwd_shifted(b, L.conv_out, B, L.cout, L.h, L.w, t->theta + L.off_gamma, t->theta + L.off_beta,
                                                   L.running_mean, L.running_var, 0.1, 1e-5, L.out_act, L.save_mean, L.save_rstd,
                                                   next ? next->x_shift[0] : nullptr, next ? next->x_shift[1] : nullptr,
                                                   have_sums ? L.stat_sums : nullptr, have_sums ? t->theta + L.off_b : nullptr));
            }
            act = L.out_act;
        } else if (L.kind == L_LINEAR) {
            // F::linear (functional.rs:54-60): x W^T + b, ReLU folded into the epilogue
            WbGemmOperand Ax{act, B, L.in, L.in, 0, false};
            WbGemmOperand Bw{t->theta + L.off_w, L.out, L.in, L.in, 0, false};
            tc::Epilogue ep{L.out_act, L.out, 0, t->theta + L.off_b, nullptr, L.relu, 0};
            { OpTimer tm(t, i, "linear_fwd_gemm"); WB_TRY(gemm(t, Ax, Bw, 1, static_cast<int>(B), L.out, L.in, ep)); }
            act = L.out_act;
        } else {
            seed_of[i] = (L.p > 0.0 && L.p < 1.0) ? dropout_seeds[di++] : 0;
            { OpTimer tm(t, i, "dropout_fwd"); WB_TRY(wb_dropout_fwd(b, act, L.out_act, B * L.out_elems, L.p, seed_of[i])); }
            act = L.out_act;
        }
    }
    // ---- loss: cross-entropy, mean over the batch (crates/weta-autograd/src/ops.rs:499-519) ---
    { OpTimer tm(t, nl, "softmax_ce"); WB_TRY(wb_softmax_ce_pitched(b, act, t->y_in, B, t->classes, nullptr, t->dlogits, t->dl_pitch, nullptr, t->loss_dev, 1.0)); }
    // ---- backward ---------------------------------------------------------------------------
    const float* g = t->dlogits;  // gradient w.r.t. the current layer's output
    int pp = 0;
    for (int i = nl - 1; i >= 0; --i) {
        Layer& L = t->layers[i];
        const float* in_act = i == 0 ? t->x_in : t->layers[i - 1].out_act;
        const bool need_dx = i > 0;
        if (L.kind == L_LINEAR) {
            float* gz = const_cast<float*>(g);
            const int64_t gld = (i == nl - 1) ? t->dl_pitch : L.out;  // row pitch of dZ (the logits' gradient is padded)
            if (L.relu && !L.relu_bwd_done) WB_TRY(relu_bwd_inplace(t, gz, L.out_act, B * L.out));
            // MatmulBw (ops.rs:821-827): dW = dZ^T X, db = sum over the batch, dX = dZ W
            // The logits layer (at most 16 outputs): its gradients on the CUDA cores.  Measured on 1024 -> 10: dX 8 us against
            // 16 us on the tensor-core path at batch 512 (equal at 4096); dW only up to 1024 samples (one block per 32
            // inputs walks the whole batch); the forward product stays on the tensor cores (a warp per row on CUDA cores
            // took 27-30 us against 15 us, at batch 512 and at 4096).
            if (wb_narrow_linear_ok(B, L.in, L.out, in_act, t->theta + L.off_w)) {
                if (B <= 1024) {
                    OpTimer tm(t, i, "linear_wgrad_gemm");
                    WB_TRY(wb_narrow_linear_wgrad(b, t->matmul_mode, gz, gld, in_act, static_cast<int>(B), L.in, L.out, t->grad + L.off_w));
                } else {
                    WbGemmOperand Az{gz, L.out, B, gld, 0, true};
                    WbGemmOperand Bx{in_act, L.in, B, L.in, 0, true};
                    tc::Epilogue epw{t->grad + L.off_w, L.in, 0, nullptr, nullptr, 0, 0};
                    OpTimer tm(t, i, "linear_wgrad_gemm");
                    WB_TRY(gemm(t, Az, Bx, 1, L.out, L.in, static_cast<int>(B), epw));
                }
                { OpTimer tm(t, i, "linear_bias_grad"); WB_TRY(column_sum(t, gz, B, L.out, gld, t->grad + L.off_b)); }
                if (need_dx) {
                    float* dx = t->gbuf[pp];
                    pp ^= 1;
                    { OpTimer tm(t, i, "linear_dgrad_gemm"); WB_TRY(wb_narrow_linear_dgrad(b, t->matmul_mode, gz, gld, t->theta + L.off_w, static_cast<int>(B), L.in, L.out, dx)); }
                    g = dx;
                }
                if (t->cb && L.range_len > 0) t->cb(t->cb_user, t->grad + L.range_begin, L.range_len);
                continue;
            }
            WbGemmOperand Az{gz, L.out, B, gld, 0, true};
            WbGemmOperand Bx{in_act, L.in, B, L.in, 0, true};
            tc::Epilogue epw{t->grad + L.off_w, L.in, 0, nullptr, nullptr, 0, 0};
            { OpTimer tm(t, i, "linear_wgrad_gemm"); WB_TRY(gemm(t, Az, Bx, 1, L.out, L.in, static_cast<int>(B), epw)); }
            { OpTimer tm(t, i, "linear_bias_grad"); WB_TRY(column_sum(t, gz, B, L.out, gld, t->grad + L.off_b)); }
            if (need_dx) {
                float* dx = t->gbuf[pp];
                pp ^= 1;
                WbGemmOperand Ad{gz, B, L.out, gld, 0, false};
                WbGemmOperand Bw{t->theta + L.off_w, L.in, L.out, L.in, 0, true};
                tc::Epilogue epx{dx, L.in, 0, nullptr, nullptr, 0, 0};
                { OpTimer tm(t, i, "linear_dgrad_gemm"); WB_TRY(gemm(t, Ad, Bw, 1, static_cast<int>(B), L.in, L.out, epx)); }
                g = dx;
            }
        } else if (L.kind == L_DROPOUT) {
            // BinaryBw Mul (ops.rs:199): dx = dy * mask.  If a ReLU'd linear layer feeds this dropout, its
            // step() factor is applied in the same pass.
            float* dx = t->gbuf[pp];
            pp ^= 1;
            const float* relu_src = nullptr;
            if (i > 0 && t->layers[i - 1].kind == L_LINEAR && t->layers[i - 1].relu) {
                relu_src = t->layers[i - 1].out_act;
                t->layers[i - 1].relu_bwd_done = true;
            }
            { OpTimer tm(t, i, "dropout_bwd"); WB_TRY(wb_dropout_relu_bwd(b, g, relu_src, dx, B * L.out_elems, L.p, seed_of[i])); }
            g = dx;
        } else {
            const int64_t hw = static_cast<int64_t>(L.h) * L.w, ck = static_cast<int64_t>(L.cin) * 9;
            // First block, 27-value contraction: its output gradient has no consumer but the weight and bias gradients,
            // which one kernel computes from the pieces of it that it builds in shared memory (conv1_bwd_fused.cu).
            if (!need_dx && !L.implicit && t->matmul_mode == WB_MM_TF32 &&
                wb_conv1_bwd_fused_ok(B, L.cout, L.h, L.w, ck, L.conv_out, g, L.cols)) {
                {
                    OpTimer tm(t, i, "bn_relu_pool_bwd");
                    WB_TRY(wb_bn_relu_pool_bwd_shifted(b, L.conv_out, g, B, L.cout, L.h, L.w, t->theta + L.off_gamma, t->theta + L.off_beta,
                                                       L.save_mean, L.save_rstd, nullptr, t->grad + L.off_gamma, t->grad + L.off_beta, nullptr, nullptr,
                                                       nullptr, L.out_act));
                }
                if (t->cb) t->cb(t->cb_user, nullptr, 0);
                {
                    OpTimer tm(t, i, "conv_wgrad_gemm");
                    WB_TRY(wb_conv1_bwd_fused(b, L.conv_out, g, L.cols, B, L.h, L.w, ck, t->theta + L.off_gamma, t->theta + L.off_beta, L.save_mean,
                                              L.save_rstd, t->grad + L.off_gamma, t->grad + L.off_beta, t->grad + L.off_w, t->grad + L.off_b));
                }
                if (t->cb && L.range_len > 0) t->cb(t->cb_user, t->grad + L.range_begin, L.range_len);
                continue;
            }
            float* dconv = t->gbuf[pp];
            pp ^= 1;
            {
                OpTimer tm(t, i, "bn_relu_pool_bwd");
                const bool fuse = L.implicit && need_dx && L.dy_shift_fused;
                WB_TRY(wb_bn_relu_pool_bwd_shifted(b, L.conv_out, g, B, L.cout, L.h, L.w, t->theta + L.off_gamma, t->theta + L.off_beta,
                                                   L.save_mean, L.save_rstd, dconv, t->grad + L.off_gamma, t->grad + L.off_beta,
                                                   t->grad + L.off_b, fuse ? t->dy_shift[0] : nullptr, fuse ? t->dy_shift[1] : nullptr, L.out_act));
            }
            // Quiet point: the memory-bound pass of this block is queued and tensor-core contractions follow, which neither
            // fill every block slot of the SMs nor live on HBM bandwidth; side-stream work started now disturbs the least.
            if (t->cb) t->cb(t->cb_user, nullptr, 0);
            if (L.implicit) {
                const WbConv3 geo{B, L.cin, L.h, L.w, L.cout};
                const float* x3[3] = {L.x_shift[0], in_act, L.x_shift[1]};
                { OpTimer tm(t, i, "conv_wgrad_gemm"); WB_TRY(wb_conv3_wgrad(b, geo, dconv, x3, L.dw_taps, t->grad + L.off_w)); }
                if (need_dx) {
                    if (!L.dy_shift_fused && !L.dgrad_plain) {
                        OpTimer tm(t, i, "conv_shift_dy");
                        WB_TRY(wb_conv3_shift_copies(b, dconv, B * L.cout * L.h, L.w, t->dy_shift[0], t->dy_shift[1]));
                    }
                    float* dx = t->gbuf[pp];
                    pp ^= 1;
                    const float* d3[3] = {L.dgrad_plain ? nullptr : t->dy_shift[0], dconv, L.dgrad_plain ? nullptr : t->dy_shift[1]};
                    { OpTimer tm(t, i, "conv_dgrad_gemm"); WB_TRY(wb_conv3_dgrad(b, geo, d3, L.w_dgrad, dx)); }
                    g = dx;
                }
            } else {
            OpTimer* wt = new OpTimer(t, i, "conv_wgrad_gemm");
            // dW[O, C*9] = sum_n dY[n] cols[n]^T: one contraction over (n, position), not a batched
            // product followed by a reduction over n (ops.rs:821-827 + sum_to_shape).
            WbGemmOperand Ad{dconv, L.cout, hw, hw, L.cout * hw, false};
            WbGemmOperand Bc{L.cols, ck, hw, hw, ck * hw, false};
            tc::Epilogue epw{t->grad + L.off_w, ck, 0, nullptr, nullptr, 0, 0};
            int s = WB_ERR_UNSUPPORTED;
            if (t->matmul_mode != WB_MM_FP32) s = wb_tc_gemm(b, Ad, Bc, 1, L.cout, static_cast<int>(ck), static_cast<int>(hw), epw, t->matmul_mode, 0, B);
            if (s == WB_ERR_UNSUPPORTED) {
                // CUDA-core path: batched dY[n] cols[n]^T into scratch, then the sum over n.
                void* tmp = nullptr;
                size_t klass = 0;
                WB_TRY(wb_arena_alloc(b, static_cast<size_t>(B) * L.cout * ck * sizeof(float), &tmp, &klass));
                WbGemmOperand Bt{L.cols, ck, hw, hw, ck * hw, false};
                tc::Epilogue ept{static_cast<float*>(tmp), ck, L.cout * ck, nullptr, nullptr, 0, 0};
                int saved = t->matmul_mode;
                t->matmul_mode = WB_MM_FP32;
                s = gemm(t, Ad, Bt, B, L.cout, static_cast<int>(ck), static_cast<int>(hw), ept);
                t->matmul_mode = saved;
                if (s == WB_OK) s = column_sum(t, static_cast<float*>(tmp), B, L.cout * ck, L.cout * ck, t->grad + L.off_w);
                wb_arena_free(b, tmp, klass);
            }
            delete wt;
            WB_TRY(s);
            if (need_dx) {
                // dcols[n] = W^T dY[n], then col2im (Im2ColBw, ops.rs:865-868)
                WbGemmOperand Aw{t->theta + L.off_w, ck, L.cout, ck, 0, true};
                WbGemmOperand Bd{dconv, hw, L.cout, hw, L.cout * hw, true};
                tc::Epilogue epc{t->dcols, hw, ck * hw, nullptr, nullptr, 0, 0};
                { OpTimer tm(t, i, "conv_dgrad_gemm"); WB_TRY(gemm(t, Aw, Bd, B, static_cast<int>(ck), static_cast<int>(hw), L.cout, epc)); }
                float* dx = t->gbuf[pp];
                pp ^= 1;
                WbView cv{};
                cv.data = t->dcols; cv.dtype = WB_F32; cv.ndim = 3;
                cv.shape[0] = B; cv.shape[1] = ck; cv.shape[2] = hw;
                cv.stride[0] = ck * hw; cv.stride[1] = hw; cv.stride[2] = 1;
                WbConvParams cp{3, 3, 1, 1, 1, 1, 1, 1};
                { OpTimer tm(t, i, "col2im"); WB_TRY(wb_col2im_into(b, &cv, &cp, L.cin, L.h, L.w, dx)); }
                g = dx;
            }
            }
        }
        if (t->cb && L.range_len > 0) t->cb(t->cb_user, t->grad + L.range_begin, L.range_len);
    }
    return WB_OK;
}

extern "C" int wb_trainer_adam_step(WbTrainer* t, double grad_scale) {
    WB_REQUIRE(t, WB_ERR_INVALID, "wb_trainer_adam_step: null trainer");
    t->t += 1;
    const WbAdamConfig& a = t->adam;
    OpTimer tm(t, static_cast<int>(t->layers.size()), "adam");
    return wb_adam_step(t->be, t->theta, t->grad, t->m, t->v, t->n_params, t->t, a.lr, a.beta1, a.beta2, a.eps, a.weight_decay, a.decoupled,
                        grad_scale);
}

// Adam over one range of the arena, issued on another backend handle's stream (same device): a data-parallel
// caller updates a bucket as soon as its gradient sum has arrived, while backward continues on the trainer's
// stream.  wb_trainer_begin_step advances and returns the step count t that every range of one step passes.
extern "C" int64_t wb_trainer_begin_step(WbTrainer* t) { return ++t->t; }

extern "C" int wb_trainer_adam_range(WbTrainer* t, WbBackend* on, int64_t offset, int64_t len, int64_t step, double grad_scale) {
    WB_REQUIRE(t && on, WB_ERR_INVALID, "wb_trainer_adam_range: null pointer");
    WB_REQUIRE(on->ordinal == t->be->ordinal, WB_ERR_INVALID, "wb_trainer_adam_range: the stream's backend is on another device");
    WB_REQUIRE(offset >= 0 && len >= 0 && offset + len <= t->n_params && step >= 1, WB_ERR_INVALID, "wb_trainer_adam_range: bad range");
    if (len == 0) return WB_OK;
    const WbAdamConfig& a = t->adam;
    return wb_adam_step(on, t->theta + offset, t->grad + offset, t->m + offset, t->v + offset, len, step, a.lr, a.beta1, a.beta2, a.eps,
                        a.weight_decay, a.decoupled, grad_scale);
}

// ---- a whole step as one CUDA graph -----------------------------------------------------------------------------
// The step of a small model is some 25-40 launches of a few microseconds each: the host's launch cost bounds it.
// wb_trainer_step replays forward + loss + backward + Adam from a graph captured once; per step it rewrites the
// arguments that change - the dropout seeds (found by the sentinel values the capture ran with) and the Adam scalars
// of step t - in the graph's kernel nodes and launches it.  The first step runs eagerly (it sizes every scratch block,
// sets kernel attributes and is the only one with Adam's first-step form); a capture that fails for any reason turns
// the feature off for this trainer and the step runs eagerly as before.
namespace {

constexpr uint64_t SEED_SENTINEL = 0x5EEDC0DE00000000ull;

void graph_drop(WbTrainer* t) {
    if (t->gexec) cudaGraphExecDestroy(t->gexec);
    if (t->graph) cudaGraphDestroy(t->graph);
    t->gexec = nullptr;
    t->graph = nullptr;
    t->g_drops.clear();
    t->g_adams.clear();
}

int eager_step(WbTrainer* t, const uint64_t* seeds, int n_seeds) {
    WB_TRY(wb_trainer_forward_backward(t, seeds, n_seeds));
    return wb_trainer_adam_step(t, 1.0);
}

// Captures one step on the trainer's stream.  Returns false (graph released, error state cleared) if anything fails.
bool graph_capture(WbTrainer* t, int n_seeds) {
    WbBackend* b = t->be;
    std::vector<uint64_t> sentinels(static_cast<size_t>(std::max(n_seeds, 1)));
    for (int i = 0; i < n_seeds; ++i) sentinels[i] = SEED_SENTINEL + static_cast<uint64_t>(i);
    const int64_t saved_t = t->t;
    if (cudaStreamBeginCapture(b->stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess) { (void)cudaGetLastError(); return false; }
    const int s = eager_step(t, sentinels.data(), n_seeds);
    cudaGraph_t g = nullptr;
    const cudaError_t e = cudaStreamEndCapture(b->stream, &g);
    t->t = saved_t;  // the captured Adam launch carries placeholder scalars; the step count advances when a step runs
    if (s != WB_OK || e != cudaSuccess || !g) {
        if (g) cudaGraphDestroy(g);
        (void)cudaGetLastError();
        return false;
    }
    t->graph = g;
    if (cudaGraphInstantiate(&t->gexec, g, 0) != cudaSuccess) { (void)cudaGetLastError(); graph_drop(t); return false; }
    size_t n_nodes = 0;
    if (cudaGraphGetNodes(g, nullptr, &n_nodes) != cudaSuccess) { (void)cudaGetLastError(); graph_drop(t); return false; }
    std::vector<cudaGraphNode_t> nodes(n_nodes);
    if (n_nodes && cudaGraphGetNodes(g, nodes.data(), &n_nodes) != cudaSuccess) { (void)cudaGetLastError(); graph_drop(t); return false; }
    std::vector<int> seen(static_cast<size_t>(std::max(n_seeds, 1)), 0);
    for (cudaGraphNode_t node : nodes) {
        cudaGraphNodeType type;
        if (cudaGraphNodeGetType(node, &type) != cudaSuccess || type != cudaGraphNodeTypeKernel) continue;
        cudaKernelNodeParams kp{};
        if (cudaGraphKernelNodeGetParams(node, &kp) != cudaSuccess || !kp.kernelParams) { (void)cudaGetLastError(); continue; }
        void** a = kp.kernelParams;
        if (kp.func == wb_dropout_kernel_func()) {
            const uint64_t seed = *static_cast<uint64_t*>(a[6]);
            if (seed < SEED_SENTINEL || seed >= SEED_SENTINEL + static_cast<uint64_t>(n_seeds)) continue;  // a mask-free use of the kernel (ReLU backward)
            WbTrainer::DropNode d{};
            d.node = node; d.p = kp; d.ordinal = static_cast<int>(seed - SEED_SENTINEL);
            d.y = *static_cast<float**>(a[0]); d.x = *static_cast<const float**>(a[1]); d.relu_src = *static_cast<const float**>(a[2]);
            d.n = *static_cast<int64_t*>(a[3]); d.kmin = *static_cast<uint64_t*>(a[4]); d.scale = *static_cast<float*>(a[5]); d.vec = *static_cast<int*>(a[7]);
            seen[d.ordinal]++;
            t->g_drops.push_back(d);
        } else if (kp.func == wb_adam_kernel_func()) {
            WbTrainer::AdamNode d{};
            d.node = node; d.p = kp;
            d.theta = *static_cast<float**>(a[0]); d.grad = *static_cast<const float**>(a[1]); d.m = *static_cast<float**>(a[2]); d.v = *static_cast<float**>(a[3]);
            d.n = *static_cast<int64_t*>(a[4]); d.vec = *static_cast<int*>(a[6]);
            t->g_adams.push_back(d);
        }
    }
    bool complete = !t->g_adams.empty();
    for (int i = 0; i < n_seeds; ++i) complete = complete && seen[i] > 0;
    if (!complete) { graph_drop(t); return false; }
    t->g_x = t->x_in;
    t->g_y = t->y_in;
    t->g_scratch = b->scratch;
    return true;
}

}  // namespace

// Whether wb_trainer_step and wb_trainer_step_host replay a captured graph (1) or issue the launches one by one (0,
// the default).  Not for trainers with a bucket callback (the data-parallel step issues work on other streams).
extern "C" int wb_trainer_use_graph(WbTrainer* t, int on) {
    WB_REQUIRE(t, WB_ERR_INVALID, "wb_trainer_use_graph: null trainer");
    t->graph_on = on != 0;
    if (!t->graph_on) graph_drop(t);
    return WB_OK;
}

// One whole step on the staged batch: wb_trainer_forward_backward followed by wb_trainer_adam_step(1.0), same results.
extern "C" int wb_trainer_step(WbTrainer* t, const uint64_t* dropout_seeds, int n_seeds) {
    WB_REQUIRE(t, WB_ERR_INVALID, "wb_trainer_step: null trainer");
    WbBackend* b = t->be;
    if (!t->graph_on || t->graph_failed || t->cb || t->timing || b->profiling || t->eager_steps < 1) {
        t->eager_steps++;
        return eager_step(t, dropout_seeds, n_seeds);
    }
    int n_drop = 0;
    for (const Layer& L : t->layers) n_drop += L.kind == L_DROPOUT && L.p > 0.0 && L.p < 1.0;
    WB_REQUIRE(n_seeds == n_drop && (n_drop == 0 || dropout_seeds), WB_ERR_INVALID, "trainer: expected %d dropout seeds, got %d", n_drop, n_seeds);
    // the capture baked in the staged batch's address and the backend's scratch block: capture again if either moved
    if (t->gexec && (t->g_x != t->x_in || t->g_y != t->y_in || t->g_scratch != b->scratch)) graph_drop(t);
    if (!t->gexec && !graph_capture(t, n_seeds)) {
        t->graph_failed = true;
        return eager_step(t, dropout_seeds, n_seeds);
    }
    t->t += 1;
    const WbAdamConfig& ac = t->adam;
    AdamK k = wb_adam_constants(t->t, ac.lr, ac.beta1, ac.beta2, ac.eps, ac.weight_decay, ac.decoupled, 1.0);
    for (WbTrainer::DropNode& d : t->g_drops) {
        uint64_t seed = dropout_seeds[d.ordinal];
        void* args[8] = {&d.y, &d.x, &d.relu_src, &d.n, &d.kmin, &d.scale, &seed, &d.vec};
        d.p.kernelParams = args;
        d.p.extra = nullptr;
        WB_CHECK_CUDA(cudaGraphExecKernelNodeSetParams(t->gexec, d.node, &d.p));
    }
    for (WbTrainer::AdamNode& d : t->g_adams) {
        void* args[7] = {&d.theta, &d.grad, &d.m, &d.v, &d.n, &k, &d.vec};
        d.p.kernelParams = args;
        d.p.extra = nullptr;
        WB_CHECK_CUDA(cudaGraphExecKernelNodeSetParams(t->gexec, d.node, &d.p));
    }
    WB_CHECK_CUDA(cudaGraphLaunch(t->gexec, b->stream));
    b->launches++;
    return WB_OK;
}

// The call a user makes per step: host batch in, loss out.  Copies the batch from (pinned) host
// memory, runs forward/backward/Adam and reads the loss back; waits for the stream.
extern "C" int wb_trainer_step_host(WbTrainer* t, const float* host_x, const int64_t* host_y, const uint64_t* dropout_seeds, int n_seeds,
                                    float* host_loss) {
    WB_REQUIRE(t && host_x && host_y, WB_ERR_INVALID, "wb_trainer_step_host: null pointer");
    WbBackend* b = t->be;
    WB_CHECK_CUDA(cudaMemcpyAsync(t->x_in, host_x, static_cast<size_t>(t->batch * t->in_elems) * sizeof(float), cudaMemcpyHostToDevice, b->stream));
    WB_CHECK_CUDA(cudaMemcpyAsync(t->y_in, host_y, static_cast<size_t>(t->batch) * sizeof(int64_t), cudaMemcpyHostToDevice, b->stream));
    WB_TRY(wb_trainer_step(t, dropout_seeds, n_seeds));
    WB_CHECK_CUDA(cudaMemcpyAsync(t->loss_pinned, t->loss_dev, sizeof(float), cudaMemcpyDeviceToHost, b->stream));
    WB_CHECK_CUDA(cudaStreamSynchronize(b->stream));
    if (host_loss) *host_loss = *t->loss_pinned;
    return WB_OK;
}

extern "C" int wb_trainer_read_loss(WbTrainer* t, float* host_loss) {
    WbBackend* b = t->be;
    WB_CHECK_CUDA(cudaMemcpyAsync(t->loss_pinned, t->loss_dev, sizeof(float), cudaMemcpyDeviceToHost, b->stream));
    WB_CHECK_CUDA(cudaStreamSynchronize(b->stream));
    *host_loss = *t->loss_pinned;
    return WB_OK;
}

extern "C" int wb_trainer_set_timing(WbTrainer* t, int on) {
    t->timing = on != 0;
    return WB_OK;
}

// Waits for the stream, then returns one line per op label: "label calls total_ms" (device time
// between the event pairs recorded since the last report).  The string stays valid until the next call.
extern "C" const char* wb_trainer_timing_report(WbTrainer* t) {
    cudaStreamSynchronize(t->be->stream);
    std::vector<double> ms(t->labels.size(), 0.0);
    std::vector<int64_t> calls(t->labels.size(), 0);
    for (auto& r : t->recs) {
        float e = 0.f;
        if (cudaEventElapsedTime(&e, r.e0, r.e1) == cudaSuccess) { ms[r.label] += e; calls[r.label]++; }
        t->event_pool.push_back(r.e0);
        t->event_pool.push_back(r.e1);
    }
    t->recs.clear();
    t->timing_text.clear();
    char line[160];
    for (size_t i = 0; i < t->labels.size(); ++i) {
        if (!calls[i]) continue;
        snprintf(line, sizeof line, "%s %lld %.6f\n", t->labels[i].c_str(), (long long)calls[i], ms[i]);
        t->timing_text += line;
    }
    return t->timing_text.c_str();
}
