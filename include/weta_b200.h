/* weta_b200.h -- C ABI of the B200-native tensor-operator backend for weta.
 *
 * Every entry point below stands in for one method of `weta_core::Backend`
 * (crates/weta-core/src/backend.rs:65-106) or for one piece of glue the reference CUDA crate
 * exposes to `weta-tensor` (crates/weta-cuda/src/lib.rs:129-156).  The citation on each
 * declaration names the reference interface it replaces.  Entry points under "extension" have
 * no trait method today: in Rust they would be default-bodied trait methods, the way `random`
 * already is (backend.rs:94-105), so existing crates keep compiling.
 *
 * Conventions (same as the trait, backend.rs:59-64):
 *   - shapes, strides and offsets count ELEMENTS, at most WB_MAX_DIMS dimensions;
 *   - inputs are strided views (stride 0 = broadcast); every op produces fresh contiguous output;
 *   - all work is asynchronous on the backend's one stream; only wb_to_host / wb_synchronize wait;
 *   - every function returns a WbStatus; on failure wb_last_error() holds the message (per thread).
 *     The reference panics where this ABI returns non-zero (e.g. lib.rs:207, 387, 518).
 *   - there is no CPU fallback: without a usable CUDA device wb_backend_create fails with
 *     WB_ERR_DEVICE_UNAVAILABLE, the counterpart of Error::DeviceUnavailable (lib.rs:131-133).
 */
#ifndef WETA_B200_H
#define WETA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WB_MAX_DIMS 8 /* crates/weta-cuda/src/lib.rs:67 */

typedef enum WbStatus {
    WB_OK = 0,
    WB_ERR_INVALID = 1,            /* bad argument (shape/dtype mismatch, null pointer) */
    WB_ERR_UNSUPPORTED = 2,        /* op not defined for this dtype (the reference panics) */
    WB_ERR_CUDA = 3,               /* a CUDA call failed */
    WB_ERR_OOM = 4,
    WB_ERR_DEVICE_UNAVAILABLE = 5, /* weta_core::Error::DeviceUnavailable */
    WB_ERR_TIMEOUT = 6             /* a bounded device-side wait ran out */
} WbStatus;

/* crates/weta-core/src/dtype.rs:9-14 */
typedef enum WbDType { WB_F32 = 0, WB_F64 = 1, WB_I64 = 2 } WbDType;

/* crates/weta-core/src/ops.rs:7-36, numbered as crates/weta-cuda/src/lib.rs:256-278.
 * AFFINE uses (p1, p2) = (mul, add); POWF, GT_SCALAR, MAX_SCALAR, MIN_SCALAR use p1. */
typedef enum WbUnaryOp {
    WB_NEG = 0, WB_EXP, WB_LOG, WB_SQRT, WB_ABS, WB_SIGN, WB_RELU, WB_STEP, WB_TANH, WB_SIGMOID, WB_ERF,
    WB_SIN, WB_COS, WB_RECIP, WB_AFFINE, WB_POWF, WB_GT_SCALAR, WB_MAX_SCALAR, WB_MIN_SCALAR
} WbUnaryOp;

/* crates/weta-core/src/ops.rs:68-82, numbered as crates/weta-cuda/src/lib.rs:280-296 */
typedef enum WbBinaryOp {
    WB_ADD = 0, WB_SUB, WB_MUL, WB_DIV, WB_POW, WB_MAXIMUM, WB_MINIMUM, WB_EQ, WB_NE, WB_LT, WB_LE, WB_GT, WB_GE
} WbBinaryOp;

/* crates/weta-core/src/ops.rs:106-112 */
typedef enum WbReduceOp { WB_SUM = 0, WB_MAX, WB_MIN, WB_ARGMAX, WB_ARGMIN } WbReduceOp;

/* crates/weta-core/src/ops.rs:154-157 */
typedef enum WbDistribution { WB_UNIFORM = 0 /* a = lo, b = hi */, WB_NORMAL = 1 /* a = mean, b = std */ } WbDistribution;

/* How float32 contractions are evaluated.  The reference calls cuBLAS in its default FP32 mode
 * (crates/weta-cuda/src/lib.rs:351-389). */
typedef enum WbMatmulMode {
    WB_MM_TF32X3 = 0, /* tcgen05 kind::tf32, three products per term: FP32-grade accuracy (default) */
    WB_MM_TF32 = 1,   /* tcgen05 kind::tf32, one product per term */
    WB_MM_FP32 = 2    /* CUDA-core FP32 FMA tiles (also what f64 and irregular layouts use) */
} WbMatmulMode;

/* A strided look at device memory: crates/weta-core/src/backend.rs:4-8 (`View`) with the layout
 * of crates/weta-core/src/layout.rs:16-21 flattened the way the reference's kernels receive it
 * (`Strides`, crates/weta-cuda/src/lib.rs:52-61).  `data` is the storage's base device pointer. */
typedef struct WbView {
    void* data;
    int32_t dtype;
    int32_t ndim;
    int64_t shape[WB_MAX_DIMS];
    int64_t stride[WB_MAX_DIMS];
    int64_t offset;
} WbView;

/* crates/weta-core/src/ops.rs:122-128 (`Im2ColParams`) */
typedef struct WbConvParams {
    int64_t kh, kw, sh, sw, ph, pw, dh, dw;
} WbConvParams;

typedef struct WbBackend WbBackend; /* crates/weta-cuda/src/lib.rs:122-127 (`CudaBackend`) */
typedef struct WbStorage WbStorage; /* crates/weta-cuda/src/lib.rs:26-48 (`CudaStorage`) */

/* ---- device and backend ------------------------------------------------------------------ */

/* weta_cuda::device_count (lib.rs:149-152): 0 when no driver or no device. */
int wb_device_count(void);
/* weta_cuda::backend(ordinal) (lib.rs:137-146, 176-192): context, stream, kernels.  The kernels
 * are AOT sm_100a code inside this library; nothing is compiled at run time. */
int wb_backend_create(int ordinal, WbBackend** out);
/* Same, but all work goes to the caller's CUDA stream (a cudaStream_t), so a host framework can
 * order its own copies and collectives against the backend's kernels. */
int wb_backend_create_on_stream(int ordinal, void* cuda_stream, WbBackend** out);
int wb_backend_destroy(WbBackend* b);
int wb_backend_ordinal(const WbBackend* b);   /* CudaStorage::ordinal (lib.rs:38-40) */
void* wb_backend_stream(const WbBackend* b);  /* the cudaStream_t every op is issued on */
int wb_synchronize(WbBackend* b);
const char* wb_last_error(void);
/* weta_cuda::profile_report (crates/weta-cuda/src/profile.rs:58-73): per-op call counts and
 * device time.  Profiling is on when wb_set_profiling(b, 1) was called or WETA_B200_PROFILE=1. */
int wb_set_profiling(WbBackend* b, int on);
const char* wb_profile_report(WbBackend* b);
int wb_set_matmul_mode(WbBackend* b, int mode);
int wb_get_matmul_mode(const WbBackend* b);
/* Number of kernels this backend has launched since creation (for launch accounting). */
int64_t wb_launch_count(const WbBackend* b);

/* ---- storage (Backend::Storage) ----------------------------------------------------------- */

/* `uninit` (lib.rs:204-208): uninitialised device storage from the stream-ordered arena.
 * Zero-length requests get one element, like the reference (lib.rs:206-207). */
int wb_alloc(WbBackend* b, int64_t len, int dtype, WbStorage** out);
/* Backend::zeros (backend.rs:74; lib.rs:457-461) */
int wb_zeros(WbBackend* b, int64_t len, int dtype, WbStorage** out);
/* Drop of CudaStorage: the block returns to the arena, ordered after queued work. */
int wb_free(WbBackend* b, WbStorage* s);
/* Wraps device memory owned by someone else (no copy, never freed by the backend). */
int wb_storage_wrap(WbBackend* b, void* device_ptr, int64_t len, int dtype, WbStorage** out);
void* wb_storage_data(const WbStorage* s);
int64_t wb_storage_len(const WbStorage* s);
int wb_storage_dtype(const WbStorage* s);
/* Backend::from_host (backend.rs:71; lib.rs:423-434): `host` holds `len` elements of `dtype`. */
int wb_from_host(WbBackend* b, const void* host, int64_t len, int dtype, WbStorage** out);
/* Backend::to_host (backend.rs:73; lib.rs:436-455): elements of the view in row-major order. */
int wb_to_host(WbBackend* b, const WbView* x, void* host_out);
/* Asynchronous variants for pinned host buffers (ordered on the backend stream, no wait). */
int wb_upload_async(WbBackend* b, const void* pinned_host, void* device_dst, int64_t bytes);
int wb_download_async(WbBackend* b, const void* device_src, void* pinned_host, int64_t bytes);
int64_t wb_arena_bytes_reserved(const WbBackend* b);

/* ---- the trait's kernels ------------------------------------------------------------------ */
/* Each op exists twice: `wb_x(..., WbStorage** out)` allocates the fresh contiguous result like
 * the trait method does; `wb_x_into(..., void* out)` writes it to caller-provided device memory
 * of the right size and allocates nothing. */

/* Backend::copy_strided (backend.rs:79; lib.rs:463-480): dst view elements <- src view elements. */
int wb_copy_strided(WbBackend* b, const WbView* src, const WbView* dst);
/* Backend::unary (backend.rs:81; lib.rs:482-494; CPU semantics crates/weta-cpu/src/lib.rs:133-203) */
int wb_unary(WbBackend* b, int op, double p1, double p2, const WbView* x, WbStorage** out);
int wb_unary_into(WbBackend* b, int op, double p1, double p2, const WbView* x, void* out);
/* Backend::binary (backend.rs:83; lib.rs:496-521; CPU semantics weta-cpu/src/lib.rs:205-241) */
int wb_binary(WbBackend* b, int op, const WbView* a, const WbView* bb, WbStorage** out);
int wb_binary_into(WbBackend* b, int op, const WbView* a, const WbView* bb, void* out);
/* Backend::reduce (backend.rs:85; lib.rs:523-580; CPU semantics weta-cpu/src/lib.rs:245-300).
 * ARGMAX/ARGMIN produce i64. */
int wb_reduce(WbBackend* b, int op, const WbView* x, int axis, WbStorage** out);
int wb_reduce_into(WbBackend* b, int op, const WbView* x, int axis, void* out);
/* Backend::matmul (backend.rs:87; lib.rs:603-628): [B,M,K] x [B,K,N] -> [B,M,N], any strides,
 * batch stride 0 allowed; f32 and f64. */
int wb_matmul(WbBackend* b, const WbView* a, const WbView* bb, WbStorage** out);
int wb_matmul_into(WbBackend* b, const WbView* a, const WbView* bb, void* out);
/* Backend::im2col (backend.rs:89; lib.rs:630-642; weta-cpu/src/lib.rs:367-408) */
int wb_im2col(WbBackend* b, const WbView* x, const WbConvParams* p, WbStorage** out);
int wb_im2col_into(WbBackend* b, const WbView* x, const WbConvParams* p, void* out);
/* Backend::col2im (backend.rs:91; lib.rs:644-656; weta-cpu/src/lib.rs:410-446) */
int wb_col2im(WbBackend* b, const WbView* cols, const WbConvParams* p, int64_t c, int64_t h, int64_t w, WbStorage** out);
int wb_col2im_into(WbBackend* b, const WbView* cols, const WbConvParams* p, int64_t c, int64_t h, int64_t w, void* out);
/* Backend::cast (backend.rs:92; lib.rs:658-679; weta-cpu/src/lib.rs:552-565); same dtype = contiguous(). */
int wb_cast(WbBackend* b, const WbView* x, int dtype, WbStorage** out);
int wb_cast_into(WbBackend* b, const WbView* x, int dtype, void* out);
/* Backend::random (backend.rs:97-105; lib.rs:582-601; crates/weta-core/src/ops.rs:164-189):
 * element i = Distribution::sample(seed, i).  Uniform fills are bit-identical to the CPU backend; Normal fills
 * evaluate ln and cos correctly rounded, which matches the CPU backend wherever its libm rounds correctly. */
int wb_random(WbBackend* b, int64_t len, int dtype, int dist, double pa, double pb, uint64_t seed, WbStorage** out);
int wb_random_into(WbBackend* b, int64_t len, int dtype, int dist, double pa, double pb, uint64_t seed, void* out);

/* ---- host RNG seed stream (crates/weta-tensor/src/random.rs:21-110) ----------------------- */
typedef struct WbPcg { uint64_t state, inc; } WbPcg;
void wb_pcg_seed(WbPcg* g, uint64_t seed); /* Rng::new */
uint32_t wb_pcg_next_u32(WbPcg* g);
uint64_t wb_pcg_next_u64(WbPcg* g);        /* the per-tensor seed */
uint64_t wb_splitmix64(uint64_t seed, uint64_t i); /* crates/weta-core/src/ops.rs:164-169 */
/* Host-side evaluation of what the Normal fill computes on the device (same source compiled for the CPU; needs no
 * GPU): correctly rounded ln(x) for x in (0, 1], cos(t) for t in [0, 8), and element i of a Normal{mean, std} fill as
 * f64 (Distribution::sample, crates/weta-core/src/ops.rs:182-186). */
double wb_host_log_rn(double x);
double wb_host_cos_rn(double t);
double wb_host_normal_sample(uint64_t seed, uint64_t i, double mean, double std);

/* ==== extension: entry points with no trait method today ===================================== */

/* Reads the device-side flag a tensor-core kernel raises when one of its bounded barrier waits
 * runs out (WB_ERR_TIMEOUT), then clears it.  Synchronises the stream.  The reference has no
 * counterpart: cuBLAS reports its own failures through the call's status (lib.rs:387). */
int wb_gemm_check(WbBackend* b);
/* Test hook: one thread waits with the GEMM kernels' bounded barrier wait on a barrier nothing arrives at, gives up
 * after `polls` polls (1..2^20) and raises the same flag; the next wb_gemm_check then returns WB_ERR_TIMEOUT. */
int wb_gemm_selftest_timeout(WbBackend* b, int polls);

/* A chain of unary / binary trait calls over one index space as ONE launch (no counterpart in the reference, which
 * launches each op by itself: crates/weta-cuda/src/lib.rs:482-521).  `inputs`: up to 8 f32 views of n elements each
 * (strided or broadcast; they may differ in shape, the linear row-major index is what they share).  `prog`: up to
 * 48 instructions, instruction k producing value k: kind 0 loads inputs[a]; kind 1 applies WbUnaryOp `op` with (p1, p2)
 * to value a; kind 2 applies WbBinaryOp `op` to values a and b (a, b < k).  Values out_regs[0..n_outputs) are stored
 * contiguously to outs[..] (up to 4).  An output may be the storage of an input read through a contiguous view.
 * Results are bit-identical to issuing the same ops one launch at a time. */
#define WB_EWF_MAX_INPUTS 8
#define WB_EWF_MAX_INSTRS 48
#define WB_EWF_MAX_OUTPUTS 4
typedef struct WbEwInstr { int32_t kind, op, a, b; double p1, p2; } WbEwInstr;
int wb_ew_fused(WbBackend* b, const WbView* inputs, int n_inputs, const WbEwInstr* prog, int n_instr, const int32_t* out_regs,
                void* const* outs, int n_outputs, int64_t n);

/* ---- fused layer ops ------------------------------------------------------------------------
 * Each stands for the chain of trait calls the reference issues for one layer; pointers are f32
 * device memory, tensors are contiguous NCHW / row-major. */

/* F::dropout in training mode (crates/weta-nn/src/functional.rs:64-74): y = x * mask with
 * mask_i = (rand_f32(seed)_i > p) / (1 - p), the mask regenerated from the seed (never stored);
 * values are bit-identical to the four-call chain random -> gt_scalar -> mul_scalar -> mul.  p = 0 gives y = x,
 * p = 1 gives y = x * 0 (functional.rs:66-71). */
int wb_dropout_fwd(WbBackend* b, const float* x, float* y, int64_t n, double p, uint64_t seed);
/* Its backward, dx = dy * mask, optionally times step(relu_out) (ReLU backward, autograd ops.rs:85). */
int wb_dropout_relu_bwd(WbBackend* b, const float* dy, const float* relu_out, float* dx, int64_t n, double p, uint64_t seed);
/* Just the mask values (0 or f32(1/(1-p))). */
int wb_dropout_mask(WbBackend* b, float* mask, int64_t n, double p, uint64_t seed);
/* Tensor::cross_entropy forward and CrossEntropyBw (crates/weta-autograd/src/ops.rs:444-519), mean
 * reduction: logits [rows, cols], labels i64 [rows].  Any of probs / dlogits / row_loss / mean_loss may
 * be null.  dlogits = (softmax - onehot) * upstream / rows. */
int wb_softmax_ce(WbBackend* b, const float* logits, const int64_t* labels, int64_t rows, int64_t cols, float* probs,
                  float* dlogits, float* row_loss, float* mean_loss, double upstream);
/* F::batch_norm in training mode (crates/weta-nn/src/functional.rs:144-180) on [n, c, hw]: batch mean,
 * biased variance -> rstd = 1/sqrt(var + eps); running stats updated with the unbiased variance. */
int wb_bn2d_stats(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t hw, double eps, double momentum, float* mean,
                  float* rstd, float* running_mean, float* running_var);
int wb_bn2d_apply(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t hw, const float* mean, const float* rstd,
                  const float* gamma, const float* beta, int relu, float* y);
/* No counterpart in the reference.  wb_bn2d_stats for callers that must not allocate device memory when
 * they call (inside an allocator hook or memory-pool callback, in a loop that has frozen its memory map,
 * or with the device's memory fully budgeted elsewhere): it takes no backend handle, runs on the current
 * device and the given cudaStream_t, and keeps its partial sums in a fixed 512 KiB array inside the library
 * instead of arena scratch.  Limit: c <= 32768 channels (else WB_ERR_INVALID).  The first call on a device
 * resolves the array's address and may load the library's device code (which takes device memory): make one
 * warm-up call per device at start-up, outside the no-allocation context and before any stream capture; two
 * host threads racing on that first call store the same address, which is harmless.  Calls share the array:
 * calls that overlap on the GPU race; keep them on one stream or order them yourself. */
int wb_bn2d_stats_noalloc(void* cuda_stream, const float* x, int64_t n, int64_t c, int64_t hw, double eps, double momentum,
                          float* mean, float* rstd, float* running_mean, float* running_var);
int wb_bn2d_fwd(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t hw, const float* gamma, const float* beta,
                float* running_mean, float* running_var, double momentum, double eps, float* y, float* save_mean, float* save_rstd);
/* The gradient autograd derives through that chain: dx, dgamma = sum(dy*xhat), dbeta = sum(dy). */
int wb_bn2d_bwd(WbBackend* b, const float* x, const float* dy, int64_t n, int64_t c, int64_t hw, const float* gamma,
                const float* save_mean, const float* save_rstd, float* dx, float* dgamma, float* dbeta);
/* BatchNorm2d -> ReLU -> MaxPool2d(2) of crates/weta/examples/mnist_cnn.rs:18-20 in one pass: x [n,c,h,w]
 * -> y_pooled [n,c,h/2,w/2].  Backward recomputes the activations from x; max-pool ties share the
 * gradient equally (crates/weta-autograd/src/ops.rs:305-314).  dbias_conv (optional) receives sum(dx)
 * per channel, the gradient of the bias of the convolution that produced x. */
int wb_bn_relu_pool_fwd(WbBackend* b, const float* x, int64_t n, int64_t c, int64_t h, int64_t w, const float* gamma,
                        const float* beta, float* running_mean, float* running_var, double momentum, double eps, float* y_pooled,
                        float* save_mean, float* save_rstd);
int wb_bn_relu_pool_bwd(WbBackend* b, const float* x, const float* dy_pooled, int64_t n, int64_t c, int64_t h, int64_t w,
                        const float* gamma, const float* beta, const float* save_mean, const float* save_rstd, float* dx,
                        float* dgamma, float* dbeta, float* dbias_conv);
/* F::linear (crates/weta-nn/src/functional.rs:54-60): y[n, out] = x[n, in] * weight[out, in]^T + bias (bias may be
 * NULL; relu != 0 applies ReLU in the same pass), in the backend's matmul mode.  Backward (MatmulBw,
 * crates/weta-autograd/src/ops.rs:821-827, and the bias's sum over the batch, ops.rs:46-58): dweight[out, in] =
 * dy^T x, dbias[out] = sum_n dy, dx[n, in] = dy * weight; any of the three outputs may be NULL. */
int wb_linear_fwd(WbBackend* b, const float* x, const float* weight, const float* bias, int64_t n, int64_t in, int64_t out, int relu,
                  float* y);
int wb_linear_bwd(WbBackend* b, const float* x, const float* weight, const float* dy, int64_t n, int64_t in, int64_t out, float* dx,
                  float* dweight, float* dbias);
/* F::max_pool2d (functional.rs:121-130) over `planes` = N*C contiguous [h, w] planes, square kernel, no padding:
 * y[planes, oh, ow] with weta's max rule (a NaN wins).  Backward (ops.rs:305-314): positions equal to their
 * window's maximum share its gradient equally; overlapping windows add. */
int wb_maxpool2d_fwd(WbBackend* b, const float* x, int64_t planes, int64_t h, int64_t w, int64_t kernel, int64_t stride, float* y);
int wb_maxpool2d_bwd(WbBackend* b, const float* x, const float* dy, int64_t planes, int64_t h, int64_t w, int64_t kernel, int64_t stride,
                     float* dx);
/* UnaryBw for ReLU (ops.rs:85): dx = dy * step(y); y is the ReLU's input or output. */
int wb_relu_bwd(WbBackend* b, const float* dy, const float* y, float* dx, int64_t n);
/* 3x3, stride 1, padding 1 convolution over contiguous NCHW f32 tensors as an implicit GEMM on the
 * tensor cores (TF32 operands, f32 accumulation; no im2col matrix in memory).  Forward replaces the
 * chain F::conv2d_ext builds (crates/weta-nn/src/functional.rs:84-106: im2col -> matmul -> add bias,
 * bias may be NULL); backward replaces MatmulBw + Im2ColBw + the sum over the batch
 * (crates/weta-autograd/src/ops.rs:821-827, 865-868): dweight [o,c,3,3] and dx [n,c,h,w], either may be
 * NULL.  Shape rules: w % 4 == 0, c % 128 == 0, o % 32 == 0; WB_ERR_UNSUPPORTED otherwise (use wb_im2col +
 * wb_matmul).  Scratch (two shifted copies of the image operand, the reordered weight) comes from the arena. */
int wb_conv3x3_fwd(WbBackend* b, const float* x, const float* weight, const float* bias, int64_t n, int64_t c, int64_t h, int64_t w,
                   int64_t o, float* y);
int wb_conv3x3_bwd(WbBackend* b, const float* x, const float* weight, const float* dy, int64_t n, int64_t c, int64_t h, int64_t w,
                   int64_t o, float* dx, float* dweight);
/* Adam::step / AdamW for one flat parameter range at step t >= 1 (crates/weta-optim/src/lib.rs:210-239,
 * 276-283), every f32 rounding of the 13-call chain kept.  grad_scale multiplies the gradient first
 * (1/world after a summing all-reduce); 1.0 leaves the chain untouched. */
int wb_adam_step(WbBackend* b, float* theta, const float* grad, float* m, float* v, int64_t n, int64_t t, double lr, double beta1,
                 double beta2, double eps, double weight_decay, int decoupled, double grad_scale);

/* ---- fused training step ---------------------------------------------------------------------
 * The step of crates/weta/examples/mnist_cnn.rs:63-73 / mnist_mlp.rs (forward, cross-entropy,
 * backward, Adam) for a sequential model made of the three layer kinds below, run as a fixed
 * sequence of fused kernels instead of ~400 trait calls.  Parameters, gradients and Adam state live
 * in one flat f32 arena, layers in reverse order; wb_trainer_tensor_range maps the reference's
 * parameter order (layer by layer: weight, bias, then BatchNorm weight, bias) onto it. */
typedef enum WbLayerKind {
    WB_LAYER_CONV_BN_RELU_POOL = 0, /* Conv2d(a -> b, 3x3, padding 1) + BatchNorm2d + ReLU + MaxPool2d(2) */
    WB_LAYER_LINEAR = 1,            /* Linear(a -> b), followed by ReLU when c != 0 */
    WB_LAYER_DROPOUT = 2            /* Dropout(p), training mode */
} WbLayerKind;
typedef struct WbLayerSpec { int32_t kind, a, b, c; double p; } WbLayerSpec;
/* Adam / AdamW hyper-parameters (crates/weta-optim/src/lib.rs:178-207, 276-283). */
typedef struct WbAdamConfig { double lr, beta1, beta2, eps, weight_decay; int32_t decoupled; } WbAdamConfig;
typedef struct WbTrainer WbTrainer;
/* Called during backward each time one layer's gradients are final: a contiguous arena range.  Also called with
 * (NULL, 0) at each "quiet point" of backward: right after a conv block's memory-bound BatchNorm pass has been queued
 * and before its tensor-core contractions, the moment at which side-stream work (a gradient exchange) disturbs the
 * step least. */
typedef void (*wb_bucket_callback)(void* user, float* grad_range, int64_t len);

/* Input is [batch, in_c, in_h, in_w] (NCHW; use in_h = in_w = 1 for flat features). */
int wb_trainer_create(WbBackend* b, const WbLayerSpec* layers, int n_layers, int64_t batch, int64_t in_c, int64_t in_h,
                      int64_t in_w, const WbAdamConfig* adam, int matmul_mode, WbTrainer** out);
int wb_trainer_destroy(WbTrainer* t);
/* Default init of crates/weta-nn/src/layers.rs:19-26 from one RNG seed per weight / bias tensor, in creation order. */
int wb_trainer_init(WbTrainer* t, const uint64_t* seeds, int n_seeds);
int64_t wb_trainer_arena_len(const WbTrainer* t);
float* wb_trainer_params(WbTrainer* t);      /* device pointers into the flat arenas */
float* wb_trainer_grads(WbTrainer* t);
float* wb_trainer_exp_avg(WbTrainer* t);
float* wb_trainer_exp_avg_sq(WbTrainer* t);
float* wb_trainer_input(WbTrainer* t);       /* staged batch: f32 [batch, in_c*in_h*in_w] */
int64_t* wb_trainer_labels(WbTrainer* t);
/* Reads the following steps' batch from caller-owned device buffers instead (the slots of a double-buffered
 * upload); NULL, NULL restores the trainer's own staging buffers.  No counterpart in the reference, which uploads
 * each batch synchronously (`Tensor::to`, crates/weta-tensor/src/tensor.rs:235-240). */
int wb_trainer_set_input(WbTrainer* t, float* x, int64_t* y);    /* staged labels: i64 [batch] */
float* wb_trainer_loss_ptr(WbTrainer* t);    /* device scalar written by forward_backward */
int wb_trainer_num_tensors(const WbTrainer* t);
int wb_trainer_tensor_range(const WbTrainer* t, int index, int64_t* offset, int64_t* len);
int wb_trainer_bn_buffers(WbTrainer* t, int conv_index, float** running_mean, float** running_var, int64_t* channels);
int wb_trainer_set_bucket_callback(WbTrainer* t, wb_bucket_callback cb, void* user);
/* Forward, mean cross-entropy and backward on the staged batch; one seed per dropout layer with 0 < p < 1, in forward
 * order (p = 0 and p = 1 need no mask and, as in crates/weta-nn/src/functional.rs:66-71, consume no seed). */
int wb_trainer_forward_backward(WbTrainer* t, const uint64_t* dropout_seeds, int n_seeds);
/* Adam over the whole arena; grad_scale = 1/world after a summing all-reduce, else 1. */
int wb_trainer_adam_step(WbTrainer* t, double grad_scale);
/* One whole step on the staged batch: wb_trainer_forward_backward followed by wb_trainer_adam_step(t, 1.0), with the same
 * results.  After wb_trainer_use_graph(t, 1) the step is captured once into a CUDA graph and replayed (one launch per
 * step instead of 25-40; the first step always runs eagerly); per step only the dropout seeds and the Adam scalars are
 * rewritten in the graph's kernel nodes.  A capture that fails, a bucket callback or per-op timing make the call issue
 * its launches one by one as before.  No counterpart in the reference (its steps are ~400 separate launches,
 * README.md:123-124). */
int wb_trainer_use_graph(WbTrainer* t, int on);
int wb_trainer_step(WbTrainer* t, const uint64_t* dropout_seeds, int n_seeds);
/* The same update range by range, on another backend handle's stream (same device), for callers that overlap
 * the optimizer with backward: wb_trainer_begin_step advances and returns the step count, which every
 * wb_trainer_adam_range call of that step passes.  The ranges of one step must tile the arena exactly once.
 * No counterpart in the reference (its optimizer walks the parameter list after backward). */
int64_t wb_trainer_begin_step(WbTrainer* t);
int wb_trainer_adam_range(WbTrainer* t, WbBackend* on, int64_t offset, int64_t len, int64_t step, double grad_scale);
/* One whole step from host memory: upload batch, forward/backward/Adam, download the loss, wait. */
int wb_trainer_step_host(WbTrainer* t, const float* host_x, const int64_t* host_y, const uint64_t* dropout_seeds, int n_seeds,
                         float* host_loss);
int wb_trainer_read_loss(WbTrainer* t, float* host_loss);
/* Per-op device timing (the counterpart of WETA_CUDA_PROFILE, crates/weta-cuda/src/profile.rs, without
 * its per-call synchronisation): event pairs are recorded around each op while timing is on;
 * the report waits for the stream and returns lines "label calls total_ms". */
int wb_trainer_set_timing(WbTrainer* t, int on);
const char* wb_trainer_timing_report(WbTrainer* t);

/* ---- data-parallel training step ---------------------------------------------------------------
 * No counterpart in the reference: its backends are per-ordinal singletons with no gradient exchange
 * (crates/weta-cuda/src/lib.rs:129-146).  One process (or host thread) per GPU, every rank a full replica built
 * from the same seeds, the batch sharded by samples; BatchNorm statistics stay per rank (the reference has no
 * SyncBN).  The one exchange sits between backward and Adam::step (crates/weta-optim/src/lib.rs:210-239): the
 * gradient arena is cut into buckets of whole layers, and as soon as backward has finished a bucket its exchange
 * and its optimizer update run on side streams while backward continues. */
#define WB_DP_ID_BYTES 128
typedef struct WbDpId { char bytes[WB_DP_ID_BYTES]; } WbDpId;
typedef enum WbDpMode {
    WB_DP_AUTO = 0,      /* PEER when the ranks can map each other's memory, else SHARDED; WETA_B200_DP_MODE overrides */
    WB_DP_ALLREDUCE = 1, /* ncclAllReduce per bucket, Adam over the whole bucket on every rank */
    WB_DP_SHARDED = 2,   /* ncclReduceScatter -> Adam on this rank's 1/world of the bucket -> ncclAllGather of the parameters */
    WB_DP_PEER = 3       /* this library's kernel: peer loads of every replica's gradient shard over NVLink, sum in rank
                            order, Adam, peer stores of the new parameters into every replica (arenas shared by CUDA IPC) */
} WbDpMode;
typedef struct WbDp WbDp;
/* Rank 0 makes the id and hands its bytes to the other ranks over any host channel (ncclGetUniqueId). */
int wb_dp_unique_id(WbDpId* out);
/* Collective: every rank calls it with the same id, world, mode and bucket_elems (<= 0: 2^20), after wb_trainer_init.
 * world == 1 needs no id and no NCCL.  The trainer's bucket callback is taken over by the handle. */
int wb_dp_create(WbTrainer* t, const WbDpId* id, int rank, int world, int mode, int64_t bucket_elems, WbDp** out);
int wb_dp_destroy(WbDp* dp);
int wb_dp_mode(const WbDp* dp);   /* the mode in use (AUTO resolved; the same on every rank) */
int wb_dp_world(const WbDp* dp);
int wb_dp_num_buckets(const WbDp* dp);
int wb_dp_bucket(const WbDp* dp, int index, int64_t* offset, int64_t* len);
/* One step on the staged batch (wb_trainer_input / wb_trainer_labels / wb_trainer_set_input): forward, loss,
 * backward with every bucket's exchange + update queued behind it; the next step waits for the last update.
 * Asynchronous; wb_dp_wait or wb_trainer_read_loss waits. */
int wb_dp_step(WbDp* dp, const uint64_t* dropout_seeds, int n_seeds);
/* Double-buffered input: wb_dp_submit queues the upload of one batch from PINNED host memory into one of two device
 * slots on a copy stream (at most two batches ahead of the steps); wb_dp_step_submitted steps on the oldest submitted
 * batch and, when host_loss is given, reads the loss back and waits.  Replaces the per-batch `Tensor::to`
 * (crates/weta-tensor/src/tensor.rs:235-240) and `loss.item()` of crates/weta/examples/mnist_cnn.rs:63-73. */
int wb_dp_submit(WbDp* dp, const float* pinned_x, const int64_t* pinned_y);
int wb_dp_step_submitted(WbDp* dp, const uint64_t* dropout_seeds, int n_seeds, float* host_loss);
/* Waits for everything queued so far.  timeout_ms > 0: a host watchdog polls completion, the status word of the
 * bounded device-side waits and ncclCommGetAsyncError; on expiry the communicator is aborted and WB_ERR_TIMEOUT
 * returned, so a rank whose peer never joined gets an error instead of a hang.  timeout_ms <= 0: no limit. */
int wb_dp_wait(WbDp* dp, int timeout_ms);
int wb_dp_set_timing(WbDp* dp, int on);
const char* wb_dp_timing_report(WbDp* dp); /* "bucket_work calls total_ms": device time of the side-stream work */
/* Pure host logic (no device needed): how per-layer arena ranges, in arena order, merge into buckets of at least
 * min_elems elements.  Returns the number of buckets (which may exceed max_buckets; only that many are written). */
int wb_dp_plan_buckets(const int64_t* range_off, const int64_t* range_len, int n, int64_t min_elems, int64_t* bucket_off, int64_t* bucket_len,
                       int max_buckets);
/* The watchdog loop by itself: polls `poll(user)` (0 = finished, 1 = still running, other = failed) every interval_us
 * until it finishes or timeout_ms have passed (0 = no limit); WB_OK, WB_ERR_TIMEOUT or WB_ERR_CUDA. */
typedef int (*wb_poll_fn)(void* user);
int wb_watchdog_wait(wb_poll_fn poll, void* user, int timeout_ms, int interval_us);
/* The PEER-mode kernel as an operation of its own: sums `world` (<= 8) gradient buffers element-wise in index order,
 * runs Adam step t (as wb_adam_step, grad_scale applied to the sum) on elements [offset, offset + len) of the parameters
 * in thetas[self] with the caller's m / v, and stores the new parameters into all `world` parameter buffers.  Buffers
 * may be local or peer mappings; all 16-byte aligned, offset and len multiples of 4. */
int wb_reduce_adam_broadcast(WbBackend* b, const float* const* grads, float* const* thetas, int world, int self, int64_t offset, int64_t len,
                             float* m, float* v, int64_t t, double lr, double beta1, double beta2, double eps, double weight_decay, int decoupled,
                             double grad_scale);
/* Exercises the bounded device-side wait of the PEER mode on one GPU: polls a flag word that nothing sets (unless
 * preset != 0) for timeout_ms (1..5000), then returns WB_ERR_TIMEOUT with the context still usable. */
int wb_dp_selftest_wait(WbBackend* b, int timeout_ms, int preset);

#ifdef __cplusplus
}
#endif
#endif /* WETA_B200_H */
