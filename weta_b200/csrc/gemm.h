// Internal GEMM service shared by Backend::matmul and the fused trainer.
#pragma once

#include "tc_gemm.cuh"

// One GEMM operand as the tensor core sees it: `rows` x `k` elements, either K-major (element
// (r, kk) at ptr + r*ld + kk) or MN-major (element (r, kk) at ptr + kk*ld + r).
struct WbGemmOperand {
    const float* ptr;
    int64_t rows, k, ld, batch_stride;  // batch_stride 0 = shared by every batch
    bool mn_major;
};

// D = A x B (+ epilogue) on the tensor cores; mode is WB_MM_TF32 or WB_MM_TF32X3.  Returns
// WB_ERR_UNSUPPORTED, without an error message, when TMA cannot read an operand (misaligned base
// or pitch): the caller then uses the CUDA-core path.  span_batch > 0: A and B are batched K-major
// operands and the contraction runs over (image, k) pairs into one [m, n] result.
int wb_tc_gemm(WbBackend* be, WbGemmOperand A, WbGemmOperand B, int64_t batch, int m, int n, int k, tc::Epilogue ep, int mode,
               int force_splits, int64_t span_batch);

// Implicit-GEMM 3x3 convolution pieces (forward / input gradient: mode 1, weight gradient: mode 2); see gemm_tcgen05.cu.
int wb_tc_conv_gemm(WbBackend* be, int mode, const float* a, const float* const img[3], int64_t batch, int64_t ch, int64_t h, int64_t w, int m,
                    tc::Epilogue ep);

// Whether mode 3 of wb_tc_conv_gemm (input gradient from the unshifted gradient tensor) takes this layer: ch = the
// contraction's channels (the layer's outputs), m = the result's rows (its inputs).
bool wb_tc_conv_mode3_ok(int64_t ch, int64_t h, int64_t w, int64_t m);

// Implicit 3x3 convolution built on wb_tc_conv_gemm (conv_implicit.cu).
struct WbConv3 { int64_t n, c, h, w, o; };
bool wb_conv3_eligible(const WbConv3& g);
int wb_conv3_shift_copies(WbBackend* b, const float* in, int64_t rows, int w, float* left, float* right);
int wb_conv3_weight_reorder(WbBackend* b, int kind, const float* src, float* dst, int o_n, int c_n, float* dst2 = nullptr);
int wb_conv3_fwd(WbBackend* b, const WbConv3& g, const float* const x3[3], const float* wr, const float* bias, float* y,
                 double* channel_sums);
int wb_conv3_wgrad(WbBackend* b, const WbConv3& g, const float* dy, const float* const x3[3], float* dwr, float* dweight);
// dy3[0] == dy3[2] == nullptr: the layer must pass wb_conv3_dgrad_needs_no_copies; the gradient is then read from dy3[1] alone.
bool wb_conv3_dgrad_needs_no_copies(const WbConv3& g);
int wb_conv3_dgrad(WbBackend* b, const WbConv3& g, const float* const dy3[3], const float* wt, float* dx);

// Tensor-map and error-flag access for tensor-core kernels outside gemm_tcgen05.cu.
int wb_tc_encode(WbBackend* be, const float* ptr, const uint64_t dims[3], const uint64_t strides[2], const uint32_t box[3], bool swizzle128,
                 CUtensorMap* map);
int wb_tc_error_flag(WbBackend* be, int** flag);

// BatchNorm+ReLU+pool backward of the first convolution block fused with that convolution's weight gradient
// (conv1_bwd_fused.cu): dconv is never written.  `cols` is the block's im2col matrix [n][ck][h*w].
bool wb_conv1_bwd_fused_ok(int64_t n, int64_t cout, int64_t h, int64_t w, int64_t ck, const float* x, const float* dy_pooled, const float* cols);
int wb_conv1_bwd_fused(WbBackend* b, const float* x, const float* dy_pooled, const float* cols, int64_t n, int64_t h, int64_t w, int64_t ck,
                       const float* gamma, const float* beta, const float* save_mean, const float* save_rstd, const float* dgamma,
                       const float* dbeta, float* dweight, float* dbias_conv);

// Tensor cores first, CUDA-core tiles otherwise (dense.cu).
int wb_gemm_dispatch(WbBackend* be, int mode, WbGemmOperand A, WbGemmOperand B, int64_t batch, int m, int n, int k, tc::Epilogue ep,
                     int64_t span_batch, bool* used_tc);

int wb_matmul_simt(WbBackend* be, const WbView* a, const WbView* b, void* out);

// Linear layers with at most 16 outputs on CUDA cores, in the arithmetic of `mode` (narrow_linear.cu).
bool wb_narrow_linear_ok(int64_t n, int64_t in, int64_t out, const float* x, const float* w);
int wb_narrow_linear_wgrad(WbBackend* b, int mode, const float* dy, int64_t dy_pitch, const float* x, int n, int in, int out, float* dw);
int wb_narrow_linear_dgrad(WbBackend* b, int mode, const float* dy, int64_t dy_pitch, const float* w, int n, int in, int out, float* dx);
