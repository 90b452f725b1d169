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

int wb_matmul_simt(WbBackend* be, const WbView* a, const WbView* b, void* out);
