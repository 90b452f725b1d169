// CUDA-core GEMM tiles for Backend::matmul: the path for f64 (gradient checks), for layouts the
// tensor-core path cannot read, and for WB_MM_FP32.  [B,M,K] x [B,K,N] -> [B,M,N] with any element
// strides, including batch stride 0 (a weight broadcast over the batch,
// crates/weta-tensor/src/tensor.rs:586-606).  Each output is one FMA chain over k ascending.
#include "common.h"

namespace simt {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

struct MMP {
    int64_t bs, m, n, k;
    int64_t a0, a1, a2, aoff;
    int64_t b0, b1, b2, boff;
};

template <class T>
__global__ void __launch_bounds__(THREADS) gemm_tiles(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b, MMP p,
                                                       int a_kfast, int b_nfast) {
    __shared__ T As[BK][BM + 4];
    __shared__ T Bs[BK][BN + 4];
    const int64_t batch = blockIdx.z;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM, n0 = static_cast<int64_t>(blockIdx.x) * BN;
    const T* A = a + p.aoff + batch * p.a0;
    const T* B = b + p.boff + batch * p.b0;
    const int tid = threadIdx.x;
    const int tr = tid / (BN / TN), tc = tid % (BN / TN);  // 16 x 16 thread grid
    T acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = T(0);
    for (int64_t k0 = 0; k0 < p.k; k0 += BK) {
        // Stage A (BM x BK) and B (BK x BN); threads run along whichever index has unit stride.
#pragma unroll
        for (int e = tid; e < BM * BK; e += THREADS) {
            int mm = a_kfast ? e / BK : e % BM;
            int kk = a_kfast ? e % BK : e / BM;
            int64_t gm = m0 + mm, gk = k0 + kk;
            As[kk][mm] = (gm < p.m && gk < p.k) ? A[gm * p.a1 + gk * p.a2] : T(0);
        }
#pragma unroll
        for (int e = tid; e < BK * BN; e += THREADS) {
            int nn = b_nfast ? e % BN : e / BK;
            int kk = b_nfast ? e / BN : e % BK;
            int64_t gn = n0 + nn, gk = k0 + kk;
            Bs[kk][nn] = (gn < p.n && gk < p.k) ? B[gk * p.b1 + gn * p.b2] : T(0);
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            T av[TM], bv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = As[kk][tr * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) bv[j] = Bs[kk][tc * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fma(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
    T* O = out + batch * p.m * p.n;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        int64_t gm = m0 + tr * TM + i;
        if (gm >= p.m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            int64_t gn = n0 + tc * TN + j;
            if (gn < p.n) O[gm * p.n + gn] = acc[i][j];
        }
    }
}

template <class T>
int run(WbBackend* be, const WbView& a, const WbView& b, T* out) {
    MMP p{a.shape[0], a.shape[1], b.shape[2], a.shape[2], a.stride[0], a.stride[1], a.stride[2], a.offset,
          b.stride[0], b.stride[1], b.stride[2], b.offset};
    if (p.bs * p.m * p.n == 0) return WB_OK;
    WB_REQUIRE(p.bs <= 65535, WB_ERR_UNSUPPORTED, "matmul: batch %lld exceeds the launch limit of this path", (long long)p.bs);
    dim3 grid(static_cast<unsigned>((p.n + BN - 1) / BN), static_cast<unsigned>((p.m + BM - 1) / BM), static_cast<unsigned>(p.bs));
    int a_kfast = p.a2 == 1 || p.a1 != 1;
    int b_nfast = p.b2 == 1 || p.b1 != 1;
    gemm_tiles<T><<<grid, THREADS, 0, be->stream>>>(out, static_cast<const T*>(a.data), static_cast<const T*>(b.data), p, a_kfast, b_nfast);
    WB_LAUNCH_OK(be);
    return WB_OK;
}

}  // namespace simt

int wb_matmul_simt(WbBackend* be, const WbView* a, const WbView* b, void* out) {
    if (a->dtype == WB_F32) return simt::run<float>(be, *a, *b, static_cast<float*>(out));
    return simt::run<double>(be, *a, *b, static_cast<double*>(out));
}
