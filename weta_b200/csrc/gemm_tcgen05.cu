// Backend::matmul entry point (crates/weta-core/src/backend.rs:87) and its dispatch between the
// tensor-core path and the CUDA-core tiles.
#include "common.h"

int wb_matmul_simt(WbBackend* be, const WbView* a, const WbView* b, void* out);

void wb_gemm_state_destroy(WbBackend* b) { (void)b; }

extern "C" int wb_matmul_into(WbBackend* b, const WbView* a, const WbView* bb, void* out) {
    WB_REQUIRE(b && a && bb && out, WB_ERR_INVALID, "wb_matmul: null pointer");
    WB_REQUIRE(a->ndim == 3 && bb->ndim == 3, WB_ERR_INVALID, "matmul: expected [B,M,K] x [B,K,N] views");
    WB_REQUIRE(a->dtype == bb->dtype, WB_ERR_INVALID, "matmul: dtype mismatch");
    WB_REQUIRE(a->dtype == WB_F32 || a->dtype == WB_F64, WB_ERR_UNSUPPORTED, "matmul: unsupported dtype i64");
    WB_REQUIRE(a->shape[0] == bb->shape[0] && a->shape[2] == bb->shape[1], WB_ERR_INVALID,
               "matmul: [%lld,%lld,%lld] x [%lld,%lld,%lld] do not contract", (long long)a->shape[0], (long long)a->shape[1],
               (long long)a->shape[2], (long long)bb->shape[0], (long long)bb->shape[1], (long long)bb->shape[2]);
    WbProfileScope ps(b, "matmul");
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
