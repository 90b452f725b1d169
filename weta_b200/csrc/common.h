// Internal definitions shared by every translation unit of libweta_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdlib>
#include <utility>
#include <cstdio>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "weta_b200.h"

#define WB_SM_COUNT_DEFAULT 148

void wb_set_error(const char* fmt, ...);

#define WB_CHECK_CUDA(expr)                                                                       \
    do {                                                                                          \
        cudaError_t _e = (expr);                                                                  \
        if (_e != cudaSuccess) {                                                                  \
            wb_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return _e == cudaErrorMemoryAllocation ? WB_ERR_OOM : WB_ERR_CUDA;                    \
        }                                                                                         \
    } while (0)

#define WB_REQUIRE(cond, status, ...)   \
    do {                                \
        if (!(cond)) {                  \
            wb_set_error(__VA_ARGS__);  \
            return (status);            \
        }                               \
    } while (0)

#define WB_TRY(expr)                   \
    do {                               \
        int _s = (expr);               \
        if (_s != WB_OK) return _s;    \
    } while (0)

// Checks the launch that was just issued and counts it.
#define WB_LAUNCH_OK(b)                                                                                \
    do {                                                                                               \
        cudaError_t _e = cudaPeekAtLastError();                                                        \
        if (_e != cudaSuccess) {                                                                       \
            (void)cudaGetLastError();                                                                  \
            wb_set_error("kernel launch failed: %s (%s:%d)", cudaGetErrorString(_e), __FILE__, __LINE__); \
            return WB_ERR_CUDA;                                                                        \
        }                                                                                              \
        (b)->launches++;                                                                               \
    } while (0)

struct WbStorage {
    void* ptr;
    int64_t len;      // elements
    int32_t dtype;
    bool owned;
    size_t bytes;     // size class it came from (0 if not owned)
};

struct WbProfileEntry {
    int64_t calls = 0;
    double ms = 0.0;
};

struct WbBackend {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    int sm_count = WB_SM_COUNT_DEFAULT;
    int matmul_mode = WB_MM_TF32X3;
    int64_t launches = 0;
    // Caching arena: freed blocks are kept per size class and handed back to later requests of
    // the same class.  One stream per backend, so reuse is automatically stream-ordered.
    std::mutex mu;
    std::multimap<size_t, void*> free_blocks;
    size_t reserved = 0;
    // profiling
    bool profiling = false;
    std::map<std::string, WbProfileEntry> profile;
    std::string profile_text;
    // scratch owned by the backend (grown on demand, reused across calls)
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    // lazily created resources of the tensor-core GEMM path
    void* gemm_state = nullptr;
    // 4096 block counters for kernels whose last block finishes a reduction (narrow_linear.cu, trainer.cu); every such
    // kernel finds them zero and leaves them zero
    void* narrow_counters = nullptr;
};

inline size_t wb_dtype_size(int dt) { return dt == WB_F32 ? 4 : 8; }

inline int64_t wb_numel(const WbView& v) {
    int64_t n = 1;
    for (int i = 0; i < v.ndim; ++i) n *= v.shape[i];
    return n;
}

inline bool wb_is_contiguous(const WbView& v) {
    int64_t expected = 1;
    for (int i = v.ndim - 1; i >= 0; --i) {
        if (v.shape[i] != 1 && v.stride[i] != expected) return false;
        expected *= v.shape[i];
    }
    return true;
}

int wb_arena_alloc(WbBackend* b, size_t bytes, void** out, size_t* klass);
void wb_arena_free(WbBackend* b, void* p, size_t klass);
int wb_scratch(WbBackend* b, size_t bytes, void** out);
const void* wb_dropout_kernel_func();  // fused.cu
const void* wb_adam_kernel_func();
// The backend's 4096 zeroed block counters (created on first use).
int wb_block_counters(WbBackend* b, unsigned int** out);
int wb_new_storage(WbBackend* b, int64_t len, int dtype, WbStorage** out);

// RAII profiling scope: when profiling is on, brackets the op with events and a sync (like the
// reference's Timer, crates/weta-cuda/src/profile.rs:31-55); otherwise it costs one branch.
struct WbProfileScope {
    WbBackend* b;
    const char* label;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    WbProfileScope(WbBackend* be, const char* l) : b(be), label(l) {
        if (b->profiling) {
            cudaEventCreate(&e0);
            cudaEventCreate(&e1);
            cudaEventRecord(e0, b->stream);
        }
    }
    ~WbProfileScope() {
        if (e0) {
            cudaEventRecord(e1, b->stream);
            cudaEventSynchronize(e1);
            float ms = 0.f;
            cudaEventElapsedTime(&ms, e0, e1);
            auto& p = b->profile[label];
            p.calls++;
            p.ms += ms;
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
        }
    }
};

// ---- iteration plans for element-wise kernels ---------------------------------------------------
// The output of every element-wise op is contiguous; the plan describes how up to three operand
// views walk alongside it after size-1 dims are dropped and mergeable neighbours are fused.
#define WB_PLAN_MAX_OPS 3

struct WbIterPlan {
    int nd;                               // collapsed rank (>= 1)
    int64_t n;                            // total elements
    int64_t size[WB_MAX_DIMS];            // collapsed sizes, outermost first
    int64_t st[WB_PLAN_MAX_OPS][WB_MAX_DIMS];
    int64_t off[WB_PLAN_MAX_OPS];
};

// Builds the collapsed plan of `nops` operand views that share one shape.
void wb_make_plan(const WbView* const* ops, int nops, WbIterPlan* plan);

// Division of a 32-bit index by a launch-invariant divisor, as a multiply-high (exact for n < 2^31).
// Programmatic dependent launch.  A kernel launched with wb_launch_pdl may be scheduled while the kernel before it in
// the stream is still running; its first statement is wb_pdl_enter(), which waits until that kernel has completed and
// its writes are visible, and then (in a kernel of few blocks) lets the kernel after it be scheduled in the same way.  What overlaps is the launch
// itself (and, in the tensor-core GEMM, the preamble it runs before its own wait): one to two microseconds per kernel,
// which is most of a small model's step.  Dependencies through events are not relaxed.
// Process-wide switch (backend.cu): off with WETA_B200_NO_PDL=1, and turned off by a data-parallel handle over more than
// one rank: with the gradient exchange running beside backward, blocks that sit on an SM waiting for the kernel before
// them take room from the exchange kernels (2 GPUs: 1.057 M samples/s without against 1.036 M with).
bool wb_pdl_allowed();
void wb_pdl_disallow();
#ifdef __CUDACC__
__device__ __forceinline__ void wb_pdl_enter() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // A small grid is a short kernel: the next kernel's blocks may as well be scheduled now.  A large one releases its
    // dependents as its blocks exit: blocks parked on the SMs for the length of a long kernel slow it down (the
    // 4096-sample step of the wide CNN lost 3 % when every kernel released its dependents at once).
    if (gridDim.x * gridDim.y * gridDim.z <= 296u) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
template <class... Params, class... Args>
inline cudaError_t wb_launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    const bool plain = !wb_pdl_allowed();
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = plain ? nullptr : &attr;
    cfg.numAttrs = plain ? 0u : 1u;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

struct FastDiv {
    uint32_t d, s;
    uint64_t mul;
    __host__ FastDiv() : d(1), s(0), mul(1ull << 32) {}
    __host__ explicit FastDiv(uint32_t div) : d(div) {
        s = 0;
        while ((1ull << s) < div) ++s;
        mul = ((1ull << (32 + s)) + div - 1) / div;
    }
    __device__ __forceinline__ uint32_t div(uint32_t n) const { return static_cast<uint32_t>((static_cast<uint64_t>(n) * mul) >> (32 + s)); }
};

