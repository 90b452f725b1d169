// Backend handle, caching arena, storage handles, host copies, profiling report, host RNG.
// Replaces the host glue of the reference CUDA crate (crates/weta-cuda/src/lib.rs:122-228, 423-461)
// with AOT-compiled code: there is no run-time compiler and no name -> function map.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include <atomic>
#include "common.h"

static thread_local char g_err[1024] = "";

void wb_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

extern "C" const char* wb_last_error(void) { return g_err; }

extern "C" int wb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

static int create_backend(int ordinal, cudaStream_t stream, bool adopt, WbBackend** out) {
    WB_REQUIRE(out != nullptr, WB_ERR_INVALID, "wb_backend_create: out is null");
    int n = wb_device_count();
    WB_REQUIRE(ordinal >= 0 && ordinal < n, WB_ERR_DEVICE_UNAVAILABLE, "no CUDA device %d (found %d)", ordinal, n);
    WB_CHECK_CUDA(cudaSetDevice(ordinal));
    cudaDeviceProp prop;
    WB_CHECK_CUDA(cudaGetDeviceProperties(&prop, ordinal));
    WB_REQUIRE(prop.major == 10, WB_ERR_DEVICE_UNAVAILABLE,
               "device %d is sm_%d%d; this library holds sm_100a code only", ordinal, prop.major, prop.minor);
    WbBackend* b = new WbBackend();
    b->ordinal = ordinal;
    b->sm_count = prop.multiProcessorCount;
    if (adopt) {
        b->stream = stream;
        b->own_stream = false;
    } else {
        cudaError_t e = cudaStreamCreateWithFlags(&b->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            delete b;
            wb_set_error("cudaStreamCreate failed: %s", cudaGetErrorString(e));
            return WB_ERR_CUDA;
        }
        b->own_stream = true;
    }
    const char* env = getenv("WETA_B200_PROFILE");
    b->profiling = env && env[0] == '1';
    *out = b;
    return WB_OK;
}

extern "C" int wb_backend_create(int ordinal, WbBackend** out) { return create_backend(ordinal, nullptr, false, out); }

extern "C" int wb_backend_create_on_stream(int ordinal, void* cuda_stream, WbBackend** out) {
    return create_backend(ordinal, static_cast<cudaStream_t>(cuda_stream), true, out);
}

void wb_gemm_state_destroy(WbBackend* b);

extern "C" int wb_backend_destroy(WbBackend* b) {
    if (!b) return WB_OK;
    cudaSetDevice(b->ordinal);
    cudaStreamSynchronize(b->stream);
    wb_gemm_state_destroy(b);
    for (auto& kv : b->free_blocks) cudaFree(kv.second);
    if (b->scratch) cudaFree(b->scratch);
    if (b->narrow_counters) cudaFree(b->narrow_counters);
    if (b->own_stream) cudaStreamDestroy(b->stream);
    delete b;
    return WB_OK;
}

extern "C" int wb_backend_ordinal(const WbBackend* b) { return b->ordinal; }
extern "C" void* wb_backend_stream(const WbBackend* b) { return b->stream; }
extern "C" int64_t wb_launch_count(const WbBackend* b) { return b->launches; }
extern "C" int64_t wb_arena_bytes_reserved(const WbBackend* b) { return static_cast<int64_t>(b->reserved); }

extern "C" int wb_synchronize(WbBackend* b) {
    WB_CHECK_CUDA(cudaStreamSynchronize(b->stream));
    return WB_OK;
}

extern "C" int wb_set_profiling(WbBackend* b, int on) {
    b->profiling = on != 0;
    return WB_OK;
}

extern "C" int wb_set_matmul_mode(WbBackend* b, int mode) {
    WB_REQUIRE(mode >= 0 && mode <= 2, WB_ERR_INVALID, "unknown matmul mode %d", mode);
    b->matmul_mode = mode;
    return WB_OK;
}

extern "C" int wb_get_matmul_mode(const WbBackend* b) { return b->matmul_mode; }

extern "C" const char* wb_profile_report(WbBackend* b) {
    // crates/weta-cuda/src/profile.rs:58-73: label, calls, total time, sorted by time.
    std::vector<std::pair<std::string, WbProfileEntry>> rows(b->profile.begin(), b->profile.end());
    std::sort(rows.begin(), rows.end(), [](const auto& x, const auto& y) { return x.second.ms > y.second.ms; });
    b->profile_text.clear();
    char line[256];
    snprintf(line, sizeof line, "%-40s %10s %12s\n", "op", "calls", "ms");
    b->profile_text += line;
    for (auto& r : rows) {
        snprintf(line, sizeof line, "%-40s %10lld %12.3f\n", r.first.c_str(), (long long)r.second.calls, r.second.ms);
        b->profile_text += line;
    }
    return b->profile_text.c_str();
}

// ---- arena --------------------------------------------------------------------------------------
// Size classes: multiples of 512 B up to 1 MiB, multiples of 1 MiB above.  A training step asks
// for the same sizes every iteration, so after the first step every request is a free-list hit.
static size_t size_class(size_t bytes) {
    if (bytes == 0) bytes = 1;
    if (bytes <= (1u << 20)) return (bytes + 511) & ~size_t(511);
    return (bytes + (1u << 20) - 1) & ~size_t((1u << 20) - 1);
}

int wb_arena_alloc(WbBackend* b, size_t bytes, void** out, size_t* klass) {
    size_t k = size_class(bytes);
    {
        std::lock_guard<std::mutex> g(b->mu);
        auto it = b->free_blocks.find(k);
        if (it != b->free_blocks.end()) {
            *out = it->second;
            *klass = k;
            b->free_blocks.erase(it);
            return WB_OK;
        }
    }
    WB_CHECK_CUDA(cudaSetDevice(b->ordinal));
    cudaError_t e = cudaMalloc(out, k);
    if (e == cudaErrorMemoryAllocation) {
        // Give cached blocks back to the driver and retry once.
        (void)cudaGetLastError();
        cudaStreamSynchronize(b->stream);
        std::lock_guard<std::mutex> g(b->mu);
        for (auto& kv : b->free_blocks) {
            cudaFree(kv.second);
            b->reserved -= kv.first;
        }
        b->free_blocks.clear();
        e = cudaMalloc(out, k);
    }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        wb_set_error("CUDA allocation of %zu bytes failed: %s", k, cudaGetErrorString(e));
        return e == cudaErrorMemoryAllocation ? WB_ERR_OOM : WB_ERR_CUDA;
    }
    {
        std::lock_guard<std::mutex> g(b->mu);
        b->reserved += k;
    }
    *klass = k;
    return WB_OK;
}

void wb_arena_free(WbBackend* b, void* p, size_t klass) {
    std::lock_guard<std::mutex> g(b->mu);
    b->free_blocks.emplace(klass, p);
}

namespace {
std::atomic<int> g_pdl_state{0};  // 0: not looked up, 1: allowed, 2: off
}
bool wb_pdl_allowed() {
    int v = g_pdl_state.load(std::memory_order_relaxed);
    if (v == 0) {
        const char* e = std::getenv("WETA_B200_NO_PDL");
        int want = (e && e[0] == '1') ? 2 : 1, expected = 0;
        g_pdl_state.compare_exchange_strong(expected, want, std::memory_order_relaxed);
        v = g_pdl_state.load(std::memory_order_relaxed);
    }
    return v == 1;
}
void wb_pdl_disallow() { g_pdl_state.store(2, std::memory_order_relaxed); }

int wb_block_counters(WbBackend* b, unsigned int** out) {
    if (!b->narrow_counters) {
        WB_CHECK_CUDA(cudaMalloc(&b->narrow_counters, 4096 * sizeof(unsigned int)));
        WB_CHECK_CUDA(cudaMemsetAsync(b->narrow_counters, 0, 4096 * sizeof(unsigned int), b->stream));
    }
    *out = static_cast<unsigned int*>(b->narrow_counters);
    return WB_OK;
}

int wb_scratch(WbBackend* b, size_t bytes, void** out) {
    if (bytes > b->scratch_bytes) {
        // Queued kernels may still read the old scratch: wait before releasing it.
        WB_CHECK_CUDA(cudaStreamSynchronize(b->stream));
        if (b->scratch) cudaFree(b->scratch);
        b->scratch = nullptr;
        b->scratch_bytes = 0;
        size_t want = size_class(bytes);
        WB_CHECK_CUDA(cudaMalloc(&b->scratch, want));
        b->scratch_bytes = want;
    }
    *out = b->scratch;
    return WB_OK;
}

int wb_new_storage(WbBackend* b, int64_t len, int dtype, WbStorage** out) {
    WB_REQUIRE(out != nullptr, WB_ERR_INVALID, "out is null");
    WB_REQUIRE(len >= 0 && dtype >= 0 && dtype <= 2, WB_ERR_INVALID, "bad length %lld or dtype %d", (long long)len, dtype);
    void* p = nullptr;
    size_t klass = 0;
    // Zero-length tensors keep one element (crates/weta-cuda/src/lib.rs:206-207).
    WB_TRY(wb_arena_alloc(b, static_cast<size_t>(len > 0 ? len : 1) * wb_dtype_size(dtype), &p, &klass));
    *out = new WbStorage{p, len, dtype, true, klass};
    return WB_OK;
}

extern "C" int wb_alloc(WbBackend* b, int64_t len, int dtype, WbStorage** out) { return wb_new_storage(b, len, dtype, out); }

extern "C" int wb_zeros(WbBackend* b, int64_t len, int dtype, WbStorage** out) {
    WbProfileScope ps(b, "zeros");
    WB_TRY(wb_new_storage(b, len, dtype, out));
    WB_CHECK_CUDA(cudaMemsetAsync((*out)->ptr, 0, static_cast<size_t>(len > 0 ? len : 1) * wb_dtype_size(dtype), b->stream));
    return WB_OK;
}

extern "C" int wb_free(WbBackend* b, WbStorage* s) {
    if (!s) return WB_OK;
    if (s->owned) wb_arena_free(b, s->ptr, s->bytes);
    delete s;
    return WB_OK;
}

extern "C" int wb_storage_wrap(WbBackend* b, void* device_ptr, int64_t len, int dtype, WbStorage** out) {
    (void)b;
    WB_REQUIRE(out && device_ptr, WB_ERR_INVALID, "wb_storage_wrap: null pointer");
    *out = new WbStorage{device_ptr, len, dtype, false, 0};
    return WB_OK;
}

extern "C" void* wb_storage_data(const WbStorage* s) { return s->ptr; }
extern "C" int64_t wb_storage_len(const WbStorage* s) { return s->len; }
extern "C" int wb_storage_dtype(const WbStorage* s) { return s->dtype; }

extern "C" int wb_from_host(WbBackend* b, const void* host, int64_t len, int dtype, WbStorage** out) {
    WbProfileScope ps(b, "from_host (upload)");
    WB_TRY(wb_new_storage(b, len, dtype, out));
    if (len > 0) {
        WB_REQUIRE(host != nullptr, WB_ERR_INVALID, "wb_from_host: host is null");
        // Pageable memory: cudaMemcpyAsync stages it before returning, so the caller's buffer is
        // free to change afterwards, like the reference's clone_htod.
        WB_CHECK_CUDA(cudaMemcpyAsync((*out)->ptr, host, static_cast<size_t>(len) * wb_dtype_size(dtype),
                                      cudaMemcpyHostToDevice, b->stream));
    }
    return WB_OK;
}

extern "C" int wb_to_host(WbBackend* b, const WbView* x, void* host_out) {
    WbProfileScope ps(b, "to_host (download)");
    WB_REQUIRE(x && host_out, WB_ERR_INVALID, "wb_to_host: null pointer");
    int64_t n = wb_numel(*x);
    if (n == 0) return WB_OK;
    size_t bytes = static_cast<size_t>(n) * wb_dtype_size(x->dtype);
    if (wb_is_contiguous(*x)) {
        const char* src = static_cast<const char*>(x->data) + x->offset * wb_dtype_size(x->dtype);
        WB_CHECK_CUDA(cudaMemcpyAsync(host_out, src, bytes, cudaMemcpyDeviceToHost, b->stream));
    } else {
        WbStorage* tmp = nullptr;
        WB_TRY(wb_cast(b, x, x->dtype, &tmp));  // contiguous(), like lib.rs:439
        cudaError_t e = cudaMemcpyAsync(host_out, tmp->ptr, bytes, cudaMemcpyDeviceToHost, b->stream);
        wb_free(b, tmp);
        WB_CHECK_CUDA(e);
    }
    WB_CHECK_CUDA(cudaStreamSynchronize(b->stream));
    return WB_OK;
}

extern "C" int wb_upload_async(WbBackend* b, const void* pinned_host, void* device_dst, int64_t bytes) {
    WB_CHECK_CUDA(cudaMemcpyAsync(device_dst, pinned_host, static_cast<size_t>(bytes), cudaMemcpyHostToDevice, b->stream));
    return WB_OK;
}

extern "C" int wb_download_async(WbBackend* b, const void* device_src, void* pinned_host, int64_t bytes) {
    WB_CHECK_CUDA(cudaMemcpyAsync(pinned_host, device_src, static_cast<size_t>(bytes), cudaMemcpyDeviceToHost, b->stream));
    return WB_OK;
}

// ---- iteration plan -----------------------------------------------------------------------------
void wb_make_plan(const WbView* const* ops, int nops, WbIterPlan* plan) {
    const WbView& v0 = *ops[0];
    int nd = 0;
    int64_t size[WB_MAX_DIMS];
    int64_t st[WB_PLAN_MAX_OPS][WB_MAX_DIMS];
    plan->n = 1;
    for (int d = 0; d < v0.ndim; ++d) {
        plan->n *= v0.shape[d];
        if (v0.shape[d] == 1) continue;  // size-1 dims never move
        size[nd] = v0.shape[d];
        for (int o = 0; o < nops; ++o) st[o][nd] = ops[o]->stride[d];
        ++nd;
    }
    // Merge dim i+1 into dim i when every operand steps over it exactly.
    int out = 0;
    for (int d = 0; d < nd; ++d) {
        if (out > 0) {
            bool merge = true;
            for (int o = 0; o < nops; ++o)
                if (st[o][out - 1] != st[o][d] * size[d]) merge = false;
            if (merge) {
                size[out - 1] *= size[d];
                for (int o = 0; o < nops; ++o) st[o][out - 1] = st[o][d];
                continue;
            }
        }
        size[out] = size[d];
        for (int o = 0; o < nops; ++o) st[o][out] = st[o][d];
        ++out;
    }
    if (out == 0) {  // scalar or all-ones shape
        size[0] = 1;
        for (int o = 0; o < nops; ++o) st[o][0] = 0;
        out = 1;
    }
    plan->nd = out;
    for (int d = 0; d < WB_MAX_DIMS; ++d) {
        plan->size[d] = d < out ? size[d] : 1;
        for (int o = 0; o < WB_PLAN_MAX_OPS; ++o) plan->st[o][d] = (o < nops && d < out) ? st[o][d] : 0;
    }
    for (int o = 0; o < WB_PLAN_MAX_OPS; ++o) plan->off[o] = o < nops ? ops[o]->offset : 0;
}

// ---- host RNG -----------------------------------------------------------------------------------
// PCG-XSH-RR exactly as crates/weta-tensor/src/random.rs:27-46.
extern "C" uint32_t wb_pcg_next_u32(WbPcg* g) {
    uint64_t old = g->state;
    g->state = old * 6364136223846793005ull + g->inc;
    uint32_t xorshifted = static_cast<uint32_t>(((old >> 18) ^ old) >> 27);
    uint32_t rot = static_cast<uint32_t>(old >> 59);
    return (xorshifted >> rot) | (xorshifted << ((32 - rot) & 31));
}

extern "C" void wb_pcg_seed(WbPcg* g, uint64_t seed) {
    g->state = 0;
    g->inc = (0xda3e39cb94b95bdbull << 1) | 1;
    wb_pcg_next_u32(g);
    g->state += seed;
    wb_pcg_next_u32(g);
}

extern "C" uint64_t wb_pcg_next_u64(WbPcg* g) {
    uint64_t hi = wb_pcg_next_u32(g);
    return (hi << 32) | wb_pcg_next_u32(g);
}

extern "C" uint64_t wb_splitmix64(uint64_t seed, uint64_t i) {
    uint64_t z = seed + (i + 1) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
