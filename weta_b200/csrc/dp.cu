// Data-parallel training step behind the C ABI: one process per GPU, every rank a full replica of the model, the
// batch sharded by samples.  The reference has no multi-GPU path (its backends are per-ordinal singletons with no
// gradient exchange, crates/weta-cuda/src/lib.rs:129-146); this file adds the one exchange a data-parallel step
// needs, between the backward pass and the optimizer of crates/weta-optim/src/lib.rs:210-239.
//
// The trainer's gradient arena is cut into buckets of whole layers (last layer first, the order backward finishes
// them).  When a bucket's gradients are final, its exchange and its optimizer update are queued on a side stream
// while backward continues on the compute stream.  Three interchangeable forms of that work:
//   ALLREDUCE  ncclAllReduce of the bucket, then Adam over the whole bucket on every rank;
//   SHARDED    ncclReduceScatter, Adam on this rank's 1/world of the bucket, ncclAllGather of the new parameters:
//              optimizer traffic and NVLink bytes per rank fall by world/1 and 2x respectively;
//   PEER       one kernel of this library: each rank reads its shard of the bucket from every replica's gradient
//              arena over NVLink (plain peer loads), adds them in rank order, runs Adam on the sum and stores the new
//              parameters into every replica's parameter arena (plain peer stores).  Arenas and flag words are
//              shared between the processes with CUDA IPC.  A bucket costs two launches and no NCCL call.
// NCCL is loaded with dlopen at the first wb_dp_create that needs it, so the library itself has no link-time
// dependency on it.  Every device-side wait is bounded by a time limit and reports through a status word; the host
// side has a watchdog (wb_dp_wait) that polls completion and the communicator's asynchronous error state.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "adam.cuh"
#include "common.h"

int wb_trainer_internal_info(WbTrainer* t, WbBackend** be, int64_t* batch, int64_t* in_elems, std::vector<std::pair<int64_t, int64_t>>* ranges,
                             std::vector<int>* conv_follows);
const WbAdamConfig* wb_trainer_adam_config(const WbTrainer* t);

namespace {

constexpr int MAX_WORLD = 8;
constexpr int MAX_BUCKETS = 64;

// ---- NCCL, loaded at run time -------------------------------------------------------------------
struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
};

NcclApi* load_nccl() {
    static NcclApi api;
    static std::mutex mu;
    std::lock_guard<std::mutex> g(mu);
    if (api.lib) return &api;
    const char* override_path = std::getenv("WETA_B200_NCCL_LIB");
    const char* names[] = {override_path, "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        if (!n || !n[0]) continue;
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) {
        wb_set_error("data parallelism over more than one rank needs NCCL: dlopen(libnccl.so.2) failed (%s); set WETA_B200_NCCL_LIB", dlerror());
        return nullptr;
    }
    bool ok = true;
    auto sym = [&](const char* name) {
        void* p = dlsym(h, name);
        if (!p) ok = false;
        return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
    api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(sym("ncclReduceScatter"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    if (!ok) {
        wb_set_error("the NCCL library that was found lacks an entry point this library needs");
        dlclose(h);
        return nullptr;
    }
    api.lib = h;
    return &api;
}

#define WB_CHECK_NCCL(api, expr)                                                                        \
    do {                                                                                                \
        ncclResult_t _r = (expr);                                                                       \
        if (_r != ncclSuccess && _r != ncclInProgress) {                                                \
            wb_set_error("%s failed: %s (%s:%d)", #expr, (api)->GetErrorString(_r), __FILE__, __LINE__); \
            return WB_ERR_CUDA;                                                                         \
        }                                                                                               \
    } while (0)

// ---- the peer-memory kernels ----------------------------------------------------------------------
// Flag words shared between the ranks (one block per rank, opened by every peer through CUDA IPC):
//   ready[b][r]  rank r's gradients of bucket b are final for step `value`
//   done[b][r]   rank r has stored its shard of bucket b's new parameters into this rank's arena for step `value`
struct PeerFlags {
    uint32_t ready[MAX_BUCKETS][MAX_WORLD];
    uint32_t done[MAX_BUCKETS][MAX_WORLD];
};

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

struct PeerPtrs {
    PeerFlags* flags[MAX_WORLD];  // every rank's flag block (own rank: the local pointer)
    const float* grad[MAX_WORLD];
    float* theta[MAX_WORLD];
};

// Thread p < world: (announce) stores `seq` into word `mine[p]`, which lives in rank p's flag block, then (wait) polls
// the local word `theirs[p]` until rank p has stored `seq` there.  Either half can be switched off.  The wait is bounded
// by `timeout_ns` of the global timer; on expiry the thread records which peer and phase it gave up on in *status
// (0 = fine) and returns, so the kernel always ends and the context stays usable.
__global__ void peer_announce_wait(PeerPtrs pp, int world, int rank, int bucket, int use_done, int announce, int wait, uint32_t seq,
                                   unsigned long long timeout_ns, uint32_t* status) {
    const int p = threadIdx.x;
    if (p >= world) return;
    if (announce) {
        __threadfence_system();
        PeerFlags* f = pp.flags[p];
        store_release_sys(use_done ? &f->done[bucket][rank] : &f->ready[bucket][rank], seq);
    }
    if (wait) {
        if (*reinterpret_cast<volatile uint32_t*>(status) != 0) return;  // an earlier wait of this step already gave up
        const PeerFlags* f = pp.flags[rank];
        const uint32_t* word = use_done ? &f->done[bucket][p] : &f->ready[bucket][p];
        const unsigned long long t0 = global_ns();
        while (static_cast<int32_t>(load_acquire_sys(word) - seq) < 0) {
            if (global_ns() - t0 > timeout_ns) {
                atomicCAS(status, 0u, 0x80000000u | (static_cast<uint32_t>(use_done) << 16) | (static_cast<uint32_t>(bucket) << 8) | static_cast<uint32_t>(p));
                return;
            }
            __nanosleep(256);
        }
    }
}

// The end-of-step wait in one launch: thread (b, p) polls done[b][p] of this rank's block for every bucket b and peer p.
__global__ void peer_wait_all_done(PeerPtrs pp, int world, int rank, int n_buckets, uint32_t seq, unsigned long long timeout_ns, uint32_t* status) {
    const int b = threadIdx.x / MAX_WORLD, p = threadIdx.x % MAX_WORLD;
    if (b >= n_buckets || p >= world) return;
    if (*reinterpret_cast<volatile uint32_t*>(status) != 0) return;
    const uint32_t* word = &pp.flags[rank]->done[b][p];
    const unsigned long long t0 = global_ns();
    while (static_cast<int32_t>(load_acquire_sys(word) - seq) < 0) {
        if (global_ns() - t0 > timeout_ns) {
            atomicCAS(status, 0u, 0x80000000u | (1u << 16) | (static_cast<uint32_t>(b) << 8) | static_cast<uint32_t>(p));
            return;
        }
        __nanosleep(256);
    }
}

struct FusedArgs {
    const float* grad[MAX_WORLD];  // the replicas' gradient arenas (peer or local pointers)
    float* theta[MAX_WORLD];       // the replicas' parameter arenas
    float *m, *v;                  // this rank's optimizer state (full-arena indexing)
    int world, self;               // `self`: index whose theta holds the current parameters of the range
    int64_t off, len;              // the range this launch owns, in arena elements; off and len multiples of 4
    AdamK k;
    // completion signal (optional): the last block to finish stores `seq` into done_word[p] for every p
    uint32_t* done_word[MAX_WORLD];
    unsigned int* block_counter;
    uint32_t seq;
    const uint32_t* status;  // when non-null and *status != 0 (a wait gave up) the kernel does nothing
};

// Gradient sum over the replicas in index order, Adam on the sum, new parameters stored into every replica: the
// reduce-scatter, the optimizer and the all-gather of one shard in one pass.  Loads from the replicas bypass L1
// (another GPU wrote them); one thread handles U groups of four consecutive elements at a time with 128-bit accesses,
// and issues the U x world replica loads of a round before it uses any of them: a peer load takes a few microseconds,
// so the bytes in flight per thread, not the link, set the rate (U = 8 / world keeps eight loads in flight).
template <int U>
__global__ void __launch_bounds__(512) reduce_adam_broadcast(FusedArgs a) {
    if (a.status && *a.status != 0) return;
    const int64_t groups = a.len / 4;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t g0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; g0 < groups; g0 += stride * U) {
        float4 part[U][MAX_WORLD];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t g = g0 + u * stride;
            if (g < groups) {
#pragma unroll
                for (int p = 0; p < MAX_WORLD; ++p)
                    if (p < a.world) part[u][p] = __ldcv(reinterpret_cast<const float4*>(a.grad[p] + a.off + g * 4));
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t g = g0 + u * stride;
            if (g >= groups) break;
            const int64_t i = a.off + g * 4;
            float4 s = part[u][0];
#pragma unroll
            for (int p = 1; p < MAX_WORLD; ++p)
                if (p < a.world) { s.x += part[u][p].x; s.y += part[u][p].y; s.z += part[u][p].z; s.w += part[u][p].w; }
            float4 th = *reinterpret_cast<const float4*>(a.theta[a.self] + i);
            float4 mi = a.k.first ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(a.m + i);
            float4 vi = a.k.first ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(a.v + i);
            adam_one(th.x, s.x, mi.x, vi.x, a.k);
            adam_one(th.y, s.y, mi.y, vi.y, a.k);
            adam_one(th.z, s.z, mi.z, vi.z, a.k);
            adam_one(th.w, s.w, mi.w, vi.w, a.k);
            *reinterpret_cast<float4*>(a.m + i) = mi;
            *reinterpret_cast<float4*>(a.v + i) = vi;
#pragma unroll
            for (int p = 0; p < MAX_WORLD; ++p)
                if (p < a.world) *reinterpret_cast<float4*>(a.theta[p] + i) = th;
        }
    }
    if (a.block_counter) {
        __threadfence_system();  // this block's stores to the replicas are ordered before the signal below
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned int arrived = atomicAdd(a.block_counter, 1u);
            if (arrived == gridDim.x - 1) {
                *a.block_counter = 0;
                __threadfence_system();
                for (int p = 0; p < a.world; ++p) store_release_sys(a.done_word[p], a.seq);
            }
        }
    }
}

void launch_reduce_adam_broadcast(const FusedArgs& a, int blocks, cudaStream_t stream) {
    if (a.world <= 2) reduce_adam_broadcast<4><<<blocks, 512, 0, stream>>>(a);
    else if (a.world <= 4) reduce_adam_broadcast<2><<<blocks, 512, 0, stream>>>(a);
    else reduce_adam_broadcast<1><<<blocks, 512, 0, stream>>>(a);
}

struct Bucket {
    int64_t off, len;
};

std::vector<Bucket> plan_buckets(const std::vector<std::pair<int64_t, int64_t>>& ranges, int64_t min_elems) {
    std::vector<Bucket> out;
    Bucket cur{0, 0};
    for (auto& r : ranges) {
        if (r.second <= 0) continue;
        if (cur.len == 0) cur = {r.first, r.second};
        else if (r.first == cur.off + cur.len) cur.len += r.second;
        else { out.push_back(cur); cur = {r.first, r.second}; }
        if (cur.len >= min_elems) { out.push_back(cur); cur = {0, 0}; }
    }
    if (cur.len > 0) out.push_back(cur);
    return out;
}

struct IpcPacket {
    cudaIpcMemHandle_t grad, theta, flags;
    int64_t grad_off, theta_off, flags_off;  // offsets of the pointers inside their allocations
};

typedef int (*cuMemGetAddressRange_fn)(unsigned long long*, size_t*, unsigned long long);

}  // namespace

struct WbDp {
    WbTrainer* tr = nullptr;
    WbBackend* be = nullptr;       // the trainer's backend (compute stream)
    WbBackend* side_be = nullptr;  // a handle on comm_stream: optimizer kernels of the exchange
    WbBackend* adam_be = nullptr;  // a handle on adam_stream (ALLREDUCE mode only)
    int rank = 0, world = 1, mode = WB_DP_ALLREDUCE;
    NcclApi* nccl = nullptr;
    ncclComm_t comm = nullptr;
    cudaStream_t comm_stream = nullptr, adam_stream = nullptr, copy_stream = nullptr;
    std::vector<Bucket> buckets;
    std::vector<int> defer;        // per bucket: a quiet point of backward follows its completion, start its work there
    std::vector<int> deferred;     // buckets complete but not yet issued
    bool defer_enabled = false;    // measured at 4 ranks: no gain (the BatchNorm pass recovers what the contractions then lose)
    bool defer_all = false;        // diagnostic (WETA_B200_DP_DEFER=2): no exchange starts before backward is over
    bool flushing = false;
    std::vector<cudaEvent_t> bucket_ready;  // recorded on the compute stream when a bucket's gradients are final
    cudaEvent_t ev_side = nullptr, ev_adam = nullptr, ev_step = nullptr;
    int64_t n_params = 0, batch = 0, in_elems = 0;
    float *theta = nullptr, *grad = nullptr, *m = nullptr, *v = nullptr;
    // state of the step being issued
    int next_bucket = 0;
    int64_t covered = 0;
    int64_t step = 0;   // Adam's step count t of the step being issued
    uint32_t seq = 0;   // how many steps this handle has issued: the value the flag words carry
    int issue_error = WB_OK;
    std::string issue_message;
    // peer mode
    PeerFlags* flags = nullptr;
    unsigned int* counters = nullptr;  // one block counter per bucket
    uint32_t* status_dev = nullptr;    // device view of the pinned status word
    uint32_t* status_host = nullptr;
    PeerPtrs peers{};
    void* opened[3 * MAX_WORLD] = {};
    int n_opened = 0;
    unsigned long long timeout_ns = 10ull * 1000 * 1000 * 1000;
    int fused_blocks = 64;
    // double-buffered upload
    float* slot_x[2] = {nullptr, nullptr};
    int64_t* slot_y[2] = {nullptr, nullptr};
    cudaEvent_t slot_ready[2] = {nullptr, nullptr}, slot_consumed[2] = {nullptr, nullptr};
    int64_t submitted = 0, stepped = 0;
    float* loss_pinned = nullptr;
    // timing of the side-stream work (optional)
    bool timing = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> timing_events;
    std::string timing_text;
};

namespace {

int issue_bucket(WbDp* dp, int bi);

void on_range(void* user, float* ptr, int64_t len) {
    WbDp* dp = static_cast<WbDp*>(user);
    if (dp->issue_error != WB_OK) return;
    if (len == 0) {  // a quiet point of backward: start the work of the buckets that were waiting for one
        if (dp->defer_all && !dp->flushing) return;
        for (int bi : dp->deferred) {
            int s = issue_bucket(dp, bi);
            if (s != WB_OK) {
                dp->issue_error = s;
                dp->issue_message = wb_last_error();
                break;
            }
        }
        dp->deferred.clear();
        return;
    }
    const int64_t off = ptr - dp->grad;
    if (off != dp->covered) {
        dp->issue_error = WB_ERR_INVALID;
        dp->issue_message = "data-parallel step: gradient ranges arrived out of arena order";
        return;
    }
    dp->covered += len;
    while (dp->next_bucket < static_cast<int>(dp->buckets.size())) {
        const Bucket& b = dp->buckets[dp->next_bucket];
        if (dp->covered < b.off + b.len) break;
        if (dp->defer_all || (dp->defer_enabled && dp->defer[dp->next_bucket])) {
            // The next ops of backward are a conv block's BatchNorm pass, which streams HBM with every block slot of
            // every SM taken: an exchange started now would share its bandwidth and push part of its single wave of
            // blocks into a second one.  Hold the bucket until that pass is queued (the quiet point that follows).
            dp->deferred.push_back(dp->next_bucket);
        } else {
            int s = issue_bucket(dp, dp->next_bucket);
            if (s != WB_OK) {
                dp->issue_error = s;
                dp->issue_message = wb_last_error();
                return;
            }
        }
        dp->next_bucket++;
    }
}

int adam_on(WbDp* dp, WbBackend* on, int64_t off, int64_t len, double scale) {
    return wb_trainer_adam_range(dp->tr, on, off, len, dp->step, scale);
}

// Queues the exchange and the optimizer update of one bucket on the side stream(s), ordered after the compute stream's
// work so far (which produced the bucket's gradients).
int issue_bucket(WbDp* dp, int bi) {
    const Bucket& b = dp->buckets[bi];
    WB_CHECK_CUDA(cudaEventRecord(dp->bucket_ready[bi], dp->be->stream));
    WB_CHECK_CUDA(cudaStreamWaitEvent(dp->comm_stream, dp->bucket_ready[bi], 0));
    cudaEvent_t t0 = nullptr, t1 = nullptr;
    if (dp->timing) {
        cudaEventCreate(&t0);
        cudaEventCreate(&t1);
        cudaEventRecord(t0, dp->comm_stream);
    }
    const double scale = 1.0 / dp->world;
    if (dp->world == 1) {
        WB_TRY(adam_on(dp, dp->side_be, b.off, b.len, 1.0));
    } else if (dp->mode == WB_DP_ALLREDUCE) {
        WB_CHECK_NCCL(dp->nccl, dp->nccl->AllReduce(dp->grad + b.off, dp->grad + b.off, static_cast<size_t>(b.len), ncclFloat, ncclSum, dp->comm, dp->comm_stream));
        WB_CHECK_CUDA(cudaEventRecord(dp->ev_side, dp->comm_stream));
        WB_CHECK_CUDA(cudaStreamWaitEvent(dp->adam_stream, dp->ev_side, 0));
        WB_TRY(adam_on(dp, dp->adam_be, b.off, b.len, scale));
    } else if (dp->mode == WB_DP_SHARDED) {
        const int64_t shard = b.len / dp->world, mine = b.off + dp->rank * shard;
        WB_CHECK_NCCL(dp->nccl, dp->nccl->ReduceScatter(dp->grad + b.off, dp->grad + mine, static_cast<size_t>(shard), ncclFloat, ncclSum, dp->comm, dp->comm_stream));
        WB_TRY(adam_on(dp, dp->side_be, mine, shard, scale));
        WB_CHECK_NCCL(dp->nccl, dp->nccl->AllGather(dp->theta + mine, dp->theta + b.off, static_cast<size_t>(shard), ncclFloat, dp->comm, dp->comm_stream));
    } else {  // WB_DP_PEER
        const uint32_t seq = dp->seq;
        peer_announce_wait<<<1, 32, 0, dp->comm_stream>>>(dp->peers, dp->world, dp->rank, bi, 0, 1, 1, seq, dp->timeout_ns, dp->status_dev);
        WB_LAUNCH_OK(dp->side_be);
        FusedArgs a{};
        for (int p = 0; p < dp->world; ++p) {
            a.grad[p] = dp->peers.grad[p];
            a.theta[p] = dp->peers.theta[p];
            a.done_word[p] = &dp->peers.flags[p]->done[bi][dp->rank];
        }
        a.m = dp->m;
        a.v = dp->v;
        a.world = dp->world;
        a.self = dp->rank;
        const int64_t shard = b.len / dp->world;
        a.off = b.off + dp->rank * shard;
        a.len = shard;
        const WbAdamConfig* cfg = wb_trainer_adam_config(dp->tr);
        a.k = wb_adam_constants(dp->step, cfg->lr, cfg->beta1, cfg->beta2, cfg->eps, cfg->weight_decay, cfg->decoupled, scale);
        a.block_counter = dp->counters + bi;
        a.seq = seq;
        a.status = dp->status_dev;
        const int64_t groups = shard / 4;
        const int blocks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(dp->fused_blocks, (groups + 511) / 512)));
        launch_reduce_adam_broadcast(a, blocks, dp->comm_stream);
        WB_LAUNCH_OK(dp->side_be);
    }
    if (dp->timing) {
        cudaEventRecord(t1, dp->comm_stream);
        dp->timing_events.push_back({t0, t1});
    }
    return WB_OK;
}

int open_peers(WbDp* dp) {
    // Exchange IPC handles of the two arenas and the flag block through the communicator, then map every peer's.
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    WB_CHECK_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres));
    WB_REQUIRE(fn && qres == cudaDriverEntryPointSuccess, WB_ERR_CUDA, "cuMemGetAddressRange is not available from this driver");
    auto range = reinterpret_cast<cuMemGetAddressRange_fn>(fn);
    auto base_of = [&](const void* p, int64_t* off) -> void* {
        unsigned long long base = 0;
        size_t size = 0;
        if (range(&base, &size, reinterpret_cast<unsigned long long>(p)) != 0) return nullptr;
        *off = static_cast<int64_t>(reinterpret_cast<unsigned long long>(p) - base);
        return reinterpret_cast<void*>(base);
    };
    IpcPacket mine{};
    void* gb = base_of(dp->grad, &mine.grad_off);
    void* tb = base_of(dp->theta, &mine.theta_off);
    void* fb = base_of(dp->flags, &mine.flags_off);
    WB_REQUIRE(gb && tb && fb, WB_ERR_CUDA, "peer mode: could not resolve the arenas' allocation bases");
    WB_CHECK_CUDA(cudaIpcGetMemHandle(&mine.grad, gb));
    WB_CHECK_CUDA(cudaIpcGetMemHandle(&mine.theta, tb));
    WB_CHECK_CUDA(cudaIpcGetMemHandle(&mine.flags, fb));
    IpcPacket* dev = nullptr;
    WB_CHECK_CUDA(cudaMalloc(&dev, sizeof(IpcPacket) * dp->world));
    WB_CHECK_CUDA(cudaMemcpyAsync(dev + dp->rank, &mine, sizeof mine, cudaMemcpyHostToDevice, dp->comm_stream));
    int s = WB_OK;
    ncclResult_t r = dp->nccl->AllGather(dev + dp->rank, dev, sizeof(IpcPacket), ncclChar, dp->comm, dp->comm_stream);
    std::vector<IpcPacket> all(dp->world);
    if (r != ncclSuccess) { wb_set_error("peer mode: handle exchange failed: %s", dp->nccl->GetErrorString(r)); s = WB_ERR_CUDA; }
    if (s == WB_OK && cudaMemcpyAsync(all.data(), dev, sizeof(IpcPacket) * dp->world, cudaMemcpyDeviceToHost, dp->comm_stream) != cudaSuccess) s = WB_ERR_CUDA;
    if (s == WB_OK && cudaStreamSynchronize(dp->comm_stream) != cudaSuccess) s = WB_ERR_CUDA;
    cudaFree(dev);
    if (s != WB_OK) { (void)cudaGetLastError(); return s; }
    for (int p = 0; p < dp->world; ++p) {
        if (p == dp->rank) {
            dp->peers.grad[p] = dp->grad;
            dp->peers.theta[p] = dp->theta;
            dp->peers.flags[p] = dp->flags;
            continue;
        }
        void *g = nullptr, *t = nullptr, *f = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&g, all[p].grad, cudaIpcMemLazyEnablePeerAccess);
        if (e == cudaSuccess) { dp->opened[dp->n_opened++] = g; e = cudaIpcOpenMemHandle(&t, all[p].theta, cudaIpcMemLazyEnablePeerAccess); }
        if (e == cudaSuccess) { dp->opened[dp->n_opened++] = t; e = cudaIpcOpenMemHandle(&f, all[p].flags, cudaIpcMemLazyEnablePeerAccess); }
        if (e == cudaSuccess) dp->opened[dp->n_opened++] = f;
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            wb_set_error("peer mode: cudaIpcOpenMemHandle for rank %d failed: %s", p, cudaGetErrorString(e));
            return WB_ERR_CUDA;
        }
        dp->peers.grad[p] = reinterpret_cast<const float*>(static_cast<char*>(g) + all[p].grad_off);
        dp->peers.theta[p] = reinterpret_cast<float*>(static_cast<char*>(t) + all[p].theta_off);
        dp->peers.flags[p] = reinterpret_cast<PeerFlags*>(static_cast<char*>(f) + all[p].flags_off);
    }
    return WB_OK;
}

void close_peers(WbDp* dp) {
    for (int i = 0; i < dp->n_opened; ++i) cudaIpcCloseMemHandle(dp->opened[i]);
    dp->n_opened = 0;
}

// Every rank learns whether all ranks succeeded at something (1) or any failed (0): a summed flag.
int all_agree(WbDp* dp, bool ok, bool* all_ok) {
    int* d = nullptr;
    WB_CHECK_CUDA(cudaMalloc(&d, sizeof(int)));
    int h = ok ? 0 : 1;
    WB_CHECK_CUDA(cudaMemcpyAsync(d, &h, sizeof h, cudaMemcpyHostToDevice, dp->comm_stream));
    ncclResult_t r = dp->nccl->AllReduce(d, d, 1, ncclInt, ncclSum, dp->comm, dp->comm_stream);
    cudaError_t e = cudaMemcpyAsync(&h, d, sizeof h, cudaMemcpyDeviceToHost, dp->comm_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(dp->comm_stream);
    cudaFree(d);
    WB_REQUIRE(r == ncclSuccess && e == cudaSuccess, WB_ERR_CUDA, "data-parallel set-up: agreement all-reduce failed");
    *all_ok = h == 0;
    return WB_OK;
}

}  // namespace

extern "C" int wb_dp_unique_id(WbDpId* out) {
    WB_REQUIRE(out, WB_ERR_INVALID, "wb_dp_unique_id: null pointer");
    static_assert(sizeof(WbDpId) == sizeof(ncclUniqueId), "id sizes differ");
    NcclApi* api = load_nccl();
    if (!api) return WB_ERR_UNSUPPORTED;
    ncclUniqueId id;
    WB_CHECK_NCCL(api, api->GetUniqueId(&id));
    std::memcpy(out->bytes, id.internal, sizeof id.internal);
    return WB_OK;
}

extern "C" int wb_dp_plan_buckets(const int64_t* range_off, const int64_t* range_len, int n, int64_t min_elems, int64_t* bucket_off,
                                  int64_t* bucket_len, int max_buckets) {
    if (!range_off || !range_len || n < 0) return -1;
    std::vector<std::pair<int64_t, int64_t>> r;
    for (int i = 0; i < n; ++i) r.push_back({range_off[i], range_len[i]});
    auto b = plan_buckets(r, min_elems);
    for (size_t i = 0; i < b.size() && static_cast<int>(i) < max_buckets; ++i) {
        if (bucket_off) bucket_off[i] = b[i].off;
        if (bucket_len) bucket_len[i] = b[i].len;
    }
    return static_cast<int>(b.size());
}

extern "C" int wb_dp_create(WbTrainer* t, const WbDpId* id, int rank, int world, int mode, int64_t bucket_elems, WbDp** out) {
    WB_REQUIRE(t && out, WB_ERR_INVALID, "wb_dp_create: null pointer");
    WB_REQUIRE(world >= 1 && world <= MAX_WORLD && rank >= 0 && rank < world, WB_ERR_INVALID, "wb_dp_create: rank %d of %d (at most %d ranks)", rank, world,
               MAX_WORLD);
    WB_REQUIRE(mode >= WB_DP_AUTO && mode <= WB_DP_PEER, WB_ERR_INVALID, "wb_dp_create: unknown mode %d", mode);
    WB_REQUIRE(world == 1 || id, WB_ERR_INVALID, "wb_dp_create: more than one rank needs the shared id");
    WbDp* dp = new WbDp();
    dp->tr = t;
    dp->rank = rank;
    dp->world = world;
    std::vector<std::pair<int64_t, int64_t>> ranges;
    std::vector<int> conv_follows;
    wb_trainer_internal_info(t, &dp->be, &dp->batch, &dp->in_elems, &ranges, &conv_follows);
    dp->n_params = wb_trainer_arena_len(t);
    dp->theta = wb_trainer_params(t);
    dp->grad = wb_trainer_grads(t);
    dp->m = wb_trainer_exp_avg(t);
    dp->v = wb_trainer_exp_avg_sq(t);
    if (bucket_elems <= 0) bucket_elems = 1 << 20;
    dp->buckets = plan_buckets(ranges, bucket_elems);
    for (const Bucket& bk : dp->buckets) {  // a bucket ends with some layer range: is a conv block still ahead of it in backward?
        int flag = 0;
        for (size_t r = 0; r < ranges.size(); ++r)
            if (ranges[r].first + ranges[r].second == bk.off + bk.len) flag = conv_follows[r];
        dp->defer.push_back(flag);
    }
    if (const char* env = std::getenv("WETA_B200_DP_DEFER")) { dp->defer_enabled = env[0] == '1'; dp->defer_all = env[0] == '2'; }
    int s = WB_OK;
    auto fail = [&](int st) { wb_dp_destroy(dp); return st; };
    if (static_cast<int>(dp->buckets.size()) > MAX_BUCKETS) { wb_set_error("wb_dp_create: %zu buckets, at most %d", dp->buckets.size(), MAX_BUCKETS); return fail(WB_ERR_INVALID); }
    if (cudaSetDevice(dp->be->ordinal) != cudaSuccess) return fail(WB_ERR_CUDA);
    // Side streams at the lowest priority: when both have blocks ready, the compute stream's kernels go first.
    int lo = 0, hi = 0;
    cudaDeviceGetStreamPriorityRange(&lo, &hi);
    if (cudaStreamCreateWithPriority(&dp->comm_stream, cudaStreamNonBlocking, lo) != cudaSuccess ||
        cudaStreamCreateWithPriority(&dp->adam_stream, cudaStreamNonBlocking, lo) != cudaSuccess ||
        cudaStreamCreateWithPriority(&dp->copy_stream, cudaStreamNonBlocking, lo) != cudaSuccess) {
        wb_set_error("wb_dp_create: stream creation failed");
        return fail(WB_ERR_CUDA);
    }
    if ((s = wb_backend_create_on_stream(dp->be->ordinal, dp->comm_stream, &dp->side_be)) != WB_OK) return fail(s);
    if ((s = wb_backend_create_on_stream(dp->be->ordinal, dp->adam_stream, &dp->adam_be)) != WB_OK) return fail(s);
    for (size_t i = 0; i < dp->buckets.size(); ++i) {
        cudaEvent_t e;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return fail(WB_ERR_CUDA);
        dp->bucket_ready.push_back(e);
    }
    if (cudaEventCreateWithFlags(&dp->ev_side, cudaEventDisableTiming) != cudaSuccess || cudaEventCreateWithFlags(&dp->ev_adam, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&dp->ev_step, cudaEventDisableTiming) != cudaSuccess)
        return fail(WB_ERR_CUDA);
    for (int k = 0; k < 2; ++k)
        if (cudaEventCreateWithFlags(&dp->slot_ready[k], cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&dp->slot_consumed[k], cudaEventDisableTiming) != cudaSuccess)
            return fail(WB_ERR_CUDA);
    if (cudaMallocHost(&dp->loss_pinned, 16) != cudaSuccess) return fail(WB_ERR_CUDA);
    if (const char* env = std::getenv("WETA_B200_DP_TIMEOUT_MS")) {
        const long ms = std::atol(env);
        if (ms > 0) dp->timeout_ns = static_cast<unsigned long long>(ms) * 1000000ull;
    }
    if (const char* env = std::getenv("WETA_B200_DP_BLOCKS")) {
        const int n = std::atoi(env);
        if (n > 0 && n <= 1024) dp->fused_blocks = n;
    }
    bool shardable = true;
    for (const Bucket& b : dp->buckets) shardable = shardable && b.len % (4 * world) == 0 && b.off % 4 == 0;
    if (world == 1) {
        dp->mode = WB_DP_ALLREDUCE;
    } else {
        wb_pdl_disallow();  // see common.h: dependents parked on the SMs slow the exchange kernels that run beside backward
        dp->nccl = load_nccl();
        if (!dp->nccl) return fail(WB_ERR_UNSUPPORTED);
        ncclUniqueId nid;
        std::memcpy(nid.internal, id->bytes, sizeof nid.internal);
        ncclResult_t r = dp->nccl->CommInitRank(&dp->comm, world, nid, rank);
        if (r != ncclSuccess) { wb_set_error("ncclCommInitRank failed: %s", dp->nccl->GetErrorString(r)); dp->comm = nullptr; return fail(WB_ERR_CUDA); }
        if (mode == WB_DP_AUTO) {
            const char* env = std::getenv("WETA_B200_DP_MODE");
            mode = env ? std::atoi(env) : WB_DP_PEER;
            if (mode < WB_DP_ALLREDUCE || mode > WB_DP_PEER) mode = WB_DP_PEER;
        }
        if (mode != WB_DP_ALLREDUCE && !shardable) mode = WB_DP_ALLREDUCE;  // a bucket does not split into aligned shards
        if (mode == WB_DP_PEER) {
            // Flag block, block counters and status word; then the handle exchange.  Every rank zeroes its flags before it
            // contributes to the exchange, so no peer can announce into a block that is still being cleared.
            bool ok = cudaMalloc(&dp->flags, sizeof(PeerFlags)) == cudaSuccess && cudaMalloc(&dp->counters, sizeof(unsigned int) * MAX_BUCKETS) == cudaSuccess &&
                      cudaHostAlloc(&dp->status_host, sizeof(uint32_t), cudaHostAllocMapped) == cudaSuccess &&
                      cudaHostGetDevicePointer(&dp->status_dev, dp->status_host, 0) == cudaSuccess;
            if (ok) {
                *dp->status_host = 0;
                ok = cudaMemset(dp->flags, 0, sizeof(PeerFlags)) == cudaSuccess && cudaMemset(dp->counters, 0, sizeof(unsigned int) * MAX_BUCKETS) == cudaSuccess &&
                     cudaDeviceSynchronize() == cudaSuccess;
            }
            if (ok) ok = open_peers(dp) == WB_OK;
            if (!ok) (void)cudaGetLastError();
            // All ranks must take the same path: if any rank could not map its peers, every rank uses NCCL shards.
            bool all_ok = false;
            if ((s = all_agree(dp, ok, &all_ok)) != WB_OK) return fail(s);
            if (!all_ok) {
                close_peers(dp);
                mode = WB_DP_SHARDED;
            }
        }
        dp->mode = mode;
    }
    wb_trainer_set_bucket_callback(t, on_range, dp);
    *out = dp;
    return WB_OK;
}

extern "C" int wb_dp_destroy(WbDp* dp) {
    if (!dp) return WB_OK;
    if (dp->be) cudaSetDevice(dp->be->ordinal);
    if (dp->tr) wb_trainer_set_bucket_callback(dp->tr, nullptr, nullptr);
    if (dp->be) cudaStreamSynchronize(dp->be->stream);
    for (cudaStream_t s : {dp->comm_stream, dp->adam_stream, dp->copy_stream})
        if (s) cudaStreamSynchronize(s);
    if (dp->comm) dp->nccl->CommDestroy(dp->comm);
    close_peers(dp);
    if (dp->side_be) wb_backend_destroy(dp->side_be);
    if (dp->adam_be) wb_backend_destroy(dp->adam_be);
    for (cudaEvent_t e : dp->bucket_ready) cudaEventDestroy(e);
    for (cudaEvent_t e : {dp->ev_side, dp->ev_adam, dp->ev_step, dp->slot_ready[0], dp->slot_ready[1], dp->slot_consumed[0], dp->slot_consumed[1]})
        if (e) cudaEventDestroy(e);
    for (auto& pr : dp->timing_events) { cudaEventDestroy(pr.first); cudaEventDestroy(pr.second); }
    for (cudaStream_t s : {dp->comm_stream, dp->adam_stream, dp->copy_stream})
        if (s) cudaStreamDestroy(s);
    if (dp->flags) cudaFree(dp->flags);
    if (dp->counters) cudaFree(dp->counters);
    if (dp->status_host) cudaFreeHost(dp->status_host);
    for (int k = 0; k < 2; ++k) {
        if (dp->slot_x[k]) cudaFree(dp->slot_x[k]);
        if (dp->slot_y[k]) cudaFree(dp->slot_y[k]);
    }
    if (dp->loss_pinned) cudaFreeHost(dp->loss_pinned);
    (void)cudaGetLastError();
    delete dp;
    return WB_OK;
}

extern "C" int wb_dp_mode(const WbDp* dp) { return dp ? dp->mode : -1; }
extern "C" int wb_dp_world(const WbDp* dp) { return dp ? dp->world : -1; }
extern "C" int wb_dp_num_buckets(const WbDp* dp) { return dp ? static_cast<int>(dp->buckets.size()) : -1; }
extern "C" int wb_dp_bucket(const WbDp* dp, int i, int64_t* off, int64_t* len) {
    WB_REQUIRE(dp && i >= 0 && i < static_cast<int>(dp->buckets.size()), WB_ERR_INVALID, "wb_dp_bucket: no bucket %d", i);
    if (off) *off = dp->buckets[i].off;
    if (len) *len = dp->buckets[i].len;
    return WB_OK;
}

// Reads the status word of the peer-mode waits and the communicator's asynchronous error state; neither blocks.
static int poll_errors(WbDp* dp) {
    if (dp->status_host && *reinterpret_cast<volatile uint32_t*>(dp->status_host) != 0) {
        const uint32_t st = *reinterpret_cast<volatile uint32_t*>(dp->status_host);
        wb_set_error("data-parallel step: rank %d gave up waiting for rank %u (%s flag of bucket %u) after %.1f s", dp->rank, st & 0xffu,
                     (st >> 16) & 1u ? "parameters-stored" : "gradients-ready", (st >> 8) & 0xffu, dp->timeout_ns * 1e-9);
        return WB_ERR_TIMEOUT;
    }
    if (dp->comm) {
        ncclResult_t async = ncclSuccess;
        ncclResult_t r = dp->nccl->CommGetAsyncError(dp->comm, &async);
        if (r != ncclSuccess || (async != ncclSuccess && async != ncclInProgress)) {
            wb_set_error("data-parallel step: NCCL reports an asynchronous error: %s", dp->nccl->GetErrorString(r != ncclSuccess ? r : async));
            return WB_ERR_CUDA;
        }
    }
    return WB_OK;
}

// One training step on the staged batch: forward, loss, backward with each bucket's exchange and optimizer update
// queued behind it, and the hand-over that makes the next step wait for the last update.  Asynchronous.
extern "C" int wb_dp_step(WbDp* dp, const uint64_t* dropout_seeds, int n_seeds) {
    WB_REQUIRE(dp, WB_ERR_INVALID, "wb_dp_step: null handle");
    WB_TRY(poll_errors(dp));
    dp->step = wb_trainer_begin_step(dp->tr);
    dp->seq += 1;
    dp->next_bucket = 0;
    dp->covered = 0;
    dp->issue_error = WB_OK;
    dp->deferred.clear();
    WB_TRY(wb_trainer_forward_backward(dp->tr, dropout_seeds, n_seeds));
    if (dp->issue_error == WB_OK && !dp->deferred.empty()) {  // no quiet point came: start them now
        dp->flushing = true;
        on_range(dp, nullptr, 0);
        dp->flushing = false;
    }
    if (dp->issue_error != WB_OK) {
        wb_set_error("%s", dp->issue_message.c_str());
        return dp->issue_error;
    }
    WB_REQUIRE(dp->next_bucket == static_cast<int>(dp->buckets.size()) && dp->covered == dp->n_params, WB_ERR_INVALID,
               "data-parallel step: gradient buckets covered %lld of %lld arena elements", (long long)dp->covered, (long long)dp->n_params);
    if (dp->world > 1 && dp->mode == WB_DP_PEER) {
        // The next step may start once every peer has stored its shards of every bucket here (which also means every
        // peer has finished reading this rank's gradients): wait for the `done` words of all buckets.
        peer_wait_all_done<<<1, MAX_BUCKETS * MAX_WORLD, 0, dp->comm_stream>>>(dp->peers, dp->world, dp->rank, static_cast<int>(dp->buckets.size()), dp->seq,
                                                                              dp->timeout_ns, dp->status_dev);
        WB_LAUNCH_OK(dp->side_be);
    }
    WB_CHECK_CUDA(cudaEventRecord(dp->ev_step, dp->comm_stream));
    WB_CHECK_CUDA(cudaStreamWaitEvent(dp->be->stream, dp->ev_step, 0));
    if (dp->world > 1 && dp->mode == WB_DP_ALLREDUCE) {
        WB_CHECK_CUDA(cudaEventRecord(dp->ev_adam, dp->adam_stream));
        WB_CHECK_CUDA(cudaStreamWaitEvent(dp->be->stream, dp->ev_adam, 0));
    }
    return WB_OK;
}

static int ensure_slots(WbDp* dp) {
    if (dp->slot_x[0]) return WB_OK;
    for (int k = 0; k < 2; ++k) {
        WB_CHECK_CUDA(cudaMalloc(&dp->slot_x[k], static_cast<size_t>(dp->batch * dp->in_elems) * sizeof(float)));
        WB_CHECK_CUDA(cudaMalloc(&dp->slot_y[k], static_cast<size_t>(dp->batch) * sizeof(int64_t)));
        WB_CHECK_CUDA(cudaEventRecord(dp->slot_consumed[k], dp->be->stream));
    }
    return WB_OK;
}

// Queues the upload of one host batch (pinned memory, so the copy is asynchronous) into the next of two device slots,
// on a copy stream: the copy of batch i+1 runs while step i computes.  The copy waits for the step that last read the slot.
extern "C" int wb_dp_submit(WbDp* dp, const float* host_x, const int64_t* host_y) {
    WB_REQUIRE(dp && host_x && host_y, WB_ERR_INVALID, "wb_dp_submit: null pointer");
    WB_REQUIRE(dp->submitted - dp->stepped < 2, WB_ERR_INVALID, "wb_dp_submit: both slots hold batches that have not been stepped yet");
    WB_TRY(ensure_slots(dp));
    const int k = static_cast<int>(dp->submitted % 2);
    WB_CHECK_CUDA(cudaStreamWaitEvent(dp->copy_stream, dp->slot_consumed[k], 0));
    WB_CHECK_CUDA(cudaMemcpyAsync(dp->slot_x[k], host_x, static_cast<size_t>(dp->batch * dp->in_elems) * sizeof(float), cudaMemcpyHostToDevice, dp->copy_stream));
    WB_CHECK_CUDA(cudaMemcpyAsync(dp->slot_y[k], host_y, static_cast<size_t>(dp->batch) * sizeof(int64_t), cudaMemcpyHostToDevice, dp->copy_stream));
    WB_CHECK_CUDA(cudaEventRecord(dp->slot_ready[k], dp->copy_stream));
    dp->submitted++;
    return WB_OK;
}

// One step on the oldest submitted batch; reads the loss back and waits for it when host_loss is given.
extern "C" int wb_dp_step_submitted(WbDp* dp, const uint64_t* dropout_seeds, int n_seeds, float* host_loss) {
    WB_REQUIRE(dp, WB_ERR_INVALID, "wb_dp_step_submitted: null handle");
    WB_REQUIRE(dp->stepped < dp->submitted, WB_ERR_INVALID, "wb_dp_step_submitted: no submitted batch to step on");
    const int k = static_cast<int>(dp->stepped % 2);
    WB_CHECK_CUDA(cudaStreamWaitEvent(dp->be->stream, dp->slot_ready[k], 0));
    WB_TRY(wb_trainer_set_input(dp->tr, dp->slot_x[k], dp->slot_y[k]));
    int s = wb_dp_step(dp, dropout_seeds, n_seeds);
    cudaEventRecord(dp->slot_consumed[k], dp->be->stream);
    wb_trainer_set_input(dp->tr, nullptr, nullptr);
    dp->stepped++;
    WB_TRY(s);
    if (host_loss) {
        WB_CHECK_CUDA(cudaMemcpyAsync(dp->loss_pinned, wb_trainer_loss_ptr(dp->tr), sizeof(float), cudaMemcpyDeviceToHost, dp->be->stream));
        WB_TRY(wb_dp_wait(dp, 0));
        *host_loss = *dp->loss_pinned;
    }
    return WB_OK;
}

// A host-side watchdog: polls `poll` (0 = finished, 1 = still running, anything else = failed) every
// `interval_us` until it finishes or `timeout_ms` have passed (0 = no limit).
extern "C" int wb_watchdog_wait(wb_poll_fn poll, void* user, int timeout_ms, int interval_us) {
    WB_REQUIRE(poll, WB_ERR_INVALID, "wb_watchdog_wait: null callback");
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const int r = poll(user);
        if (r == 0) return WB_OK;
        if (r != 1) {
            if (r != WB_ERR_TIMEOUT && r != WB_ERR_CUDA) wb_set_error("watchdog: the watched operation reported failure %d", r);
            return r == WB_ERR_TIMEOUT ? WB_ERR_TIMEOUT : WB_ERR_CUDA;
        }
        if (timeout_ms > 0 && std::chrono::steady_clock::now() - t0 > std::chrono::milliseconds(timeout_ms)) {
            wb_set_error("watchdog: no completion within %d ms", timeout_ms);
            return WB_ERR_TIMEOUT;
        }
        if (interval_us > 0) std::this_thread::sleep_for(std::chrono::microseconds(interval_us));
        else std::this_thread::yield();
    }
}

static int poll_step(void* user) {
    WbDp* dp = static_cast<WbDp*>(user);
    int s = poll_errors(dp);
    if (s != WB_OK) return s;
    cudaError_t e = cudaStreamQuery(dp->be->stream);
    if (e == cudaErrorNotReady) return 1;
    if (e != cudaSuccess) {
        wb_set_error("data-parallel step: the compute stream reports %s", cudaGetErrorString(e));
        return WB_ERR_CUDA;
    }
    // the compute stream waits for the side streams at the end of every step, so it drains last
    return poll_errors(dp);
}

// Waits until everything queued by the steps so far has finished.  With timeout_ms > 0 it gives up after that long
// and aborts the communicator, so a rank whose peer never joined a collective returns an error instead of hanging.
extern "C" int wb_dp_wait(WbDp* dp, int timeout_ms) {
    WB_REQUIRE(dp, WB_ERR_INVALID, "wb_dp_wait: null handle");
    if (timeout_ms <= 0) {
        WB_CHECK_CUDA(cudaStreamSynchronize(dp->be->stream));
        return poll_errors(dp);
    }
    int s = wb_watchdog_wait(poll_step, dp, timeout_ms, 50);
    if (s == WB_ERR_TIMEOUT && dp->comm) {
        std::string msg = wb_last_error();
        dp->nccl->CommAbort(dp->comm);  // ends NCCL kernels that are still waiting for the missing rank
        dp->comm = nullptr;
        wb_set_error("%s; the communicator was aborted", msg.c_str());
    }
    return s;
}

extern "C" int wb_dp_set_timing(WbDp* dp, int on) {
    WB_REQUIRE(dp, WB_ERR_INVALID, "wb_dp_set_timing: null handle");
    dp->timing = on != 0;
    return WB_OK;
}

// Device time of the side-stream work (exchange + optimizer) of the buckets issued since the last report:
// one line "bucket_work calls total_ms".  Waits for the streams.
extern "C" const char* wb_dp_timing_report(WbDp* dp) {
    cudaStreamSynchronize(dp->comm_stream);
    double ms = 0.0;
    int calls = 0;
    for (auto& pr : dp->timing_events) {
        float e = 0.f;
        if (cudaEventElapsedTime(&e, pr.first, pr.second) == cudaSuccess) { ms += e; calls++; }
        cudaEventDestroy(pr.first);
        cudaEventDestroy(pr.second);
    }
    dp->timing_events.clear();
    char line[96];
    snprintf(line, sizeof line, "bucket_work %d %.6f\n", calls, ms);
    dp->timing_text = line;
    return dp->timing_text.c_str();
}

// The PEER-mode kernel as a stand-alone operation: sums `world` gradient buffers element-wise in index order, runs
// Adam step t on elements [offset, offset + len) of the parameters held in thetas[self] with this caller's m / v, and
// stores the result into all `world` parameter buffers.  The pointers may be peer mappings or local buffers.
extern "C" int wb_reduce_adam_broadcast(WbBackend* b, const float* const* grads, float* const* thetas, int world, int self, int64_t offset, int64_t len,
                                        float* m, float* v, int64_t t, double lr, double beta1, double beta2, double eps, double weight_decay,
                                        int decoupled, double grad_scale) {
    WB_REQUIRE(b && grads && thetas && m && v, WB_ERR_INVALID, "wb_reduce_adam_broadcast: null pointer");
    WB_REQUIRE(world >= 1 && world <= MAX_WORLD && self >= 0 && self < world, WB_ERR_INVALID, "wb_reduce_adam_broadcast: %d buffers (1..%d)", world, MAX_WORLD);
    WB_REQUIRE(t >= 1 && offset >= 0 && len >= 0 && offset % 4 == 0 && len % 4 == 0, WB_ERR_INVALID,
               "wb_reduce_adam_broadcast: offset and length must be multiples of 4 elements");
    if (len == 0) return WB_OK;
    FusedArgs a{};
    uintptr_t bits = reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v);
    for (int p = 0; p < world; ++p) {
        WB_REQUIRE(grads[p] && thetas[p], WB_ERR_INVALID, "wb_reduce_adam_broadcast: null buffer %d", p);
        a.grad[p] = grads[p];
        a.theta[p] = thetas[p];
        bits |= reinterpret_cast<uintptr_t>(grads[p]) | reinterpret_cast<uintptr_t>(thetas[p]);
    }
    WB_REQUIRE((bits & 15) == 0, WB_ERR_INVALID, "wb_reduce_adam_broadcast: every buffer must be 16-byte aligned");
    a.m = m;
    a.v = v;
    a.world = world;
    a.self = self;
    a.off = offset;
    a.len = len;
    a.k = wb_adam_constants(t, lr, beta1, beta2, eps, weight_decay, decoupled, grad_scale);
    const int64_t groups = len / 4;
    const int blocks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(4 * b->sm_count, (groups + 511) / 512)));
    launch_reduce_adam_broadcast(a, blocks, b->stream);
    WB_LAUNCH_OK(b);
    return WB_OK;
}

// Test hook of the bounded device-side wait: one launch of the announce/wait kernel as rank 0 of a two-rank job whose
// second rank does not exist, so nothing ever sets the word it polls.  Returns WB_ERR_TIMEOUT once the limit has
// passed (the kernel has returned by then and the context stays usable), WB_OK if `preset` filled the word first.
extern "C" int wb_dp_selftest_wait(WbBackend* b, int timeout_ms, int preset) {
    WB_REQUIRE(b && timeout_ms > 0 && timeout_ms <= 5000, WB_ERR_INVALID, "wb_dp_selftest_wait: timeout must be 1..5000 ms");
    WB_CHECK_CUDA(cudaSetDevice(b->ordinal));
    PeerFlags* flags = nullptr;
    uint32_t *status_host = nullptr, *status_dev = nullptr;
    WB_CHECK_CUDA(cudaMalloc(&flags, sizeof(PeerFlags)));
    cudaError_t e = cudaMemsetAsync(flags, 0, sizeof(PeerFlags), b->stream);
    if (e == cudaSuccess) e = cudaHostAlloc(&status_host, sizeof(uint32_t), cudaHostAllocMapped);
    if (e == cudaSuccess) e = cudaHostGetDevicePointer(&status_dev, status_host, 0);
    if (e != cudaSuccess) { cudaFree(flags); if (status_host) cudaFreeHost(status_host); WB_CHECK_CUDA(e); }
    *status_host = 0;
    if (preset) {
        const uint32_t one = 1;
        cudaMemcpyAsync(&flags->ready[0][1], &one, sizeof one, cudaMemcpyHostToDevice, b->stream);
    }
    PeerPtrs pp{};
    pp.flags[0] = flags;
    pp.flags[1] = flags;  // the absent rank's block: this rank's announcement lands in its own block, harmlessly
    peer_announce_wait<<<1, 32, 0, b->stream>>>(pp, 2, 0, 0, 0, 1, 1, 1u, static_cast<unsigned long long>(timeout_ms) * 1000000ull, status_dev);
    b->launches++;
    e = cudaStreamSynchronize(b->stream);
    const uint32_t st = *status_host;
    cudaFree(flags);
    cudaFreeHost(status_host);
    WB_CHECK_CUDA(e);
    if (st != 0) {
        wb_set_error("bounded wait ran out after %d ms waiting for rank %u", timeout_ms, st & 0xffu);
        return WB_ERR_TIMEOUT;
    }
    return WB_OK;
}
