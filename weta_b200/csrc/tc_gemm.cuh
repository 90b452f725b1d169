// TF32 tensor-core GEMM for sm_100a: TMA -> 128B-swizzled shared-memory ring -> tcgen05.mma
// (kind::tf32, accumulator in TMEM) -> tcgen05.ld epilogue.
//
// Persistent CTAs (one per SM) each walk a list of 128 x BN output tiles.  Warp 0 (one elected lane)
// issues the TMA loads, warp 1 (one lane) issues the MMAs into one of two TMEM accumulators, and four
// epilogue warps read the other accumulator back (a warp may read TMEM lanes 32*(warp%4)..+31, i.e. 32
// tile rows) and store it, so one tile's epilogue overlaps the next tile's main loop.  Operands may be K-major
// (contraction index contiguous) or MN-major (row/column index contiguous); both are described to
// the tensor core through the shared-memory matrix descriptor, so no operand is ever transposed
// in memory.  A "segment" is one (A map, B map, K extent) triple; up to three segments accumulate
// into the same TMEM tile, which is how the 3xTF32 mode runs hi*hi + hi*lo + lo*hi in one launch.
//
// Every wait on an mbarrier is bounded: after SPIN_LIMIT polls the waiter raises the error flag
// in global memory and leaves; the other roles then run out as well, TMEM is released, and the
// host reports WB_ERR_TIMEOUT.  No loads here use cluster-wide delivery; each CTA fetches its own
// tiles.
#pragma once

#include <cuda.h>
#include <type_traits>

#include "common.h"

namespace tc {

constexpr int BM = 128;
constexpr int BK = 32;                 // 32 tf32 = 128 bytes = one swizzle row
constexpr int UMMA_K = 8;              // K per tcgen05.mma for tf32
// warp 0: TMA, warp 1: MMA + TMEM owner, then EPW epilogue warps (8, or 16 for contractions of one or two K blocks,
// whose time is the epilogue's instruction stream)
constexpr int threads_for(int epw) { return 64 + 32 * epw; }
constexpr uint32_t SPIN_LIMIT = 1u << 26;

struct Segment {
    CUtensorMap a;
    CUtensorMap b;
};

struct Epilogue {
    float* out;            // row-major [M, ldd] (+ batch * batch_stride_d)
    int64_t ldd;
    int64_t batch_stride_d;
    const float* bias_n;   // per output column, may be null
    const float* bias_m;   // per output row, may be null
    int relu;
    int accumulate;        // out += result instead of out = result
    // Optional per-row statistics, added (atomically, in double) over the whole launch: row_stats[2*row] += sum,
    // row_stats[2*row + 1] += sum of squares, both of the accumulator BEFORE bias_m is added, i.e. of the stored
    // value minus its row's bias (a large bias then costs the sum of squares no digits).  The caller zeroes the
    // array.  For a convolution whose rows are output channels these are the sums batch normalisation needs, so
    // the activation is not read again to get them.  Not available with split-K, bias_n or relu.
    double* row_stats = nullptr;
};

struct Args {
    Segment seg[3];
    int num_segments;
    int m, n;
    int k_blocks;          // BK-blocks of the contraction, per segment
    int splits;            // split-K factor: blockIdx.z = batch * splits + split
    int batched_a, batched_b;  // 0: operand shared by every batch (TMA coordinate 0)
    int kpb;                   // K blocks per image when the contraction spans the batch, else 0
    int tiles_m, tiles_n, total_tiles;  // tile list walked by the persistent CTAs
    FastDiv div_tiles_m, div_tiles_n, div_splits;  // the same counts as multiply-shift divisors: a tile index is taken apart by one
                                                   // thread per role before its first copy, MMA or store can start
    // Implicit-GEMM convolution (3x3, stride 1, padding 1, NCHW).  The B operand is not a matrix in memory
    // but windows of an image tensor [n][c][h*w]: a run of pixels moved by (ky-1) rows is the same run at
    // flattened offset (ky-1)*w, which TMA can start at when w is a multiple of 4; the horizontal move by
    // kx-1 would misalign the box, so seg[kx].b maps a copy of the tensor already shifted by kx-1 columns.
    //   conv_mode 1 (forward, input gradient): A = reordered weights [M][tap][c], K index = (tap, c);
    //     B chunks are 32 pixels x 32 channels, N-major.
    //   conv_mode 2 (weight gradient): M index = (tap, c): A is one box of BM channels x 32 pixels of the tap's
    //     window (seg[kx].a maps the shifted copies), K-major; B = dY [o][pixels] per image; K index = (image, pixel block).
    //   conv_mode 3 (input gradient without shifted copies, MT = 3 kernels): the horizontal move is applied to the
    //     RESULT instead of the operand.  Row block kx of a tile accumulates P_kx[m][q] = sum over (ky, c) of
    //     A[m][(ky, kx)][c] * img[c][q + (ky-1)*w] from the unshifted tensor (seg[0].b); the epilogue stores
    //     P_1[m][q] + P_0[m][q-1] + P_2[m][q+1], dropping the terms that would cross an image row's ends.  The
    //     neighbours are registers of the same thread: tiles are 128 pixels wide and w divides 32, so a 32-column
    //     chunk of the accumulator never ends inside an image row.
    int conv_mode, conv_w, conv_cb;  // conv_cb: 32-channel blocks per tap (modes 1, 3) / BM-channel blocks per tap (mode 2)
    Epilogue ep;
    int64_t split_stride_d;    // distance between split-K partial outputs
    int* error_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// Bounded wait.  Returns false if the phase never completed within `limit` polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = SPIN_LIMIT) {
    uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < limit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Shared-memory matrix descriptor, SWIZZLE_128B, descriptor version 1 (sm_100).
//   bits [0,14)  start address >> 4      bits [16,30) leading-dim byte offset >> 4
//   bits [32,46) stride-dim byte offset >> 4   bits [46,48) version = 1   bits [61,64) layout = 2 (128B swizzle)
// Layout field: 2 = 128B swizzle of 16-byte chunks (K-major operands); layout 1 = 128B swizzle of 32-byte chunks,
//   the only swizzled layout the tensor core accepts for MN-major 32-bit operands.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(layout) << 61;
    return d;
}

// Instruction descriptor for kind::tf32 with an f32 accumulator:
//   [4,6) D format = 1 (f32)   [7,10) A format = 2 (tf32)   [10,13) B format = 2 (tf32)
//   [15] A major (0 = K, 1 = MN)   [16] B major   [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int a_mn, int b_mn) {
    return (1u << 4) | (2u << 7) | (2u << 10) | (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives on `bar` once every MMA issued so far by this thread has finished reading shared memory.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster act as one 256-row MMA --------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Shared::cluster address of the same shared-memory location in CTA `cta` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(cta));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load issued by either CTA of a pair; the bytes are counted on the barrier at cluster address `bar`
// (the leader CTA's), which cta_group::2 allows to live in the other CTA than the destination.
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
        : "memory");
}
// D[256 x N] (+)= A[256 x 8] B[8 x N]: rows 0-127 of A and D live in the leader CTA, rows 128-255 in its peer;
// each CTA's shared memory holds N/2 rows of B.  Issued by the leader only.
__device__ __forceinline__ void umma_tf32_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Completion of the pair's MMAs issued so far, signalled on the barrier at cluster address `bar` (either CTA's).
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr) : "memory");
}

// Issues the TMEM load of 32 columns of this warp's 32 lanes; the registers are valid after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }


template <int BN, int STAGES, int CTAS, int EPW, int MT, int HALO = 0>
struct SharedStorage {
    // Stage buffers first: each must start on a 1024-byte boundary for the 128B swizzle.
    alignas(1024) float a[STAGES][MT * BM * BK];   // MT row blocks of BM rows, one after the other
    alignas(1024) float b[STAGES][(BN / CTAS + 32 * HALO) * BK];  // a CTA of a pair holds half of the tile's B rows
    // Epilogue staging, one 32 x 32 slab per epilogue warp; 16-byte chunk j of row r sits at chunk j ^ (r & 7),
    // so the row-per-lane writes and the row-segment reads are both free of bank conflicts without padding.
    alignas(128) float stage[EPW][32 * 32];
    alignas(8) uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[4];   // one pair of barriers per TMEM accumulator: 512 / BN of them
    uint64_t tmem_empty[4];
    uint32_t tmem_base;
};

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Persistent kernel: gridDim.x CTAs (one per SM) walk the tile list round-robin.  Ten warps:
//   warp 0      TMA producer (one lane)            smem ring, STAGES deep
//   warp 1      MMA issuer (one lane); owns TMEM   512 / BN accumulators of BN columns, used in turn
//   warps 2..9  epilogue: TMEM -> registers -> shared staging -> coalesced global stores
// so the stores of tile i overlap the loads and MMAs of tile i+1.
// A_MN: A tile arrives as BM/32 boxes of [32 m][BK k-rows]; otherwise one box of [BM rows][BK k].
// CTAS = 2: launched as clusters of two CTAs that share one (2*BM) x BN tile.  Each loads its own BM rows of A
// and its own BN/2 rows of B (a third fewer bytes per flop through L2 than two independent BM x BN tiles); the
// even CTA (the leader) issues cta_group::2 MMAs that read both CTAs' shared memory and write both CTAs' TMEM;
// each CTA stores its own BM rows of the result.  Barriers: `full` and `tmem_empty` are the leader's (the peer's
// loads and epilogue warps signal them remotely), `empty` and `tmem_full` exist in both CTAs and the leader's
// commits signal each of them.
// MT = 2 (single CTAs only): one CTA owns a (2*BM) x BN tile as two BM-row blocks that share every B box - the
// same third fewer operand bytes per flop as a CTA pair, inside one SM.  Both TMEM accumulators belong to the one
// tile, so its epilogue does not overlap the next tile's MMAs: used for contractions whose tiles run long.
// HALO = 1 (conv_mode 1 on images 16 pixels wide, one split): the three taps of one kernel column share their
// pixels.  Rows come two to a 32-pixel chunk, so the windows of the upper and the lower tap (one image row up, one
// down) are the same chunks, one chunk apart, of a single copy that starts one image row early and is one chunk
// longer; only the middle tap needs a copy of its own.  The K blocks of a (channel block, kernel column) then run in
// the order middle, upper, lower; the lower tap's ring slot carries weights only and its MMAs read the pixels from
// the upper tap's slot, which is handed back together with its own.  Two pixel copies instead of three per kernel
// column: a fifth fewer operand bytes through L2 on 128 x 256 tiles.  (Works for CTA pairs too; measured no gain there.)
//
// CSPLIT = 1: split-K inside a thread-block cluster, for outputs of so few tiles that most SMs would idle while each
// busy one pulls a whole contraction's operands through its own L2 port (a 128 x 128 tile takes in 32 KB per K block
// at about 50 bytes per clock, whatever the tensor cores could do).  The grid is one cluster of `splits` (2, 4 or 8)
// CTAs per tile, one tile per cluster; CTA r accumulates K blocks [r * k_blocks / splits, (r + 1) * k_blocks / splits),
// writes its accumulator into its own shared memory (the operand ring, idle by then) and, after a cluster barrier,
// sums rows [r * 128 / splits, (r + 1) * 128 / splits) of all the CTAs' partial tiles through distributed shared
// memory in rank order (one order, every run), applies the epilogue and stores them: no partial results in global
// memory and no second launch.  A second cluster barrier keeps every CTA's shared memory alive until its peers have
// read it.  (Sending the rows to their owners with remote stores instead, which needs no second barrier, was slower:
// 3 us for the exchange against 0.7 + 2.3 us for barrier and remote reads on a 512^3 product.)
template <int BN, int STAGES, bool A_MN, bool B_MN, int CTAS, int EPW, int MT, int HALO = 0, int CSPLIT = 0>
__global__ void __launch_bounds__(threads_for(EPW), 1) gemm_tf32_kernel(const __grid_constant__ Args args) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    using SS = SharedStorage<BN, STAGES, CTAS, EPW, MT, HALO>;
    static_assert(CSPLIT == 0 || (CTAS == 1 && MT == 1 && HALO == 0 && BN == 128 && EPW == 8), "cluster split-K: plain 128 x 128 tiles");
    constexpr int RED_LD = BN + 4;  // floats between rows of the partial tile in shared memory (padded against bank conflicts)
    static_assert(CSPLIT == 0 || BM * RED_LD <= STAGES * MT * BM * BK, "the partial tile must fit the A ring");

    static_assert(MT == 1 || (MT == 2 && CTAS == 1 && BN == 256) || (MT == 3 && CTAS == 1 && BN == 128 && B_MN && !A_MN && HALO == 0),
                  "two row blocks per CTA: single CTAs with 256-wide tiles; three (conv_mode 3): 128-wide tiles");
    static_assert(HALO == 0 || (MT == 1 && B_MN && !A_MN && STAGES >= 3), "shared tap windows: implicit convolution tiles only");
    SS& ss = *reinterpret_cast<SS*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int B_ROWS = BN / CTAS;   // B rows this CTA loads
    constexpr int TILE_M = MT == 3 ? BM : BM * CTAS * MT;   // output rows per tile (the three blocks of conv_mode 3 are the same rows)
    constexpr int NACC = 512 / BN;      // accumulators in TMEM (all 512 columns), used round-robin: 2 or 4 tiles in flight

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb_per = static_cast<int>(args.div_splits.div(static_cast<uint32_t>(args.k_blocks + args.splits - 1)));
    const int rank = CTAS == 2 ? static_cast<int>(cluster_ctarank()) : 0;
    const int first_tile = static_cast<int>(blockIdx.x) / CTAS, tile_step = static_cast<int>(gridDim.x) / CTAS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&ss.full[s], 1);
            mbar_init(&ss.empty[s], 1);
        }
        for (int a = 0; a < NACC; ++a) {
            mbar_init(&ss.tmem_full[a], 1);
            mbar_init(&ss.tmem_empty[a], EPW * CTAS);  // one arrival per epilogue warp (of both CTAs of a pair)
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if constexpr (CTAS == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ss.tmem_base)), "r"(512)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ss.tmem_base)), "r"(512)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (CTAS == 2) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = ss.tmem_base;
    bool ok = true;
    // Launched as a programmatic dependent of the kernel before it in the stream: everything above (barriers, TMEM,
    // and the launch itself) may run while that kernel is still finishing; nothing below touches global memory before
    // it has completed and its writes are visible.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // Only a short product (one tile per CTA at most, a short contraction) releases its dependents now; blocks parked
    // on the SMs for the length of a long one would slow it down, so that one releases them as its CTAs exit.
    if (args.total_tiles <= static_cast<int>(gridDim.x) && args.k_blocks * args.num_segments <= 64)
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Tile t -> (n block, m block, z = batch * splits + split); n fastest so neighbouring CTAs share A.
    auto decode = [&](int t, int& m0, int& n0, int& batch, int& split, int& kb_begin, int& kb_end) {
        const uint32_t ut = static_cast<uint32_t>(t);
        if constexpr (CSPLIT) {
            // split fastest: the CTAs of a cluster are the splits of one tile, and the K blocks are dealt out evenly
            const uint32_t q = args.div_splits.div(ut), r = args.div_tiles_n.div(q), b = args.div_tiles_m.div(r);
            split = static_cast<int>(ut - q * args.splits);
            n0 = static_cast<int>(q - r * args.tiles_n) * BN;
            m0 = static_cast<int>(r - b * args.tiles_m) * TILE_M;
            batch = static_cast<int>(b);
            kb_begin = static_cast<int>(args.div_splits.div(static_cast<uint32_t>(split * args.k_blocks)));
            kb_end = static_cast<int>(args.div_splits.div(static_cast<uint32_t>((split + 1) * args.k_blocks)));
            return;
        }
        const uint32_t r = args.div_tiles_n.div(ut), z = args.div_tiles_m.div(r), bz = args.div_splits.div(z);
        m0 = static_cast<int>(r - z * args.tiles_m) * TILE_M;
        n0 = static_cast<int>(ut - r * args.tiles_n) * BN;
        batch = static_cast<int>(bz);
        split = static_cast<int>(z - bz * args.splits);
        kb_begin = split * kb_per;
        kb_end = min(args.k_blocks, kb_begin + kb_per);
    };

    if (warp == 0) {
        if (lane == 0) {
            // ---- TMA producer ---------------------------------------------------------------
            // Walks this CTA's (tile, segment, K block) sequence and fills the shared-memory ring.  (Asking L2 to
            // fetch boxes further ahead with cp.async.bulk.prefetch.tensor was tried and made every contraction
            // slower: the kernel is bound by the bytes the SM pulls through L2, and a prefetch pulls them twice.)
            struct Cursor { int t, sg, kb, m0, n0, batch, split, kb_begin, kb_end; };
            auto start = [&](Cursor& c, int t) {
                c.t = t;
                c.sg = 0;
                if (t < args.total_tiles) {
                    decode(t, c.m0, c.n0, c.batch, c.split, c.kb_begin, c.kb_end);
                    c.kb = c.kb_begin;
                }
            };
            auto next = [&](Cursor& c) {
                if (++c.kb >= c.kb_end) {
                    c.kb = c.kb_begin;
                    if (++c.sg >= args.num_segments) start(c, c.t + tile_step);
                }
            };
            // Row blocks of the tile that hold rows of the matrix (the last tile of an odd block count has one).
            auto blocks_of = [&](const Cursor& c) { return MT == 3 ? 3 : ((MT == 2 && c.m0 + BM < args.m) ? 2 : 1); };
            // One K block of operands into ring slot s.
            auto issue = [&](const int s, const Cursor& c) {
                const CUtensorMap* ma = &args.seg[c.sg].a;
                const CUtensorMap* mb = &args.seg[c.sg].b;
                // This CTA's rows of A and of B inside the tile.
                const int m0 = c.m0 + rank * BM, n0 = c.n0 + rank * B_ROWS, batch = c.batch, kb = c.kb;
                uint64_t* bar = &ss.full[s];
                const uint32_t leader_bar = CTAS == 2 ? map_to_cta(smem_u32(bar), 0) : 0;
                auto copy = [&](float* dst, const CUtensorMap* map, int x, int y, int z) {
                    if constexpr (CTAS == 2) tma_load_3d_pair(dst, map, leader_bar, x, y, z);
                    else tma_load_3d(dst, map, bar, x, y, z);
                };
                // kpb > 0: the contraction runs over (image, position) pairs of a batched K-major
                // operand pair, kpb blocks per image (a convolution's weight gradient); the image
                // index becomes the third TMA coordinate and each image's tail is zero-filled.
                const int k0 = (args.kpb > 0 ? kb % args.kpb : kb) * BK;
                const int kz = args.kpb > 0 ? kb / args.kpb : 0;
                const int za = args.kpb > 0 ? kz : (args.batched_a ? batch : 0);
                const int zb = args.kpb > 0 ? kz : (args.batched_b ? batch : 0);
                if constexpr (MT == 3) {
                    // kb = channel block * 3 + ky; the three kernel columns are the three row blocks
                    const int cb = kb / 3, ky = kb - cb * 3;
#pragma unroll
                    for (int kx = 0; kx < 3; ++kx) copy(&ss.a[s][kx * BM * BK], ma, ((ky * 3 + kx) * args.conv_cb + cb) * BK, m0, 0);
                    const int x0 = n0 + (ky - 1) * args.conv_w;
#pragma unroll
                    for (int ch = 0; ch < B_ROWS / 32; ++ch) copy(&ss.b[s][ch * 32 * BK], mb, x0 + ch * 32, cb * 32, batch);
                } else if constexpr (HALO == 1) {
                    // kb = (channel block * 3 + kx) * 3 + r; r = 0: middle tap (ky = 1) with its own pixels, r = 1: upper
                    // tap (ky = 0) with the long copy that starts one image row early, r = 2: lower tap (ky = 2), weights only.
                    const int cb = kb / 9, j = kb - cb * 9;
                    const int kx = j / 3, r = j - kx * 3;
                    const int tap = (r == 0 ? 1 : (r == 1 ? 0 : 2)) * 3 + kx;
                    copy(&ss.a[s][0], ma, (tap * args.conv_cb + cb) * BK, m0, 0);
                    if (r < 2) {
                        const CUtensorMap* mx = &args.seg[kx].b;
                        const int x0 = n0 - (r == 1 ? args.conv_w : 0);
                        const int chunks = B_ROWS / 32 + (r == 1 ? 1 : 0);
                        for (int ch = 0; ch < chunks; ++ch) copy(&ss.b[s][ch * 32 * BK], mx, x0 + ch * 32, cb * 32, batch);
                    }
                } else if (args.conv_mode == 1) {
                    // kb = channel block * 9 + tap, tap = ky*3 + kx: the nine taps of a channel block follow one
                    // another, so the rows a tap shares with the previous ones (same pixels, moved by a row) are
                    // still in L2.  The window of tap (ky, kx) over a run of pixels is the same run, moved (ky-1)
                    // image rows, of the copy shifted by kx-1; positions before the first / after the last pixel
                    // are zero-filled by TMA, which is the padding.  A's columns are ordered (tap, channel).
                    const int cb = kb / 9, tap = kb - cb * 9;
                    const int ky = tap / 3, kx = tap - ky * 3;
                    for (int sub = 0; sub < blocks_of(c); ++sub) copy(&ss.a[s][sub * BM * BK], ma, (tap * args.conv_cb + cb) * BK, m0 + sub * BM, 0);
                    const CUtensorMap* mx = &args.seg[kx].b;
                    const int x0 = n0 + (ky - 1) * args.conv_w;
#pragma unroll
                    for (int ch = 0; ch < B_ROWS / 32; ++ch) copy(&ss.b[s][ch * 32 * BK], mx, x0 + ch * 32, cb * 32, batch);
                } else if (args.conv_mode == 2) {
                    // M tile = tap * conv_cb + channel block of BM; K block = 32 pixels of image kz.
                    for (int sub = 0; sub < blocks_of(c); ++sub) {
                        const int mbi = m0 / BM + sub;
                        const int tap = mbi / args.conv_cb, cb = mbi - tap * args.conv_cb;
                        const int ky = tap / 3, kx = tap - ky * 3;
                        copy(&ss.a[s][sub * BM * BK], &args.seg[kx].a, k0 + (ky - 1) * args.conv_w, cb * BM, kz);
                    }
                    copy(&ss.b[s][0], mb, k0, n0, kz);
                } else {
                    for (int sub = 0; sub < blocks_of(c); ++sub) {
                        if constexpr (A_MN) {
#pragma unroll
                            for (int ch = 0; ch < BM / 32; ++ch) copy(&ss.a[s][sub * BM * BK + ch * 32 * BK], ma, m0 + sub * BM + ch * 32, k0, za);
                        } else {
                            copy(&ss.a[s][sub * BM * BK], ma, k0, m0 + sub * BM, za);
                        }
                    }
                    if constexpr (B_MN) {
#pragma unroll
                        for (int ch = 0; ch < B_ROWS / 32; ++ch) copy(&ss.b[s][ch * 32 * BK], mb, n0 + ch * 32, k0, zb);
                    } else {
                        copy(&ss.b[s][0], mb, k0, n0, zb);
                    }
                }
            };
            Cursor cur;
            start(cur, first_tile);
            for (int it = 0; cur.t < args.total_tiles; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(&ss.empty[s], ph ^ 1)) { ok = false; break; }
                if (rank == 0) {  // the leader's barrier counts both CTAs' bytes
                    int b_rows = B_ROWS;
                    if constexpr (HALO == 1) {
                        const int r = cur.kb % 3;
                        b_rows = r == 0 ? B_ROWS : (r == 1 ? B_ROWS + 32 : 0);
                    }
                    mbar_expect_tx(&ss.full[s], static_cast<uint32_t>((blocks_of(cur) * BM * BK + b_rows * BK) * sizeof(float)) * CTAS);
                }
                issue(s, cur);
                next(cur);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer (the leader CTA of a pair) ----------------------------------------
            constexpr uint32_t idesc = make_idesc(BM * CTAS, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
            // A completion is signalled in this CTA and, for a pair, at the same barrier of the peer.
            auto commit = [&](uint64_t* bar) {
                if constexpr (CTAS == 2) {
                    umma_commit_pair(smem_u32(bar));
                    umma_commit_pair(map_to_cta(smem_u32(bar), 1));
                } else {
                    umma_commit(bar);
                }
            };
            int it = 0, tile_iter = 0;
            for (int t = first_tile; t < args.total_tiles && ok; t += tile_step, ++tile_iter) {
                int m0, n0, batch, split, kb_begin, kb_end;
                decode(t, m0, n0, batch, split, kb_begin, kb_end);
                // MT == 1: the tiles take the accumulators in turn.  MT == 2: row block `sub` of every tile uses accumulator `sub`.
                const int acc = MT >= 2 ? 0 : tile_iter % NACC;
                const uint32_t use = static_cast<uint32_t>(MT >= 2 ? tile_iter : tile_iter / NACC);
                const int nsub = MT == 3 ? 3 : ((MT == 2 && m0 + BM < args.m) ? 2 : 1);  // row blocks that hold rows of the matrix
                // Wait until the epilogue has drained the accumulator(s) (passes at once on first use).
                if (!mbar_wait(&ss.tmem_empty[acc], (use & 1) ^ 1)) { ok = false; break; }
                if (MT == 2 && !mbar_wait(&ss.tmem_empty[1], (use & 1) ^ 1)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
                const int iters = (kb_end - kb_begin) * args.num_segments;
                for (int i = 0; i < iters; ++i, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&ss.full[s], ph)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t b_base = smem_u32(&ss.b[s][0]);
                    int halo_r = 0;
                    if constexpr (HALO == 1) {
                        halo_r = (kb_begin + i) % 3;
                        // the lower tap reads the upper tap's copy, one chunk (two image rows) further on
                        if (halo_r == 2) b_base = smem_u32(&ss.b[(it + STAGES - 1) % STAGES][0]) + 32 * BK * 4;
                    }
                    for (int sub = 0; sub < nsub; ++sub) {
                        const uint32_t a_base = smem_u32(&ss.a[s][sub * BM * BK]);
                        const uint32_t d = tmem_d + static_cast<uint32_t>(sub * BN);
#pragma unroll
                        for (int ks = 0; ks < BK / UMMA_K; ++ks) {
                            // K-major: rows of 128 B, 8-row groups 1024 B apart (SBO); a K step of 8 elements is +32 B
                            //          inside the swizzle row.
                            // MN-major: each K index is a 128 B row of 32 consecutive M/N elements; rows come in
                            //          groups of 4 (512 B apart, SBO), 32-element M/N blocks are 32*BK*4 B apart (LBO);
                            //          a K step of 8 is two groups = +1024 B.
                            uint64_t ad = A_MN ? make_smem_desc(a_base + ks * 1024, 32 * BK * 4, 512, 1) : make_smem_desc(a_base + ks * 32, 16, 1024, 2);
                            uint64_t bd = B_MN ? make_smem_desc(b_base + ks * 1024, 32 * BK * 4, 512, 1) : make_smem_desc(b_base + ks * 32, 16, 1024, 2);
                            if constexpr (CTAS == 2) umma_tf32_pair(d, ad, bd, idesc, (i > 0 || ks > 0) ? 1u : 0u);
                            else umma_tf32(d, ad, bd, idesc, (i > 0 || ks > 0) ? 1u : 0u);
                        }
                    }
                    // frees this stage once the MMAs above have read it (the upper tap's stage stays until the lower tap is done)
                    if (HALO == 1 && halo_r == 2) commit(&ss.empty[(it + STAGES - 1) % STAGES]);
                    if (HALO == 0 || halo_r != 1) commit(&ss.empty[s]);
                }
                if (!ok) break;
                commit(&ss.tmem_full[acc]);  // accumulator complete once every MMA above has retired
                if (MT == 2) commit(&ss.tmem_full[1]);
            }
        }
    } else {
        // ---- epilogue warps ---------------------------------------------------------------------
        // A warp may read the TMEM lanes 32*(warp % 4) .. +31 only; the EPW / 4 warps that share a lane group
        // take an equal share of the tile's columns each.
        const int lg = warp & 3;
        const int half = (warp - 2) >> 2;
        constexpr int HALF_N = BN / (EPW / 4);
        float* stage = &ss.stage[warp - 2][0];
        const bool vec_ok = (args.ep.ldd % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.ep.out) & 15) == 0) &&
                            (args.ep.batch_stride_d % 4 == 0) && (args.split_stride_d % 4 == 0);
        const int sw = lane & 7;  // this lane's row (lane) & 7 when writing a staged row
        // Per-row statistics: f32 partial sums per tile, carried in double across the tiles this thread sees of
        // the same row, flushed with two atomics when the row changes and at the end.
        double* const row_stats = args.ep.row_stats;
        double st1 = 0.0, st2 = 0.0;
        int st_row = -1;
        auto flush_stats = [&]() {
            if (st_row >= 0 && st_row < args.m) {
                atomicAdd(row_stats + 2 * st_row, st1);
                atomicAdd(row_stats + 2 * st_row + 1, st2);
            }
            st1 = st2 = 0.0;
        };
        int tile_iter = 0;
        for (int t = first_tile; t < args.total_tiles && ok; t += tile_step, ++tile_iter) {
            int tile_m0, n0, batch, split, kb_begin, kb_end;
            decode(t, tile_m0, n0, batch, split, kb_begin, kb_end);
          if constexpr (CSPLIT) {
            // The partial tile goes to shared memory as it is; the sum over the cluster follows the role branches.
            if (!mbar_wait(&ss.tmem_full[0], 0)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(half * HALF_N) + (static_cast<uint32_t>(lg * 32) << 16);
            float* dst = &ss.a[0][0] + (lg * 32 + lane) * RED_LD + half * HALF_N;
#pragma unroll 1
            for (int c = 0; c < HALF_N; c += 32) {
                uint32_t raw[32];
                tmem_ld32_issue(tmem_d + c, raw);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    *reinterpret_cast<float4*>(dst + c + 4 * i) = make_float4(__uint_as_float(raw[4 * i]), __uint_as_float(raw[4 * i + 1]),
                                                                              __uint_as_float(raw[4 * i + 2]), __uint_as_float(raw[4 * i + 3]));
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          } else if constexpr (MT == 3) {
            // conv_mode 3: the tile's three accumulators (kernel columns 0, 1, 2 at TMEM columns 0, BN, 2 * BN) are read
            // together and combined with a move of one pixel each way; plain stores only (no bias, no statistics).
            if (!mbar_wait(&ss.tmem_full[0], static_cast<uint32_t>(tile_iter) & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int cbase = half * HALF_N;
            const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(cbase) + (static_cast<uint32_t>(lg * 32) << 16);
            float* out_base = args.ep.out + static_cast<int64_t>(batch) * args.ep.batch_stride_d;
            const int wmask = args.conv_w - 1;  // w is a power of two that divides 32
            const bool fast = vec_ok && tile_m0 + lg * 32 + 32 <= args.m && n0 + cbase + HALF_N <= args.n;
#pragma unroll 1
            for (int c = 0; c < HALF_N; c += 32) {
                const int col0 = n0 + cbase + c;
                uint32_t r0[32], r1[32], r2[32];
                tmem_ld32_issue(tmem_d + c, r0);
                tmem_ld32_issue(tmem_d + BN + c, r1);
                tmem_ld32_issue(tmem_d + 2 * BN + c, r2);
                tmem_ld_wait();
                if (c + 32 >= HALF_N) {
                    // Last TMEM read of this warp for the tile: hand the accumulators back before the stores.
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ss.tmem_empty[0]);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float v[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = 4 * i + e, x = j & wmask;  // column c + j starts a chunk-aligned run: its x is j mod w
                        float acc = __uint_as_float(r1[j]);
                        if (j > 0 && x != 0) acc += __uint_as_float(r0[j > 0 ? j - 1 : 0]);
                        if (j < 31 && x != wmask) acc += __uint_as_float(r2[j < 31 ? j + 1 : 31]);
                        v[e] = acc;
                    }
                    *reinterpret_cast<float4*>(stage + lane * 32 + ((i ^ sw) << 2)) = make_float4(v[0], v[1], v[2], v[3]);
                }
                __syncwarp();
                if (col0 < args.n) {
                    const int rsub = lane >> 3, cc = lane & 7;
                    if (fast) {
                        float* p = out_base + static_cast<int64_t>(tile_m0 + lg * 32 + rsub) * args.ep.ldd + col0 + cc * 4;
                        const int64_t step = static_cast<int64_t>(args.ep.ldd) * 4;
#pragma unroll
                        for (int it8 = 0; it8 < 8; ++it8) {
                            const int r = it8 * 4 + rsub;
                            *reinterpret_cast<float4*>(p + it8 * step) = *reinterpret_cast<const float4*>(stage + r * 32 + ((cc ^ (r & 7)) << 2));
                        }
                    } else {
#pragma unroll 1
                        for (int it8 = 0; it8 < 8; ++it8) {
                            const int r = it8 * 4 + rsub;
                            const int grow = tile_m0 + lg * 32 + r, gcol = col0 + cc * 4;
                            if (grow < args.m && gcol < args.n) {
                                const float4 val = *reinterpret_cast<const float4*>(stage + r * 32 + ((cc ^ (r & 7)) << 2));
                                float* p = out_base + static_cast<int64_t>(grow) * args.ep.ldd + gcol;
                                const float e4[4] = {val.x, val.y, val.z, val.w};
                                for (int j = 0; j < 4 && gcol + j < args.n; ++j) p[j] = e4[j];
                            }
                        }
                    }
                }
                __syncwarp();
            }
          } else
          for (int sub = 0; sub < MT && ok; ++sub) {
            const int m0 = tile_m0 + rank * BM + sub * BM;  // this CTA's (this row block's) rows of the tile
            const int acc = MT == 2 ? sub : tile_iter % NACC;
            const uint32_t use = static_cast<uint32_t>(MT == 2 ? tile_iter : tile_iter / NACC);
            if (!mbar_wait(&ss.tmem_full[acc], use & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int cbase = half * HALF_N;
            const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN + cbase) + (static_cast<uint32_t>(lg * 32) << 16);
            const int row = m0 + lg * 32 + lane;
            float* out_base = args.ep.out + static_cast<int64_t>(batch) * args.ep.batch_stride_d + static_cast<int64_t>(split) * args.split_stride_d;
            const float bm = (args.ep.bias_m && row < args.m) ? args.ep.bias_m[row] : 0.f;
            const float* bias_n = args.ep.bias_n;
            const bool relu = args.ep.relu != 0;
            // Whole 32-row x HALF_N-column slab inside the matrix, vector stores possible, plain overwrite.
            const bool fast = vec_ok && !args.ep.accumulate && m0 + lg * 32 + 32 <= args.m && n0 + cbase + HALF_N <= args.n;
            // The loop below is fully unrolled and every TMEM load is issued unconditionally (columns past the
            // matrix edge are allocated accumulator columns, just unused), so the registers of a load in flight
            // are never merged with other values before its wait.
            // Two compiled copies of the tile drain, with and without the row statistics, so that the common case
            // carries none of the statistics' code.
            auto drain = [&](auto stats_tag) {
                constexpr bool STATS = decltype(stats_tag)::value;
                if (STATS && row != st_row) {
                    flush_stats();
                    st_row = row;
                }
                float2 q1[4], q2[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) q1[u] = q2[u] = make_float2(0.f, 0.f);
                const float2 bm2 = make_float2(bm, bm);
                uint32_t raw[32];
                tmem_ld32_issue(tmem_d, raw);
#pragma unroll
                for (int c = 0; c < HALF_N; c += 32) {
                    const int col0 = n0 + cbase + c;
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        // Packed f32x2 arithmetic: one instruction per two values.
                        const float2 rlo = make_float2(__uint_as_float(raw[4 * i]), __uint_as_float(raw[4 * i + 1]));
                        const float2 rhi = make_float2(__uint_as_float(raw[4 * i + 2]), __uint_as_float(raw[4 * i + 3]));
                        float2 lo = __fadd2_rn(rlo, bm2);
                        float2 hi = __fadd2_rn(rhi, bm2);
                        if (bias_n) {
                            const int col = col0 + 4 * i;
                            if (col + 0 < args.n) lo.x += bias_n[col + 0];
                            if (col + 1 < args.n) lo.y += bias_n[col + 1];
                            if (col + 2 < args.n) hi.x += bias_n[col + 2];
                            if (col + 3 < args.n) hi.y += bias_n[col + 3];
                        }
                        if (relu) { lo.x = fmaxf(lo.x, 0.f); lo.y = fmaxf(lo.y, 0.f); hi.x = fmaxf(hi.x, 0.f); hi.y = fmaxf(hi.y, 0.f); }
                        if constexpr (STATS) {
                            const int col = col0 + 4 * i;
                            if (fast || col + 3 < args.n) {
                                // four independent chains each: the adds of one chunk do not wait on one another
                                q1[i & 3] = __fadd2_rn(q1[i & 3], __fadd2_rn(rlo, rhi));
                                q2[i & 3] = __ffma2_rn(rlo, rlo, q2[i & 3]);
                                q2[(i + 2) & 3] = __ffma2_rn(rhi, rhi, q2[(i + 2) & 3]);
                            } else {
                                const float e[4] = {rlo.x, rlo.y, rhi.x, rhi.y};
                                for (int j = 0; j < 4; ++j)
                                    if (col + j < args.n) { q1[0].x += e[j]; q2[0].x += e[j] * e[j]; }
                            }
                        }
                        const float4 r = make_float4(lo.x, lo.y, hi.x, hi.y);
                        *reinterpret_cast<float4*>(stage + lane * 32 + ((i ^ sw) << 2)) = r;
                    }
                    // The registers are free again: fetch the next 32 columns while this slab is stored.
                    if (c + 32 < HALF_N) {
                        tmem_ld32_issue(tmem_d + c + 32, raw);
                    } else {
                        // Last TMEM read of this warp for the tile: hand the accumulator back before the stores.
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            if constexpr (CTAS == 2) mbar_arrive_cluster(map_to_cta(smem_u32(&ss.tmem_empty[acc]), 0));
                            else mbar_arrive(&ss.tmem_empty[acc]);
                        }
                    }
                    __syncwarp();
                    if (col0 >= args.n) continue;  // warp-uniform: nothing of this slab lies inside the matrix
                    // Each store instruction of the warp writes four 128-byte row segments.
                    const int rsub = lane >> 3, cc = lane & 7;
                    if (fast) {
                        float* p = out_base + static_cast<int64_t>(m0 + lg * 32 + rsub) * args.ep.ldd + col0 + cc * 4;
                        const int64_t step = static_cast<int64_t>(args.ep.ldd) * 4;
#pragma unroll
                        for (int it8 = 0; it8 < 8; ++it8) {
                            const int r = it8 * 4 + rsub;
                            *reinterpret_cast<float4*>(p + it8 * step) = *reinterpret_cast<const float4*>(stage + r * 32 + ((cc ^ (r & 7)) << 2));
                        }
                    } else {
#pragma unroll 1
                        for (int it8 = 0; it8 < 8; ++it8) {
                            const int r = it8 * 4 + rsub;
                            const int grow = m0 + lg * 32 + r, gcol = col0 + cc * 4;
                            if (grow < args.m && gcol < args.n) {
                                float4 val = *reinterpret_cast<const float4*>(stage + r * 32 + ((cc ^ (r & 7)) << 2));
                                float* p = out_base + static_cast<int64_t>(grow) * args.ep.ldd + gcol;
                                if (vec_ok && gcol + 4 <= args.n) {
                                    if (args.ep.accumulate) {
                                        float4 o = *reinterpret_cast<const float4*>(p);
                                        val.x += o.x; val.y += o.y; val.z += o.z; val.w += o.w;
                                    }
                                    *reinterpret_cast<float4*>(p) = val;
                                } else {
                                    const float e[4] = {val.x, val.y, val.z, val.w};
                                    for (int j = 0; j < 4 && gcol + j < args.n; ++j) p[j] = args.ep.accumulate ? p[j] + e[j] : e[j];
                                }
                            }
                        }
                    }
                    __syncwarp();
                }
                if constexpr (STATS) {
                    const float2 p1 = __fadd2_rn(__fadd2_rn(q1[0], q1[1]), __fadd2_rn(q1[2], q1[3]));
                    const float2 p2 = __fadd2_rn(__fadd2_rn(q2[0], q2[1]), __fadd2_rn(q2[2], q2[3]));
                    st1 += p1.x + p1.y;
                    st2 += p2.x + p2.y;
                }
            };
            if (row_stats) drain(std::true_type{});
            else drain(std::false_type{});
          }
        }
        if (row_stats) flush_stats();
    }
    if constexpr (CSPLIT) {
        // Every CTA of the cluster has its partial tile in shared memory after this barrier (a CTA whose wait ran out
        // arrives too, with the error flag set below; the tile is then garbage and reported as such).
        __syncthreads();
        cluster_sync_all();
        if (warp >= 2 && static_cast<int>(blockIdx.x) < args.total_tiles) {
            int m0, n0, batch, split, kb_begin, kb_end;
            decode(static_cast<int>(blockIdx.x), m0, n0, batch, split, kb_begin, kb_end);
            const uint32_t red_base = smem_u32(&ss.a[0][0]);
            float* out_base = args.ep.out + static_cast<int64_t>(batch) * args.ep.batch_stride_d;
            const bool vec_ok = (args.ep.ldd % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.ep.out) & 15) == 0) && (args.ep.batch_stride_d % 4 == 0);
            // A thread sums BM * BN / 4 / (32 * EPW) / PARTS groups of four columns, each from PARTS CTAs: sixteen remote
            // loads whatever the cluster size, all issued before the first is used.
            auto reduce = [&](auto parts_tag) {
                constexpr int PARTS = decltype(parts_tag)::value, ROWS = BM / PARTS, ITEMS = ROWS * (BN / 4) / (32 * EPW);
                float4 part[ITEMS][PARTS];
#pragma unroll
                for (int it = 0; it < ITEMS; ++it) {
                    const int idx = static_cast<int>(threadIdx.x) - 64 + it * 32 * EPW;
                    const uint32_t off = red_base + static_cast<uint32_t>(((split * ROWS + idx / (BN / 4)) * RED_LD + 4 * (idx % (BN / 4))) * sizeof(float));
#pragma unroll
                    for (int p = 0; p < PARTS; ++p)
                        asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                     : "=f"(part[it][p].x), "=f"(part[it][p].y), "=f"(part[it][p].z), "=f"(part[it][p].w)
                                     : "r"(map_to_cta(off, static_cast<uint32_t>(p)))
                                     : "memory");
                }
#pragma unroll
                for (int it = 0; it < ITEMS; ++it) {
                    const int idx = static_cast<int>(threadIdx.x) - 64 + it * 32 * EPW;
                    const int row = m0 + split * ROWS + idx / (BN / 4), col = n0 + 4 * (idx % (BN / 4));
                    if (row >= args.m || col >= args.n) continue;
                    float v[4] = {part[it][0].x, part[it][0].y, part[it][0].z, part[it][0].w};
#pragma unroll
                    for (int p = 1; p < PARTS; ++p) { v[0] += part[it][p].x; v[1] += part[it][p].y; v[2] += part[it][p].z; v[3] += part[it][p].w; }
                    const float bm = args.ep.bias_m ? args.ep.bias_m[row] : 0.f;
                    float* dst = out_base + static_cast<int64_t>(row) * args.ep.ldd + col;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        v[j] += bm;
                        if (args.ep.bias_n && col + j < args.n) v[j] += args.ep.bias_n[col + j];
                        if (args.ep.relu) v[j] = fmaxf(v[j], 0.f);
                    }
                    if (vec_ok && col + 4 <= args.n) {
                        float4 o = make_float4(v[0], v[1], v[2], v[3]);
                        if (args.ep.accumulate) {
                            const float4 old = *reinterpret_cast<const float4*>(dst);
                            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                        }
                        *reinterpret_cast<float4*>(dst) = o;
                    } else {
                        for (int j = 0; j < 4 && col + j < args.n; ++j) dst[j] = args.ep.accumulate ? dst[j] + v[j] : v[j];
                    }
                }
            };
            if (args.splits == 8) reduce(std::integral_constant<int, 8>{});
            else if (args.splits == 4) reduce(std::integral_constant<int, 4>{});
            else reduce(std::integral_constant<int, 2>{});
        }
    }
    if (!ok) {
        atomicExch(args.error_flag, 1);
        // Give copies and MMAs that are still in flight time to finish before the CTA retires.
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000) {}
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (CTAS == 2 || CSPLIT != 0) cluster_sync_all();  // no CTA frees TMEM or leaves while a peer may still signal it or read its shared memory
    if (warp == 1) {
        if constexpr (CTAS == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

}  // namespace tc
