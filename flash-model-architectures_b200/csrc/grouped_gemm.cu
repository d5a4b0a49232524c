// Grouped GEMM for the MoE expert MLPs on sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM ->
// fused epilogue. Persistent CTA PAIRS (clusters of two CTAs on two SMs, tcgen05 cta_group::2): a
// pair computes a 256x256 accumulator tile, each CTA holding 128 rows of it in its own TMEM. Per
// 64-deep K block each CTA loads its own 128 rows of A and HALF of the B tile (128 of the 256
// columns); the MMA issued by the leader CTA reads both halves. Against one CTA per 128x256 tile this
// cuts the shared-memory traffic per FLOP by a third, which is what bounds the tensor pipe.
// Warp roles in every CTA:
//   warp 0      TMA producer (one lane issues cp.async.bulk.tensor loads; both CTAs signal the
//               leader's "full" barrier)
//   warp 1      TMEM allocation; in the leader CTA also the MMA issuer (one lane issues
//               tcgen05.mma / tcgen05.commit, committing to the barriers of both CTAs)
//   warps 2..5  epilogue: tcgen05.ld of the fp32 accumulator, fused math, global stores
// Shared memory holds kStages operand stages; TMEM holds two 128x256 fp32 accumulators per CTA so
// the epilogue of tile i overlaps the main loop of tile i+1. No load is multicast.
// A second tile shape, 256x512 per pair (template parameter kWide: two N = 256 MMAs per K step share
// the A tile, one accumulator over all 512 TMEM columns, three 48 KB stages), serves the plain-store
// kernels whose reductions are long enough to make its unhidden epilogue cheap.
//
// Three problem shapes run through the same skeleton:
//   rows NT   C[r, n] = sum_k A[r, k] W[e(r), n, k]    A, W K-major          (forward)
//   rows NN   C[r, n] = sum_k A[r, k] W[e(r), k, n]    A K-major, W N-major  (input gradient)
//   wgrad     dW[e, m, n] = sum_{r in e} X[r, m] Y[r, n]   both operands MN-major, ragged K
//
// Every device-side wait is bounded: when it runs out the kernel records a code in the caller's
// status word, all roles leave their loops, TMEM is released and the kernel returns.
#include <cuda.h>
#include <mutex>

#include "common.cuh"

namespace xma {
namespace gemm {

constexpr int kBlockM = 128;   // accumulator rows per CTA
constexpr int kPairM = 256;    // accumulator rows per CTA pair
constexpr int kBlockN = 256;   // accumulator columns (both CTAs)
constexpr int kHalfN = 128;    // B columns each CTA loads
constexpr int kBlockK = 64;    // 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kStages = 5;
constexpr int kWideStages = 3; // stages of the 256x512 variant (48 KB each)
constexpr int kWideMinK = 4096; // reduction length from which the 256x512 variant is used
constexpr int kWideMinRowsWgrad = 2048; // mean rows per expert from which the weight gradient uses it
constexpr int64_t kWideMinElemsWgrad = int64_t(1) << 23; // or elements of one expert's weight matrix
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kGroupM = 16;    // pair-tiles (256 rows each) swept together so their operands stay in L2

constexpr uint32_t kABytes = kBlockM * kBlockK * 2;  // 16 KB
constexpr uint32_t kBBytes = kHalfN * kBlockK * 2;   // 16 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kChunkBytes = 64 * kBlockK * 2;   // one 64-wide MN-major chunk: 8 KB
constexpr uint32_t kStoreBoxRows = 32;                       // one epilogue warp's rows
constexpr uint32_t kStoreBoxBytes = kStoreBoxRows * 64 * 2;  // 32 rows x 64 columns: 4 KB
constexpr uint32_t kStagingTiles = 3;                        // staging tiles per epilogue warp
constexpr uint32_t kStagingBytes = 4 * kStagingTiles * kStoreBoxBytes;
constexpr uint32_t kBarrierBytes = 256;
constexpr uint32_t kPrefixBytes = (kMaxExperts + 1) * 4;  // per-expert prefix of pair-tiles
// Dynamic shared memory of a kernel variant: operand stages, epilogue staging, alignment slack,
// barriers, the per-expert prefix of pair-tiles.
template <bool kWide>
constexpr uint32_t smem_bytes() {
    return (kWide ? kWideStages * (kABytes + 2 * kBBytes) : kStages * kStageBytes) + kStagingBytes + 1024 +
           kBarrierBytes + kPrefixBytes;
}

constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s
// Upper bound the hardware may keep a polling warp suspended inside one try_wait (it still wakes as
// soon as the phase completes): waiting warps then issue almost nothing.
constexpr uint32_t kTryWaitSuspendNs = 20000;

enum Mode { kRowsNT = 0, kRowsNN = 1, kWgrad = 2 };
// Epilogue that is not part of the public xma_epilogue enum: the router front end (logits, top-k and
// softmax of one token per accumulator row), reached through xma_router_gate_topk only.
constexpr int kEpiRouter = 100;
constexpr int kRouterMaxK = 8;
constexpr int kSelfTestCode = 199;  // status code written by xma_selftest_bounded_wait

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kTryWaitSuspendNs)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait. Returns false when the wait ran out or another role already gave up. kSleepNs > 0
// backs off between polls (roles that can afford ~100 ns of wake-up latency).
template <int kSleepNs = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int32_t* status,
                                          int code, uint64_t limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (kSleepNs > 0) __nanosleep(kSleepNs);
        if ((++spins & 0x3ffu) == 0) {
            if (*abort_flag) return false;
            if (global_timer_ns() - start > limit_ns) {
                *abort_flag = 1;
                if (status != nullptr) atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}

// Bulk tensor stores (shared -> global), tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
// Bulk tensor reduce: global[box] += shared tile (float32 add).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
    asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most kPending of this thread's bulk groups still READ their shared-memory source.
template <int kPending>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format): 128-byte swizzle, 1024-byte aligned tiles.
//   bits  0-13 start address >> 4      bits 16-29 leading byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 descriptor version (1)     bits 61-63 layout (2 = SWIZZLE_128B)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor for kind::f16: fp32 accumulate, A/B both bf16 (format 1) or fp16 (format 0).
//   bits 4-5 D format (1 = f32)  7-9 A format  10-12 B format  15 A major (1 = MN)  16 B major
//   bits 17-22 N >> 3            24-28 M >> 4
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool a_mn_major, bool b_mn_major, int ab_format) {
    return (1u << 4) | (static_cast<uint32_t>(ab_format) << 7) | (static_cast<uint32_t>(ab_format) << 10) |
           (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------
// Kernel parameters and tile schedule
// ---------------------------------------------------------------------------------------------

struct Params {
    const int32_t* padded_offsets;  // [E + 1], multiples of kBlockM
    int num_experts;
    int m_pairs;  // wgrad: ceil(M / 256)
    int n_tiles;
    int64_t n;    // columns of the accumulator problem (N)
    int64_t k;    // reduction length for the rows modes
    int64_t m;    // wgrad: rows of dW per expert
    int64_t cap;  // rows modes: rows of A and C (padded capacity)
    void* c;
    void* aux;
    const int32_t* row_src;
    const void* row_scale;
    float* d_row_scale;
    int32_t* status;
    int ab_format;  // 1 = bf16, 0 = fp16
    int group_m;    // pair-tiles swept together (rasterisation)
    int accumulate; // float32 output: add to C instead of overwriting it
    int single_rows;       // padded_offsets == nullptr: one expert owning rows [0, single_rows) (router mode)
    int64_t rows_valid;    // router mode: tokens (rows at or past it are padding and produce no output)
    int top_k;             // router mode
    int64_t* selected;     // router mode: int64 [T, top_k]
};

// What one CTA does for one work item (a 256 x 256 accumulator tile of the pair).
struct Tile {
    int expert;
    int m0;       // first accumulator row of THIS CTA (rows modes: padded row; wgrad: dW row)
    bool valid;   // false: this CTA only feeds the pair's MMA and stores nothing
    int n_tile;
    int k_begin;  // wgrad: first padded row of the expert
    int num_kb;
};

// First padded row of expert i (i = E: one past the last). Without an offsets array there is a single
// expert that owns rows [0, single_rows).
__device__ __forceinline__ int seg_begin(const Params& p, int i) {
    return p.padded_offsets != nullptr ? p.padded_offsets[i] : (i == 0 ? 0 : p.single_rows);
}

// Rows modes: an expert with t 128-row tiles contributes ceil(t / 2) pair-tiles; `prefix[e]` counts
// the pair-tiles of the experts before e (prefix[E] = all of them). A pair-tile never mixes experts:
// when t is odd the second CTA of the last pair repeats the first CTA's rows and stores nothing.
// Rasterisation: m fastest inside a group of kGroupM pair-tiles, then n, then the next group, so the
// CTA pairs that run at the same time share a few A tiles and a few B tiles through L2.
template <int kMode>
__device__ __forceinline__ Tile get_tile(const Params& p, const int32_t* prefix, int item, uint32_t cta_rank) {
    Tile r;
    int m_items, local = item, expert = 0;
    if (kMode == kWgrad) {
        const int per_expert = p.m_pairs * p.n_tiles;
        expert = item / per_expert;
        local = item - expert * per_expert;
        m_items = p.m_pairs;
    } else {
        m_items = prefix[p.num_experts];
    }
    const int group_span = p.group_m * p.n_tiles;
    const int group = local / group_span;
    const int first_m = group * p.group_m;
    const int rows_in_group = min(p.group_m, m_items - first_m);
    const int in_group = local - group * group_span;
    const int n_tile = in_group / rows_in_group;
    const int m_item = first_m + in_group - n_tile * rows_in_group;
    r.n_tile = n_tile;
    if (kMode == kWgrad) {
        r.expert = expert;
        r.m0 = m_item * kPairM + static_cast<int>(cta_rank) * kBlockM;
        r.valid = r.m0 < p.m;
        r.k_begin = seg_begin(p, expert);
        r.num_kb = (seg_begin(p, expert + 1) - r.k_begin) / kBlockK;
    } else {
        // expert e with prefix[e] <= m_item < prefix[e + 1]
        int lo = 0, hi = p.num_experts - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (prefix[mid] <= m_item) lo = mid; else hi = mid - 1;
        }
        const int begin = seg_begin(p, lo);
        const int tiles = (seg_begin(p, lo + 1) - begin) / kBlockM;
        const int first = 2 * (m_item - prefix[lo]);
        const bool has_second = first + 1 < tiles;
        r.expert = lo;
        r.valid = cta_rank == 0 || has_second;
        r.m0 = begin + (first + ((cta_rank == 1 && has_second) ? 1 : 0)) * kBlockM;
        r.k_begin = 0;
        r.num_kb = static_cast<int>((p.k + kBlockK - 1) / kBlockK);
    }
    return r;
}

__device__ __forceinline__ float sigmoidf_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&v));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
    return __half22float2(*reinterpret_cast<__half2*>(&v));
}

// Load 32 consecutive elements of one row (64 bytes) with a per-8-column bound check.
template <typename T>
__device__ __forceinline__ void load_row32(const T* src, uint32_t (&packed)[16], int64_t col0, int64_t ncols) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (col0 + q * 8 < ncols) v = *reinterpret_cast<const uint4*>(src + q * 8);
        packed[q * 4 + 0] = v.x;
        packed[q * 4 + 1] = v.y;
        packed[q * 4 + 2] = v.z;
        packed[q * 4 + 3] = v.w;
    }
}

// Writes 32 packed columns of this lane's row into half `half` (0/1) of a 32x64 staging tile laid out
// with the 128-byte swizzle a bulk tensor store expects (16-byte chunk index XOR row % 8).
__device__ __forceinline__ void stage_row32(uint32_t tile_addr, int lane, int half, const uint32_t (&packed)[16]) {
    const uint32_t row_addr = tile_addr + static_cast<uint32_t>(lane) * 128;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint32_t dst = row_addr + static_cast<uint32_t>(((half * 4 + q) ^ (lane & 7)) * 16);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[q * 4 + 0]), "r"(packed[q * 4 + 1]),
                     "r"(packed[q * 4 + 2]), "r"(packed[q * 4 + 3])
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The kernel (launched as clusters of two CTAs)
// ---------------------------------------------------------------------------------------------

// kWide: the pair computes a 256 x 512 tile (two N = 256 MMAs per K step that share the A tile: 48 KB of
// operands per stage instead of 2 x 32 KB for the same work) into ONE accumulator that takes all 512
// TMEM columns, so the epilogue does not overlap the next tile's main loop. Used for the plain-store
// rows kernels with long reductions (K >= kWideMinK), where the main loop of a tile is tens of times
// longer than its epilogue: the step is bound by the board power limit, and the operand feed from L2
// is what most of that power goes to.
template <typename T, int kMode, int kEpi, bool kWide = false>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_d,
                    const Params p) {
    constexpr bool kAMn = (kMode == kWgrad);
    constexpr bool kBMn = (kMode != kRowsNT);
    static_assert(!kWide || kEpi == XMA_EPI_STORE, "the wide tile exists for the plain-store kernels");
    constexpr int BN = kWide ? 2 * kBlockN : kBlockN;  // accumulator columns of a tile
    constexpr int SUB = BN / kBlockN;                  // N = 256 MMAs per K step
    constexpr int STAGES = kWide ? kWideStages : kStages;
    constexpr uint32_t STAGE_BYTES = kABytes + SUB * kBBytes;
    constexpr int NBUF = kWide ? 1 : 2;                // accumulators in TMEM

    extern __shared__ uint8_t smem_raw[];
    // Operand tiles need 1024-byte alignment for the 128-byte swizzle. Both CTAs of the pair compute
    // the same offsets, so a shared-memory address means the same object in either CTA.
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t staging_base = smem_base + STAGES * STAGE_BYTES;  // epilogue tiles for TMA stores
    const uint32_t bar_base = staging_base + kStagingBytes;
    const uint32_t full_bar = bar_base;                      // STAGES x 8 B (the leader's are used)
    const uint32_t empty_bar = bar_base + 8 * STAGES;        // STAGES x 8 B
    const uint32_t tmem_full_bar = bar_base + 16 * STAGES;   // 2 x 8 B
    const uint32_t tmem_empty_bar = tmem_full_bar + 16;      // 2 x 8 B (the leader's are used)
    const uint32_t tmem_slot = tmem_empty_bar + 16;          // 4 B
    uint8_t* bar_gen = smem_gen + STAGES * STAGE_BYTES + kStagingBytes;
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(bar_gen + 16 * STAGES + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_gen + 16 * STAGES + 40);
    int32_t* prefix = reinterpret_cast<int32_t*>(bar_gen + kBarrierBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_ctarank();
    const bool leader = cta_rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);   // the leader's arrive.expect_tx; both CTAs' TMA bytes
            mbar_init(empty_bar + 8 * s, 1);  // one tcgen05.commit from the leader
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tmem_full_bar + 8 * b, 1);   // one tcgen05.commit from the leader
            mbar_init(tmem_empty_bar + 8 * b, 8);  // four epilogue warps of each CTA
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        prefetch_tmap(&tmap_c);
        if (kEpi == XMA_EPI_SWIGLU) prefetch_tmap(&tmap_d);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    if (kMode != kWgrad && warp == 2) {
        // prefix[e] = pair-tiles of the experts before e
        int running = 0;
        for (int e0 = 0; e0 < p.num_experts; e0 += 32) {
            const int e = e0 + lane;
            int v = 0;
            if (e < p.num_experts) v = ((seg_begin(p, e + 1) - seg_begin(p, e)) / kBlockM + 1) / 2;
            int incl = v;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, incl, off);
                if (lane >= off) incl += o;
            }
            if (e < p.num_experts) prefix[e + 1] = running + incl;
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) prefix[0] = 0;
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_gen;

    const int num_items = kMode == kWgrad ? p.num_experts * p.m_pairs * p.n_tiles : prefix[p.num_experts] * p.n_tiles;
    const int first_item = blockIdx.x >> 1;
    const int item_stride = gridDim.x >> 1;

    if (warp == 0) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = first_item; ok && t < num_items; t += item_stride) {
            const Tile tile = get_tile<kMode>(p, prefix, t, cta_rank);
            for (int kb = 0; ok && kb < tile.num_kb; ++kb) {
                ok = mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, p.status, 101);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
                    const uint32_t b_dst = a_dst + kABytes;
                    // All bytes of the stage, from both CTAs, complete on the leader's barrier.
                    const uint32_t bar = map_to_cta(full_bar + 8 * stage, 0);
                    if (leader) mbar_expect_tx(full_bar + 8 * stage, 2 * STAGE_BYTES);
                    // B rows (accumulator columns) this CTA loads for the first N = 256 MMA; the second
                    // MMA of a wide tile takes the rows kBlockN further on.
                    const int n_half = tile.n_tile * BN + static_cast<int>(cta_rank) * kHalfN;
                    if (kMode == kWgrad) {
                        const int krow = tile.k_begin + kb * kBlockK;
#pragma unroll
                        for (int c = 0; c < kBlockM / 64; ++c)
                            tma_load_2d(a_dst + c * kChunkBytes, &tmap_a, bar, tile.m0 + 64 * c, krow);
#pragma unroll
                        for (int h = 0; h < SUB; ++h)
#pragma unroll
                            for (int c = 0; c < kHalfN / 64; ++c)
                                tma_load_2d(b_dst + h * kBBytes + c * kChunkBytes, &tmap_b, bar,
                                            n_half + h * kBlockN + 64 * c, krow);
                    } else {
                        const int kcol = kb * kBlockK;
                        tma_load_2d(a_dst, &tmap_a, bar, kcol, tile.m0);
                        if (kMode == kRowsNT) {
                            if (kEpi == XMA_EPI_SWIGLU) {
                                // accumulator columns [0,128) = up rows [j0, j0+128) of W[e] (leader's half),
                                // columns [128,256) = gate rows [I+j0, I+j0+128) (the peer's half)
                                const int half = static_cast<int>(p.n / 2);
                                const int j0 = tile.n_tile * kHalfN;
                                tma_load_3d(b_dst, &tmap_b, bar, kcol, (leader ? 0 : half) + j0, tile.expert);
                            } else {
#pragma unroll
                                for (int h = 0; h < SUB; ++h)
                                    tma_load_3d(b_dst + h * kBBytes, &tmap_b, bar, kcol, n_half + h * kBlockN, tile.expert);
                            }
                        } else {
#pragma unroll
                            for (int h = 0; h < SUB; ++h)
#pragma unroll
                                for (int c = 0; c < kHalfN / 64; ++c)
                                    tma_load_3d(b_dst + h * kBBytes + c * kChunkBytes, &tmap_b, bar,
                                                n_half + h * kBlockN + 64 * c, kcol, tile.expert);
                        }
                    }
                }
                __syncwarp();
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1 && leader) {
        // ------------------------------ MMA issuer (leader CTA only) ------------------------------
        const uint32_t idesc = make_idesc(kPairM, kBlockN, kAMn, kBMn, p.ab_format);
        int stage = 0;
        uint32_t phase = 0;
        int local = 0;
        bool ok = true;
        for (int t = first_item; ok && t < num_items; t += item_stride, ++local) {
            const Tile tile = get_tile<kMode>(p, prefix, t, cta_rank);
            const int buf = local % NBUF;
            const uint32_t buf_phase = (local / NBUF) & 1u;
            ok = mbar_wait(tmem_empty_bar + 8 * buf, buf_phase ^ 1u, abort_flag, p.status, 102);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tmem_d = tmem_base + buf * kBlockN;
            for (int kb = 0; ok && kb < tile.num_kb; ++kb) {
                ok = mbar_wait(full_bar + 8 * stage, phase, abort_flag, p.status, 103);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
                    const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
                    for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
                        // K-major: 32 bytes per 16-element K step inside the swizzle row.
                        // MN-major: 16 K rows of 128 bytes per step; chunks of 64 MN elements are kChunkBytes apart.
                        const uint64_t adesc = kAMn ? make_smem_desc(a_addr + kk * 2048, kChunkBytes, 1024)
                                                    : make_smem_desc(a_addr + kk * 32, 0, 1024);
#pragma unroll
                        for (int h = 0; h < SUB; ++h) {
                            const uint32_t bh = b_addr + h * kBBytes;
                            const uint64_t bdesc = kBMn ? make_smem_desc(bh + kk * 2048, kChunkBytes, 1024)
                                                        : make_smem_desc(bh + kk * 32, 0, 1024);
                            umma_bf16(tmem_d + h * kBlockN, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
                        }
                    }
                    // Free the stage in both CTAs when these MMAs retire.
                    umma_commit(empty_bar + 8 * stage);
                    umma_commit(map_to_cta(empty_bar + 8 * stage, 1));
                }
                __syncwarp();
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            if (ok && lane == 0) {
                umma_commit(tmem_full_bar + 8 * buf);
                umma_commit(map_to_cta(tmem_full_bar + 8 * buf, 1));
            }
            __syncwarp();
        }
    } else if (warp >= 2) {
        // ------------------------------ epilogue (both CTAs) ------------------------------
        const int quarter = warp & 3;  // TMEM lanes this warp may read: [32*quarter, 32*quarter+32)
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t leader_tmem_empty = map_to_cta(tmem_empty_bar, 0);
        int local = 0;
        bool ok = true;
        for (int t = first_item; ok && t < num_items; t += item_stride, ++local) {
            const Tile tile = get_tile<kMode>(p, prefix, t, cta_rank);
            const int buf = local % NBUF;
            const uint32_t buf_phase = (local / NBUF) & 1u;
            const int64_t row = tile.m0 + row_in_tile;
            // swiglu backward reads the saved pre-activation: fetch the first 32 columns of this
            // thread's row while the tile's MMAs are still running.
            uint32_t pu[16], pg[16];
            if (kEpi == XMA_EPI_SWIGLU_BWD && tile.valid) {
                const int64_t n0 = static_cast<int64_t>(tile.n_tile) * kBlockN;
                const T* pre_row = static_cast<const T*>(p.aux) + row * (2 * p.n);
                load_row32<T>(pre_row + n0, pu, n0, p.n);
                load_row32<T>(pre_row + p.n + n0, pg, n0, p.n);
            }
            ok = mbar_wait(tmem_full_bar + 8 * buf, buf_phase, abort_flag, p.status, 104);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + buf * kBlockN + (static_cast<uint32_t>(quarter * 32) << 16);

            if (!tile.valid) {
                // nothing to store: this CTA only supplied operands
            } else if (kEpi == XMA_EPI_STORE) {
                const int64_t ncols = p.n;
                const int64_t col_base = static_cast<int64_t>(tile.n_tile) * BN;
                if (tile.num_kb == 0) {
                    // An expert without rows (weight gradient only): the tile is zeros. One warp
                    // instruction writes one 512-byte row segment, fully coalesced.
#pragma unroll
                    for (int h = 0; h < SUB; ++h) {
                        const int64_t col = col_base + h * kBlockN + lane * 8;
                        T* base = static_cast<T*>(p.c) + (static_cast<int64_t>(tile.expert) * p.m + tile.m0 + quarter * 32) * p.n + col;
                        if (col < ncols) {
                            for (int r = 0; r < 32; ++r)
                                if (tile.m0 + quarter * 32 + r < p.m) *reinterpret_cast<uint4*>(base + r * p.n) = make_uint4(0, 0, 0, 0);
                        }
                    }
                } else {
                    // 64 columns at a time: TMEM -> registers -> this warp's 32x64 staging tile
                    // (128-byte swizzle, so the 32 row writes of one instruction spread over all
                    // banks) -> one bulk tensor store. The store clips rows and columns that fall
                    // outside the output, so tails need no predicates. Two staging tiles per warp:
                    // a tile is rewritten only after the store issued from it has read it.
                    const uint32_t my_staging = staging_base + static_cast<uint32_t>(warp - 2) * kStagingTiles * kStoreBoxBytes;
                    const int row0 = tile.m0 + quarter * 32;
#pragma unroll 1
                    for (int ch = 0; ch < BN / 64; ++ch) {
                        const int64_t col0 = col_base + ch * 64;
                        if (col0 >= ncols) break;  // warp-uniform
                        uint32_t lo[32], hi[32];
                        tmem_ld32(taddr + ch * 64, lo);
                        tmem_ld32(taddr + ch * 64 + 32, hi);
                        const uint32_t buf_addr = my_staging + static_cast<uint32_t>(ch & 1) * kStoreBoxBytes;
                        if (lane == 0) bulk_wait_read<1>();  // the store that last used this tile is done with it
                        __syncwarp();
                        tmem_ld_wait();
                        const uint32_t row_addr = buf_addr + static_cast<uint32_t>(lane) * 128;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const uint32_t* src = c < 4 ? &lo[c * 8] : &hi[(c - 4) * 8];
                            const uint32_t v0 = pack2<T>(__uint_as_float(src[0]), __uint_as_float(src[1]));
                            const uint32_t v1 = pack2<T>(__uint_as_float(src[2]), __uint_as_float(src[3]));
                            const uint32_t v2 = pack2<T>(__uint_as_float(src[4]), __uint_as_float(src[5]));
                            const uint32_t v3 = pack2<T>(__uint_as_float(src[6]), __uint_as_float(src[7]));
                            const uint32_t dst = row_addr + static_cast<uint32_t>((c ^ (lane & 7)) * 16);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v0), "r"(v1), "r"(v2), "r"(v3)
                                         : "memory");
                        }
                        fence_proxy_async();  // the generic-proxy writes above become visible to the bulk store
                        __syncwarp();
                        if (lane == 0) {
                            if (kMode == kWgrad)
                                tma_store_3d(&tmap_c, buf_addr, static_cast<int>(col0), row0, tile.expert);
                            else
                                tma_store_2d(&tmap_c, buf_addr, static_cast<int>(col0), row0);
                            bulk_commit();
                        }
                    }
                }
            } else if (kEpi == XMA_EPI_STORE_F32) {
                // float32 output: one 32-column TMEM load fills one 128-byte row of a 32x32 float32
                // staging tile; the bulk store (or reduce-add) clips at the edges of the output.
                const int64_t ncols = p.n;
                const int64_t col_base = static_cast<int64_t>(tile.n_tile) * kBlockN;
                if (tile.num_kb == 0) {
                    // An expert without rows (weight gradient only): zeros, unless accumulating.
                    if (!p.accumulate) {
                        float* base = static_cast<float*>(p.c) +
                                      (static_cast<int64_t>(tile.expert) * p.m + tile.m0 + quarter * 32) * p.n;
                        for (int part = 0; part < 2; ++part) {
                            const int64_t col = col_base + part * 128 + lane * 4;
                            if (col < ncols) {
                                for (int r = 0; r < 32; ++r)
                                    if (tile.m0 + quarter * 32 + r < p.m)
                                        *reinterpret_cast<float4*>(base + r * p.n + col) = make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                        }
                    }
                } else {
                    const uint32_t my_staging = staging_base + static_cast<uint32_t>(warp - 2) * kStagingTiles * kStoreBoxBytes;
                    const int row0 = tile.m0 + quarter * 32;
#pragma unroll 1
                    for (int ch = 0; ch < kBlockN / 32; ++ch) {
                        const int64_t col0 = col_base + ch * 32;
                        if (col0 >= ncols) break;  // warp-uniform
                        uint32_t acc[32];
                        tmem_ld32(taddr + ch * 32, acc);
                        const uint32_t buf_addr = my_staging + static_cast<uint32_t>(ch & 1) * kStoreBoxBytes;
                        if (lane == 0) bulk_wait_read<1>();  // the store that last used this tile is done with it
                        __syncwarp();
                        tmem_ld_wait();
                        const uint32_t row_addr = buf_addr + static_cast<uint32_t>(lane) * 128;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            const uint32_t dst = row_addr + static_cast<uint32_t>((c ^ (lane & 7)) * 16);
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(acc[c * 4]),
                                         "r"(acc[c * 4 + 1]), "r"(acc[c * 4 + 2]), "r"(acc[c * 4 + 3])
                                         : "memory");
                        }
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            if (kMode == kWgrad) {
                                if (p.accumulate)
                                    tma_reduce_add_3d(&tmap_c, buf_addr, static_cast<int>(col0), row0, tile.expert);
                                else
                                    tma_store_3d(&tmap_c, buf_addr, static_cast<int>(col0), row0, tile.expert);
                            } else {
                                if (p.accumulate)
                                    tma_reduce_add_2d(&tmap_c, buf_addr, static_cast<int>(col0), row0);
                                else
                                    tma_store_2d(&tmap_c, buf_addr, static_cast<int>(col0), row0);
                            }
                            bulk_commit();
                        }
                    }
                }
            } else if (kEpi == kEpiRouter) {
                // acc row = the logits of one token over all E <= 256 experts (one n tile). The logits
                // are rounded to the storage type and leave through bulk stores as in EPI_STORE; the
                // same rounded values feed a running top-8 list (descending, a later expert passes an
                // earlier one only when strictly greater: ties go to the lowest expert id, like
                // router_topk_softmax_kernel), then the softmax over the first top_k entries.
                const int num_e = static_cast<int>(p.n);
                const uint32_t my_staging = staging_base + static_cast<uint32_t>(warp - 2) * kStagingTiles * kStoreBoxBytes;
                const int row0 = tile.m0 + quarter * 32;
                float best_v[kRouterMaxK];
                int best_e[kRouterMaxK];
#pragma unroll
                for (int j = 0; j < kRouterMaxK; ++j) {
                    best_v[j] = -INFINITY;
                    best_e[j] = 0;
                }
#pragma unroll 1
                for (int ch = 0; ch < kBlockN / 64; ++ch) {
                    const int col0 = ch * 64;
                    if (col0 >= num_e) break;  // warp-uniform
                    uint32_t lo[32], hi[32];
                    tmem_ld32(taddr + ch * 64, lo);
                    tmem_ld32(taddr + ch * 64 + 32, hi);
                    const uint32_t buf_addr = my_staging + static_cast<uint32_t>(ch & 1) * kStoreBoxBytes;
                    if (lane == 0) bulk_wait_read<1>();
                    __syncwarp();
                    tmem_ld_wait();
                    const uint32_t row_addr = buf_addr + static_cast<uint32_t>(lane) * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const uint32_t* src = c < 4 ? &lo[c * 8] : &hi[(c - 4) * 8];
                        uint32_t v[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            v[q] = pack2<T>(__uint_as_float(src[2 * q]), __uint_as_float(src[2 * q + 1]));
                            const float2 f = unpack2<T>(v[q]);
                            const int e0 = col0 + c * 8 + 2 * q;
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const float val = h == 0 ? f.x : f.y;
                                const int e = e0 + h;
                                if (e < num_e && val > best_v[kRouterMaxK - 1]) {
                                    best_v[kRouterMaxK - 1] = val;
                                    best_e[kRouterMaxK - 1] = e;
#pragma unroll
                                    for (int sft = kRouterMaxK - 1; sft > 0; --sft) {
                                        if (best_v[sft] > best_v[sft - 1]) {
                                            const float tv = best_v[sft];
                                            best_v[sft] = best_v[sft - 1];
                                            best_v[sft - 1] = tv;
                                            const int te = best_e[sft];
                                            best_e[sft] = best_e[sft - 1];
                                            best_e[sft - 1] = te;
                                        }
                                    }
                                }
                            }
                        }
                        const uint32_t dst = row_addr + static_cast<uint32_t>((c ^ (lane & 7)) * 16);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3])
                                     : "memory");
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tmap_c, buf_addr, col0, row0);  // clips columns >= E and rows >= T
                        bulk_commit();
                    }
                }
                if (row < p.rows_valid) {
                    // softmax over the first top_k entries in float32; the sum is taken in the order of
                    // the warp butterfly of router_topk_softmax_kernel so both kernels agree bit for bit.
                    float ex[kRouterMaxK];
#pragma unroll
                    for (int j = 0; j < kRouterMaxK; ++j) ex[j] = j < p.top_k ? expf(best_v[j] - best_v[0]) : 0.f;
                    const float sum = ((ex[0] + ex[4]) + (ex[2] + ex[6])) + ((ex[1] + ex[5]) + (ex[3] + ex[7]));
                    T* w_out = static_cast<T*>(p.aux) + row * p.top_k;
                    float* p_out = p.d_row_scale + row * p.top_k;
                    int64_t* s_out = p.selected + row * p.top_k;
#pragma unroll
                    for (int j = 0; j < kRouterMaxK; ++j) {
                        if (j < p.top_k) {
                            const float prob = ex[j] / sum;
                            w_out[j] = Elem<T>::from_float(prob);
                            p_out[j] = prob;
                            s_out[j] = best_e[j];
                        }
                    }
                }
            } else if (kEpi == XMA_EPI_SWIGLU) {
                // acc columns [0,128) = up, [128,256) = gate, for activation columns j0 .. j0+127.
                const int64_t j0 = static_cast<int64_t>(tile.n_tile) * kHalfN;
                float scale = 1.f;
                if (p.row_scale != nullptr) {
                    const int32_t flat = p.row_src[row];
                    scale = flat >= 0 ? Elem<T>::to_float(static_cast<const T*>(p.row_scale)[flat]) : 0.f;
                }
                // Three staging tiles per warp: up and gate pre-activations and the activation, 64
                // columns each, leave through bulk tensor stores (tmap_c views the pre-activation as
                // [row][up|gate][column], tmap_d is the activation).
                const uint32_t t_up = staging_base + static_cast<uint32_t>(warp - 2) * kStagingTiles * kStoreBoxBytes;
                const uint32_t t_gate = t_up + kStoreBoxBytes, t_act = t_gate + kStoreBoxBytes;
                const int row0 = tile.m0 + quarter * 32;
#pragma unroll 1
                for (int grp = 0; grp < kHalfN / 64; ++grp) {
                    if (lane == 0) bulk_wait_read<0>();  // the previous group's stores have read the tiles
                    __syncwarp();
#pragma unroll 1
                    for (int sub = 0; sub < 2; ++sub) {
                        const int ch = grp * 2 + sub;
                        uint32_t up[32], gate[32];
                        tmem_ld32(taddr + ch * 32, up);
                        tmem_ld32(taddr + kHalfN + ch * 32, gate);
                        tmem_ld_wait();
                        uint32_t pu[16], pg[16], ph[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            // Round the pre-activation to the storage type first, as the reference does
                            // between the up projection and the activation.
                            pu[j] = pack2<T>(__uint_as_float(up[2 * j]), __uint_as_float(up[2 * j + 1]));
                            pg[j] = pack2<T>(__uint_as_float(gate[2 * j]), __uint_as_float(gate[2 * j + 1]));
                            const float2 u = unpack2<T>(pu[j]);
                            const float2 g = unpack2<T>(pg[j]);
                            const float h0 = u.x * g.x * sigmoidf_fast(g.x);
                            const float h1 = u.y * g.y * sigmoidf_fast(g.y);
                            ph[j] = pack2<T>(scale * h0, scale * h1);
                        }
                        stage_row32(t_up, lane, sub, pu);
                        stage_row32(t_gate, lane, sub, pg);
                        stage_row32(t_act, lane, sub, ph);
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        const int col0 = static_cast<int>(j0) + grp * 64;
                        tma_store_3d(&tmap_c, t_up, col0, 0, row0);
                        tma_store_3d(&tmap_c, t_gate, col0, 1, row0);
                        tma_store_2d(&tmap_d, t_act, col0, row0);
                        bulk_commit();
                    }
                }
            } else {
                // XMA_EPI_SWIGLU_BWD: acc = dY W2 (unscaled) for activation columns [n0, n0+256).
                const int64_t inter = p.n;
                const int64_t n0 = static_cast<int64_t>(tile.n_tile) * kBlockN;
                const T* pre_row = static_cast<const T*>(p.aux) + row * (2 * inter);
                const uint32_t t_du = staging_base + static_cast<uint32_t>(warp - 2) * kStagingTiles * kStoreBoxBytes;
                const uint32_t t_dg = t_du + kStoreBoxBytes;
                const int row0 = tile.m0 + quarter * 32;
                int32_t flat = -1;
                float scale = 1.f;
                if (p.row_src != nullptr) flat = p.row_src[row];
                if (p.row_scale != nullptr) scale = flat >= 0 ? Elem<T>::to_float(static_cast<const T*>(p.row_scale)[flat]) : 0.f;
                float dscale = 0.f;
#pragma unroll 1
                for (int ch = 0; ch < kBlockN / 32; ++ch) {
                    const int64_t col0 = n0 + ch * 32;
                    if (col0 >= inter) break;  // warp-uniform
                    uint32_t acc[32];
                    tmem_ld32(taddr + ch * 32, acc);
                    if ((ch & 1) == 0) {  // a new 64-column group: its two staging tiles must be free
                        if (lane == 0) bulk_wait_read<0>();
                        __syncwarp();
                    }
                    // Next chunk's pre-activation is requested before this chunk's math (the loads
                    // are predicated off past the last column).
                    uint32_t nu[16], ng[16];
                    load_row32<T>(pre_row + col0 + 32, nu, ch + 1 < kBlockN / 32 ? col0 + 32 : inter, inter);
                    load_row32<T>(pre_row + inter + col0 + 32, ng, ch + 1 < kBlockN / 32 ? col0 + 32 : inter, inter);
                    tmem_ld_wait();
                    uint32_t du[16], dg[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float2 u = unpack2<T>(pu[j]);
                        const float2 g = unpack2<T>(pg[j]);
                        const float a0 = __uint_as_float(acc[2 * j]), a1 = __uint_as_float(acc[2 * j + 1]);
                        const float s0 = sigmoidf_fast(g.x), s1 = sigmoidf_fast(g.y);
                        const float silu0 = g.x * s0, silu1 = g.y * s1;
                        dscale = fmaf(a0, u.x * silu0, dscale);
                        dscale = fmaf(a1, u.y * silu1, dscale);
                        const float dh0 = scale * a0, dh1 = scale * a1;
                        du[j] = pack2<T>(dh0 * silu0, dh1 * silu1);
                        dg[j] = pack2<T>(dh0 * u.x * (s0 + silu0 * (1.f - s0)), dh1 * u.y * (s1 + silu1 * (1.f - s1)));
                    }
                    stage_row32(t_du, lane, ch & 1, du);
                    stage_row32(t_dg, lane, ch & 1, dg);
                    if ((ch & 1) == 1 || col0 + 32 >= inter) {
                        // d(pre-activation) is viewed as [row][up|gate][column]: the stores clip at
                        // `inter`, so a group that straddles the last column writes only valid ones.
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) {
                            const int gcol = static_cast<int>(n0) + (ch >> 1) * 64;
                            tma_store_3d(&tmap_c, t_du, gcol, 0, row0);
                            tma_store_3d(&tmap_c, t_dg, gcol, 1, row0);
                            bulk_commit();
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        pu[j] = nu[j];
                        pg[j] = ng[j];
                    }
                }
                // One partial per row and n tile, summed in tile order by reduce_row_partials_kernel:
                // the router-weight gradient does not depend on the order the tiles finish in.
                if (p.d_row_scale != nullptr) p.d_row_scale[static_cast<int64_t>(tile.n_tile) * p.cap + row] = dscale;
            }

            // Hand the accumulator buffer back to the leader's MMA issuer.
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_tmem_empty + 8 * buf);
        }
    }

    if (warp >= 2 && lane == 0) bulk_wait_read<0>();
    // Neither CTA may leave while its peer can still signal its barriers or read its shared memory.
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// rank-2 or rank-3 tiled map, 128-byte swizzle, zero fill out of bounds. dims/box are innermost first.
static bool make_tmap(CUtensorMap* map, int dtype, const void* base, int rank, const uint64_t* dims,
                      const uint64_t* strides_bytes /*rank-1 entries*/, const uint32_t* box) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t gdims[3];
    cuuint64_t gstrides[2];
    cuuint32_t gbox[3];
    cuuint32_t estr[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
    }
    for (int i = 0; i < rank - 1; ++i) gstrides[i] = strides_bytes[i];
    const CUtensorMapDataType dt = dtype == kDtypeBF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                   : dtype == kDtypeF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                        : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const CUresult r = fn(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides, gbox, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Clusters of two CTAs that can be resident at once for this kernel on the current device. One
// instantiation (and one cache) per kernel instantiation: the shared-memory attribute is per kernel.
template <typename T, int kMode, int kEpi, bool kWide = false>
static int resident_pairs() {
    auto kernel = grouped_gemm_kernel<T, kMode, kEpi, kWide>;
    constexpr uint32_t kSmemBytes = smem_bytes<kWide>();
    constexpr int kMaxDevices = 64;
    static int cached[kMaxDevices];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes)) !=
            cudaSuccess) {
            cudaGetLastError();
            return -1;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(sm_count() & ~1), 1, 1);
        cfg.blockDim = dim3(kThreads, 1, 1);
        cfg.dynamicSmemBytes = kSmemBytes;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters <= 0) {
            cudaGetLastError();
            clusters = sm_count() / 2;
        }
        cached[dev] = clusters;
    }
    return cached[dev];
}

template <typename T, int kMode, int kEpi, bool kWide = false>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& td,
                  const Params& p, int64_t max_items, cudaStream_t stream) {
    auto kernel = grouped_gemm_kernel<T, kMode, kEpi, kWide>;
    constexpr uint32_t kSmemBytes = smem_bytes<kWide>();
    int64_t pairs = resident_pairs<T, kMode, kEpi, kWide>();
    if (pairs <= 0) return XMA_ERR_LAUNCH;
    if (pairs > max_items) pairs = max_items;
    if (pairs < 1) pairs = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kernel, ta, tb, tc, td, p) != cudaSuccess) {
        cudaGetLastError();
        return XMA_ERR_LAUNCH;
    }
    return launch_status();
}

template <typename T>
static int run_rows(int layout, int epilogue, int dtype, const void* a, const void* w, const int32_t* padded_offsets,
                    int64_t cap, int num_experts, int64_t n, int64_t k, void* c, void* aux, const int32_t* row_src,
                    const void* row_scale, float* d_row_scale, int32_t* status, cudaStream_t stream) {
    CUtensorMap ta, tb;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(k), static_cast<uint64_t>(cap)};
        const uint64_t strides[1] = {static_cast<uint64_t>(k) * 2};
        const uint32_t box[2] = {kBlockK, kBlockM};
        if (!make_tmap(&ta, dtype, a, 2, dims, strides, box)) return XMA_ERR_DRIVER;
    }
    if (layout == XMA_GEMM_NT) {
        const uint64_t dims[3] = {static_cast<uint64_t>(k), static_cast<uint64_t>(n), static_cast<uint64_t>(num_experts)};
        const uint64_t strides[2] = {static_cast<uint64_t>(k) * 2, static_cast<uint64_t>(n) * static_cast<uint64_t>(k) * 2};
        const uint32_t box[3] = {kBlockK, kHalfN, 1};
        if (!make_tmap(&tb, dtype, w, 3, dims, strides, box)) return XMA_ERR_DRIVER;
    } else {
        const uint64_t dims[3] = {static_cast<uint64_t>(n), static_cast<uint64_t>(k), static_cast<uint64_t>(num_experts)};
        const uint64_t strides[2] = {static_cast<uint64_t>(n) * 2, static_cast<uint64_t>(n) * static_cast<uint64_t>(k) * 2};
        const uint32_t box[3] = {64, kBlockK, 1};
        if (!make_tmap(&tb, dtype, w, 3, dims, strides, box)) return XMA_ERR_DRIVER;
    }
    // Output maps for the epilogue's bulk stores (boxes of 64 columns x 32 rows).
    CUtensorMap tc, td = ta;
    const bool out_f32 = epilogue == XMA_EPI_STORE_F32 || epilogue == XMA_EPI_ADD_F32;
    if (out_f32) {
        const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(cap)};
        const uint64_t strides[1] = {static_cast<uint64_t>(n) * 4};
        const uint32_t box[2] = {32, kStoreBoxRows};
        if (!make_tmap(&tc, kDtypeF32, c, 2, dims, strides, box)) return XMA_ERR_DRIVER;
    } else if (epilogue == XMA_EPI_STORE) {
        const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(cap)};
        const uint64_t strides[1] = {static_cast<uint64_t>(n) * 2};
        const uint32_t box[2] = {64, kStoreBoxRows};
        if (!make_tmap(&tc, dtype, c, 2, dims, strides, box)) return XMA_ERR_DRIVER;
    } else {
        // pre-activation / its gradient [cap, 2*half] viewed as [cap][2][half]
        const uint64_t half = static_cast<uint64_t>(epilogue == XMA_EPI_SWIGLU ? n / 2 : n);
        const uint64_t dims[3] = {half, 2, static_cast<uint64_t>(cap)};
        const uint64_t strides[2] = {half * 2, half * 4};
        const uint32_t box[3] = {64, 1, kStoreBoxRows};
        if (!make_tmap(&tc, dtype, c, 3, dims, strides, box)) return XMA_ERR_DRIVER;
        if (epilogue == XMA_EPI_SWIGLU) {
            const uint64_t adims[2] = {half, static_cast<uint64_t>(cap)};
            const uint64_t astrides[1] = {half * 2};
            const uint32_t abox[2] = {64, kStoreBoxRows};
            if (!make_tmap(&td, dtype, aux, 2, adims, astrides, abox)) return XMA_ERR_DRIVER;
        }
    }
    Params p{};
    p.padded_offsets = padded_offsets;
    p.num_experts = num_experts;
    p.n = n;
    p.k = k;
    p.cap = cap;
    p.c = c;
    p.aux = aux;
    p.row_src = row_src;
    p.row_scale = row_scale;
    p.d_row_scale = d_row_scale;
    p.status = status;
    p.ab_format = dtype == kDtypeBF16 ? 1 : 0;
    p.accumulate = epilogue == XMA_EPI_ADD_F32 ? 1 : 0;
    p.group_m = kGroupM;
    // Long reductions with a plain store take the 256 x 512 tile (see the kernel's comment).
    const bool wide = epilogue == XMA_EPI_STORE && k >= kWideMinK && n >= 2 * kBlockN;
    p.n_tiles = static_cast<int>(epilogue == XMA_EPI_SWIGLU ? ceil_div(n / 2, kHalfN)
                                                           : ceil_div(n, wide ? 2 * kBlockN : kBlockN));
    const int64_t max_items = (cap / kBlockM) * p.n_tiles;
    if (out_f32) {
        if (layout == XMA_GEMM_NT) return launch<T, kRowsNT, XMA_EPI_STORE_F32>(ta, tb, tc, td, p, max_items, stream);
        return launch<T, kRowsNN, XMA_EPI_STORE_F32>(ta, tb, tc, td, p, max_items, stream);
    }
    if (wide) {
        if (layout == XMA_GEMM_NT) return launch<T, kRowsNT, XMA_EPI_STORE, true>(ta, tb, tc, td, p, max_items, stream);
        return launch<T, kRowsNN, XMA_EPI_STORE, true>(ta, tb, tc, td, p, max_items, stream);
    }
    if (layout == XMA_GEMM_NT) {
        if (epilogue == XMA_EPI_STORE) return launch<T, kRowsNT, XMA_EPI_STORE>(ta, tb, tc, td, p, max_items, stream);
        if (epilogue == XMA_EPI_SWIGLU) return launch<T, kRowsNT, XMA_EPI_SWIGLU>(ta, tb, tc, td, p, max_items, stream);
    } else {
        if (epilogue == XMA_EPI_STORE) return launch<T, kRowsNN, XMA_EPI_STORE>(ta, tb, tc, td, p, max_items, stream);
        if (epilogue == XMA_EPI_SWIGLU_BWD) return launch<T, kRowsNN, XMA_EPI_SWIGLU_BWD>(ta, tb, tc, td, p, max_items, stream);
    }
    return XMA_ERR_UNSUPPORTED;
}

// Router front end: logits = x @ w_gate^T (one "expert" owning every token row), top-k and softmax in
// the epilogue.
template <typename T>
static int run_router(int dtype, const void* x, const void* w_gate, int64_t num_tokens, int64_t hidden, int num_experts,
                      int top_k, void* logits, void* topk_weights, float* topk_probs, int64_t* selected,
                      int32_t* status, cudaStream_t stream) {
    CUtensorMap ta, tb, tc;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(hidden), static_cast<uint64_t>(num_tokens)};
        const uint64_t strides[1] = {static_cast<uint64_t>(hidden) * 2};
        const uint32_t box[2] = {kBlockK, kBlockM};
        if (!make_tmap(&ta, dtype, x, 2, dims, strides, box)) return XMA_ERR_DRIVER;
    }
    {
        const uint64_t dims[3] = {static_cast<uint64_t>(hidden), static_cast<uint64_t>(num_experts), 1};
        const uint64_t strides[2] = {static_cast<uint64_t>(hidden) * 2,
                                     static_cast<uint64_t>(num_experts) * static_cast<uint64_t>(hidden) * 2};
        const uint32_t box[3] = {kBlockK, kHalfN, 1};
        if (!make_tmap(&tb, dtype, w_gate, 3, dims, strides, box)) return XMA_ERR_DRIVER;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(num_experts), static_cast<uint64_t>(num_tokens)};
        const uint64_t strides[1] = {static_cast<uint64_t>(num_experts) * 2};
        const uint32_t box[2] = {64, kStoreBoxRows};
        if (!make_tmap(&tc, dtype, logits, 2, dims, strides, box)) return XMA_ERR_DRIVER;
    }
    Params p{};
    p.padded_offsets = nullptr;
    p.num_experts = 1;
    p.single_rows = static_cast<int>(ceil_div(num_tokens, kBlockM) * kBlockM);
    p.rows_valid = num_tokens;
    p.n = num_experts;
    p.k = hidden;
    p.n_tiles = 1;
    p.c = logits;
    p.aux = topk_weights;
    p.d_row_scale = topk_probs;
    p.selected = selected;
    p.top_k = top_k;
    p.status = status;
    p.ab_format = dtype == kDtypeBF16 ? 1 : 0;
    p.group_m = kGroupM;
    return launch<T, kRowsNT, kEpiRouter>(ta, tb, tc, ta, p, ceil_div(p.single_rows / kBlockM, 2), stream);
}

template <typename T>
static int run_wgrad(int dtype, const void* x, const void* y, const int32_t* padded_offsets, int64_t cap, int num_experts,
                     int64_t m, int64_t n, void* dw, bool out_f32, bool accumulate, int32_t* status, cudaStream_t stream) {
    CUtensorMap ta, tb;
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(m), static_cast<uint64_t>(cap)};
        const uint64_t strides[1] = {static_cast<uint64_t>(m) * 2};
        const uint32_t box[2] = {64, kBlockK};
        if (!make_tmap(&ta, dtype, x, 2, dims, strides, box)) return XMA_ERR_DRIVER;
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(n), static_cast<uint64_t>(cap)};
        const uint64_t strides[1] = {static_cast<uint64_t>(n) * 2};
        const uint32_t box[2] = {64, kBlockK};
        if (!make_tmap(&tb, dtype, y, 2, dims, strides, box)) return XMA_ERR_DRIVER;
    }
    CUtensorMap tc;
    {
        const uint64_t esize = out_f32 ? 4 : 2;
        const uint64_t dims[3] = {static_cast<uint64_t>(n), static_cast<uint64_t>(m), static_cast<uint64_t>(num_experts)};
        const uint64_t strides[2] = {static_cast<uint64_t>(n) * esize, static_cast<uint64_t>(n) * static_cast<uint64_t>(m) * esize};
        const uint32_t box[3] = {out_f32 ? 32u : 64u, kStoreBoxRows, 1};
        if (!make_tmap(&tc, out_f32 ? kDtypeF32 : dtype, dw, 3, dims, strides, box)) return XMA_ERR_DRIVER;
    }
    Params p{};
    p.padded_offsets = padded_offsets;
    p.num_experts = num_experts;
    p.m_pairs = static_cast<int>(ceil_div(m, kPairM));
    // The reduction runs over an expert's rows, known only on the device. Long reductions (by the mean)
    // take the wide tile for its lighter operand feed; so do large weight matrices whatever the mean,
    // where experts with few rows make the per-tile hand-over and the stores the cost and half as many
    // tiles are cheaper (measured: +4 % at 4096 x 7168 and 7168 x 2048 with a Zipf load, -6 % at
    // 2048 x 2048 with 1024-row experts).
    const bool wide = !out_f32 && n >= 2 * kBlockN &&
                      (cap / num_experts >= kWideMinRowsWgrad || m * n >= kWideMinElemsWgrad);
    p.n_tiles = static_cast<int>(ceil_div(n, wide ? 2 * kBlockN : kBlockN));
    p.m = m;
    p.n = n;
    p.c = dw;
    p.status = status;
    p.ab_format = dtype == kDtypeBF16 ? 1 : 0;
    p.group_m = kGroupM;
    const int64_t total = static_cast<int64_t>(num_experts) * p.m_pairs * p.n_tiles;
    if (total >= (int64_t(1) << 31)) return XMA_ERR_UNSUPPORTED;
    p.accumulate = accumulate ? 1 : 0;
    if (out_f32) return launch<T, kWgrad, XMA_EPI_STORE_F32>(ta, tb, tc, ta, p, total, stream);
    if (wide) return launch<T, kWgrad, XMA_EPI_STORE, true>(ta, tb, tc, ta, p, total, stream);
    return launch<T, kWgrad, XMA_EPI_STORE>(ta, tb, tc, ta, p, total, stream);
}

// float32 -> (hi, lo) bf16 pair with src = hi + lo up to 2^-16 relative. HBM-bound: 4 bytes read and
// 4 written per element, 16-byte loads, 8-byte stores.
__global__ void __launch_bounds__(256)
split_f32_kernel(const float* __restrict__ src, int64_t count, __nv_bfloat16* __restrict__ hi, __nv_bfloat16* __restrict__ lo) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t quads = count / 4;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < quads; i += stride) {
        const float4 v = reinterpret_cast<const float4*>(src)[i];
        const __nv_bfloat162 h01 = __floats2bfloat162_rn(v.x, v.y), h23 = __floats2bfloat162_rn(v.z, v.w);
        const float2 f01 = __bfloat1622float2(h01), f23 = __bfloat1622float2(h23);
        const __nv_bfloat162 l01 = __floats2bfloat162_rn(v.x - f01.x, v.y - f01.y);
        const __nv_bfloat162 l23 = __floats2bfloat162_rn(v.z - f23.x, v.w - f23.y);
        uint2 ph, pl;
        ph.x = *reinterpret_cast<const uint32_t*>(&h01);
        ph.y = *reinterpret_cast<const uint32_t*>(&h23);
        pl.x = *reinterpret_cast<const uint32_t*>(&l01);
        pl.y = *reinterpret_cast<const uint32_t*>(&l23);
        reinterpret_cast<uint2*>(hi)[i] = ph;
        reinterpret_cast<uint2*>(lo)[i] = pl;
    }
    // tail (count % 4 elements)
    const int64_t tail = quads * 4 + static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (tail < count) {
        const float v = src[tail];
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        hi[tail] = h;
        lo[tail] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
}

// out[row_src[r]] = sum over n tiles of partials[tile][r], tiles in ascending order (one thread per
// row, consecutive threads on consecutive addresses of every tile's slice).
__global__ void __launch_bounds__(256)
reduce_row_partials_kernel(const float* __restrict__ partials, int n_tiles, int64_t cap, const int32_t* __restrict__ row_src,
                           const int32_t* __restrict__ rows_in_use, float* __restrict__ out) {
    const int64_t rows = rows_in_use != nullptr ? min(static_cast<int64_t>(*rows_in_use), cap) : cap;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; r < rows; r += stride) {
        const int32_t flat = row_src[r];
        if (flat < 0) continue;
        float sum = 0.f;
        for (int t = 0; t < n_tiles; ++t) sum += partials[static_cast<int64_t>(t) * cap + r];
        out[flat] = sum;
    }
}

// out[i] = sum_s partials[s][i] (s ascending), rounded to T: the second step of a reduction split over
// row segments (router weight gradient).
template <typename T>
__global__ void __launch_bounds__(256)
sum_partials_kernel(const float* __restrict__ partials, int splits, int64_t count, T* __restrict__ out) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        float sum = 0.f;
        for (int s = 0; s < splits; ++s) sum += partials[static_cast<int64_t>(s) * count + i];
        out[i] = Elem<T>::from_float(sum);
    }
}

// One thread waits, with the GEMM kernels' own bounded wait, on a barrier that nothing ever arrives
// at: the wait runs out after `limit_ns`, the code lands in the status word and the kernel returns.
__global__ void bounded_wait_selftest_kernel(int32_t* status, uint64_t limit_ns) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    fence_barrier_init();
    mbar_wait(smem_u32(&bar), 0, &abort_flag, status, kSelfTestCode, limit_ns);
}

}  // namespace gemm
}  // namespace xma

extern "C" {

int xma_split_f32(const float* src, int64_t count, void* hi, void* lo, void* stream) {
    if (count < 0 || (count > 0 && (!src || !hi || !lo))) return XMA_ERR_BAD_ARG;
    if (count == 0) return XMA_OK;
    if (!xma::aligned16(src) || (reinterpret_cast<uintptr_t>(hi) & 7) || (reinterpret_cast<uintptr_t>(lo) & 7))
        return XMA_ERR_BAD_ARG;
    const int64_t quads = count / 4 > 0 ? count / 4 : 1;
    const int64_t want = xma::ceil_div(quads, 256);
    const int64_t cap_blocks = static_cast<int64_t>(xma::sm_count()) * 8;
    const unsigned blocks = static_cast<unsigned>(want < cap_blocks ? want : cap_blocks);
    xma::gemm::split_f32_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, count, static_cast<__nv_bfloat16*>(hi), static_cast<__nv_bfloat16*>(lo));
    return xma::launch_status();
}

int xma_selftest_bounded_wait(int32_t* status, int64_t limit_ns, void* stream) {
    if (!status || limit_ns <= 0 || limit_ns > 1000000000ll) return XMA_ERR_BAD_ARG;
    xma::gemm::bounded_wait_selftest_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
        status, static_cast<uint64_t>(limit_ns));
    return xma::launch_status();
}

int xma_sum_partials(const float* partials, int32_t splits, int64_t count, int32_t dtype, void* out, void* stream) {
    if (!partials || !out || splits <= 0 || count <= 0) return XMA_ERR_BAD_ARG;
    const int64_t want = xma::ceil_div(count, 256);
    const int64_t max_blocks = static_cast<int64_t>(xma::sm_count()) * 8;
    const unsigned blocks = static_cast<unsigned>(want < max_blocks ? want : max_blocks);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case xma::kDtypeBF16:
            xma::gemm::sum_partials_kernel<<<blocks, 256, 0, s>>>(partials, splits, count, static_cast<__nv_bfloat16*>(out));
            break;
        case xma::kDtypeF16:
            xma::gemm::sum_partials_kernel<<<blocks, 256, 0, s>>>(partials, splits, count, static_cast<__half*>(out));
            break;
        case xma::kDtypeF32:
            xma::gemm::sum_partials_kernel<<<blocks, 256, 0, s>>>(partials, splits, count, static_cast<float*>(out));
            break;
        default:
            return XMA_ERR_UNSUPPORTED;
    }
    return xma::launch_status();
}

int xma_reduce_row_partials(const float* partials, int32_t n_tiles, int64_t cap, const int32_t* row_src,
                            const int32_t* rows_in_use, float* out, void* stream) {
    if (!partials || !row_src || !out || n_tiles <= 0 || cap <= 0) return XMA_ERR_BAD_ARG;
    const int64_t want = xma::ceil_div(cap, 256);
    const int64_t max_blocks = static_cast<int64_t>(xma::sm_count()) * 8;
    xma::gemm::reduce_row_partials_kernel<<<static_cast<unsigned>(want < max_blocks ? want : max_blocks), 256, 0,
                                            static_cast<cudaStream_t>(stream)>>>(partials, n_tiles, cap, row_src,
                                                                                 rows_in_use, out);
    return xma::launch_status();
}

int xma_grouped_gemm(int32_t layout, int32_t epilogue, int32_t dtype, const void* a, const void* w,
                     const int32_t* padded_offsets, int64_t cap, int32_t num_experts, int64_t n, int64_t k, void* c,
                     void* aux, const int32_t* row_src, const void* row_scale, float* d_row_scale, int32_t* status,
                     void* stream) {
    if (!a || !w || !padded_offsets || !c || cap <= 0 || cap % XMA_BLOCK_M != 0 || num_experts <= 0 || n <= 0 || k <= 0)
        return XMA_ERR_BAD_ARG;
    if (!xma::aligned16(a) || !xma::aligned16(w) || !xma::aligned16(c) || (aux && !xma::aligned16(aux)))
        return XMA_ERR_BAD_ARG;
    if (dtype != xma::kDtypeBF16 && dtype != xma::kDtypeF16) return XMA_ERR_UNSUPPORTED;
    if (n % 8 != 0 || k % 8 != 0 || num_experts > xma::kMaxExperts) return XMA_ERR_UNSUPPORTED;
    if (layout != XMA_GEMM_NT && layout != XMA_GEMM_NN) return XMA_ERR_BAD_ARG;
    if (epilogue == XMA_EPI_SWIGLU) {
        if (layout != XMA_GEMM_NT || !aux) return XMA_ERR_BAD_ARG;
        if (n % 2 != 0 || (n / 2) % xma::gemm::kHalfN != 0) return XMA_ERR_UNSUPPORTED;
    } else if (epilogue == XMA_EPI_SWIGLU_BWD) {
        if (layout != XMA_GEMM_NN || !aux) return XMA_ERR_BAD_ARG;
    } else if (epilogue != XMA_EPI_STORE && epilogue != XMA_EPI_STORE_F32 && epilogue != XMA_EPI_ADD_F32) {
        return XMA_ERR_BAD_ARG;
    }
    if ((row_scale || d_row_scale) && !row_src) return XMA_ERR_BAD_ARG;
    if (cap / XMA_BLOCK_M * xma::ceil_div(n, 128) >= (int64_t(1) << 31)) return XMA_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == xma::kDtypeBF16)
        return xma::gemm::run_rows<__nv_bfloat16>(layout, epilogue, dtype, a, w, padded_offsets, cap, num_experts, n, k, c,
                                                  aux, row_src, row_scale, d_row_scale, status, s);
    return xma::gemm::run_rows<__half>(layout, epilogue, dtype, a, w, padded_offsets, cap, num_experts, n, k, c, aux,
                                       row_src, row_scale, d_row_scale, status, s);
}

int xma_router_gate_topk(int32_t dtype, const void* x, const void* w_gate, int64_t num_tokens, int64_t hidden,
                         int32_t num_experts, int32_t top_k, void* logits, void* topk_weights, float* topk_probs_f32,
                         int64_t* selected, int32_t* status, void* stream) {
    if (num_tokens < 0 || hidden <= 0 || num_experts <= 0 || top_k <= 0) return XMA_ERR_BAD_ARG;
    if (dtype != xma::kDtypeBF16 && dtype != xma::kDtypeF16) return XMA_ERR_UNSUPPORTED;
    if (num_experts > xma::gemm::kBlockN || num_experts % 8 != 0 || hidden % 8 != 0 || top_k > xma::gemm::kRouterMaxK ||
        top_k > num_experts || num_tokens >= (int64_t(1) << 31) - XMA_BLOCK_M)
        return XMA_ERR_UNSUPPORTED;
    if (num_tokens == 0) return XMA_OK;
    if (!x || !w_gate || !logits || !topk_weights || !topk_probs_f32 || !selected) return XMA_ERR_BAD_ARG;
    if (!xma::aligned16(x) || !xma::aligned16(w_gate) || !xma::aligned16(logits)) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == xma::kDtypeBF16)
        return xma::gemm::run_router<__nv_bfloat16>(dtype, x, w_gate, num_tokens, hidden, num_experts, top_k, logits,
                                                    topk_weights, topk_probs_f32, selected, status, s);
    return xma::gemm::run_router<__half>(dtype, x, w_gate, num_tokens, hidden, num_experts, top_k, logits, topk_weights,
                                         topk_probs_f32, selected, status, s);
}

int xma_grouped_wgrad(int32_t dtype, const void* x, const void* y, const int32_t* padded_offsets, int64_t cap,
                      int32_t num_experts, int64_t m, int64_t n, void* dw, int32_t* status, void* stream) {
    if (!x || !y || !padded_offsets || !dw || cap <= 0 || cap % XMA_BLOCK_M != 0 || num_experts <= 0 || m <= 0 || n <= 0)
        return XMA_ERR_BAD_ARG;
    if (!xma::aligned16(x) || !xma::aligned16(y) || !xma::aligned16(dw)) return XMA_ERR_BAD_ARG;
    if (dtype != xma::kDtypeBF16 && dtype != xma::kDtypeF16) return XMA_ERR_UNSUPPORTED;
    if (m % 8 != 0 || n % 8 != 0) return XMA_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == xma::kDtypeBF16)
        return xma::gemm::run_wgrad<__nv_bfloat16>(dtype, x, y, padded_offsets, cap, num_experts, m, n, dw, false, false,
                                                   status, s);
    return xma::gemm::run_wgrad<__half>(dtype, x, y, padded_offsets, cap, num_experts, m, n, dw, false, false, status, s);
}

int xma_grouped_wgrad_f32(int32_t dtype, const void* x, const void* y, const int32_t* padded_offsets, int64_t cap,
                          int32_t num_experts, int64_t m, int64_t n, float* dw, int32_t accumulate, int32_t* status,
                          void* stream) {
    // Rows at or past `cap` are read as zeros (the tensor maps end there), so `cap` may be any row count
    // here; the segments in padded_offsets must still begin and end on multiples of 64 rows.
    if (!x || !y || !padded_offsets || !dw || cap <= 0 || num_experts <= 0 || m <= 0 || n <= 0)
        return XMA_ERR_BAD_ARG;
    if (!xma::aligned16(x) || !xma::aligned16(y) || !xma::aligned16(dw)) return XMA_ERR_BAD_ARG;
    if (dtype != xma::kDtypeBF16 && dtype != xma::kDtypeF16) return XMA_ERR_UNSUPPORTED;
    if (m % 8 != 0 || n % 8 != 0) return XMA_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == xma::kDtypeBF16)
        return xma::gemm::run_wgrad<__nv_bfloat16>(dtype, x, y, padded_offsets, cap, num_experts, m, n, dw, true,
                                                   accumulate != 0, status, s);
    return xma::gemm::run_wgrad<__half>(dtype, x, y, padded_offsets, cap, num_experts, m, n, dw, true, accumulate != 0,
                                        status, s);
}

}  // extern "C"
