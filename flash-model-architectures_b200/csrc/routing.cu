// Routing kernels of the MoE hot path: expert histogram, router top-k + softmax (forward and
// backward) and the stable counting sort that builds the padded expert order.
//
// All of it is integer / HBM-bound work: vectorised 16-byte loads, warp-private shared-memory
// counters, warp match/ballot ranking, no tensor cores.
#include <limits.h>
#include <math.h>
#include <mutex>

#include "common.cuh"

namespace xma {

// ------------------------------------------------------------------------------------------------
// continuous_count: out[b] = #{i : ids[i] == b}
//
// HBM-bound integer work. Three ways to count, by the number of bins:
//   bins <= 8     per-thread counters packed into one 64-bit register (eight 8-bit fields, spilled
//                 into eight 32-bit registers every 240 ids): no shared-memory traffic per id at all;
//   bins <= 1024  shared-memory counters laid out [bin][lane]: a lane only ever touches its own bank,
//                 so a warp's 32 updates never conflict, whatever the ids are (sorted ids, MoE's
//                 case, included);
//   larger        as many lane-replicated copies as fit, `stride` (odd) words apart.
// Two ways to produce the result:
//   one thread-block cluster (inputs up to kCountClusterMaxIds ids): the CTAs sum their histograms
//                 through distributed shared memory and CTA 0 stores out[] - one launch, no memset,
//                 no global atomics;
//   a grid of blocks after a memset, one global atomicAdd per bin and block.
// ------------------------------------------------------------------------------------------------

constexpr int kCountThreads = 512;
constexpr int kCountMaxSmemEntries = 8192;  // 32 KB of uint32 counters without opting in to more
constexpr int kCountLaneBins = 1024;        // up to here the [bin][lane] layout is used (128 KB)
constexpr int kCountPackedBins = 8;
constexpr int64_t kCountClusterMaxIds = int64_t(1) << 18;  // beyond, 16 SMs cannot pull the ids fast enough

__device__ __forceinline__ uint32_t count_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t count_cluster_size() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void count_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Word at the same shared-memory address in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t count_ld_remote(const uint32_t* local, uint32_t rank) {
    uint32_t addr, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(addr)
                 : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(local))), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

enum CountMode { kCountPacked = 0, kCountLane = 1, kCountReplicated = 2 };

template <typename IdT, int kMode>
struct Counter {
    uint32_t* hist;
    int bins, stride, rep, lane;
    uint64_t packed;
    uint32_t tot[kCountPackedBins];
    int pending;

    __device__ __forceinline__ void init(uint32_t* h, int bins_, int reps, int stride_) {
        hist = h;
        bins = bins_;
        stride = stride_;
        lane = threadIdx.x & 31;
        rep = lane % reps;
        packed = 0;
        pending = 0;
#pragma unroll
        for (int b = 0; b < kCountPackedBins; ++b) tot[b] = 0;
    }
    __device__ __forceinline__ void spill() {
#pragma unroll
        for (int b = 0; b < kCountPackedBins; ++b) tot[b] += static_cast<uint32_t>(packed >> (8 * b)) & 0xffu;
        packed = 0;
        pending = 0;
    }
    // Ids outside [0, bins) are ignored (documented behaviour of continuous_count,
    // xma/functional/continuous_count/__init__.py:15-16).
    __device__ __forceinline__ void add(IdT id) {
        if (kMode == kCountPacked) {
            const bool ok = id >= 0 && id < static_cast<IdT>(bins);
            packed += static_cast<uint64_t>(ok) << ((static_cast<uint32_t>(id) & 7u) * 8u);
        } else if (id >= 0 && id < static_cast<IdT>(bins)) {
            if (kMode == kCountLane) atomicAdd(&hist[static_cast<int>(id) * 32 + lane], 1u);
            else atomicAdd(&hist[rep * stride + static_cast<int>(id)], 1u);
        }
    }
    // Call after every batch of at most 16 ids per thread.
    __device__ __forceinline__ void batch_done(int ids_in_batch) {
        if (kMode == kCountPacked) {
            pending += ids_in_batch;
            if (pending > 255 - 16) spill();
        }
    }
    // Packed mode: the warp adds its totals into hist[b] (one shared atomic per bin and warp).
    __device__ __forceinline__ void finish() {
        if (kMode == kCountPacked) {
            spill();
#pragma unroll
            for (int b = 0; b < kCountPackedBins; ++b) {
                uint32_t v = tot[b];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                if (lane == 0 && b < bins && v) atomicAdd(&hist[b], v);
            }
        }
    }
    // Total of bin b over this block's copies (after __syncthreads()).
    __device__ __forceinline__ uint32_t total(int b, int reps) const {
        if (kMode == kCountPacked) return hist[b];
        uint32_t sum = 0;
        if (kMode == kCountLane) {
            // A lane group of 32 consecutive words: read rotated so that the threads of a warp, which
            // hold consecutive bins, start in different banks.
            for (int r = 0; r < 32; ++r) sum += hist[b * 32 + ((r + b) & 31)];
        } else {
            for (int r = 0; r < reps; ++r) sum += hist[r * stride + b];
        }
        return sum;
    }
};

// kCluster: the grid is ONE cluster; CTA 0 writes out[] (no memset before, no atomics).
// Otherwise out[] was zeroed before the launch and every block adds its totals.
template <typename IdT, int kMode, bool kCluster>
__global__ void __launch_bounds__(kCountThreads)
continuous_count_kernel(const IdT* __restrict__ ids, int64_t n, uint32_t* __restrict__ out, int bins,
                        int reps, int stride, int64_t head, int64_t nvec) {
    extern __shared__ uint32_t hist[];
    constexpr int kPerVec = 16 / sizeof(IdT);
    const int words = kMode == kCountPacked ? bins : kMode == kCountLane ? bins * 32 : reps * stride;
    // In cluster mode the block totals are parked after the counters for the peers to read.
    uint32_t* block_tot = hist + words;
    for (int i = threadIdx.x; i < words; i += blockDim.x) hist[i] = 0;
    __syncthreads();

    Counter<IdT, kMode> counter;
    counter.init(hist, bins, reps, stride);
    const int64_t gtid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int64_t gthreads = static_cast<int64_t>(gridDim.x) * blockDim.x;

    // Body: 16-byte vectors starting at the first 16-byte aligned element. Four independent 16-byte
    // loads are in flight per thread before any counter is touched.
    const uint4* body = reinterpret_cast<const uint4*>(ids + head);
    constexpr int kUnroll = 4;
    for (int64_t v0 = gtid; v0 < nvec; v0 += gthreads * kUnroll) {
        uint4 raw[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int64_t v = v0 + u * gthreads;
            if (v < nvec) raw[u] = __ldg(body + v);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            if (v0 + u * gthreads < nvec) {
                const IdT* e = reinterpret_cast<const IdT*>(&raw[u]);
#pragma unroll
                for (int j = 0; j < kPerVec; ++j) counter.add(e[j]);
            }
        }
        counter.batch_done(kUnroll * kPerVec);
    }
    // Unaligned head and the tail that does not fill a vector: scalar loads.
    const int64_t tail_start = head + nvec * kPerVec;
    const int64_t scalar = head + (n - tail_start);
    for (int64_t s = gtid; s < scalar; s += gthreads) {
        const int64_t i = s < head ? s : tail_start + (s - head);
        counter.add(ids[i]);
        counter.batch_done(1);
    }
    counter.finish();
    __syncthreads();

    if (!kCluster) {
        for (int b = threadIdx.x; b < bins; b += blockDim.x) {
            const uint32_t sum = counter.total(b, reps);
            if (sum) atomicAdd(&out[b], sum);
        }
    } else {
        for (int b = threadIdx.x; b < bins; b += blockDim.x) block_tot[b] = counter.total(b, reps);
        count_cluster_sync();  // every CTA's totals are in place (release/acquire at cluster scope)
        if (count_cluster_rank() == 0) {
            const uint32_t ctas = count_cluster_size();
            for (int b = threadIdx.x; b < bins; b += blockDim.x) {
                uint32_t sum = 0;
                for (uint32_t c = 0; c < ctas; ++c) sum += count_ld_remote(&block_tot[b], c);
                out[b] = sum;
            }
        }
        count_cluster_sync();  // no CTA leaves while CTA 0 may still read its shared memory
    }
}

// ------------------------------------------------------------------------------------------------
// Router top-k + softmax over the selected logits
// ------------------------------------------------------------------------------------------------

constexpr int kRouterWarps = 8;

template <typename T, int VPL>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_softmax_kernel(const T* __restrict__ logits, int64_t num_tokens, int num_experts, int top_k,
                           T* __restrict__ weights, float* __restrict__ probs, int64_t* __restrict__ selected) {
    const int lane = threadIdx.x & 31;
    const int64_t token = static_cast<int64_t>(blockIdx.x) * kRouterWarps + (threadIdx.x >> 5);
    if (token >= num_tokens) return;
    const T* row = logits + token * num_experts;

    // Lane l holds experts l, l+32, l+64, ... so the row is read with coalesced loads.
    float v[VPL];
    uint32_t taken = 0;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int e = lane + 32 * i;
        if (e < num_experts) {
            v[i] = Elem<T>::to_float(row[e]);
        } else {
            v[i] = -INFINITY;
            taken |= 1u << i;
        }
    }

    float my_val = 0.f;
    int my_idx = 0;
    for (int j = 0; j < top_k; ++j) {
        // Lane-local best among the experts not taken yet; the strict '>' keeps the lowest id.
        float bv = -INFINITY;
        int be = INT_MAX;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const bool free_slot = !((taken >> i) & 1u);
            if (free_slot && (be == INT_MAX || v[i] > bv)) {
                bv = v[i];
                be = lane + 32 * i;
            }
        }
        // Warp argmax: larger value wins, equal values go to the lower expert id.
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oe = __shfl_xor_sync(0xffffffffu, be, off);
            if (oe != INT_MAX && (be == INT_MAX || ov > bv || (ov == bv && oe < be))) {
                bv = ov;
                be = oe;
            }
        }
        if (lane == j) {
            my_val = bv;
            my_idx = be;
        }
        if ((be & 31) == lane) taken |= 1u << (be >> 5);
    }

    // softmax over the k selected logits in float32 (xma/layers/moe/__init__.py:200).
    const float vmax = __shfl_sync(0xffffffffu, my_val, 0);
    float ex = lane < top_k ? expf(my_val - vmax) : 0.f;
    float sum = ex;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane < top_k) {
        const float p = ex / sum;
        const int64_t o = token * top_k + lane;
        weights[o] = Elem<T>::from_float(p);
        probs[o] = p;
        selected[o] = my_idx;
    }
}

template <typename T, int VPL>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_softmax_backward_kernel(const T* __restrict__ d_weights, const float* __restrict__ probs,
                                    const int64_t* __restrict__ selected, int64_t num_tokens, int num_experts,
                                    int top_k, T* __restrict__ d_logits) {
    const int lane = threadIdx.x & 31;
    const int64_t token = static_cast<int64_t>(blockIdx.x) * kRouterWarps + (threadIdx.x >> 5);
    if (token >= num_tokens) return;

    float p = 0.f, dw = 0.f;
    int sel = -1;
    if (lane < top_k) {
        const int64_t o = token * top_k + lane;
        p = probs[o];
        dw = Elem<T>::to_float(d_weights[o]);
        sel = static_cast<int>(selected[o]);
    }
    float dot = p * dw;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    const float g = p * (dw - dot);

    float acc[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) acc[i] = 0.f;
    for (int j = 0; j < top_k; ++j) {
        const int sj = __shfl_sync(0xffffffffu, sel, j);
        const float gj = __shfl_sync(0xffffffffu, g, j);
#pragma unroll
        for (int i = 0; i < VPL; ++i)
            if (sj == lane + 32 * i) acc[i] += gj;
    }
    T* row = d_logits + token * num_experts;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        const int e = lane + 32 * i;
        if (e < num_experts) row[e] = Elem<T>::from_float(acc[i]);
    }
}

// ------------------------------------------------------------------------------------------------
// Stable counting sort -> padded expert order
//
// The n ids are cut into `segs` contiguous segments, one warp per segment, so that "earlier
// segment, then earlier position inside the segment" is exactly ascending flat index: the sort is
// stable by construction.
//   1. index_hist_kernel     per-segment histograms              seg_hist[s][e]
//   2. index_scan_kernel     per expert, exclusive scan over s   seg_base[s][e] = rows of e before s
//   3. index_offsets_kernel  counts -> offsets, padded offsets, tile -> expert map
//   4. index_fill_kernel     padding rows of row_src, sorted_expert_idxs
//   5. index_scatter_kernel  rank every id inside its warp with match_any and write the indices
// ------------------------------------------------------------------------------------------------

constexpr int kIndexWarps = 8;
constexpr int kIndexMaxSegs = 8192;
constexpr int kIndexMinSegLen = 1024;

struct IndexPlan {
    int segs;
    int64_t seg_len;  // multiple of 32
};

inline IndexPlan index_plan(int64_t n) {
    IndexPlan p;
    int64_t segs = ceil_div(n, kIndexMinSegLen);
    if (segs < 1) segs = 1;
    if (segs > kIndexMaxSegs) segs = kIndexMaxSegs;
    int64_t len = ceil_div(n > 0 ? n : 1, segs);
    len = ceil_div(len, 32) * 32;
    p.seg_len = len;
    p.segs = static_cast<int>(n > 0 ? ceil_div(n, len) : 1);
    return p;
}

template <typename IdT>
__global__ void __launch_bounds__(kIndexWarps * 32)
index_hist_kernel(const IdT* __restrict__ ids, int64_t n, int num_experts, int segs, int64_t seg_len,
                  int32_t* __restrict__ seg_hist) {
    extern __shared__ int32_t smem_hist[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = blockIdx.x * kIndexWarps + warp;
    int32_t* h = smem_hist + warp * num_experts;
    for (int e = lane; e < num_experts; e += 32) h[e] = 0;
    __syncwarp();
    if (seg < segs) {
        const int64_t begin = seg * seg_len;
        const int64_t end = min(begin + seg_len, n);
        for (int64_t i0 = begin + lane; i0 < end; i0 += 32 * 4) {
            IdT id[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) id[u] = i0 + 32 * u < end ? ids[i0 + 32 * u] : static_cast<IdT>(-1);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (id[u] >= 0 && id[u] < static_cast<IdT>(num_experts)) atomicAdd(&h[static_cast<int>(id[u])], 1);
        }
        __syncwarp();
        for (int e = lane; e < num_experts; e += 32) seg_hist[static_cast<int64_t>(seg) * num_experts + e] = h[e];
    }
}

// Exclusive scan of the per-segment histograms over the segments, one block per expert: seg_base[s][e]
// = rows of expert e in segments before s; expert_frequency[e] = the total. A thread owns up to
// kScanPerThread consecutive segments (all their counts are requested before any is used), the block
// scans the per-thread sums.
constexpr int kScanThreads = 256;
constexpr int kScanPerThread = 32;

__global__ void __launch_bounds__(kScanThreads)
index_scan_kernel(const int32_t* __restrict__ seg_hist, int32_t* __restrict__ seg_base, int num_experts, int segs,
                  uint32_t* __restrict__ expert_frequency) {
    __shared__ int32_t warp_sums[kScanThreads / 32];
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int32_t running = 0;
    for (int round0 = 0; round0 < segs; round0 += kScanThreads * kScanPerThread) {
        const int round_len = min(segs - round0, kScanThreads * kScanPerThread);
        const int per = (round_len + kScanThreads - 1) / kScanThreads;  // <= kScanPerThread
        const int first = round0 + threadIdx.x * per;
        const int last = min(first + per, round0 + round_len);
        int32_t v[kScanPerThread];
#pragma unroll
        for (int u = 0; u < kScanPerThread; ++u)
            v[u] = (u < per && first + u < last) ? seg_hist[static_cast<int64_t>(first + u) * num_experts + e] : 0;
        int32_t mine = 0;
#pragma unroll
        for (int u = 0; u < kScanPerThread; ++u) mine += v[u];
        int32_t incl = mine;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int32_t o = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += o;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        int32_t before = running + incl - mine;
        int32_t total = 0;
#pragma unroll
        for (int w = 0; w < kScanThreads / 32; ++w) {
            const int32_t ws = warp_sums[w];
            if (w < warp) before += ws;
            total += ws;
        }
#pragma unroll
        for (int u = 0; u < kScanPerThread; ++u) {
            if (u < per && first + u < last) seg_base[static_cast<int64_t>(first + u) * num_experts + e] = before;
            before += v[u];
        }
        running += total;
        __syncthreads();  // warp_sums is rewritten by the next round
    }
    if (threadIdx.x == 0) expert_frequency[e] = static_cast<uint32_t>(running);
}

// One block of kMaxExperts threads: thread e owns expert e.
__global__ void __launch_bounds__(kMaxExperts)
index_offsets_kernel(const uint32_t* __restrict__ expert_frequency, int num_experts, int block_m,
                     int32_t* __restrict__ expert_offsets, int32_t* __restrict__ padded_offsets,
                     int32_t* __restrict__ tile_expert, int max_tiles) {
    __shared__ int32_t s_cnt[kMaxExperts];
    __shared__ int32_t s_pad[kMaxExperts];
    const int e = threadIdx.x;
    const int32_t c = e < num_experts ? static_cast<int32_t>(expert_frequency[e]) : 0;
    const int32_t pc = (c + block_m - 1) / block_m * block_m;
    s_cnt[e] = c;
    s_pad[e] = pc;
    __syncthreads();
    // Hillis-Steele inclusive scans of both arrays.
    for (int off = 1; off < kMaxExperts; off <<= 1) {
        const int32_t a = e >= off ? s_cnt[e - off] : 0;
        const int32_t b = e >= off ? s_pad[e - off] : 0;
        __syncthreads();
        s_cnt[e] += a;
        s_pad[e] += b;
        __syncthreads();
    }
    const int32_t pad_end = s_pad[e];
    const int32_t pad_begin = pad_end - pc;
    if (e < num_experts) {
        expert_offsets[e] = s_cnt[e];
        padded_offsets[e] = pad_begin;
        if (e == num_experts - 1) padded_offsets[num_experts] = pad_end;
    }
    if (tile_expert != nullptr && e == 0) tile_expert[max_tiles] = s_pad[num_experts - 1] / block_m;
}

// The fill pass over rows [first_p0, cap) in steps of `stride`, 4 consecutive rows per thread. s_off
// (inclusive end offsets), s_pad (padded begin offsets, E + 1 entries) and s_cnt (row counts) are in
// shared memory.
__device__ __forceinline__ void fill_rows(int32_t first_p0, int32_t stride, const int32_t* s_off, const int32_t* s_pad,
                                          const int32_t* s_cnt, int num_experts, int64_t n64, int64_t cap64, int block_m,
                                          int32_t* __restrict__ row_src, int32_t* __restrict__ sorted_expert_idxs,
                                          int32_t* __restrict__ tile_expert) {
    // Every thread owns kFillRun = 4 consecutive rows: one binary search per table at the start of the
    // run, then the owner only moves forward; the four expert ids leave as one 16-byte store, so a
    // warp writes 512 contiguous bytes per instruction. Row numbers fit 32 bits (checked at the entry
    // point) and all the arithmetic is 32-bit: an ncu capture of the 64-bit version showed the kernel
    // issue-bound at 120 instructions per row.
    constexpr int kFillRun = 4;
    const int32_t n = static_cast<int32_t>(n64), cap = static_cast<int32_t>(cap64);
    const int32_t rows_used = s_pad[num_experts];
    const int block_shift = (block_m & (block_m - 1)) == 0 ? __ffs(block_m) - 1 : -1;
    const bool vec_ok = sorted_expert_idxs != nullptr && (reinterpret_cast<uintptr_t>(sorted_expert_idxs) & 15) == 0;
    const int last = num_experts - 1;
    // (the increment cannot overflow: p0 jumps to cap when fewer than `stride` rows are left)
    for (int32_t p0 = first_p0; p0 < cap;
         p0 = cap - p0 > stride ? p0 + stride : cap) {
        // ---- expert id of sorted position p (positions below n) ----
        if (sorted_expert_idxs != nullptr && p0 < n) {
            int lo = 0, hi = last;  // smallest e with s_off[e] > p0 (offsets are inclusive end offsets)
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (s_off[mid] > p0) hi = mid; else lo = mid + 1;
            }
            int32_t ids_out[kFillRun];
            if (s_off[lo] > p0 + (kFillRun - 1)) {  // the whole run lies inside one expert
#pragma unroll
                for (int u = 0; u < kFillRun; ++u) ids_out[u] = lo;
            } else {
                int owner = lo;
#pragma unroll
                for (int u = 0; u < kFillRun; ++u) {
                    while (owner < last && s_off[owner] <= p0 + u) ++owner;
                    ids_out[u] = owner;
                }
            }
            if (vec_ok && p0 + kFillRun <= n) {
                *reinterpret_cast<int4*>(sorted_expert_idxs + p0) = make_int4(ids_out[0], ids_out[1], ids_out[2], ids_out[3]);
            } else {
#pragma unroll
                for (int u = 0; u < kFillRun; ++u)
                    if (p0 + u < n) sorted_expert_idxs[p0 + u] = ids_out[u];
            }
        }
        // ---- padded order: -1 for padding rows, expert of every tile ----
        const bool row_vec_ok = (reinterpret_cast<uintptr_t>(row_src) & 15) == 0 && p0 + kFillRun <= cap;
        if (p0 >= rows_used) {
            // past the rows in use: all padding, no expert
            if (row_vec_ok) {
                *reinterpret_cast<int4*>(row_src + p0) = make_int4(-1, -1, -1, -1);
            } else {
#pragma unroll
                for (int u = 0; u < kFillRun; ++u)
                    if (p0 + u < cap) row_src[p0 + u] = -1;
            }
            if (tile_expert != nullptr) {
#pragma unroll
                for (int u = 0; u < kFillRun; ++u) {
                    const int32_t p = p0 + u;
                    if (p < cap && (block_shift >= 0 ? (p & (block_m - 1)) == 0 : p % block_m == 0))
                        tile_expert[block_shift >= 0 ? p >> block_shift : p / block_m] = -1;
                }
            }
            continue;
        }
        int owner;
        {
            int lo = 0, hi = last;  // largest e with s_pad[e] <= p0
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (s_pad[mid] <= p0) lo = mid; else hi = mid - 1;
            }
            owner = lo;
        }
        if (block_shift >= 2) {
            // Segments are multiples of a power of two >= 4 rows, so the run stays inside one expert's
            // segment and only its first row can start a tile.
            const int32_t first = p0 - s_pad[owner], cnt = s_cnt[owner];
            if (first >= cnt && row_vec_ok) {
                *reinterpret_cast<int4*>(row_src + p0) = make_int4(-1, -1, -1, -1);
            } else {
#pragma unroll
                for (int u = 0; u < kFillRun; ++u)
                    if (first + u >= cnt) row_src[p0 + u] = -1;
            }
            if (tile_expert != nullptr && (p0 & (block_m - 1)) == 0) tile_expert[p0 >> block_shift] = owner;
        } else {
#pragma unroll
            for (int u = 0; u < kFillRun; ++u) {
                const int32_t p = p0 + u;
                if (p >= cap) break;
                bool padding = p >= rows_used;
                int tile_owner = -1;
                if (!padding) {
                    while (owner < last && s_pad[owner + 1] <= p) ++owner;
                    tile_owner = owner;
                    padding = p - s_pad[owner] >= s_cnt[owner];
                }
                if (padding) row_src[p] = -1;
                if (tile_expert != nullptr) {
                    if (block_shift >= 0) {
                        if ((p & (block_m - 1)) == 0) tile_expert[p >> block_shift] = tile_owner;
                    } else if (p % block_m == 0) {
                        tile_expert[p / block_m] = tile_owner;
                    }
                }
            }
        }
    }
}

__global__ void __launch_bounds__(256)
index_fill_kernel(const uint32_t* __restrict__ expert_frequency, const int32_t* __restrict__ expert_offsets,
                  const int32_t* __restrict__ padded_offsets, int num_experts, int64_t n64, int64_t cap64, int block_m,
                  int32_t* __restrict__ row_src, int32_t* __restrict__ sorted_expert_idxs,
                  int32_t* __restrict__ tile_expert) {
    __shared__ int32_t s_off[kMaxExperts];
    __shared__ int32_t s_pad[kMaxExperts + 1];
    __shared__ int32_t s_cnt[kMaxExperts];
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
        s_off[e] = expert_offsets[e];
        s_cnt[e] = static_cast<int32_t>(expert_frequency[e]);
    }
    for (int e = threadIdx.x; e <= num_experts; e += blockDim.x) s_pad[e] = padded_offsets[e];
    __syncthreads();
    fill_rows(static_cast<int32_t>(blockIdx.x * blockDim.x + threadIdx.x) * 4, static_cast<int32_t>(gridDim.x * blockDim.x) * 4,
              s_off, s_pad, s_cnt, num_experts, n64, cap64, block_m, row_src, sorted_expert_idxs, tile_expert);
}

template <typename IdT>
__global__ void __launch_bounds__(kIndexWarps * 32)
index_scatter_kernel(const IdT* __restrict__ ids, int64_t n, int num_experts, int segs, int64_t seg_len,
                     const int32_t* __restrict__ seg_hist, const int32_t* __restrict__ expert_offsets,
                     const uint32_t* __restrict__ expert_frequency, const int32_t* __restrict__ padded_offsets,
                     int32_t* __restrict__ sorted_scattered_idxs, int32_t* __restrict__ row_src,
                     int32_t* __restrict__ inv_row) {
    extern __shared__ int32_t smem_cnt[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = blockIdx.x * kIndexWarps + warp;
    if (seg >= segs) return;
    int32_t* cnt = smem_cnt + warp * num_experts;  // rows of expert e that precede the next id of this warp
    for (int e = lane; e < num_experts; e += 32) cnt[e] = seg_hist[static_cast<int64_t>(seg) * num_experts + e];
    __syncwarp();
    const int64_t begin = seg * seg_len;
    const int64_t end = min(begin + seg_len, n);
    const uint32_t lt_mask = (1u << lane) - 1u;
    IdT next_raw = begin + lane < end ? ids[begin + lane] : static_cast<IdT>(-1);
    for (int64_t i0 = begin; i0 < end; i0 += 32) {
        const int64_t i = i0 + lane;
        const IdT raw = next_raw;
        next_raw = i + 32 < end ? ids[i + 32] : static_cast<IdT>(-1);  // in flight during this group's ranking
        int id = -1;
        if (i < end && raw >= 0 && raw < static_cast<IdT>(num_experts)) id = static_cast<int>(raw);
        const uint32_t peers = __match_any_sync(0xffffffffu, id);
        const int rank = __popc(peers & lt_mask);
        int32_t base = 0;
        if (id >= 0) base = cnt[id];
        __syncwarp();
        if (id >= 0 && rank == 0) cnt[id] = base + __popc(peers);
        __syncwarp();
        if (id >= 0) {
            const int32_t pos = base + rank;
            const int32_t first = expert_offsets[id] - static_cast<int32_t>(expert_frequency[id]);
            const int32_t prow = padded_offsets[id] + pos;
            sorted_scattered_idxs[first + pos] = static_cast<int32_t>(i);
            row_src[prow] = static_cast<int32_t>(i);
            inv_row[i] = prow;
        }
    }
}

// Staged form of the scatter for segments of at most kStagedSegLen ids: the warp first sorts its
// segment by expert into shared memory (flat index and expert id at the segment-local sorted
// position), then writes every expert's run to its two destinations with consecutive lanes on
// consecutive addresses. The direct kernel above issues two 4-byte scattered stores per id instead.
constexpr int kStagedWarps = 4;
constexpr int kStagedSegLen = 2048;

template <typename IdT>
__global__ void __launch_bounds__(kStagedWarps * 32)
index_scatter_staged_kernel(const IdT* __restrict__ ids, int64_t n, int num_experts, int segs, int64_t seg_len,
                            const int32_t* __restrict__ seg_hist, const int32_t* __restrict__ seg_base,
                            const int32_t* __restrict__ expert_offsets, const uint32_t* __restrict__ expert_frequency,
                            const int32_t* __restrict__ padded_offsets, int32_t* __restrict__ sorted_scattered_idxs,
                            int32_t* __restrict__ row_src, int32_t* __restrict__ inv_row) {
    extern __shared__ int32_t smem_staged[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = blockIdx.x * kStagedWarps + warp;
    // per warp: stage_i[kStagedSegLen] (16 bit, index inside the segment) | stage_e[kStagedSegLen] (16 bit) |
    //           loc[E] | cursor[E] | ubase[E] | pbase[E];  per block, after the warps: first_row[E] | first_padded[E]
    const int per_warp = kStagedSegLen + 4 * num_experts;
    uint16_t* stage_i = reinterpret_cast<uint16_t*>(smem_staged + warp * per_warp);
    uint16_t* stage_e = stage_i + kStagedSegLen;
    int32_t* loc = smem_staged + warp * per_warp + kStagedSegLen;
    int32_t* cursor = loc + num_experts;
    int32_t* ubase = cursor + num_experts;
    int32_t* pbase = ubase + num_experts;
    int32_t* first_row = smem_staged + kStagedWarps * per_warp;  // first sorted position of expert e
    int32_t* first_padded = first_row + num_experts;             // first padded row of expert e
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
        first_row[e] = expert_offsets[e] - static_cast<int32_t>(expert_frequency[e]);
        first_padded[e] = padded_offsets[e];
    }
    __syncthreads();
    if (seg >= segs) return;

    int32_t running = 0;
    for (int e0 = 0; e0 < num_experts; e0 += 32) {
        const int e = e0 + lane;
        int32_t c = 0;
        if (e < num_experts) {
            const int64_t at = static_cast<int64_t>(seg) * num_experts + e;
            c = seg_hist[at];
            const int32_t before = seg_base[at];  // rows of e in earlier segments
            ubase[e] = first_row[e] + before;
            pbase[e] = first_padded[e] + before;
        }
        int32_t incl = c;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int32_t o = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += o;
        }
        if (e < num_experts) {
            loc[e] = running + incl - c;
            cursor[e] = running + incl - c;
        }
        running += __shfl_sync(0xffffffffu, incl, 31);
    }
    __syncwarp();

    // Four groups of 32 ids per step: their loads and warp matches are independent, only the cursor
    // updates of one group wait for the group before.
    constexpr int kGroups = 4;
    const int64_t begin = seg * seg_len;
    const int64_t end = min(begin + seg_len, n);
    const uint32_t lt_mask = (1u << lane) - 1u;
    IdT next_raw[kGroups];
#pragma unroll
    for (int u = 0; u < kGroups; ++u)
        next_raw[u] = begin + 32 * u + lane < end ? ids[begin + 32 * u + lane] : static_cast<IdT>(-1);
    for (int64_t i0 = begin; i0 < end; i0 += 32 * kGroups) {
        int id[kGroups];
        uint32_t peers[kGroups];
#pragma unroll
        for (int u = 0; u < kGroups; ++u) {
            const int64_t i = i0 + 32 * u + lane;
            const IdT raw = next_raw[u];
            id[u] = (i < end && raw >= 0 && raw < static_cast<IdT>(num_experts)) ? static_cast<int>(raw) : -1;
        }
#pragma unroll
        for (int u = 0; u < kGroups; ++u) {
            const int64_t i = i0 + 32 * (kGroups + u) + lane;
            next_raw[u] = i < end ? ids[i] : static_cast<IdT>(-1);
        }
#pragma unroll
        for (int u = 0; u < kGroups; ++u) peers[u] = __match_any_sync(0xffffffffu, id[u]);
#pragma unroll
        for (int u = 0; u < kGroups; ++u) {
            const int rank = __popc(peers[u] & lt_mask);
            int32_t base = 0;
            if (id[u] >= 0) base = cursor[id[u]];
            __syncwarp();
            if (id[u] >= 0 && rank == 0) cursor[id[u]] = base + __popc(peers[u]);
            __syncwarp();
            if (id[u] >= 0) {
                const int64_t i = i0 + 32 * u + lane;
                const int32_t lp = base + rank;
                stage_i[lp] = static_cast<uint16_t>(i - begin);
                stage_e[lp] = static_cast<uint16_t>(id[u]);
                inv_row[i] = pbase[id[u]] + (lp - loc[id[u]]);
            }
        }
    }
    __syncwarp();
    for (int32_t q = lane; q < running; q += 32) {
        const int e = stage_e[q];
        const int32_t r = q - loc[e];
        const int32_t i = static_cast<int32_t>(begin + stage_i[q]);
        sorted_scattered_idxs[ubase[e] + r] = i;
        row_src[pbase[e] + r] = i;
    }
}

// Single-launch form for MoE-sized inputs (E <= kSmallMaxExperts): ONE thread-block cluster of 1 to 16
// CTAs of 32 warps does all five passes, warp w of CTA c owning the (32 c + w)-th contiguous segment.
// The ids are read from global memory once, in the histogram pass, and parked in shared memory as
// 16-bit values for the ranking pass. Per expert, the rows that precede a warp are (rows in earlier
// CTAs, summed from the peers' totals through distributed shared memory) + (rows in earlier warps of
// its CTA). The five-kernel form above is bound by its launches at these sizes (30-38 us for a few
// microseconds of work) and a single block by the latency of 64 dependent steps per warp.
constexpr int kSmallWarps = 32;
constexpr int kSmallIdsPerCta = 32768;  // ids one CTA parks in shared memory (64 KB)
constexpr int kSmallMaxCtas = 16;
constexpr int kSmallMaxExperts = 256;
constexpr uint16_t kSmallNoId = 0xffffu;

template <typename IdT>
__global__ void __launch_bounds__(kSmallWarps * 32)
index_small_kernel(const IdT* __restrict__ ids, int32_t n, int num_experts, int block_m, int64_t cap, int max_tiles,
                   uint32_t* __restrict__ expert_frequency, int32_t* __restrict__ expert_offsets,
                   int32_t* __restrict__ sorted_expert_idxs, int32_t* __restrict__ sorted_scattered_idxs,
                   int32_t* __restrict__ padded_offsets, int32_t* __restrict__ row_src, int32_t* __restrict__ inv_row,
                   int32_t* __restrict__ tile_expert) {
    extern __shared__ int32_t smem_small[];
    int32_t* hist = smem_small;                         // [32][E]: per-warp counts, then exclusive bases inside the CTA
    int32_t* cta_tot = hist + kSmallWarps * num_experts;  // [E] rows of this CTA (read by the peers)
    int32_t* cta_base = cta_tot + num_experts;          // [E] rows in earlier CTAs
    int32_t* s_cnt = cta_base + num_experts;            // [E]
    int32_t* s_off = s_cnt + num_experts;               // [E] inclusive end offsets
    int32_t* s_pad = s_off + num_experts;               // [E + 1] first padded row
    uint16_t* parked = reinterpret_cast<uint16_t*>(s_pad + num_experts + 1);  // [32][seg_len] this CTA's ids
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t ctas = count_cluster_size(), cta = count_cluster_rank();
    const int32_t total_warps = static_cast<int32_t>(ctas) * kSmallWarps;
    const int32_t seg_len = ((n + total_warps - 1) / total_warps + 31) / 32 * 32;  // <= kSmallIdsPerCta / 32
    const int32_t gw = static_cast<int32_t>(cta) * kSmallWarps + warp;
    const int32_t begin = static_cast<int32_t>(min(static_cast<int64_t>(gw) * seg_len, static_cast<int64_t>(n)));
    const int32_t end = min(begin + seg_len, n);
    uint16_t* mine = parked + warp * seg_len;

    // 1. per-warp histograms
    for (int i = threadIdx.x; i < kSmallWarps * num_experts; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    int32_t* h = hist + warp * num_experts;
    constexpr int kLoads = 8;  // independent loads in flight per lane (a 256-id segment is one round)
    for (int32_t i0 = begin + lane; i0 < end; i0 += 32 * kLoads) {
        IdT raw[kLoads];
#pragma unroll
        for (int u = 0; u < kLoads; ++u) raw[u] = i0 + 32 * u < end ? ids[i0 + 32 * u] : static_cast<IdT>(-1);
#pragma unroll
        for (int u = 0; u < kLoads; ++u) {
            if (i0 + 32 * u < end) {
                const bool ok = raw[u] >= 0 && raw[u] < static_cast<IdT>(num_experts);
                mine[i0 + 32 * u - begin] = ok ? static_cast<uint16_t>(raw[u]) : kSmallNoId;
                if (ok) atomicAdd(&h[static_cast<int>(raw[u])], 1);
            }
        }
    }
    __syncthreads();
    // 2. per expert, exclusive scan over the warps of this CTA
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
        int32_t running = 0;
        for (int w = 0; w < kSmallWarps; ++w) {
            const int32_t c = hist[w * num_experts + e];
            hist[w * num_experts + e] = running;
            running += c;
        }
        cta_tot[e] = running;
    }
    count_cluster_sync();  // all CTAs' totals are in place
    for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
        // All the peers' totals are requested before any is used (a remote load takes a few hundred
        // cycles; one after the other they would dominate the kernel at 256 experts).
        int32_t t[kSmallMaxCtas];
#pragma unroll
        for (uint32_t c = 0; c < kSmallMaxCtas; ++c)
            t[c] = c < ctas ? static_cast<int32_t>(count_ld_remote(reinterpret_cast<const uint32_t*>(&cta_tot[e]), c)) : 0;
        int32_t before = 0, total = 0;
#pragma unroll
        for (uint32_t c = 0; c < kSmallMaxCtas; ++c) {
            if (c < cta) before += t[c];
            total += t[c];
        }
        cta_base[e] = before;
        s_cnt[e] = total;
    }
    // This CTA is done with its peers' shared memory; the matching wait is at the very end, so that no
    // CTA leaves while a slower peer still reads its totals.
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    __syncthreads();
    // 3. offsets and padded offsets (warp 0, 32 experts per step)
    if (warp == 0) {
        int32_t run_off = 0, run_pad = 0;
        for (int e0 = 0; e0 < num_experts; e0 += 32) {
            const int e = e0 + lane;
            const int32_t c = e < num_experts ? s_cnt[e] : 0;
            const int32_t pc = (c + block_m - 1) / block_m * block_m;
            int32_t incl_c = c, incl_p = pc;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int32_t oc = __shfl_up_sync(0xffffffffu, incl_c, off);
                const int32_t op = __shfl_up_sync(0xffffffffu, incl_p, off);
                if (lane >= off) {
                    incl_c += oc;
                    incl_p += op;
                }
            }
            if (e < num_experts) {
                s_off[e] = run_off + incl_c;
                s_pad[e] = run_pad + incl_p - pc;
            }
            run_off += __shfl_sync(0xffffffffu, incl_c, 31);
            run_pad += __shfl_sync(0xffffffffu, incl_p, 31);
        }
        if (lane == 0) s_pad[num_experts] = run_pad;
    }
    __syncthreads();
    if (cta == 0) {
        for (int e = threadIdx.x; e < num_experts; e += blockDim.x) {
            expert_frequency[e] = static_cast<uint32_t>(s_cnt[e]);
            expert_offsets[e] = s_off[e];
            padded_offsets[e] = s_pad[e];
        }
        if (threadIdx.x == 0) {
            padded_offsets[num_experts] = s_pad[num_experts];
            if (tile_expert != nullptr) tile_expert[max_tiles] = s_pad[num_experts] / block_m;
        }
    }
    // 4. padding rows, expert of every sorted position and of every tile
    fill_rows(static_cast<int32_t>(cta * blockDim.x + threadIdx.x) * 4, static_cast<int32_t>(ctas * blockDim.x) * 4, s_off, s_pad,
              s_cnt, num_experts, n, cap, block_m, row_src, sorted_expert_idxs, tile_expert);
    // 5. ranks inside the warp's segment (match_any keeps the order of the ids) and the three index stores
    const uint32_t lt_mask = (1u << lane) - 1u;
    for (int32_t i0 = begin; i0 < end; i0 += 32) {
        const int32_t i = i0 + lane;
        int id = -1;
        if (i < end) {
            const uint16_t v = mine[i - begin];
            if (v != kSmallNoId) id = v;
        }
        const uint32_t peers = __match_any_sync(0xffffffffu, id);
        const int rank = __popc(peers & lt_mask);
        int32_t base = 0;
        if (id >= 0) base = h[id];
        __syncwarp();
        if (id >= 0 && rank == 0) h[id] = base + __popc(peers);
        __syncwarp();
        if (id >= 0) {
            const int32_t pos = cta_base[id] + base + rank;
            const int32_t prow = s_pad[id] + pos;
            sorted_scattered_idxs[s_off[id] - s_cnt[id] + pos] = i;
            row_src[prow] = i;
            inv_row[i] = prow;
        }
    }
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// CTAs of the cluster index_small_kernel can run with on this device (16 with the non-portable opt-in,
// else 8, else 1 = a single block without a cluster), cached per id type and device.
template <typename IdT>
int index_small_max_ctas() {
    constexpr int kMaxDevices = 64;
    static int cached[kMaxDevices];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 1;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] != 0) return cached[dev];
    auto kernel = index_small_kernel<IdT>;
    const size_t smem = (static_cast<size_t>(kSmallWarps + 5) * kSmallMaxExperts + 1) * sizeof(int32_t) +
                        static_cast<size_t>(kSmallIdsPerCta) * sizeof(uint16_t);
    int found = 1;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) == cudaSuccess) {
        const bool allow16 = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        for (int ctas : {16, 8}) {
            if (ctas == 16 && !allow16) continue;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
            cfg.blockDim = dim3(kSmallWarps * 32, 1, 1);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = static_cast<unsigned>(ctas);
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters >= 1) {
                found = ctas;
                break;
            }
        }
    } else {
        found = -1;  // not even one block with the parked ids: the five-kernel form serves everything
    }
    cudaGetLastError();
    cached[dev] = found;
    return found;
}

template <typename T>
int launch_topk(const void* logits, int64_t num_tokens, int num_experts, int top_k, void* weights, float* probs,
                int64_t* selected, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>(ceil_div(num_tokens, kRouterWarps));
    const int vpl = static_cast<int>(ceil_div(num_experts, 32));
#define XMA_TOPK_CASE(V)                                                                              \
    router_topk_softmax_kernel<T, V><<<grid, kRouterWarps * 32, 0, stream>>>(                         \
        static_cast<const T*>(logits), num_tokens, num_experts, top_k, static_cast<T*>(weights), probs, selected)
    if (vpl <= 1) XMA_TOPK_CASE(1);
    else if (vpl <= 2) XMA_TOPK_CASE(2);
    else if (vpl <= 4) XMA_TOPK_CASE(4);
    else if (vpl <= 8) XMA_TOPK_CASE(8);
    else if (vpl <= 16) XMA_TOPK_CASE(16);
    else XMA_TOPK_CASE(32);
#undef XMA_TOPK_CASE
    return launch_status();
}

template <typename T>
int launch_topk_backward(const void* d_weights, const float* probs, const int64_t* selected, int64_t num_tokens,
                         int num_experts, int top_k, void* d_logits, cudaStream_t stream) {
    const unsigned grid = static_cast<unsigned>(ceil_div(num_tokens, kRouterWarps));
    const int vpl = static_cast<int>(ceil_div(num_experts, 32));
#define XMA_TOPK_BWD_CASE(V)                                                                          \
    router_topk_softmax_backward_kernel<T, V><<<grid, kRouterWarps * 32, 0, stream>>>(                \
        static_cast<const T*>(d_weights), probs, selected, num_tokens, num_experts, top_k, static_cast<T*>(d_logits))
    if (vpl <= 1) XMA_TOPK_BWD_CASE(1);
    else if (vpl <= 2) XMA_TOPK_BWD_CASE(2);
    else if (vpl <= 4) XMA_TOPK_BWD_CASE(4);
    else if (vpl <= 8) XMA_TOPK_BWD_CASE(8);
    else if (vpl <= 16) XMA_TOPK_BWD_CASE(16);
    else XMA_TOPK_BWD_CASE(32);
#undef XMA_TOPK_BWD_CASE
    return launch_status();
}

// Largest cluster the device runs for `kernel` with this much shared memory, trying 16 CTAs (needs the
// non-portable opt-in) and then 8; 0 when neither can be scheduled. Cached per kernel and device.
template <typename Kernel>
int count_cluster_ctas(Kernel kernel, size_t smem) {
    constexpr int kMaxDevices = 64;
    static int cached[kMaxDevices];
    static size_t cached_smem[kMaxDevices];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] != 0 && cached_smem[dev] >= smem) return cached[dev] < 0 ? 0 : cached[dev];
    int found = -1;
    const bool allow16 = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
    if (!allow16) cudaGetLastError();
    for (int ctas : {16, 8}) {
        if (ctas == 16 && !allow16) continue;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
        cfg.blockDim = dim3(kCountThreads, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = static_cast<unsigned>(ctas);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters >= 1) {
            found = ctas;
            break;
        }
        cudaGetLastError();
    }
    cached[dev] = found;
    cached_smem[dev] = smem;
    return found < 0 ? 0 : found;
}

template <typename IdT, int kMode>
int launch_count_mode(const IdT* ids, int64_t n, uint32_t* out, int bins, int reps, int stride, size_t words,
                      cudaStream_t stream) {
    constexpr int kPerVec = 16 / sizeof(IdT);
    // Elements before the first 16-byte boundary are read with scalar loads.
    const uintptr_t addr = reinterpret_cast<uintptr_t>(ids);
    int64_t head = static_cast<int64_t>(((16 - (addr & 15)) & 15) / sizeof(IdT));
    if (head > n) head = n;
    const int64_t nvec = (n - head) / kPerVec;

    if (n <= kCountClusterMaxIds) {
        auto kernel = continuous_count_kernel<IdT, kMode, true>;
        const size_t smem = (words + static_cast<size_t>(bins)) * sizeof(uint32_t);
        bool ok = true;
        if (smem > 48 * 1024)
            ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) == cudaSuccess;
        int ctas = ok ? count_cluster_ctas(kernel, smem) : 0;
        if (ctas > 0) {
            // One CTA per 8192 ids (one round of four 16-byte loads per thread), up to the whole cluster.
            while (ctas > 1 && static_cast<int64_t>(ctas / 2) * 8192 >= n) ctas /= 2;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
            cfg.blockDim = dim3(kCountThreads, 1, 1);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = static_cast<unsigned>(ctas);
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaLaunchKernelEx(&cfg, kernel, ids, n, out, bins, reps, stride, head, nvec) == cudaSuccess)
                return launch_status();
            cudaGetLastError();  // fall through to the grid form
        } else {
            cudaGetLastError();
        }
    }
    auto kernel = continuous_count_kernel<IdT, kMode, false>;
    const size_t smem = words * sizeof(uint32_t);
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
            return XMA_ERR_UNSUPPORTED;
    }
    int64_t blocks = ceil_div(nvec > 0 ? nvec : 1, static_cast<int64_t>(kCountThreads) * 4);
    const int64_t max_blocks = static_cast<int64_t>(sm_count()) * (smem > 56 * 1024 ? 1 : 4);
    if (blocks > max_blocks) blocks = max_blocks;
    if (blocks < 1) blocks = 1;
    if (cudaMemsetAsync(out, 0, sizeof(uint32_t) * bins, stream) != cudaSuccess) return XMA_ERR_LAUNCH;
    kernel<<<static_cast<unsigned>(blocks), kCountThreads, smem, stream>>>(ids, n, out, bins, reps, stride, head, nvec);
    return launch_status();
}

template <typename IdT>
int launch_count(const void* ids_v, int64_t n, uint32_t* out, int bins, cudaStream_t stream) {
    const IdT* ids = static_cast<const IdT*>(ids_v);
    if (bins <= kCountPackedBins)
        return launch_count_mode<IdT, kCountPacked>(ids, n, out, bins, 1, 1, static_cast<size_t>(bins), stream);
    if (bins <= kCountLaneBins)
        return launch_count_mode<IdT, kCountLane>(ids, n, out, bins, 32, 1, static_cast<size_t>(bins) * 32, stream);
    int reps = 32;
    while (reps > 1 && static_cast<int64_t>(reps) * (bins | 1) > kCountMaxSmemEntries) reps >>= 1;
    const int stride = bins | 1;
    return launch_count_mode<IdT, kCountReplicated>(ids, n, out, bins, reps, stride, static_cast<size_t>(reps) * stride, stream);
}

template <typename IdT>
int launch_index_build(const void* ids_v, int64_t n, int num_experts, uint32_t* expert_frequency,
                       int32_t* expert_offsets, int32_t* sorted_expert_idxs, int32_t* sorted_scattered_idxs,
                       int32_t* padded_offsets, int32_t* row_src, int32_t* inv_row, int32_t* tile_expert,
                       int block_m, void* workspace, cudaStream_t stream) {
    const IdT* ids = static_cast<const IdT*>(ids_v);
    // One cluster launch while the ids fit the shared memory of the largest cluster the device runs.
    const int max_ctas = num_experts <= kSmallMaxExperts ? index_small_max_ctas<IdT>() : -1;
    if (n > 0 && max_ctas > 0 && n <= static_cast<int64_t>(max_ctas) * kSmallIdsPerCta) {
        int ctas = 1;
        while (static_cast<int64_t>(ctas) * 8192 < n && ctas < max_ctas) ctas *= 2;  // ~256 ids per warp
        const int32_t total_warps = ctas * kSmallWarps;
        const int32_t seg_len = ((static_cast<int32_t>(n) + total_warps - 1) / total_warps + 31) / 32 * 32;
        const int64_t cap_small = xma_padded_capacity(n, num_experts, block_m);
        const size_t smem_small = (static_cast<size_t>(kSmallWarps + 5) * num_experts + 1) * sizeof(int32_t) +
                                  static_cast<size_t>(kSmallWarps) * seg_len * sizeof(uint16_t);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
        cfg.blockDim = dim3(kSmallWarps * 32, 1, 1);
        cfg.dynamicSmemBytes = smem_small;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = static_cast<unsigned>(ctas);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, index_small_kernel<IdT>, ids, static_cast<int32_t>(n), num_experts,
                               static_cast<int>(block_m), cap_small, static_cast<int>(cap_small / block_m), expert_frequency,
                               expert_offsets, sorted_expert_idxs, sorted_scattered_idxs, padded_offsets, row_src, inv_row,
                               tile_expert) != cudaSuccess) {
            cudaGetLastError();
            return XMA_ERR_LAUNCH;
        }
        return launch_status();
    }
    const IndexPlan plan = index_plan(n);
    int32_t* seg_hist = static_cast<int32_t*>(workspace);
    int32_t* seg_base = seg_hist + static_cast<int64_t>(plan.segs) * num_experts;
    const int64_t cap = xma_padded_capacity(n, num_experts, block_m);
    const int max_tiles = static_cast<int>(cap / block_m);
    const unsigned seg_blocks = static_cast<unsigned>(ceil_div(plan.segs, kIndexWarps));
    const size_t smem = static_cast<size_t>(kIndexWarps) * num_experts * sizeof(int32_t);

    index_hist_kernel<IdT><<<seg_blocks, kIndexWarps * 32, smem, stream>>>(ids, n, num_experts, plan.segs,
                                                                          plan.seg_len, seg_hist);
    index_scan_kernel<<<static_cast<unsigned>(num_experts), kScanThreads, 0, stream>>>(seg_hist, seg_base, num_experts,
                                                                                      plan.segs, expert_frequency);
    index_offsets_kernel<<<1, kMaxExperts, 0, stream>>>(expert_frequency, num_experts, block_m, expert_offsets,
                                                       padded_offsets, tile_expert, max_tiles);
    int64_t fill_blocks = ceil_div(cap, 256 * 4);
    const int64_t max_fill = static_cast<int64_t>(sm_count()) * 8;
    if (fill_blocks > max_fill) fill_blocks = max_fill;
    index_fill_kernel<<<static_cast<unsigned>(fill_blocks), 256, 0, stream>>>(
        expert_frequency, expert_offsets, padded_offsets, num_experts, n, cap, block_m, row_src, sorted_expert_idxs,
        tile_expert);
    if (n > 0) {
        const size_t staged_smem =
            (static_cast<size_t>(kStagedWarps) * (kStagedSegLen + 4 * num_experts) + 2 * num_experts) * sizeof(int32_t);
        bool staged = plan.seg_len <= kStagedSegLen;
        if (staged && staged_smem > 48 * 1024)
            staged = cudaFuncSetAttribute(index_scatter_staged_kernel<IdT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(staged_smem)) == cudaSuccess;
        if (staged) {
            index_scatter_staged_kernel<IdT><<<static_cast<unsigned>(ceil_div(plan.segs, kStagedWarps)),
                                               kStagedWarps * 32, staged_smem, stream>>>(
                ids, n, num_experts, plan.segs, plan.seg_len, seg_hist, seg_base, expert_offsets, expert_frequency,
                padded_offsets, sorted_scattered_idxs, row_src, inv_row);
        } else {
            index_scatter_kernel<IdT><<<seg_blocks, kIndexWarps * 32, smem, stream>>>(
                ids, n, num_experts, plan.segs, plan.seg_len, seg_base, expert_offsets, expert_frequency,
                padded_offsets, sorted_scattered_idxs, row_src, inv_row);
        }
    }
    return launch_status();
}

// ------------------------------------------------------------------------------------------------
// Built-in scratch for xma_moe_index_build_static
//
// Some hosts of this library may not allocate device memory at all: a plugin running inside a
// serving process whose memory pool is sized and frozen at start-up, or code that runs where the
// allocator must not be entered (a callback on a stream, a region being recorded into a graph by
// the caller). For them the per-segment histograms of the counting sort live in this fixed array
// instead of a caller-provided workspace. Every GPU that loads the library holds the array
// (kStaticScratchElems * 4 bytes = 4 MiB) until the process exits.
// ------------------------------------------------------------------------------------------------

constexpr int64_t kStaticScratchElems = int64_t(1) << 20;
static __device__ __align__(256) int32_t g_index_scratch[kStaticScratchElems];

// In host code `g_index_scratch` is only a handle for the runtime, not a device address: the
// address the kernels can use comes from cudaGetSymbolAddress, looked up once per device with
// that device current.
static int static_scratch_address(int32_t** out) {
    constexpr int kMaxDevices = 64;
    static int32_t* cached[kMaxDevices];
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return XMA_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        int32_t* ptr = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_index_scratch) != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();  // leave no sticky error behind
            return XMA_ERR_LAUNCH;
        }
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return XMA_OK;
}

}  // namespace xma

extern "C" {

int64_t xma_padded_capacity(int64_t n, int32_t num_experts, int32_t block_m) {
    if (n < 0) n = 0;
    if (block_m < 1) block_m = 1;
    return (xma::ceil_div(n, block_m) + num_experts) * block_m;
}

int64_t xma_moe_index_small_limit(void) {
    const int ctas = xma::index_small_max_ctas<int32_t>();
    const int ctas64 = xma::index_small_max_ctas<int64_t>();
    const int least = ctas < ctas64 ? ctas : ctas64;
    return least > 0 ? static_cast<int64_t>(least) * xma::kSmallIdsPerCta : 0;
}

int64_t xma_moe_index_workspace_bytes(int64_t n, int32_t num_experts) {
    const xma::IndexPlan plan = xma::index_plan(n);
    return (2 * static_cast<int64_t>(plan.segs) * num_experts + 64) * static_cast<int64_t>(sizeof(int32_t));
}

int xma_continuous_count(const void* ids, int32_t id_is_int64, int64_t n, uint32_t* out, int32_t bins, void* stream) {
    if (out == nullptr || bins <= 0 || n < 0 || (n > 0 && ids == nullptr)) return XMA_ERR_BAD_ARG;
    if (bins > 16384) return XMA_ERR_UNSUPPORTED;  // same ceiling as forward.cu:12 of the reference op
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return id_is_int64 ? xma::launch_count<int64_t>(ids, n, out, bins, s) : xma::launch_count<int32_t>(ids, n, out, bins, s);
}

int xma_router_topk_softmax(const void* logits, int32_t dtype, int64_t num_tokens, int32_t num_experts, int32_t top_k,
                            void* topk_weights, float* topk_probs_f32, int64_t* selected, void* stream) {
    if (num_tokens < 0 || num_experts <= 0 || top_k <= 0) return XMA_ERR_BAD_ARG;
    if (top_k > 32 || top_k > num_experts || num_experts > xma::kMaxExperts) return XMA_ERR_UNSUPPORTED;
    if (num_tokens == 0) return XMA_OK;
    if (!logits || !topk_weights || !topk_probs_f32 || !selected) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case xma::kDtypeBF16:
            return xma::launch_topk<__nv_bfloat16>(logits, num_tokens, num_experts, top_k, topk_weights, topk_probs_f32, selected, s);
        case xma::kDtypeF16:
            return xma::launch_topk<__half>(logits, num_tokens, num_experts, top_k, topk_weights, topk_probs_f32, selected, s);
        case xma::kDtypeF32:
            return xma::launch_topk<float>(logits, num_tokens, num_experts, top_k, topk_weights, topk_probs_f32, selected, s);
        default:
            return XMA_ERR_UNSUPPORTED;
    }
}

int xma_router_topk_softmax_backward(const void* d_weights, int32_t dtype, const float* topk_probs_f32,
                                     const int64_t* selected, int64_t num_tokens, int32_t num_experts, int32_t top_k,
                                     void* d_logits, void* stream) {
    if (num_tokens < 0 || num_experts <= 0 || top_k <= 0) return XMA_ERR_BAD_ARG;
    if (top_k > 32 || top_k > num_experts || num_experts > xma::kMaxExperts) return XMA_ERR_UNSUPPORTED;
    if (num_tokens == 0) return XMA_OK;
    if (!d_weights || !topk_probs_f32 || !selected || !d_logits) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case xma::kDtypeBF16:
            return xma::launch_topk_backward<__nv_bfloat16>(d_weights, topk_probs_f32, selected, num_tokens, num_experts, top_k, d_logits, s);
        case xma::kDtypeF16:
            return xma::launch_topk_backward<__half>(d_weights, topk_probs_f32, selected, num_tokens, num_experts, top_k, d_logits, s);
        case xma::kDtypeF32:
            return xma::launch_topk_backward<float>(d_weights, topk_probs_f32, selected, num_tokens, num_experts, top_k, d_logits, s);
        default:
            return XMA_ERR_UNSUPPORTED;
    }
}

int xma_moe_index_build(const void* ids, int32_t id_is_int64, int64_t n, int32_t num_experts,
                        uint32_t* expert_frequency, int32_t* expert_offsets, int32_t* sorted_expert_idxs,
                        int32_t* sorted_scattered_idxs, int32_t* padded_offsets, int32_t* row_src, int32_t* inv_row,
                        int32_t* tile_expert, int32_t block_m, void* workspace, void* stream) {
    if (n < 0 || num_experts <= 0 || block_m < 1) return XMA_ERR_BAD_ARG;
    if (num_experts > xma::kMaxExperts || n >= (int64_t(1) << 31) - (int64_t(num_experts) + 1) * block_m - 8)
        return XMA_ERR_UNSUPPORTED;
    if (!expert_frequency || !expert_offsets || !padded_offsets || !row_src || !workspace) return XMA_ERR_BAD_ARG;
    if (n > 0 && (!ids || !sorted_scattered_idxs || !inv_row)) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return id_is_int64 ? xma::launch_index_build<int64_t>(ids, n, num_experts, expert_frequency, expert_offsets,
                                                          sorted_expert_idxs, sorted_scattered_idxs, padded_offsets,
                                                          row_src, inv_row, tile_expert, block_m, workspace, s)
                       : xma::launch_index_build<int32_t>(ids, n, num_experts, expert_frequency, expert_offsets,
                                                          sorted_expert_idxs, sorted_scattered_idxs, padded_offsets,
                                                          row_src, inv_row, tile_expert, block_m, workspace, s);
}

int xma_moe_index_build_static(const void* ids, int32_t id_is_int64, int64_t n, int32_t num_experts,
                               uint32_t* expert_frequency, int32_t* expert_offsets, int32_t* sorted_expert_idxs,
                               int32_t* sorted_scattered_idxs, int32_t* padded_offsets, int32_t* row_src,
                               int32_t* inv_row, int32_t* tile_expert, int32_t block_m, void* stream) {
    if (n < 0 || num_experts <= 0) return XMA_ERR_BAD_ARG;
    // The scratch need is known from the sizes alone; refuse before touching the device.
    if (xma_moe_index_workspace_bytes(n, num_experts) > xma_moe_index_static_scratch_bytes())
        return XMA_ERR_SCRATCH_TOO_SMALL;
    int32_t* scratch = nullptr;
    const int rc = xma::static_scratch_address(&scratch);
    if (rc != XMA_OK) return rc;
    // Every histogram entry a call reads is written by the same call first (index_hist_kernel fills
    // all segs * num_experts counters it uses), so what an earlier call left behind never matters
    // and nothing has to be cleared.
    return xma_moe_index_build(ids, id_is_int64, n, num_experts, expert_frequency, expert_offsets, sorted_expert_idxs,
                               sorted_scattered_idxs, padded_offsets, row_src, inv_row, tile_expert, block_m, scratch,
                               stream);
}

int64_t xma_moe_index_static_scratch_bytes(void) {
    return xma::kStaticScratchElems * static_cast<int64_t>(sizeof(int32_t));
}

}  // extern "C"
