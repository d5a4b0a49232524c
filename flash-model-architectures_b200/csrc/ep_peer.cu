// Expert-parallel dispatch and combine over NVLink peer memory (one process per GPU, buffers of the
// other ranks mapped into this process). The token gather and the send are ONE kernel: a warp reads
// a token row once and stores its k copies straight into the destination ranks' row buffers, at the
// row where the destination's grouped GEMM expects it (padded expert order, grouped by source rank
// inside an expert). The way back is a pull: the combine kernel sums a token's k result rows from
// the owners' buffers with plain peer loads. No multicast, no TMA on peer memory. Ranks meet at
// ep_barrier_kernel / ep_exchange_counts_kernel: every rank stores a sequence number into a flag word
// of every peer and waits, with a time limit, until its own flag words have reached that number. A
// wait that runs out writes a code into the caller's status word and the kernel returns; the data
// kernels never wait for anything.
#include <limits.h>

#include "common.cuh"

namespace xma {

constexpr int kEpWarps = 8;
constexpr int kEpUnroll = 4;

// counts_all[s][e]: rows rank s routes to global expert e. Experts are owned in contiguous blocks of
// experts_per_rank. For every global expert e, owned by rank d as local expert el:
//   total[e]        = sum_s counts_all[s][e]
//   offsets_d[el]   = sum over d's earlier local experts of roundup(total, XMA_BLOCK_M)
//   dest_base[e]    = offsets_d[el] + sum_{s < rank} counts_all[s][e]   (where THIS rank's rows for e start)
// and for this rank as an owner: local_padded_offsets[0..experts_per_rank], local_totals[el].
//
// counts_all rows are `row_stride` ints apart; entry num_experts of a row, when row_stride allows it,
// is that rank's buffer generation. The plan is refused (status code, every dest_base entry negative,
// no local rows) when the generations differ or when some owner would receive more padded rows than
// `cap`: the dispatch kernel then stores nothing and nobody writes past a buffer.
constexpr int kEpCodeGeneration = 301;  // ranks sized their buffers in different calls
constexpr int kEpCodeOverflow = 302;    // an owner would receive more rows than its buffers hold
constexpr int kEpCodeRowRange = 303;    // a dispatch or pull met a row outside [0, cap)
constexpr int kEpCodeBarrier = 304;     // a rank did not reach a barrier within the time limit
constexpr int32_t kEpRefusedRow = INT32_MIN / 2;

__global__ void __launch_bounds__(kMaxExperts)
ep_plan_kernel(const int32_t* __restrict__ counts_all, int row_stride, int world, int rank, int num_experts,
               int experts_per_rank, int64_t cap, int32_t* __restrict__ local_padded_offsets,
               int32_t* __restrict__ local_totals, int32_t* __restrict__ dest_base, int32_t* __restrict__ status) {
    __shared__ int32_t s_padded[kMaxExperts];
    __shared__ int s_refused;
    const int e = threadIdx.x;
    if (e == 0) s_refused = 0;
    int32_t total = 0, before_me = 0;
    if (e < num_experts) {
        for (int s = 0; s < world; ++s) {
            const int32_t c = counts_all[s * row_stride + e];
            if (s < rank) before_me += c;
            total += c;
        }
    }
    s_padded[e] = (total + XMA_BLOCK_M - 1) / XMA_BLOCK_M * XMA_BLOCK_M;
    __syncthreads();
    const int owner = e / experts_per_rank, el = e - owner * experts_per_rank;
    int32_t offset = 0;
    if (e < num_experts) {
        for (int i = owner * experts_per_rank; i < e; ++i) offset += s_padded[i];
        if (el == experts_per_rank - 1 && static_cast<int64_t>(offset) + s_padded[e] > cap) {
            s_refused = 1;
            if (status != nullptr) atomicCAS(status, 0, kEpCodeOverflow);
        }
    }
    if (row_stride > num_experts && e < world && counts_all[e * row_stride + num_experts] != counts_all[rank * row_stride + num_experts]) {
        s_refused = 1;
        if (status != nullptr) atomicCAS(status, 0, kEpCodeGeneration);
    }
    __syncthreads();
    if (e >= num_experts) return;
    const bool refused = s_refused != 0;
    dest_base[e] = refused ? kEpRefusedRow : offset + before_me;
    if (owner == rank) {
        local_padded_offsets[el] = refused ? 0 : offset;
        local_totals[el] = refused ? 0 : total;
        if (el == experts_per_rank - 1) local_padded_offsets[experts_per_rank] = refused ? 0 : offset + s_padded[e];
    }
}

__device__ __forceinline__ uint64_t ep_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Thread r < world of the calling block: tell rank r that this rank reached barrier `seq`, then wait
// until rank r said the same. flags are int32[world] per rank (peer_flags[r] = rank r's array as
// mapped here); rank s writes entry s of every array. Sequence numbers only grow (compared modulo
// 2^32). Returns false when the wait ran out.
__device__ __forceinline__ bool ep_meet(const int64_t* __restrict__ peer_flags, int rank, int world, int32_t seq,
                                        uint64_t limit_ns, int32_t* status) {
    const int r = threadIdx.x;
    if (r >= world) return true;
    int32_t* theirs = reinterpret_cast<int32_t*>(peer_flags[r]) + rank;
    const int32_t* mine = reinterpret_cast<const int32_t*>(peer_flags[rank]) + r;
    __threadfence_system();
    asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(theirs), "r"(seq) : "memory");
    const uint64_t start = ep_timer_ns();
    uint32_t spins = 0;
    for (;;) {
        int32_t seen;
        asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if (seen - seq >= 0) return true;
        if ((++spins & 0x3fu) == 0 && ep_timer_ns() - start > limit_ns) {
            if (status != nullptr) atomicCAS(status, 0, kEpCodeBarrier);
            return false;
        }
        __nanosleep(100);
    }
}

__global__ void __launch_bounds__(32)
ep_barrier_kernel(const int64_t* __restrict__ peer_flags, int rank, int world, int32_t seq, uint64_t limit_ns,
                  int32_t* __restrict__ status) {
    ep_meet(peer_flags, rank, world, seq, limit_ns, status);
}

// All-gather of one short row of ints per rank without a library collective: every rank stores its
// row (counts[0..num_counts) followed by `tag`) into slot `rank` of every peer's table, then the ranks
// meet. When the kernel ends this rank's table holds every rank's row.
__global__ void __launch_bounds__(256)
ep_exchange_counts_kernel(const int32_t* __restrict__ counts, int num_counts, int32_t tag,
                          const int64_t* __restrict__ peer_tables, const int64_t* __restrict__ peer_flags, int rank,
                          int world, int32_t seq, uint64_t limit_ns, int32_t* __restrict__ status) {
    const int row_len = num_counts + 1;
    for (int i = threadIdx.x; i < world * row_len; i += blockDim.x) {
        const int r = i / row_len, j = i - r * row_len;
        reinterpret_cast<int32_t*>(peer_tables[r])[rank * row_len + j] = j < num_counts ? counts[j] : tag;
    }
    __threadfence_system();
    __syncthreads();
    if (!ep_meet(peer_flags, rank, world, seq, limit_ns, status) && threadIdx.x < world) {
        // Rank threadIdx.x never arrived: its slot may hold an older call's counts. Spoil its tag so that
        // the plan built from this table is refused and nothing is sent anywhere.
        reinterpret_cast<int32_t*>(peer_tables[rank])[threadIdx.x * row_len + num_counts] = tag - 1;
    }
}

// row_src[r] = r for rows that receive a routed row, -1 for padding rows (and rows past the rows in
// use); padding rows inside the rows in use are zeroed in `rows` (and in `rows2` when given).
template <typename T>
__global__ void __launch_bounds__(kEpWarps * 32)
ep_prepare_rows_kernel(const int32_t* __restrict__ local_padded_offsets, const int32_t* __restrict__ local_totals,
                       int experts_per_rank, int64_t cap, int64_t cols, int32_t* __restrict__ row_src,
                       T* __restrict__ rows, T* __restrict__ rows2) {
    __shared__ int32_t s_off[kMaxExperts + 1];
    for (int i = threadIdx.x; i <= experts_per_rank; i += blockDim.x) s_off[i] = local_padded_offsets[i];
    __syncthreads();
    constexpr int kPer = Vec16<T>::kCount;
    const int lane = threadIdx.x & 31;
    const int64_t nvec = cols / kPer;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * kEpWarps;
    const int64_t in_use = s_off[experts_per_rank];
    Vec16<T> z;
#pragma unroll
    for (int j = 0; j < kPer; ++j) z.v[j] = Elem<T>::from_float(0.f);
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * kEpWarps + (threadIdx.x >> 5); r < cap; r += warps) {
        bool padding = r >= in_use;
        if (!padding) {
            int lo = 0, hi = experts_per_rank - 1;  // largest el with s_off[el] <= r
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (s_off[mid] <= r) lo = mid; else hi = mid - 1;
            }
            padding = r - s_off[lo] >= local_totals[lo];
        }
        if (lane == 0) row_src[r] = padding ? -1 : static_cast<int32_t>(r);
        if (padding && r < in_use) {
            for (int64_t c = lane; c < nvec; c += 32) {
                store16(rows + r * cols + c * kPer, z);
                if (rows2 != nullptr) store16(rows2 + r * cols + c * kPer, z);
            }
        }
    }
}

// Fused gather + send. One warp per token: lane j < top_k works out where copy j goes
//   expert e = selected[t][j], owner d = e / experts_per_rank,
//   row = dest_base[e] + (position of (t, j) among this rank's rows for e),
// records (d, row) for the way back, and the warp then reads the token row once and stores it into
// the k destination buffers (16-byte stores over NVLink for remote owners). `scale`, when given, is
// pushed too: peer_scale[d][row] = scale[t][j].
template <typename T>
__global__ void __launch_bounds__(kEpWarps * 32)
ep_dispatch_rows_kernel(const T* __restrict__ src, int64_t cols, int64_t num_tokens, int top_k,
                        const int64_t* __restrict__ selected, const int32_t* __restrict__ inv_sorted,
                        const int32_t* __restrict__ expert_offsets, const uint32_t* __restrict__ expert_frequency,
                        const int32_t* __restrict__ dest_base, int experts_per_rank,
                        const int64_t* __restrict__ peer_rows, const T* __restrict__ scale,
                        const int64_t* __restrict__ peer_scale, int32_t* __restrict__ dest_rank,
                        int32_t* __restrict__ dest_row, bool record, int64_t cap, int32_t* __restrict__ status,
                        int split) {
    constexpr int kPer = Vec16<T>::kCount;
    const int lane = threadIdx.x & 31;
    const int64_t nvec = cols / kPer;
    // `split` (a power of two dividing kEpWarps) warps share a token, each moving a contiguous part of
    // the row: with few tokens per rank one warp per token leaves the links idle between its rounds.
    const int part = (threadIdx.x >> 5) & (split - 1);
    const int64_t part_len = (nvec + split - 1) / split;
    const int64_t v_begin = part * part_len, v_end = min(v_begin + part_len, nvec);
    const int64_t groups = static_cast<int64_t>(gridDim.x) * (kEpWarps / split);
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * (kEpWarps / split) + ((threadIdx.x >> 5) / split); t < num_tokens;
         t += groups) {
        unsigned long long my_dst = 0;
        if (lane < top_k) {
            const int64_t q = t * top_k + lane;
            int d, row;
            if (record) {
                const int e = static_cast<int>(selected[q]);
                const int32_t first = expert_offsets[e] - static_cast<int32_t>(expert_frequency[e]);
                d = e / experts_per_rank;
                row = dest_base[e] + (inv_sorted[q] - first);
                if (part == 0) {
                    dest_rank[q] = d;
                    dest_row[q] = row;
                }
            } else {
                d = dest_rank[q];
                row = dest_row[q];
            }
            if (row >= 0 && row < cap) {
                my_dst = static_cast<unsigned long long>(peer_rows[d]) + static_cast<unsigned long long>(row) * cols * sizeof(T);
                if (scale != nullptr && part == 0) reinterpret_cast<T*>(peer_scale[d])[row] = scale[q];
            } else if (status != nullptr) {
                atomicCAS(status, 0, kEpCodeRowRange);  // a refused plan: this copy is dropped, nothing is stored
            }
        }
        const T* in = src + t * cols;
        // Same trip count for every lane: the shuffles below need the whole warp.
        for (int64_t base = v_begin; base < v_end; base += 32 * kEpUnroll) {
            const int64_t c0 = base + lane;
            Vec16<T> buf[kEpUnroll];
#pragma unroll
            for (int u = 0; u < kEpUnroll; ++u) {
                const int64_t c = c0 + 32 * u;
                if (c < v_end) buf[u] = load16(in + c * kPer);
            }
            for (int j = 0; j < top_k; ++j) {
                T* out = reinterpret_cast<T*>(__shfl_sync(0xffffffffu, my_dst, j));
                if (out == nullptr) continue;  // warp-uniform
#pragma unroll
                for (int u = 0; u < kEpUnroll; ++u) {
                    const int64_t c = c0 + 32 * u;
                    if (c < v_end) store16(out + c * kPer, buf[u]);
                }
            }
        }
    }
    __threadfence_system();  // the rows are visible to the owners before this kernel counts as done
}

// Fused receive + combine: out[t] = sum_j rows_of_rank(dest_rank[t][j])[dest_row[t][j]], float32 sums,
// plain (peer) loads.
template <typename T>
__global__ void __launch_bounds__(kEpWarps * 32)
ep_combine_pull_kernel(const int64_t* __restrict__ peer_rows, int64_t cols, const int32_t* __restrict__ dest_rank,
                       const int32_t* __restrict__ dest_row, int64_t num_tokens, int top_k, T* __restrict__ out,
                       int64_t cap, int split) {
    constexpr int kPer = Vec16<T>::kCount;
    const int lane = threadIdx.x & 31;
    const int64_t nvec = cols / kPer;
    // `split` warps share a token (see ep_dispatch_rows_kernel): a peer load takes microseconds, and a
    // warp that walks a whole row alone pays that latency once per 512 bytes.
    const int part = (threadIdx.x >> 5) & (split - 1);
    const int64_t part_len = (nvec + split - 1) / split;
    const int64_t v_begin = part * part_len, v_end = min(v_begin + part_len, nvec);
    const int64_t groups = static_cast<int64_t>(gridDim.x) * (kEpWarps / split);
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * (kEpWarps / split) + ((threadIdx.x >> 5) / split); t < num_tokens;
         t += groups) {
        unsigned long long my_src = 0;
        if (lane < top_k) {
            const int64_t q = t * top_k + lane;
            // A row outside the buffer (left by a refused plan) reads this rank's row 0 instead of a
            // wild address; the refusal itself is already in the status word.
            const int32_t row = dest_row[q];
            const bool inside = row >= 0 && row < cap;
            my_src = static_cast<unsigned long long>(peer_rows[inside ? dest_rank[q] : 0]) +
                     static_cast<unsigned long long>(inside ? row : 0) * cols * sizeof(T);
        }
        T* o = out + t * cols;
        // Same trip count for every lane (the shuffles need the whole warp); lanes past the last
        // vector read column 0 again and store nothing.
        for (int64_t base = v_begin; base < v_end; base += 32) {
            const bool live = base + lane < v_end;
            const int64_t c = live ? base + lane : 0;
            float acc[kPer];
#pragma unroll
            for (int j = 0; j < kPer; ++j) acc[j] = 0.f;
            int s = 0;
            for (; s + 2 <= top_k; s += 2) {
                const T* r0 = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, my_src, s));
                const T* r1 = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, my_src, s + 1));
                Vec16<T> a, b;
                *reinterpret_cast<uint4*>(&a) = *reinterpret_cast<const uint4*>(r0 + c * kPer);
                *reinterpret_cast<uint4*>(&b) = *reinterpret_cast<const uint4*>(r1 + c * kPer);
#pragma unroll
                for (int j = 0; j < kPer; ++j) acc[j] += Elem<T>::to_float(a.v[j]) + Elem<T>::to_float(b.v[j]);
            }
            for (; s < top_k; ++s) {
                const T* r0 = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, my_src, s));
                Vec16<T> a;
                *reinterpret_cast<uint4*>(&a) = *reinterpret_cast<const uint4*>(r0 + c * kPer);
#pragma unroll
                for (int j = 0; j < kPer; ++j) acc[j] += Elem<T>::to_float(a.v[j]);
            }
            if (live) {
                Vec16<T> r;
#pragma unroll
                for (int j = 0; j < kPer; ++j) r.v[j] = Elem<T>::from_float(acc[j]);
                store16(o + c * kPer, r);
            }
        }
    }
}

// out[q] = float32 word dest_row[q] of rank dest_rank[q]'s array (router-weight gradients on the way back).
__global__ void ep_pull_scalars_kernel(const int64_t* __restrict__ peer_f32, const int32_t* __restrict__ dest_rank,
                                       const int32_t* __restrict__ dest_row, int64_t n, float* __restrict__ out,
                                       int64_t cap) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t q = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; q < n; q += stride) {
        const int32_t row = dest_row[q];
        out[q] = (row >= 0 && row < cap) ? reinterpret_cast<const float*>(peer_f32[dest_rank[q]])[row] : 0.f;
    }
}

// Warps per token for the row movers: enough warps to keep every SM busy (about 32 per SM) while every
// warp still has at least one full round of 32 16-byte vectors.
inline int ep_split(int64_t tokens, int64_t vectors_per_row) {
    int split = 1;
    const int64_t want = static_cast<int64_t>(sm_count()) * 32;
    while (split < kEpWarps && tokens * split < want && vectors_per_row / (2 * split) >= 32) split *= 2;
    return split;
}

inline unsigned ep_grid(int64_t rows) {
    int64_t blocks = ceil_div(rows > 0 ? rows : 1, kEpWarps);
    const int64_t max_blocks = static_cast<int64_t>(sm_count()) * 8;
    return static_cast<unsigned>(blocks > max_blocks ? max_blocks : blocks);
}

}  // namespace xma

#define XMA_EP_DISPATCH(dtype, CALL)                                     \
    switch (dtype) {                                                     \
        case xma::kDtypeBF16: { using T = __nv_bfloat16; CALL; break; }  \
        case xma::kDtypeF16: { using T = __half; CALL; break; }          \
        case xma::kDtypeF32: { using T = float; CALL; break; }           \
        default: return XMA_ERR_UNSUPPORTED;                             \
    }

extern "C" {

int xma_ep_plan(const int32_t* counts_all, int32_t row_stride, int32_t world, int32_t rank, int32_t num_experts,
                int64_t cap, int32_t* local_padded_offsets, int32_t* local_totals, int32_t* dest_base, int32_t* status,
                void* stream) {
    if (!counts_all || !local_padded_offsets || !local_totals || !dest_base) return XMA_ERR_BAD_ARG;
    if (world <= 0 || rank < 0 || rank >= world || num_experts <= 0 || num_experts % world != 0) return XMA_ERR_BAD_ARG;
    if (row_stride < num_experts || cap <= 0) return XMA_ERR_BAD_ARG;
    if (num_experts > xma::kMaxExperts || world > xma::kMaxExperts) return XMA_ERR_UNSUPPORTED;
    xma::ep_plan_kernel<<<1, xma::kMaxExperts, 0, static_cast<cudaStream_t>(stream)>>>(
        counts_all, row_stride, world, rank, num_experts, num_experts / world, cap, local_padded_offsets, local_totals,
        dest_base, status);
    return xma::launch_status();
}

int xma_ep_barrier(const int64_t* peer_flags, int32_t rank, int32_t world, int32_t seq, int64_t limit_ns,
                   int32_t* status, void* stream) {
    if (!peer_flags || world <= 0 || world > 32 || rank < 0 || rank >= world || limit_ns <= 0) return XMA_ERR_BAD_ARG;
    xma::ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(peer_flags, rank, world, seq,
                                                                           static_cast<uint64_t>(limit_ns), status);
    return xma::launch_status();
}

int xma_ep_exchange_counts(const int32_t* counts, int32_t num_counts, int32_t tag, const int64_t* peer_tables,
                           const int64_t* peer_flags, int32_t rank, int32_t world, int32_t seq, int64_t limit_ns,
                           int32_t* status, void* stream) {
    if (!counts || !peer_tables || !peer_flags || num_counts <= 0 || limit_ns <= 0) return XMA_ERR_BAD_ARG;
    if (world <= 0 || world > 32 || rank < 0 || rank >= world) return XMA_ERR_BAD_ARG;
    xma::ep_exchange_counts_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        counts, num_counts, tag, peer_tables, peer_flags, rank, world, seq, static_cast<uint64_t>(limit_ns), status);
    return xma::launch_status();
}

int xma_ep_prepare_rows(const int32_t* local_padded_offsets, const int32_t* local_totals, int32_t experts_per_rank,
                        int64_t cap, int32_t dtype, int64_t cols, int32_t* row_src, void* rows, void* rows2,
                        void* stream) {
    if (!local_padded_offsets || !local_totals || !row_src || !rows || cap <= 0 || experts_per_rank <= 0)
        return XMA_ERR_BAD_ARG;
    if (experts_per_rank > xma::kMaxExperts || cols <= 0 || (cols * xma::dtype_size(dtype)) % 16 != 0)
        return XMA_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    XMA_EP_DISPATCH(dtype, (xma::ep_prepare_rows_kernel<T><<<xma::ep_grid(cap), xma::kEpWarps * 32, 0, s>>>(
                               local_padded_offsets, local_totals, experts_per_rank, cap, cols, row_src,
                               static_cast<T*>(rows), static_cast<T*>(rows2))));
    return xma::launch_status();
}

int xma_ep_dispatch_rows(const void* src, int32_t dtype, int64_t cols, int64_t num_tokens, int32_t top_k,
                         const int64_t* selected, const int32_t* inv_sorted, const int32_t* expert_offsets,
                         const uint32_t* expert_frequency, const int32_t* dest_base, int32_t experts_per_rank,
                         const int64_t* peer_rows, const void* scale, const int64_t* peer_scale, int32_t* dest_rank,
                         int32_t* dest_row, int32_t record, int64_t cap, int32_t* status, void* stream) {
    if (num_tokens < 0 || top_k <= 0 || experts_per_rank <= 0 || cap <= 0) return XMA_ERR_BAD_ARG;
    if (top_k > 32 || cols <= 0 || (cols * xma::dtype_size(dtype)) % 16 != 0) return XMA_ERR_UNSUPPORTED;
    if (num_tokens == 0) return XMA_OK;
    if (!src || !peer_rows || !dest_rank || !dest_row || (scale && !peer_scale)) return XMA_ERR_BAD_ARG;
    if (record && (!selected || !inv_sorted || !expert_offsets || !expert_frequency || !dest_base)) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int split = xma::ep_split(num_tokens, cols * xma::dtype_size(dtype) / 16);
    XMA_EP_DISPATCH(dtype, (xma::ep_dispatch_rows_kernel<T><<<xma::ep_grid(num_tokens * split), xma::kEpWarps * 32, 0, s>>>(
                               static_cast<const T*>(src), cols, num_tokens, top_k, selected, inv_sorted, expert_offsets,
                               expert_frequency, dest_base, experts_per_rank, peer_rows, static_cast<const T*>(scale),
                               peer_scale, dest_rank, dest_row, record != 0, cap, status, split)));
    return xma::launch_status();
}

int xma_ep_combine_pull(const int64_t* peer_rows, int32_t dtype, int64_t cols, const int32_t* dest_rank,
                        const int32_t* dest_row, int64_t num_tokens, int32_t top_k, void* out, int64_t cap, void* stream) {
    if (num_tokens < 0 || top_k <= 0 || cap <= 0) return XMA_ERR_BAD_ARG;
    if (top_k > 32 || cols <= 0 || (cols * xma::dtype_size(dtype)) % 16 != 0) return XMA_ERR_UNSUPPORTED;
    if (num_tokens == 0) return XMA_OK;
    if (!peer_rows || !dest_rank || !dest_row || !out) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int split = xma::ep_split(num_tokens, cols * xma::dtype_size(dtype) / 16);
    XMA_EP_DISPATCH(dtype, (xma::ep_combine_pull_kernel<T><<<xma::ep_grid(num_tokens * split), xma::kEpWarps * 32, 0, s>>>(
                               peer_rows, cols, dest_rank, dest_row, num_tokens, top_k, static_cast<T*>(out), cap, split)));
    return xma::launch_status();
}

int xma_ep_pull_scalars(const int64_t* peer_f32, const int32_t* dest_rank, const int32_t* dest_row, int64_t n,
                        float* out, int64_t cap, void* stream) {
    if (n < 0 || cap <= 0) return XMA_ERR_BAD_ARG;
    if (n == 0) return XMA_OK;
    if (!peer_f32 || !dest_rank || !dest_row || !out) return XMA_ERR_BAD_ARG;
    const int64_t blocks = xma::ceil_div(n, 256);
    xma::ep_pull_scalars_kernel<<<static_cast<unsigned>(blocks > 4096 ? 4096 : blocks), 256, 0,
                                  static_cast<cudaStream_t>(stream)>>>(peer_f32, dest_rank, dest_row, n, out, cap);
    return xma::launch_status();
}

}  // extern "C"
