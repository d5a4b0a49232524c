// Expert-parallel dispatch and combine over NVLink peer memory (one process per GPU, buffers of the
// other ranks mapped into this process). The token gather and the send are ONE kernel: a warp reads
// a token row once and stores its k copies straight into the destination ranks' row buffers, at the
// row where the destination's grouped GEMM expects it (padded expert order, grouped by source rank
// inside an expert). The way back is a pull: the combine kernel sums a token's k result rows from
// the owners' buffers with plain peer loads. No multicast, no TMA on peer memory; every kernel here
// runs to completion on its own (no kernel waits for another rank) and ranks meet at stream-ordered
// collectives issued by the host between phases.
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
__global__ void __launch_bounds__(kMaxExperts)
ep_plan_kernel(const int32_t* __restrict__ counts_all, int world, int rank, int num_experts, int experts_per_rank,
               int32_t* __restrict__ local_padded_offsets, int32_t* __restrict__ local_totals,
               int32_t* __restrict__ dest_base) {
    __shared__ int32_t s_padded[kMaxExperts];
    const int e = threadIdx.x;
    int32_t total = 0, before_me = 0;
    if (e < num_experts) {
        for (int s = 0; s < world; ++s) {
            const int32_t c = counts_all[s * num_experts + e];
            if (s < rank) before_me += c;
            total += c;
        }
    }
    s_padded[e] = (total + XMA_BLOCK_M - 1) / XMA_BLOCK_M * XMA_BLOCK_M;
    __syncthreads();
    if (e >= num_experts) return;
    const int owner = e / experts_per_rank, el = e - owner * experts_per_rank;
    int32_t offset = 0;
    for (int i = owner * experts_per_rank; i < e; ++i) offset += s_padded[i];
    dest_base[e] = offset + before_me;
    if (owner == rank) {
        local_padded_offsets[el] = offset;
        local_totals[el] = total;
        if (el == experts_per_rank - 1) local_padded_offsets[experts_per_rank] = offset + s_padded[e];
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
                        int32_t* __restrict__ dest_row, bool record) {
    constexpr int kPer = Vec16<T>::kCount;
    const int lane = threadIdx.x & 31;
    const int64_t nvec = cols / kPer;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * kEpWarps;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * kEpWarps + (threadIdx.x >> 5); t < num_tokens; t += warps) {
        unsigned long long my_dst = 0;
        if (lane < top_k) {
            const int64_t q = t * top_k + lane;
            int d, row;
            if (record) {
                const int e = static_cast<int>(selected[q]);
                const int32_t first = expert_offsets[e] - static_cast<int32_t>(expert_frequency[e]);
                d = e / experts_per_rank;
                row = dest_base[e] + (inv_sorted[q] - first);
                dest_rank[q] = d;
                dest_row[q] = row;
            } else {
                d = dest_rank[q];
                row = dest_row[q];
            }
            my_dst = static_cast<unsigned long long>(peer_rows[d]) + static_cast<unsigned long long>(row) * cols * sizeof(T);
            if (scale != nullptr) reinterpret_cast<T*>(peer_scale[d])[row] = scale[q];
        }
        const T* in = src + t * cols;
        // Same trip count for every lane: the shuffles below need the whole warp.
        for (int64_t base = 0; base < nvec; base += 32 * kEpUnroll) {
            const int64_t c0 = base + lane;
            Vec16<T> buf[kEpUnroll];
#pragma unroll
            for (int u = 0; u < kEpUnroll; ++u) {
                const int64_t c = c0 + 32 * u;
                if (c < nvec) buf[u] = load16(in + c * kPer);
            }
            for (int j = 0; j < top_k; ++j) {
                T* out = reinterpret_cast<T*>(__shfl_sync(0xffffffffu, my_dst, j));
#pragma unroll
                for (int u = 0; u < kEpUnroll; ++u) {
                    const int64_t c = c0 + 32 * u;
                    if (c < nvec) store16(out + c * kPer, buf[u]);
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
                       const int32_t* __restrict__ dest_row, int64_t num_tokens, int top_k, T* __restrict__ out) {
    constexpr int kPer = Vec16<T>::kCount;
    const int lane = threadIdx.x & 31;
    const int64_t nvec = cols / kPer;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * kEpWarps;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * kEpWarps + (threadIdx.x >> 5); t < num_tokens; t += warps) {
        unsigned long long my_src = 0;
        if (lane < top_k) {
            const int64_t q = t * top_k + lane;
            my_src = static_cast<unsigned long long>(peer_rows[dest_rank[q]]) +
                     static_cast<unsigned long long>(dest_row[q]) * cols * sizeof(T);
        }
        T* o = out + t * cols;
        // Same trip count for every lane (the shuffles need the whole warp); lanes past the last
        // vector read column 0 again and store nothing.
        for (int64_t base = 0; base < nvec; base += 32) {
            const bool live = base + lane < nvec;
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
                                       const int32_t* __restrict__ dest_row, int64_t n, float* __restrict__ out) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t q = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; q < n; q += stride)
        out[q] = reinterpret_cast<const float*>(peer_f32[dest_rank[q]])[dest_row[q]];
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

int xma_ep_plan(const int32_t* counts_all, int32_t world, int32_t rank, int32_t num_experts,
                int32_t* local_padded_offsets, int32_t* local_totals, int32_t* dest_base, void* stream) {
    if (!counts_all || !local_padded_offsets || !local_totals || !dest_base) return XMA_ERR_BAD_ARG;
    if (world <= 0 || rank < 0 || rank >= world || num_experts <= 0 || num_experts % world != 0) return XMA_ERR_BAD_ARG;
    if (num_experts > xma::kMaxExperts) return XMA_ERR_UNSUPPORTED;
    xma::ep_plan_kernel<<<1, xma::kMaxExperts, 0, static_cast<cudaStream_t>(stream)>>>(
        counts_all, world, rank, num_experts, num_experts / world, local_padded_offsets, local_totals, dest_base);
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
                         int32_t* dest_row, int32_t record, void* stream) {
    if (num_tokens < 0 || top_k <= 0 || experts_per_rank <= 0) return XMA_ERR_BAD_ARG;
    if (top_k > 32 || cols <= 0 || (cols * xma::dtype_size(dtype)) % 16 != 0) return XMA_ERR_UNSUPPORTED;
    if (num_tokens == 0) return XMA_OK;
    if (!src || !peer_rows || !dest_rank || !dest_row || (scale && !peer_scale)) return XMA_ERR_BAD_ARG;
    if (record && (!selected || !inv_sorted || !expert_offsets || !expert_frequency || !dest_base)) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    XMA_EP_DISPATCH(dtype, (xma::ep_dispatch_rows_kernel<T><<<xma::ep_grid(num_tokens), xma::kEpWarps * 32, 0, s>>>(
                               static_cast<const T*>(src), cols, num_tokens, top_k, selected, inv_sorted, expert_offsets,
                               expert_frequency, dest_base, experts_per_rank, peer_rows, static_cast<const T*>(scale),
                               peer_scale, dest_rank, dest_row, record != 0)));
    return xma::launch_status();
}

int xma_ep_combine_pull(const int64_t* peer_rows, int32_t dtype, int64_t cols, const int32_t* dest_rank,
                        const int32_t* dest_row, int64_t num_tokens, int32_t top_k, void* out, void* stream) {
    if (num_tokens < 0 || top_k <= 0) return XMA_ERR_BAD_ARG;
    if (top_k > 32 || cols <= 0 || (cols * xma::dtype_size(dtype)) % 16 != 0) return XMA_ERR_UNSUPPORTED;
    if (num_tokens == 0) return XMA_OK;
    if (!peer_rows || !dest_rank || !dest_row || !out) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    XMA_EP_DISPATCH(dtype, (xma::ep_combine_pull_kernel<T><<<xma::ep_grid(num_tokens), xma::kEpWarps * 32, 0, s>>>(
                               peer_rows, cols, dest_rank, dest_row, num_tokens, top_k, static_cast<T*>(out))));
    return xma::launch_status();
}

int xma_ep_pull_scalars(const int64_t* peer_f32, const int32_t* dest_rank, const int32_t* dest_row, int64_t n,
                        float* out, void* stream) {
    if (n < 0) return XMA_ERR_BAD_ARG;
    if (n == 0) return XMA_OK;
    if (!peer_f32 || !dest_rank || !dest_row || !out) return XMA_ERR_BAD_ARG;
    const int64_t blocks = xma::ceil_div(n, 256);
    xma::ep_pull_scalars_kernel<<<static_cast<unsigned>(blocks > 4096 ? 4096 : blocks), 256, 0,
                                  static_cast<cudaStream_t>(stream)>>>(peer_f32, dest_rank, dest_row, n, out);
    return xma::launch_status();
}

}  // extern "C"
