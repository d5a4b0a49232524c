// Row movement kernels of the MoE hot path: gather into padded expert order, top-k combine and the
// gradient of the combine weights. Pure HBM-bound copies: one warp per row, 16-byte accesses,
// several independent loads in flight per lane.
#include "common.cuh"

namespace xma {

constexpr int kRowWarps = 8;
constexpr int kRowUnroll = 4;

// dst[p, :] = src[row_src[p] / fan_out, :] * coeff[row_src[p]]   (zeros for padding rows)
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
permute_rows_kernel(const T* __restrict__ src, int64_t cols, const int32_t* __restrict__ row_src,
                    const int32_t* __restrict__ rows_in_use, int64_t max_rows, int fan_out,
                    const T* __restrict__ coeff, T* __restrict__ dst) {
    constexpr int kPer = Vec16<T>::kCount;
    const int lane = threadIdx.x & 31;
    const int64_t rows_used = rows_in_use != nullptr ? min(static_cast<int64_t>(*rows_in_use), max_rows) : max_rows;
    const int64_t nvec = cols / kPer;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * kRowWarps;
    for (int64_t p = static_cast<int64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5); p < rows_used; p += warps) {
        const int32_t flat = row_src[p];
        T* out = dst + p * cols;
        if (flat < 0) {
            Vec16<T> z;
#pragma unroll
            for (int j = 0; j < kPer; ++j) z.v[j] = Elem<T>::from_float(0.f);
            for (int64_t c = lane; c < nvec; c += 32) store16(out + c * kPer, z);
            continue;
        }
        const T* in = src + static_cast<int64_t>(flat / fan_out) * cols;
        const bool scaled = coeff != nullptr;
        const float scale = scaled ? Elem<T>::to_float(coeff[flat]) : 1.f;
        for (int64_t c0 = lane; c0 < nvec; c0 += 32 * kRowUnroll) {
            Vec16<T> buf[kRowUnroll];
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) {
                const int64_t c = c0 + 32 * u;
                if (c < nvec) buf[u] = load16(in + c * kPer);
            }
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) {
                const int64_t c = c0 + 32 * u;
                if (c < nvec) {
                    if (scaled) {
#pragma unroll
                        for (int j = 0; j < kPer; ++j)
                            buf[u].v[j] = Elem<T>::from_float(Elem<T>::to_float(buf[u].v[j]) * scale);
                    }
                    store16(out + c * kPer, buf[u]);
                }
            }
        }
    }
}

// Source-major form of the same gather: one warp reads a source row ONCE and writes its fan_out
// copies to dst[inv_row[t*fan_out + j]]. When the source does not fit in L2 the destination-major
// kernel above re-reads every source row from HBM once per copy; this one reads it once. Padding
// rows are zeroed by the warps that run past the last source row.
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
scatter_rows_kernel(const T* __restrict__ src, int64_t cols, const int32_t* __restrict__ row_src,
                    const int32_t* __restrict__ inv_row, const int32_t* __restrict__ rows_in_use, int64_t max_rows,
                    int64_t num_src_rows, int fan_out, const T* __restrict__ coeff, T* __restrict__ dst) {
    constexpr int kPer = Vec16<T>::kCount;
    const int lane = threadIdx.x & 31;
    const int64_t rows_used = rows_in_use != nullptr ? min(static_cast<int64_t>(*rows_in_use), max_rows) : max_rows;
    const int64_t nvec = cols / kPer;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * kRowWarps;
    const int64_t warp_id = static_cast<int64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5);
    for (int64_t t = warp_id; t < num_src_rows; t += warps) {
        // Lane j keeps the j-th destination row and coefficient of this source row (fan_out <= 32).
        int32_t my_dst = -1;
        float my_scale = 1.f;
        if (lane < fan_out) {
            my_dst = inv_row[t * fan_out + lane];
            if (coeff != nullptr) my_scale = Elem<T>::to_float(coeff[t * fan_out + lane]);
        }
        const T* in = src + t * cols;
        // The trip count is the same for every lane (the shuffles below need the whole warp); a lane
        // past the last vector only skips its loads and stores.
        for (int64_t base = 0; base < nvec; base += 32 * kRowUnroll) {
            const int64_t c0 = base + lane;
            Vec16<T> buf[kRowUnroll];
#pragma unroll
            for (int u = 0; u < kRowUnroll; ++u) {
                const int64_t c = c0 + 32 * u;
                if (c < nvec) buf[u] = load16(in + c * kPer);
            }
            for (int j = 0; j < fan_out; ++j) {
                const int32_t row = __shfl_sync(0xffffffffu, my_dst, j);
                const float scale = __shfl_sync(0xffffffffu, my_scale, j);
                T* out = dst + static_cast<int64_t>(row) * cols;
#pragma unroll
                for (int u = 0; u < kRowUnroll; ++u) {
                    const int64_t c = c0 + 32 * u;
                    if (c < nvec) {
                        Vec16<T> v = buf[u];
                        if (coeff != nullptr) {
#pragma unroll
                            for (int e = 0; e < kPer; ++e) v.v[e] = Elem<T>::from_float(Elem<T>::to_float(v.v[e]) * scale);
                        }
                        store16(out + c * kPer, v);
                    }
                }
            }
        }
    }
    // Padding rows in use: zeros.
    Vec16<T> z;
#pragma unroll
    for (int e = 0; e < kPer; ++e) z.v[e] = Elem<T>::from_float(0.f);
    for (int64_t p = warp_id; p < rows_used; p += warps) {
        if (row_src[p] >= 0) continue;
        T* out = dst + p * cols;
        for (int64_t c = lane; c < nvec; c += 32) store16(out + c * kPer, z);
    }
}

// out[t, :] = sum_j weights[t, j] * rows[inv_row[t*k + j], :]
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
combine_rows_kernel(const T* __restrict__ rows, int64_t cols, const int32_t* __restrict__ inv_row,
                    const T* __restrict__ weights, int64_t num_tokens, int top_k, T* __restrict__ out) {
    constexpr int kPer = Vec16<T>::kCount;
    const int lane = threadIdx.x & 31;
    const int64_t nvec = cols / kPer;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * kRowWarps;
    for (int64_t t = static_cast<int64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5); t < num_tokens; t += warps) {
        // Lane j keeps the j-th source row and weight of this token (top_k <= 32).
        int32_t my_row = 0;
        float my_w = 1.f;
        if (lane < top_k) {
            my_row = inv_row[t * top_k + lane];
            if (weights != nullptr) my_w = Elem<T>::to_float(weights[t * top_k + lane]);
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
                const int32_t r0 = __shfl_sync(0xffffffffu, my_row, s);
                const int32_t r1 = __shfl_sync(0xffffffffu, my_row, s + 1);
                const float w0 = __shfl_sync(0xffffffffu, my_w, s);
                const float w1 = __shfl_sync(0xffffffffu, my_w, s + 1);
                const Vec16<T> a = load16(rows + static_cast<int64_t>(r0) * cols + c * kPer);
                const Vec16<T> b = load16(rows + static_cast<int64_t>(r1) * cols + c * kPer);
#pragma unroll
                for (int j = 0; j < kPer; ++j) {
                    acc[j] = fmaf(w0, Elem<T>::to_float(a.v[j]), acc[j]);
                    acc[j] = fmaf(w1, Elem<T>::to_float(b.v[j]), acc[j]);
                }
            }
            for (; s < top_k; ++s) {
                const int32_t r0 = __shfl_sync(0xffffffffu, my_row, s);
                const float w0 = __shfl_sync(0xffffffffu, my_w, s);
                const Vec16<T> a = load16(rows + static_cast<int64_t>(r0) * cols + c * kPer);
#pragma unroll
                for (int j = 0; j < kPer; ++j) acc[j] = fmaf(w0, Elem<T>::to_float(a.v[j]), acc[j]);
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

// d_weights[t, j] = <rows[inv_row[t*k + j], :], d_out[t, :]>
template <typename T>
__global__ void __launch_bounds__(kRowWarps * 32)
combine_rows_backward_weights_kernel(const T* __restrict__ rows, int64_t cols, const int32_t* __restrict__ inv_row,
                                     const T* __restrict__ d_out, int64_t num_tokens, int top_k,
                                     T* __restrict__ d_weights) {
    constexpr int kPer = Vec16<T>::kCount;
    const int lane = threadIdx.x & 31;
    const int64_t nvec = cols / kPer;
    const int64_t pairs = num_tokens * top_k;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * kRowWarps;
    for (int64_t q = static_cast<int64_t>(blockIdx.x) * kRowWarps + (threadIdx.x >> 5); q < pairs; q += warps) {
        const T* a = rows + static_cast<int64_t>(inv_row[q]) * cols;
        const T* b = d_out + (q / top_k) * cols;
        float acc = 0.f;
        for (int64_t c = lane; c < nvec; c += 32) {
            const Vec16<T> x = load16(a + c * kPer);
            const Vec16<T> y = load16(b + c * kPer);
#pragma unroll
            for (int j = 0; j < kPer; ++j) acc = fmaf(Elem<T>::to_float(x.v[j]), Elem<T>::to_float(y.v[j]), acc);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) d_weights[q] = Elem<T>::from_float(acc);
    }
}

inline unsigned row_grid(int64_t rows) {
    int64_t blocks = ceil_div(rows > 0 ? rows : 1, kRowWarps);
    const int64_t max_blocks = static_cast<int64_t>(sm_count()) * 8;
    if (blocks > max_blocks) blocks = max_blocks;
    return static_cast<unsigned>(blocks);
}

template <typename T>
int launch_permute(const void* src, int64_t cols, const int32_t* row_src, const int32_t* inv_row,
                   const int32_t* rows_in_use, int64_t max_rows, int64_t num_src_rows, int fan_out, const void* coeff,
                   void* dst, cudaStream_t stream) {
    if (inv_row != nullptr && fan_out > 1 && fan_out <= 32 && num_src_rows > 0) {
        scatter_rows_kernel<T><<<row_grid(num_src_rows), kRowWarps * 32, 0, stream>>>(
            static_cast<const T*>(src), cols, row_src, inv_row, rows_in_use, max_rows, num_src_rows, fan_out,
            static_cast<const T*>(coeff), static_cast<T*>(dst));
        return launch_status();
    }
    permute_rows_kernel<T><<<row_grid(max_rows), kRowWarps * 32, 0, stream>>>(
        static_cast<const T*>(src), cols, row_src, rows_in_use, max_rows, fan_out, static_cast<const T*>(coeff),
        static_cast<T*>(dst));
    return launch_status();
}

template <typename T>
int launch_combine(const void* rows, int64_t cols, const int32_t* inv_row, const void* weights, int64_t num_tokens,
                   int top_k, void* out, cudaStream_t stream) {
    combine_rows_kernel<T><<<row_grid(num_tokens), kRowWarps * 32, 0, stream>>>(
        static_cast<const T*>(rows), cols, inv_row, static_cast<const T*>(weights), num_tokens, top_k,
        static_cast<T*>(out));
    return launch_status();
}

template <typename T>
int launch_combine_bwd_w(const void* rows, int64_t cols, const int32_t* inv_row, const void* d_out, int64_t num_tokens,
                         int top_k, void* d_weights, cudaStream_t stream) {
    combine_rows_backward_weights_kernel<T><<<row_grid(num_tokens * top_k), kRowWarps * 32, 0, stream>>>(
        static_cast<const T*>(rows), cols, inv_row, static_cast<const T*>(d_out), num_tokens, top_k,
        static_cast<T*>(d_weights));
    return launch_status();
}

inline bool row_args_ok(int dtype, int64_t cols) {
    return cols > 0 && (cols * dtype_size(dtype)) % 16 == 0;
}

}  // namespace xma

#define XMA_DISPATCH_DTYPE(dtype, CALL)                          \
    switch (dtype) {                                             \
        case xma::kDtypeBF16: { using T = __nv_bfloat16; return CALL; } \
        case xma::kDtypeF16: { using T = __half; return CALL; }  \
        case xma::kDtypeF32: { using T = float; return CALL; }   \
        default: return XMA_ERR_UNSUPPORTED;                     \
    }

extern "C" {

int xma_permute_rows(const void* src, int32_t dtype, int64_t cols, const int32_t* row_src, const int32_t* inv_row,
                     const int32_t* rows_in_use, int64_t max_rows, int64_t num_src_rows, int32_t fan_out,
                     const void* coeff, void* dst, void* stream) {
    if (max_rows < 0 || fan_out <= 0) return XMA_ERR_BAD_ARG;
    if (max_rows == 0) return XMA_OK;
    // src may be NULL when no row is routed here (every row_src entry in use is then negative).
    if (!row_src || !dst) return XMA_ERR_BAD_ARG;
    if (!xma::row_args_ok(dtype, cols)) return XMA_ERR_UNSUPPORTED;
    if (!xma::aligned16(src) || !xma::aligned16(dst)) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    XMA_DISPATCH_DTYPE(dtype, xma::launch_permute<T>(src, cols, row_src, inv_row, rows_in_use, max_rows, num_src_rows, fan_out, coeff, dst, s));
}

int xma_combine_rows(const void* rows, int32_t dtype, int64_t cols, const int32_t* inv_row, const void* weights,
                     int64_t num_tokens, int32_t top_k, void* out, void* stream) {
    if (num_tokens < 0 || top_k <= 0) return XMA_ERR_BAD_ARG;
    if (top_k > 32 || !xma::row_args_ok(dtype, cols)) return XMA_ERR_UNSUPPORTED;
    if (num_tokens == 0) return XMA_OK;
    if (!rows || !inv_row || !out || !xma::aligned16(rows) || !xma::aligned16(out)) return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    XMA_DISPATCH_DTYPE(dtype, xma::launch_combine<T>(rows, cols, inv_row, weights, num_tokens, top_k, out, s));
}

int xma_combine_rows_backward_weights(const void* rows, int32_t dtype, int64_t cols, const int32_t* inv_row,
                                      const void* d_out, int64_t num_tokens, int32_t top_k, void* d_weights,
                                      void* stream) {
    if (num_tokens < 0 || top_k <= 0) return XMA_ERR_BAD_ARG;
    if (!xma::row_args_ok(dtype, cols)) return XMA_ERR_UNSUPPORTED;
    if (num_tokens == 0) return XMA_OK;
    if (!rows || !inv_row || !d_out || !d_weights || !xma::aligned16(rows) || !xma::aligned16(d_out))
        return XMA_ERR_BAD_ARG;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    XMA_DISPATCH_DTYPE(dtype, xma::launch_combine_bwd_w<T>(rows, cols, inv_row, d_out, num_tokens, top_k, d_weights, s));
}

}  // extern "C"
