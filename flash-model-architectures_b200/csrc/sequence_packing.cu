// pack_sequence / unpack_sequence: copies between a padded batch [B, S, N] and a packed token stream
// [total, N] described by cu_seqlens (the step that produces the [T, H] stream the MoE layer
// consumes). HBM-bound row copies: one warp per (batch, position) row, 16-byte accesses. Unlike the
// reference, which zero-fills the padded output in a separate pass before scattering into it, the
// unpack kernel writes the padding zeros itself, so every output byte is written exactly once.
#include "common.cuh"

namespace xma {

constexpr int kPackWarps = 8;

template <typename IntT>
__device__ __forceinline__ bool packed_index(const IntT* __restrict__ cu_seqlens, int64_t b, int64_t s, int64_t seq,
                                             bool pad_left, int64_t* token) {
    const int64_t start = static_cast<int64_t>(cu_seqlens[b]);
    const int64_t len = static_cast<int64_t>(cu_seqlens[b + 1]) - start;
    const int64_t first = pad_left ? seq - len : 0;  // first position of the row that holds a token
    if (s < first || s >= first + len) return false;
    *token = start + (s - first);
    return true;
}

// kPack: out[token] = x[b, s];  !kPack: out[b, s] = x[token], zeros on padding positions.
template <typename IntT, bool kPack>
__global__ void __launch_bounds__(kPackWarps * 32)
pack_unpack_sequence_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ out,
                            const IntT* __restrict__ cu_seqlens, int64_t batch, int64_t seq, int64_t row_bytes,
                            bool pad_left, bool vectorised) {
    const int lane = threadIdx.x & 31;
    const int64_t rows = batch * seq;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * kPackWarps;
    for (int64_t r = static_cast<int64_t>(blockIdx.x) * kPackWarps + (threadIdx.x >> 5); r < rows; r += warps) {
        const int64_t b = r / seq, s = r - b * seq;
        int64_t token = 0;
        const bool holds_token = packed_index<IntT>(cu_seqlens, b, s, seq, pad_left, &token);
        const uint8_t* src = nullptr;
        uint8_t* dst = nullptr;
        if (kPack) {
            if (!holds_token) continue;
            src = x + r * row_bytes;
            dst = out + token * row_bytes;
        } else {
            dst = out + r * row_bytes;
            if (holds_token) src = x + token * row_bytes;
        }
        if (vectorised) {
            const int64_t nvec = row_bytes / 16;
            for (int64_t c0 = lane; c0 < nvec; c0 += 32 * 4) {
                uint4 buf[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int64_t c = c0 + 32 * u;
                    buf[u] = make_uint4(0, 0, 0, 0);
                    if (c < nvec && src != nullptr) buf[u] = __ldg(reinterpret_cast<const uint4*>(src) + c);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int64_t c = c0 + 32 * u;
                    if (c < nvec) reinterpret_cast<uint4*>(dst)[c] = buf[u];
                }
            }
        } else {
            for (int64_t c = lane; c < row_bytes; c += 32) dst[c] = src != nullptr ? src[c] : uint8_t(0);
        }
    }
}

template <bool kPack>
int launch_pack(const void* x, void* out, const void* cu_seqlens, int cu_is_int64, int64_t batch, int64_t seq,
                int64_t row_bytes, int pad_left, cudaStream_t stream) {
    const bool vec = row_bytes % 16 == 0 && aligned16(x) && aligned16(out);
    int64_t blocks = ceil_div(batch * seq, kPackWarps);
    const int64_t max_blocks = static_cast<int64_t>(sm_count()) * 8;
    if (blocks > max_blocks) blocks = max_blocks;
    const unsigned grid = static_cast<unsigned>(blocks < 1 ? 1 : blocks);
    if (cu_is_int64)
        pack_unpack_sequence_kernel<int64_t, kPack><<<grid, kPackWarps * 32, 0, stream>>>(
            static_cast<const uint8_t*>(x), static_cast<uint8_t*>(out), static_cast<const int64_t*>(cu_seqlens), batch,
            seq, row_bytes, pad_left != 0, vec);
    else
        pack_unpack_sequence_kernel<int32_t, kPack><<<grid, kPackWarps * 32, 0, stream>>>(
            static_cast<const uint8_t*>(x), static_cast<uint8_t*>(out), static_cast<const int32_t*>(cu_seqlens), batch,
            seq, row_bytes, pad_left != 0, vec);
    return launch_status();
}

}  // namespace xma

extern "C" {

int xma_pack_sequence(const void* x, const void* cu_seqlens, int32_t cu_is_int64, int64_t batch, int64_t seq,
                      int64_t row_bytes, int32_t pad_left, void* out, void* stream) {
    if (batch < 0 || seq < 0 || row_bytes <= 0) return XMA_ERR_BAD_ARG;
    if (batch == 0 || seq == 0) return XMA_OK;
    if (!x || !cu_seqlens || !out) return XMA_ERR_BAD_ARG;
    return xma::launch_pack<true>(x, out, cu_seqlens, cu_is_int64, batch, seq, row_bytes, pad_left,
                                  static_cast<cudaStream_t>(stream));
}

int xma_unpack_sequence(const void* x, const void* cu_seqlens, int32_t cu_is_int64, int64_t batch, int64_t seq,
                        int64_t row_bytes, int32_t pad_left, void* out, void* stream) {
    if (batch < 0 || seq < 0 || row_bytes <= 0) return XMA_ERR_BAD_ARG;
    if (batch == 0 || seq == 0) return XMA_OK;
    if (!cu_seqlens || !out) return XMA_ERR_BAD_ARG;  // x may be NULL when no sequence holds a token
    return xma::launch_pack<false>(x, out, cu_seqlens, cu_is_int64, batch, seq, row_bytes, pad_left,
                                   static_cast<cudaStream_t>(stream));
}

}  // extern "C"
