/*
 * C ABI of libxma_b200: sm_100a kernels for the Mixture-of-Experts hot path of
 * open-lm-engine/flash-model-architectures ("XMA").
 *
 * Conventions (all entry points):
 *   - every pointer is a DEVICE pointer unless the parameter name starts with `host_`;
 *   - the caller owns every buffer (inputs, outputs and workspaces); the library never allocates
 *     device memory and keeps no per-call state;
 *   - `stream` is a `cudaStream_t` passed as `void*`; the call only enqueues work on it;
 *   - the return value is an `xma_status` (0 = ok); `xma_status_string` names it;
 *   - rows of 2-D operands are contiguous; base pointers are 16-byte aligned.
 *
 * Element type codes (`dtype`): 0 = bfloat16, 1 = float16, 2 = float32.
 * Index type codes (`id_is_int64`): 0 = int32, 1 = int64.
 *
 * "Padded expert order": the T*k (token, slot) rows sorted by expert id, stably (ascending flat
 * index t*k+slot inside one expert), with each expert's segment starting on a multiple of
 * block_m rows (XMA_BLOCK_M for the grouped GEMMs; 1 gives the plain sorted order, used to fill
 * expert-parallel send buffers). Rows that pad a segment hold zeros. It is described by
 *   padded_offsets int32[E+1]   first padded row of each expert (last entry: rows in use)
 *   row_src        int32[cap]   flat index t*k+slot held by a padded row, -1 for a padding row
 *   inv_row        int32[T*k]   padded row of a flat index
 *   tile_expert    int32[cap/block_m + 1]  expert id of each block_m-row tile, -1 past the end; the
 *                               LAST entry holds the number of tiles in use
 * with cap = xma_padded_capacity(T*k, E, block_m).
 */
#ifndef XMA_B200_H_
#define XMA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XMA_BLOCK_M 128
#define XMA_BLOCK_N 256 /* accumulator columns of one grouped-GEMM tile */

typedef enum {
    XMA_OK = 0,
    XMA_ERR_BAD_ARG = 1,        /* null pointer, negative size, misaligned pointer */
    XMA_ERR_UNSUPPORTED = 2,    /* shape or dtype outside what the kernels cover */
    XMA_ERR_LAUNCH = 3,         /* the CUDA runtime refused the launch (cudaGetLastError) */
    XMA_ERR_DRIVER = 4,         /* tensor-map encode or driver entry point failed */
    XMA_ERR_DEVICE_TIMEOUT = 5, /* a bounded device-side wait ran out (read from a status word) */
    XMA_ERR_SCRATCH_TOO_SMALL = 6 /* the problem needs more scratch than the library's built-in buffer */
} xma_status;

/* Human-readable name of a status code. Never NULL. */
const char* xma_status_string(int status);

/* ABI version; bumped when a signature changes. */
int xma_abi_version(void);

/* Rows a padded-expert-order buffer must hold for n = T*k routed rows, E experts and segments
 * aligned to block_m rows: (ceil(n / block_m) + E) * block_m. */
int64_t xma_padded_capacity(int64_t n, int32_t num_experts, int32_t block_m);

/* Largest n for which xma_moe_index_build (with at most 256 experts) runs as ONE kernel launch, a
 * thread-block cluster that never touches the workspace, on the current device; 0 if that form is
 * not available. Larger inputs take five launches and use the workspace. */
int64_t xma_moe_index_small_limit(void);

/* Bytes of workspace xma_moe_index_build needs. */
int64_t xma_moe_index_workspace_bytes(int64_t n, int32_t num_experts);

/*
 * Histogram of ids in [0, bins): out[b] = #{i : ids[i] == b}. Ids outside the range are ignored.
 * Replaces continuous_count_cuda (xma/functional/continuous_count/cuda_implementation/forward.cu:115-167,
 * bound at ops.cpp:7-15). `out` (uint32[bins]) is fully overwritten.
 */
int xma_continuous_count(const void* ids, int32_t id_is_int64, int64_t n, uint32_t* out, int32_t bins,
                         void* stream);

/*
 * Router top-k with softmax over the k selected logits (xma/layers/moe/__init__.py:190-203,268-274).
 *   logits          [T, E] of `dtype`
 *   topk_weights    [T, k] of `dtype`   softmax(float(top-k logits)) rounded to dtype
 *   topk_probs_f32  [T, k] float32      the same probabilities before rounding (saved for backward)
 *   selected        [T, k] int64        expert ids, by descending logit; ties: lowest id first
 * Requires 1 <= k <= 32, k <= E <= 1024.
 */
int xma_router_topk_softmax(const void* logits, int32_t dtype, int64_t num_tokens, int32_t num_experts,
                            int32_t top_k, void* topk_weights, float* topk_probs_f32, int64_t* selected,
                            void* stream);

/*
 * Backward of xma_router_topk_softmax (autograd of xma/layers/moe/__init__.py:192-201):
 *   d_logits[t, selected[t,j]] = p_tj * (dw_tj - sum_l p_tl dw_tl), zero elsewhere.
 *   d_weights [T, k] of `dtype`, topk_probs_f32 [T, k] float32, selected [T, k] int64,
 *   d_logits [T, E] of `dtype` (fully overwritten).
 */
int xma_router_topk_softmax_backward(const void* d_weights, int32_t dtype, const float* topk_probs_f32,
                                     const int64_t* selected, int64_t num_tokens, int32_t num_experts,
                                     int32_t top_k, void* d_logits, void* stream);

/*
 * Stable counting sort of the flattened expert ids and construction of the padded expert order.
 * Replaces selected_experts.flatten().sort(), continuous_count and cumsum at
 * xma/layers/moe/__init__.py:218-225.
 *   ids                    int32/int64 [n]  (n = T*k), values in [0, E)
 *   expert_frequency       uint32 [E]       rows per expert
 *   expert_offsets         int32  [E]       inclusive cumulative sum of expert_frequency
 *   sorted_expert_idxs     int32  [n]       ids in ascending order           (may be NULL)
 *   sorted_scattered_idxs  int32  [n]       flat index of each sorted row, stable
 *   padded_offsets, row_src, inv_row, tile_expert: see the header comment (tile_expert may be NULL)
 *   block_m                alignment of the expert segments, >= 1
 *   workspace              xma_moe_index_workspace_bytes(n, E) bytes
 * Requires E <= 1024 and n < 2^31.
 */
int xma_moe_index_build(const void* ids, int32_t id_is_int64, int64_t n, int32_t num_experts,
                        uint32_t* expert_frequency, int32_t* expert_offsets, int32_t* sorted_expert_idxs,
                        int32_t* sorted_scattered_idxs, int32_t* padded_offsets, int32_t* row_src,
                        int32_t* inv_row, int32_t* tile_expert, int32_t block_m, void* workspace, void* stream);

/*
 * xma_moe_index_build for callers that cannot allocate device memory. It has no counterpart in the
 * reference, whose Python side allocates whatever its kernels need.
 *
 * Who needs it: a host that embeds this library where no allocation may happen at call time, for
 * example a serving process whose device memory pool is carved up once at start-up and then
 * frozen, or a caller that issues the routing step from a place where entering an allocator is not
 * allowed. xma_moe_index_build needs a workspace for its per-segment histograms; this variant keeps
 * that workspace in a fixed array inside the library instead. Inputs and outputs are still the
 * caller's buffers and the results are identical to xma_moe_index_build's.
 *
 *   - The array is xma_moe_index_static_scratch_bytes() = 4 MiB; every GPU that loads the library
 *     holds it until the process exits. A problem whose xma_moe_index_workspace_bytes(n, E) exceeds
 *     it is refused with XMA_ERR_SCRATCH_TOO_SMALL and nothing is launched (T*k = 262144 rows over
 *     256 experts needs 0.5 MiB; the limit is reached near T*k * E = 5 * 10^8).
 *   - The call never allocates or frees: no cudaMalloc / cudaFree, no allocating library routine.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current). Make that first call outside any stream capture.
 *   - All calls on one device share the one array. Calls that may overlap on the GPU (different
 *     streams without an ordering between them) race on it; order them. Nothing needs clearing
 *     between calls: each call overwrites every scratch word before it reads it.
 */
int xma_moe_index_build_static(const void* ids, int32_t id_is_int64, int64_t n, int32_t num_experts,
                               uint32_t* expert_frequency, int32_t* expert_offsets, int32_t* sorted_expert_idxs,
                               int32_t* sorted_scattered_idxs, int32_t* padded_offsets, int32_t* row_src,
                               int32_t* inv_row, int32_t* tile_expert, int32_t block_m, void* stream);

/* Size in bytes of the built-in scratch array xma_moe_index_build_static uses. */
int64_t xma_moe_index_static_scratch_bytes(void);

/*
 * Gather rows into padded expert order (the `group` kernel,
 * xma/layers/moe/triton_implementation/group_kernel.py:12-100):
 *   dst[p, :] = src[row_src[p] / fan_out, :] * (coeff ? coeff[row_src[p]] : 1), zeros when row_src[p] < 0.
 * Rows p < min(*rows_in_use, max_rows) are written (all max_rows rows when rows_in_use is NULL);
 * rows_in_use is a device word, normally &padded_offsets[E].
 *   src [num_src_rows, cols], dst [max_rows, cols], coeff [num_src_rows * fan_out] of `dtype` or NULL.
 *   inv_row int32[num_src_rows * fan_out] or NULL: when given (and 1 < fan_out <= 32) the copy runs
 *   source-major, reading each source row once and writing its fan_out copies; the result is the same.
 * cols * sizeof(dtype) must be a multiple of 16.
 */
int xma_permute_rows(const void* src, int32_t dtype, int64_t cols, const int32_t* row_src, const int32_t* inv_row,
                     const int32_t* rows_in_use, int64_t max_rows, int64_t num_src_rows, int32_t fan_out,
                     const void* coeff, void* dst, void* stream);

/*
 * Top-k combine (torch.bmm at xma/layers/moe/triton_implementation/__init__.py:39-43; index_add at
 * xma/layers/moe/__init__.py:260-262):
 *   out[t, :] = sum_j (weights ? weights[t, j] : 1) * rows[inv_row[t*k + j], :], accumulated in float32.
 *   rows [cap, cols], weights [T, k] of `dtype` or NULL, out [T, cols].
 */
int xma_combine_rows(const void* rows, int32_t dtype, int64_t cols, const int32_t* inv_row,
                     const void* weights, int64_t num_tokens, int32_t top_k, void* out, void* stream);

/*
 * Gradient of xma_combine_rows with respect to `weights`
 * (torch.bmm at xma/layers/moe/triton_implementation/__init__.py:83):
 *   d_weights[t, j] = <rows[inv_row[t*k + j], :], d_out[t, :]>   (float32 accumulate, `dtype` out)
 */
int xma_combine_rows_backward_weights(const void* rows, int32_t dtype, int64_t cols, const int32_t* inv_row,
                                      const void* d_out, int64_t num_tokens, int32_t top_k, void* d_weights,
                                      void* stream);

/* Epilogues of xma_grouped_gemm. */
typedef enum {
    XMA_EPI_STORE = 0,        /* C = acc                                                            */
    XMA_EPI_SWIGLU = 1,       /* forward up-projection: acc = [up | gate]; writes the pre-activation
                                 and row_scale * up * silu(gate)                                   */
    XMA_EPI_SWIGLU_BWD = 2,   /* backward of the down-projection input: acc = d(h)/row_scale; writes
                                 d(pre-activation) and accumulates d(row_scale)                    */
    XMA_EPI_STORE_F32 = 3,    /* C (float32) = acc                                                   */
    XMA_EPI_ADD_F32 = 4       /* C (float32) += acc (bulk tensor reduce-add)                         */
} xma_epilogue;

/* Operand layouts of xma_grouped_gemm. */
typedef enum {
    XMA_GEMM_NT = 0,  /* C[r, n] = sum_k A[r, k] * W[e(r), n, k]   (forward: W is [E, N, K])        */
    XMA_GEMM_NN = 1   /* C[r, n] = sum_k A[r, k] * W[e(r), k, n]   (input gradient: W is [E, K, N]) */
} xma_gemm_layout;

/*
 * Grouped GEMM over rows in padded expert order; tcgen05 tensor cores (CTA pairs, cta_group::2),
 * fp32 accumulation in TMEM.
 * Replaces scatter2scatter (xma/layers/moe/triton_implementation/scatter_kernel.py:54-183) for the
 * up projection, the down projection and both input-gradient products
 * (xma/layers/moe/triton_implementation/__init__.py:14-59,131-140), with the swiglu forward/backward
 * (xma/functional/swiglu/__init__.py:34-43, cuda_implementation/backward.py:76-80) and the
 * router-weight scaling in the epilogue.
 *
 *   a            [cap, K] `dtype` (bf16 or fp16), padded expert order
 *   w            [E, N, K] (layout NT) or [E, K, N] (layout NN), `dtype`
 *   padded_offsets  int32[E+1] as in the header comment (segments aligned to XMA_BLOCK_M)
 *   c            EPI_STORE:      [cap, N]
 *                EPI_STORE_F32 / EPI_ADD_F32: float32 [cap, N] whatever `dtype` is (the float32
 *                                parameter path: three bf16 passes over split operands, see
 *                                xma_split_f32)
 *                EPI_SWIGLU:     pre-activation [cap, N] (N = 2*I: up columns then gate columns)
 *                EPI_SWIGLU_BWD: d(pre-activation) [cap, 2*N] (N = I)
 *   aux          EPI_SWIGLU:     out, activation [cap, N/2] = row_scale * up * silu(gate)
 *                EPI_SWIGLU_BWD: in, the saved pre-activation [cap, 2*N]
 *   row_src      int32[cap]; used with row_scale (may be NULL when row_scale is NULL)
 *   row_scale    [T*k] `dtype`, indexed by row_src, or NULL (= 1)
 *   d_row_scale  EPI_SWIGLU_BWD: float32 [ceil(N / XMA_BLOCK_N)][cap] partial sums, or NULL to skip:
 *                entry [j][r] receives sum over the columns n of column tile j of
 *                acc[r, n] * (up * silu(gate))[r, n]. Every entry of a row in use is written (no
 *                zeroing by the caller, no atomics); xma_reduce_row_partials adds the tiles up in
 *                a fixed order, so the router-weight gradient is the same in every run, like the
 *                bmm at xma/layers/moe/triton_implementation/__init__.py:83.
 *   status       int32 device word; a device-side wait that runs out writes a non-zero code there
 *
 * Requires K % 8 == 0, N % 8 == 0 and E <= 1024; EPI_SWIGLU requires (N/2) % 128 == 0.
 */
int xma_grouped_gemm(int32_t layout, int32_t epilogue, int32_t dtype, const void* a, const void* w,
                     const int32_t* padded_offsets, int64_t cap, int32_t num_experts, int64_t n, int64_t k,
                     void* c, void* aux, const int32_t* row_src, const void* row_scale, float* d_row_scale,
                     int32_t* status, void* stream);

/*
 * out[row_src[r]] = sum_j partials[j][r] for the rows r < *rows_in_use (all `cap` rows when
 * rows_in_use is NULL) with row_src[r] >= 0, j ascending: the second step of the router-weight
 * gradient (d_row_scale of xma_grouped_gemm). partials float32 [n_tiles][cap], out float32.
 * No reference counterpart as a kernel (the reference gets d_gates from one bmm,
 * xma/layers/moe/triton_implementation/__init__.py:83).
 */
int xma_reduce_row_partials(const float* partials, int32_t n_tiles, int64_t cap, const int32_t* row_src,
                            const int32_t* rows_in_use, float* out, void* stream);

/*
 * out[i] = sum_s partials[s][i], s ascending, rounded to `dtype`: the last step of a product whose
 * reduction dimension was split into row segments (the router weight gradient d(logits)^T x, computed by
 * xma_grouped_wgrad_f32 with every segment in the place of an expert). partials float32 [splits][count].
 * No reference counterpart (the reference leaves this product to autograd of nn.Linear,
 * xma/layers/moe/__init__.py:192).
 */
int xma_sum_partials(const float* partials, int32_t splits, int64_t count, int32_t dtype, void* out, void* stream);

/*
 * Self-test of the bounded device-side wait the GEMM kernels use: one thread waits on a barrier that
 * nothing arrives at; after limit_ns (at most 1 s; the check runs every few microseconds) the kernel
 * writes code 199 into *status and returns, leaving the context usable. No reference counterpart.
 */
int xma_selftest_bounded_wait(int32_t* status, int64_t limit_ns, void* stream);

/*
 * Per-expert weight gradient: dw[e, m, n] = sum_{r in expert e} x[r, m] * y[r, n], zeros for an expert
 * without rows. Replaces group_bwd_W and the zeros_like fill
 * (xma/layers/moe/triton_implementation/group_backward_kernel.py:13-125,
 *  xma/layers/moe/triton_implementation/__init__.py:121-129).
 *   x [cap, M], y [cap, N] in padded expert order with zero padding rows; dw [E, M, N] `dtype`.
 * Requires M % 8 == 0 and N % 8 == 0.
 */
int xma_grouped_wgrad(int32_t dtype, const void* x, const void* y, const int32_t* padded_offsets, int64_t cap,
                      int32_t num_experts, int64_t m, int64_t n, void* dw, int32_t* status, void* stream);

/*
 * The same product with a float32 result: dw float32 [E, M, N]; accumulate != 0 adds to dw instead of
 * overwriting it (an expert without rows is then left as it is). Here `cap` may be any positive row
 * count: rows at or past it read as zeros, and the segments in padded_offsets need only begin and end
 * on multiples of 64 rows (used with row segments in the place of experts to split a long reduction).
 */
int xma_grouped_wgrad_f32(int32_t dtype, const void* x, const void* y, const int32_t* padded_offsets, int64_t cap,
                          int32_t num_experts, int64_t m, int64_t n, float* dw, int32_t accumulate, int32_t* status,
                          void* stream);

/*
 * float32 operands for the tensor cores: hi = bf16(src), lo = bf16(src - hi), so that
 * src = hi + lo up to 2^-16 relative. A float32 product is then the sum of three bf16 products with
 * float32 accumulation, a_hi*b_hi + a_hi*b_lo + a_lo*b_hi (EPI_STORE_F32 for the first, EPI_ADD_F32 for
 * the other two): closer to float32 than the TF32 products of the reference's Triton kernels
 * (allow_tf32, xma/layers/moe/triton_implementation/scatter_kernel.py:49). No reference counterpart.
 *   src float32[count]; hi, lo bf16[count]; count % 4 == 0 is not required.
 */
int xma_split_f32(const float* src, int64_t count, void* hi, void* lo, void* stream);

/*
 * Router front end in one kernel: logits = x @ w_gate^T on the tensor cores (the grouped GEMM's
 * main loop with every token row in one group), and in its epilogue the logits rounded to `dtype`
 * and stored, top-k over the rounded logits (ties to the lowest expert id) and the softmax over the
 * selected values in float32. Replaces self.gate(x) + topk + softmax
 * (xma/layers/moe/__init__.py:192-201, 268-274): the [T, E] logits are written once and never read
 * back. Given the same logits the three routing outputs equal xma_router_topk_softmax's bit for bit.
 *   x [T, H], w_gate [E, H] `dtype` (bf16 or fp16); logits [T, E] `dtype`; topk_weights [T, k] `dtype`;
 *   topk_probs_f32 float32 [T, k]; selected int64 [T, k].
 * Requires E % 8 == 0, E <= 256, H % 8 == 0, k <= 8.
 */
int xma_router_gate_topk(int32_t dtype, const void* x, const void* w_gate, int64_t num_tokens, int64_t hidden,
                         int32_t num_experts, int32_t top_k, void* logits, void* topk_weights, float* topk_probs_f32,
                         int64_t* selected, int32_t* status, void* stream);

/*
 * Stand-alone packed swiglu (xma/functional/swiglu_packed.py:33-120; math of
 * xma/functional/swiglu/__init__.py:34-43 and cuda_implementation/backward.py:76-80):
 *   x [rows, 2*half] = [up | gate];  y [rows, half] = up * silu(gate), float32 inside.
 *   backward: dx = [dy * silu(gate) | dy * up * (s + gate*s*(1-s))], s = sigmoid(gate).
 */
int xma_swiglu_packed_forward(const void* x, int32_t dtype, int64_t rows, int64_t half, void* y, void* stream);
int xma_swiglu_packed_backward(const void* x, const void* dy, int32_t dtype, int64_t rows, int64_t half, void* dx,
                               void* stream);

/*
 * Unpacked swiglu (xma/functional/swiglu/__init__.py:29-120; kernels it replaces:
 * cuda_implementation/forward.py:15-72, backward.py:15-93): gate, up, y, dy, dgate, dup are
 * contiguous tensors of `count` elements of `dtype`; y = up * silu(gate) in float32.
 */
int xma_swiglu_forward(const void* gate, const void* up, int32_t dtype, int64_t count, void* y, void* stream);
int xma_swiglu_backward(const void* gate, const void* up, const void* dy, int32_t dtype, int64_t count, void* dgate,
                        void* dup, void* stream);

/*
 * Expert parallelism over NVLink peer memory. The reference has no parallelism; these entry points
 * have no counterpart there. One process per GPU; `peer_*` arguments are DEVICE arrays of `world`
 * addresses (int64), entry r being rank r's buffer as mapped into this process (CUDA IPC); entry
 * `rank` is the local buffer. The data kernels (dispatch, pull) never wait for another rank; the
 * ranks meet in xma_ep_barrier / xma_ep_exchange_counts, whose waits are bounded.
 *
 * xma_ep_barrier: one small kernel; this rank stores `seq` into word `rank` of every peer's flag
 * array (peer_flags[r] -> int32[world], zero before the first use) and waits until its own words
 * have all reached `seq` (sequence numbers grow by one per barrier, compared modulo 2^32). A wait
 * longer than limit_ns writes code 304 into *status and the kernel returns. world <= 32.
 *
 * xma_ep_exchange_counts: all-gather of one row of ints per rank without a library collective: this
 * rank's row (counts[0..num_counts) followed by `tag`) is stored into slot `rank` of every peer's
 * table (peer_tables[r] -> int32[world][num_counts + 1]), then the ranks meet as in xma_ep_barrier.
 *
 * xma_ep_plan: from counts_all int32[world][row_stride] (entries [s][0..E): rows rank s routes to
 * every global expert; experts owned in contiguous blocks of E/world; entry [s][E], when
 * row_stride > E, is rank s's buffer generation) computes, for this rank as an owner,
 * local_padded_offsets int32[E/world + 1] and local_totals int32[E/world] (rows each local expert
 * receives), and as a sender dest_base int32[E]: the row of the owner's buffer where this rank's
 * first row for expert e lands (expert segments aligned to XMA_BLOCK_M, sources in rank order).
 * If the generations differ (code 301) or an owner would receive more than `cap` padded rows
 * (code 302) the plan is refused: the code goes to *status, every dest_base entry is negative and
 * the local offsets are zero, so the kernels that follow move nothing.
 *
 * xma_ep_prepare_rows: row_src[r] = r for rows that receive a routed row, -1 otherwise; zeroes the
 * padding rows in use of `rows` (and `rows2` when not NULL).
 *
 * xma_ep_dispatch_rows: fused gather + send. Copy j of token t goes to row
 * dest_base[e] + (its position among this rank's rows for e) of the owner of e = selected[t][j];
 * (owner, row) is recorded in dest_rank / dest_row when `record` is non-zero and re-used otherwise
 * (backward pass). `scale` [T*k] is pushed to peer_scale[owner][row] when given. A copy whose row
 * is outside [0, cap) is dropped and code 303 written to *status (bounds check, nothing traps).
 *
 * xma_ep_combine_pull: out[t] = sum_j buffer(dest_rank[t][j])[dest_row[t][j]] (float32 sums, peer loads).
 * xma_ep_pull_scalars: out[q] = float32 array of rank dest_rank[q], entry dest_row[q].
 * Both read this rank's row 0 / return 0 for a row outside [0, cap).
 */
/*
 * pack_sequence / unpack_sequence (xma/functional/sequence_packing/cuda_implementation/kernel.cu:45-132,
 * bound at ops.cpp:7-16): copies between a padded batch [batch, seq, row] and the packed token stream
 * [cu_seqlens[batch], row]. cu_seqlens is int32 or int64 [batch + 1]; pad_left != 0 means the tokens of
 * a sequence sit at the END of its row of the padded batch. row_bytes is the size of one token's data.
 * xma_unpack_sequence writes every byte of `out`, zeros on the padding positions (the reference
 * zero-fills first and scatters afterwards).
 */
int xma_pack_sequence(const void* x, const void* cu_seqlens, int32_t cu_is_int64, int64_t batch, int64_t seq,
                      int64_t row_bytes, int32_t pad_left, void* out, void* stream);
int xma_unpack_sequence(const void* x, const void* cu_seqlens, int32_t cu_is_int64, int64_t batch, int64_t seq,
                        int64_t row_bytes, int32_t pad_left, void* out, void* stream);

/* Maps another process's device allocation into this process for the CURRENT device, with peer access
 * enabled: handle64 is that allocation's 64-byte cudaIpcMemHandle_t. Host-side call, no stream. */
int xma_ipc_open_handle(const void* handle64, void** device_ptr);
/* The 64-byte cudaIpcMemHandle_t of the device allocation that starts at allocation_base. Host-side call. */
int xma_ipc_get_handle(const void* allocation_base, void* handle64);
/* Unmaps what xma_ipc_open_handle returned. Host-side call; no kernel may still use the mapping. */
int xma_ipc_close_handle(void* device_ptr);
int xma_ep_barrier(const int64_t* peer_flags, int32_t rank, int32_t world, int32_t seq, int64_t limit_ns,
                   int32_t* status, void* stream);
int xma_ep_exchange_counts(const int32_t* counts, int32_t num_counts, int32_t tag, const int64_t* peer_tables,
                           const int64_t* peer_flags, int32_t rank, int32_t world, int32_t seq, int64_t limit_ns,
                           int32_t* status, void* stream);
int xma_ep_plan(const int32_t* counts_all, int32_t row_stride, int32_t world, int32_t rank, int32_t num_experts,
                int64_t cap, int32_t* local_padded_offsets, int32_t* local_totals, int32_t* dest_base, int32_t* status,
                void* stream);
int xma_ep_prepare_rows(const int32_t* local_padded_offsets, const int32_t* local_totals, int32_t experts_per_rank,
                        int64_t cap, int32_t dtype, int64_t cols, int32_t* row_src, void* rows, void* rows2,
                        void* stream);
int xma_ep_dispatch_rows(const void* src, int32_t dtype, int64_t cols, int64_t num_tokens, int32_t top_k,
                         const int64_t* selected, const int32_t* inv_sorted, const int32_t* expert_offsets,
                         const uint32_t* expert_frequency, const int32_t* dest_base, int32_t experts_per_rank,
                         const int64_t* peer_rows, const void* scale, const int64_t* peer_scale, int32_t* dest_rank,
                         int32_t* dest_row, int32_t record, int64_t cap, int32_t* status, void* stream);
int xma_ep_combine_pull(const int64_t* peer_rows, int32_t dtype, int64_t cols, const int32_t* dest_rank,
                        const int32_t* dest_row, int64_t num_tokens, int32_t top_k, void* out, int64_t cap, void* stream);
int xma_ep_pull_scalars(const int64_t* peer_f32, const int32_t* dest_rank, const int32_t* dest_row, int64_t n,
                        float* out, int64_t cap, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* XMA_B200_H_ */
