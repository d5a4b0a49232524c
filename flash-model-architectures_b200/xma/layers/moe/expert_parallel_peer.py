"""Expert parallelism with the dispatch and the combine fused into kernels over NVLink peer memory.

Same contract as `expert_parallel.py` (experts sharded in contiguous blocks, tokens stay on their
home rank, result equal to the single-GPU layer), different data movement:

  forward   route locally -> one small kernel stores this rank's per-expert counts into every
            peer's table and meets the other ranks (flag words in peer memory, bounded wait) ->
            every rank derives, without touching the host, where each of its rows lands in the
            owners' buffers -> ONE kernel gathers each token row and stores its k copies (and their
            router weights) straight into the owners' row buffers in padded expert order (beside
            it, on a second stream, this rank zeroes the padding rows of its own buffer) ->
            barrier -> the fused grouped GEMMs run on the received rows in place (swiglu and router
            weight in the epilogue; beside the first one a second stream copies the received rows
            for the backward pass) -> barrier -> ONE kernel pulls each token's k result rows from
            the owners and sums them.
  backward  (barrier, only if no forward pass has run since the backward pass before) -> the dispatch
            kernel moves the output-gradient rows to the owners -> barrier ->
            the two input-gradient GEMMs -> on a second stream: barrier, the pull kernel for the
            input-gradient rows and a pull of the router-weight gradients, while the first stream
            runs the two weight-gradient GEMMs (a third of the pass) -> the streams join.

There is no host synchronisation, no library collective, no variable-size all-to-all, no second
sort and no regrouping copy on the receiving side. A barrier is a one-warp kernel (`xma_ep_barrier`):
it stores a sequence number into a flag word of every peer and waits until its own flag words carry
that number, for at most `barrier_timeout_s`; after that it writes a code into the status word and
returns, and `xma.check_status()` raises on the host.

Every rank must call the layer the same number of times, in the same order. Buffers are sized,
collectively, for the largest token count any rank has passed so far; they grow (collectively
again) when a rank passes more tokens than that, which every rank must then do in the same call.
The device-side plan refuses to move anything (status codes 301 / 302) if ranks disagree on the
buffer generation or if a rank would receive more rows than its buffers hold.
"""

from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

from ... import _native as N
from ... import ops
from ...ops import _launch
from .peer_memory import PeerBuffer
from .routing import build_expert_index


class PeerExpertParallelState:
    """Buffers one MoE layer keeps for the peer-memory path (sized on first use, collectively)."""

    barrier_timeout_s = 10.0

    def __init__(self, group, num_experts: int) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.num_experts = num_experts
        self.experts_per_rank = num_experts // self.world
        self.key = None
        self.capacity_tokens = 0
        self.generation = 0
        self.seq = 0
        self.last_routing = None
        self.backward_since_forward = False  # a backward pass ran and no forward pass (with its meetings) since
        self._buffers: list[PeerBuffer] = []

    def ensure(self, tokens_per_rank: int, top_k: int, hidden: int, dtype: torch.dtype, device: torch.device) -> None:
        key = (top_k, hidden, dtype)
        if self.key == key and tokens_per_rank <= self.capacity_tokens:
            return
        # Collective from here on: every rank is in this call together.
        most = torch.tensor([max(tokens_per_rank, self.capacity_tokens if self.key == key else 0)],
                            dtype=torch.int64, device=device)
        dist.all_reduce(most, op=dist.ReduceOp.MAX, group=self.group)
        capacity_tokens = int(most.item())
        self.release()
        # Worst case: every routed row of every rank lands on one rank.
        rows = capacity_tokens * self.world * top_k
        self.cap = N.padded_capacity(rows, self.experts_per_rank)
        mk = lambda numel, dt, zero=False: PeerBuffer(numel, dt, device, self.group, zero=zero)
        self.rows_in = mk(self.cap * hidden, dtype)       # x rows as received
        self.rows_out = mk(self.cap * hidden, dtype)      # expert outputs; in the backward pass the dx rows
        self.rows_grad = mk(self.cap * hidden, dtype)     # dy rows as received
        self.scale = mk(self.cap, dtype)                  # router weight per received row
        self.d_scale = mk(self.cap, torch.float32)        # its gradient
        self.counts = mk(self.world * (self.num_experts + 1), torch.int32)  # every rank's counts + generation
        self.flags = mk(self.world, torch.int32, zero=True)                 # barrier sequence numbers
        self._buffers = [self.rows_in, self.rows_out, self.rows_grad, self.scale, self.d_scale, self.counts, self.flags]
        self.status = N.status_word(device)
        self.side_stream = torch.cuda.Stream(device)  # the backward pass pulls gradient rows on it, under the wgrads
        self.capacity_tokens = capacity_tokens
        self.generation += 1
        self.key = key

    def release(self) -> None:
        """Unmaps the peers' buffers and drops this rank's. Collective (every rank leaves its kernels first)."""
        if not self._buffers:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for buffer in self._buffers:
            buffer.close()
        self._buffers = []
        dist.barrier(group=self.group)  # nobody frees memory a peer still has mapped

    def _next_seq(self) -> int:
        self.seq = (self.seq + 1) & 0x7FFFFFFF
        return self.seq

    def _limit_ns(self) -> int:
        return int(self.barrier_timeout_s * 1e9)

    def barrier(self) -> None:
        """Kernels queued after it start only when every rank's earlier kernels are done (or the time limit ran out)."""
        _launch("xma_ep_barrier", self.flags.table, N.ptr(self.flags.table), self.rank, self.world, self._next_seq(),
                self._limit_ns(), N.ptr(self.status))

    def exchange_counts(self, expert_frequency: torch.Tensor) -> torch.Tensor:
        """All-gather of the per-expert row counts (and the buffer generation) through peer memory; also a barrier."""
        _launch("xma_ep_exchange_counts", expert_frequency, N.ptr(expert_frequency), self.num_experts, self.generation,
                N.ptr(self.counts.table), N.ptr(self.flags.table), self.rank, self.world, self._next_seq(),
                self._limit_ns(), N.ptr(self.status))
        return self.counts.view(self.world, self.num_experts + 1)


@contextlib.contextmanager
def _on_second_stream(state: PeerExpertParallelState, device: torch.device):
    """The enclosed launches go to the layer's second stream, behind everything queued on the current
    stream so far; `_join` makes the current stream wait for them."""
    state.side_stream.wait_stream(torch.cuda.current_stream(device))
    saved, N.profiler.prefix = N.profiler.prefix, "overlapped_"  # a per-kernel table keeps them apart
    try:
        with torch.cuda.stream(state.side_stream):
            yield
    finally:
        N.profiler.prefix = saved


def _join(state: PeerExpertParallelState, device: torch.device) -> None:
    torch.cuda.current_stream(device).wait_stream(state.side_stream)


def _plan(state: PeerExpertParallelState, counts_all: torch.Tensor):
    dev = counts_all.device
    i32 = dict(dtype=torch.int32, device=dev)
    lpo = torch.empty(state.experts_per_rank + 1, **i32)
    totals = torch.empty(state.experts_per_rank, **i32)
    dest_base = torch.empty(state.num_experts, **i32)
    _launch("xma_ep_plan", counts_all, N.ptr(counts_all), counts_all.size(1), state.world, state.rank, state.num_experts,
            state.cap, N.ptr(lpo), N.ptr(totals), N.ptr(dest_base), N.ptr(state.status))
    return lpo, totals, dest_base


def _prepare(state, lpo, totals, rows: torch.Tensor, row_src: torch.Tensor) -> None:
    """Zeroes the padding rows of `rows` and fills `row_src` (the row's own index, -1 for padding)."""
    _launch("xma_ep_prepare_rows", rows, N.ptr(lpo), N.ptr(totals), state.experts_per_rank, state.cap,
            N.dtype_code(rows.dtype), rows.size(1), N.ptr(row_src), N.ptr(rows), None)


class _PeerFusedSwigluExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_fc, w_proj, router_weights, selected, state: PeerExpertParallelState):
        x = x.contiguous()
        w_fc, w_proj = w_fc.contiguous(), w_proj.contiguous()
        router_weights = router_weights.contiguous()
        selected = selected.contiguous()
        T, H = x.shape
        k = selected.size(1)
        inter = w_fc.size(1) // 2
        dev = x.device
        state.ensure(T, k, H, x.dtype, dev)
        cap = state.cap

        home = build_expert_index(selected, state.num_experts, block_m=1)
        # The exchange is also the barrier that keeps this pass's dispatch from overwriting rows a
        # slower rank still reads for the pass before.
        counts_all = state.exchange_counts(home.expert_frequency.view(torch.int32))
        lpo, totals, dest_base = _plan(state, counts_all)

        rows_in = state.rows_in.view(cap, H)
        # Zeroing this rank's padding rows touches none of the rows the peers send: it runs beside the dispatch.
        row_src = torch.empty(cap, dtype=torch.int32, device=dev)
        with _on_second_stream(state, dev):
            _prepare(state, lpo, totals, rows_in, row_src)
        dest_rank = torch.empty(T * k, dtype=torch.int32, device=dev)
        dest_row = torch.empty(T * k, dtype=torch.int32, device=dev)
        _launch("xma_ep_dispatch_rows", x, N.ptr(x), N.dtype_code(x.dtype), H, T, k, N.ptr(selected), N.ptr(home.inv_row),
                N.ptr(home.expert_offsets), N.ptr(home.expert_frequency), N.ptr(dest_base), state.experts_per_rank,
                N.ptr(state.rows_in.table), N.ptr(router_weights), N.ptr(state.scale.table), N.ptr(dest_rank),
                N.ptr(dest_row), 1, cap, N.ptr(state.status))
        _join(state, dev)
        state.barrier()
        state.backward_since_forward = False

        opts = dict(dtype=x.dtype, device=dev)
        # The shared buffers are overwritten by the next forward pass: the backward pass reads a private
        # copy of the received rows. Only the rows in use are copied (a device-side count; the rest of
        # `xg` is never read), on the second stream, beside the first GEMM.
        xg = torch.empty(cap, H, **opts)
        with _on_second_stream(state, dev):
            ops.permute_rows_cuda(rows_in, row_src, lpo[state.experts_per_rank:], None, xg, 1, None)

        pre = torch.empty(cap, 2 * inter, **opts)
        act = torch.empty(cap, inter, **opts)
        scale = state.scale.view(cap)
        ops.grouped_gemm_cuda(rows_in, w_fc, lpo, pre, act, row_src, scale, None, N.GEMM_NT, N.EPI_SWIGLU)
        rows_out = state.rows_out.view(cap, H)
        ops.grouped_gemm_cuda(act, w_proj, lpo, rows_out, None, None, None, None, N.GEMM_NT, N.EPI_STORE)
        state.barrier()

        y = torch.empty(T, H, **opts)
        _launch("xma_ep_combine_pull", y, N.ptr(state.rows_out.table), N.dtype_code(x.dtype), H, N.ptr(dest_rank),
                N.ptr(dest_row), T, k, N.ptr(y), cap)
        _join(state, dev)  # `xg` is this stream's again; the peers may overwrite `rows_in` after the next meeting
        ctx.save_for_backward(xg, pre, act, w_fc, w_proj, scale.clone(), row_src, lpo, totals, dest_rank, dest_row)
        ctx.state = state
        ctx.dims = (T, H, k)
        state.last_routing = (dest_rank, dest_row, lpo)  # for checks outside the layer; nothing here reads it
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, pre, act, w_fc, w_proj, scale, row_src, lpo, totals, dest_rank, dest_row = ctx.saved_tensors
        state: PeerExpertParallelState = ctx.state
        T, H, k = ctx.dims
        cap = state.cap
        if pre.size(0) != cap:
            raise RuntimeError("the expert-parallel buffers were resized between this pass's forward and backward")
        dy = dy.contiguous()
        dev = dy.device
        opts = dict(dtype=dy.dtype, device=dev)
        inter = act.size(1)

        # The peers' weight-gradient GEMMs of the backward pass before must be done with the rows this
        # pass's dispatch is about to overwrite. The meetings of a forward pass in between see to that; only
        # when two backward passes follow each other directly (fwd, fwd, bwd, bwd) an extra meeting is needed.
        # Every rank makes the same calls in the same order, so every rank decides the same.
        if state.backward_since_forward:
            state.barrier()
        state.backward_since_forward = True
        rows_grad = state.rows_grad.view(cap, H)
        with _on_second_stream(state, dev):
            _prepare(state, lpo, totals, rows_grad, row_src)
        _launch("xma_ep_dispatch_rows", dy, N.ptr(dy), N.dtype_code(dy.dtype), H, T, k, None, None, None, None, None,
                state.experts_per_rank, N.ptr(state.rows_grad.table), None, None, N.ptr(dest_rank), N.ptr(dest_row), 0,
                cap, N.ptr(state.status))
        _join(state, dev)
        state.barrier()

        d_pre = torch.empty_like(pre)
        partials = torch.empty(N.gemm_n_tiles(inter), cap, dtype=torch.float32, device=dev)
        ops.grouped_gemm_cuda(rows_grad, w_proj, lpo, d_pre, pre, row_src, scale, partials, N.GEMM_NN, N.EPI_SWIGLU_BWD)
        # row_src is the identity on the rows in use: the sums land at their own row of the shared array.
        # Nothing on this stream reads them: the second stream adds them up beside the next GEMM, ahead of
        # its meeting with the peers, who pull them after it.
        with _on_second_stream(state, dev):
            ops.reduce_row_partials_cuda(partials, row_src, lpo[state.experts_per_rank:], state.d_scale.view(cap))
        # The input-gradient rows go to the buffer the forward pass used for the experts' outputs (free
        # until the next forward pass's second GEMM, which comes after two more meetings), so that the
        # received output-gradient rows stay intact for the weight gradient below.
        rows_dx = state.rows_out.view(cap, H)
        ops.grouped_gemm_cuda(d_pre, w_fc, lpo, rows_dx, None, None, None, None, N.GEMM_NN, N.EPI_STORE)

        # Everything the peers wait for is done: meet them and pull on the second stream while this
        # stream computes the weight gradients, which no other rank needs.
        dx = torch.empty(T, H, **opts)
        d_weights = torch.empty(T * k, dtype=torch.float32, device=dev)
        with _on_second_stream(state, dev):
            state.barrier()
            _launch("xma_ep_combine_pull", dx, N.ptr(state.rows_out.table), N.dtype_code(dy.dtype), H, N.ptr(dest_rank),
                    N.ptr(dest_row), T, k, N.ptr(dx), cap)
            _launch("xma_ep_pull_scalars", d_weights, N.ptr(state.d_scale.table), N.ptr(dest_rank), N.ptr(dest_row),
                    T * k, N.ptr(d_weights), cap)

        dw_proj = torch.empty_like(w_proj)
        ops.grouped_wgrad_cuda(rows_grad, act, lpo, dw_proj)
        dw_fc = torch.empty_like(w_fc)
        ops.grouped_wgrad_cuda(d_pre, xg, lpo, dw_fc)
        # dx and d_weights were allocated on this stream and are handed to it again here; every later
        # use of their memory is ordered after the second stream's work.
        _join(state, dev)
        return dx, dw_fc, dw_proj, d_weights.view(T, k).to(dy.dtype), None, None


def peer_expert_parallel_swiglu_experts(hidden_states, w_fc_local, w_proj_local, router_weights, selected_experts,
                                        state: PeerExpertParallelState) -> torch.Tensor:
    return _PeerFusedSwigluExperts.apply(hidden_states, w_fc_local, w_proj_local, router_weights, selected_experts, state)
