"""Expert parallelism with the dispatch and the combine fused into kernels over NVLink peer memory.

Same contract as `expert_parallel.py` (experts sharded in contiguous blocks, tokens stay on their
home rank, result equal to the single-GPU layer), different data movement:

  forward   route locally -> all-gather the per-expert counts (E ints, the only NCCL payload) ->
            every rank derives, without touching the host, where each of its rows lands in the
            owners' buffers -> ONE kernel gathers each token row and stores its k copies (and their
            router weights) straight into the owners' row buffers in padded expert order ->
            barrier -> the fused grouped GEMMs run on the received rows in place (swiglu and router
            weight in the epilogue) -> barrier -> ONE kernel pulls each token's k result rows from
            the owners and sums them.
  backward  the same two kernels with the roles of the buffers swapped, plus a pull of the
            router-weight gradients.

There is no host synchronisation, no variable-size all-to-all, no second sort and no regrouping copy
on the receiving side. Ranks only meet at stream-ordered NCCL collectives (one all-gather of counts
and two 4-byte all-reduces per direction); no kernel waits for another rank.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ... import _native as N
from ... import ops
from ...ops import _launch
from .peer_memory import PeerBuffer
from .routing import build_expert_index


class PeerExpertParallelState:
    """Buffers one MoE layer keeps for the peer-memory path (sized on first use, collectively)."""

    def __init__(self, group, num_experts: int) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.num_experts = num_experts
        self.experts_per_rank = num_experts // self.world
        self.key = None

    def ensure(self, tokens_per_rank: int, top_k: int, hidden: int, dtype: torch.dtype, device: torch.device) -> None:
        key = (tokens_per_rank, top_k, hidden, dtype)
        if self.key == key:
            return
        # Worst case: every routed row of every rank lands on one rank.
        rows = tokens_per_rank * self.world * top_k
        self.cap = N.padded_capacity(rows, self.experts_per_rank)
        self.rows_in = PeerBuffer(self.cap * hidden, dtype, device, self.group)      # x rows, then dy rows' results
        self.rows_out = PeerBuffer(self.cap * hidden, dtype, device, self.group)     # expert outputs
        self.rows_grad = PeerBuffer(self.cap * hidden, dtype, device, self.group)    # dy rows in, dx rows out
        self.scale = PeerBuffer(self.cap, dtype, device, self.group)                 # router weight per received row
        self.d_scale = PeerBuffer(self.cap, torch.float32, device, self.group)       # its gradient
        self.token = torch.zeros(1, dtype=torch.int32, device=device)
        self.key = key

    def barrier(self) -> None:
        """Stream-ordered: kernels queued after it start only when every rank's earlier kernels are done."""
        dist.all_reduce(self.token, group=self.group)


def _plan(state: PeerExpertParallelState, counts_all: torch.Tensor):
    dev = counts_all.device
    i32 = dict(dtype=torch.int32, device=dev)
    lpo = torch.empty(state.experts_per_rank + 1, **i32)
    totals = torch.empty(state.experts_per_rank, **i32)
    dest_base = torch.empty(state.num_experts, **i32)
    _launch("xma_ep_plan", counts_all, N.ptr(counts_all), state.world, state.rank, state.num_experts, N.ptr(lpo),
            N.ptr(totals), N.ptr(dest_base))
    return lpo, totals, dest_base


def _prepare(state, lpo, totals, rows: torch.Tensor, row_src: torch.Tensor | None):
    if row_src is None:
        row_src = torch.empty(state.cap, dtype=torch.int32, device=rows.device)
    _launch("xma_ep_prepare_rows", rows, N.ptr(lpo), N.ptr(totals), state.experts_per_rank, state.cap,
            N.dtype_code(rows.dtype), rows.size(1), N.ptr(row_src), N.ptr(rows), None)
    return row_src


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
        counts_all = torch.empty(state.world, state.num_experts, dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(counts_all, home.expert_frequency.view(torch.int32), group=state.group)
        lpo, totals, dest_base = _plan(state, counts_all)

        rows_in = state.rows_in.view(cap, H)
        row_src = _prepare(state, lpo, totals, rows_in, None)
        dest_rank = torch.empty(T * k, dtype=torch.int32, device=dev)
        dest_row = torch.empty(T * k, dtype=torch.int32, device=dev)
        _launch("xma_ep_dispatch_rows", x, N.ptr(x), N.dtype_code(x.dtype), H, T, k, N.ptr(selected), N.ptr(home.inv_row),
                N.ptr(home.expert_offsets), N.ptr(home.expert_frequency), N.ptr(dest_base), state.experts_per_rank,
                N.ptr(state.rows_in.table), N.ptr(router_weights), N.ptr(state.scale.table), N.ptr(dest_rank),
                N.ptr(dest_row), 1)
        state.barrier()

        opts = dict(dtype=x.dtype, device=dev)
        pre = torch.empty(cap, 2 * inter, **opts)
        act = torch.empty(cap, inter, **opts)
        scale = state.scale.view(cap)
        ops.grouped_gemm_cuda(rows_in, w_fc, lpo, pre, act, row_src, scale, None, N.GEMM_NT, N.EPI_SWIGLU)
        rows_out = state.rows_out.view(cap, H)
        ops.grouped_gemm_cuda(act, w_proj, lpo, rows_out, None, None, None, None, N.GEMM_NT, N.EPI_STORE)
        state.barrier()

        y = torch.empty(T, H, **opts)
        _launch("xma_ep_combine_pull", y, N.ptr(state.rows_out.table), N.dtype_code(x.dtype), H, N.ptr(dest_rank),
                N.ptr(dest_row), T, k, N.ptr(y))

        # The shared buffers are overwritten by the next forward pass: keep private copies of what
        # the backward pass reads.
        ctx.save_for_backward(rows_in.clone(), pre, act, w_fc, w_proj, scale.clone(), row_src, lpo, totals, dest_rank,
                              dest_row)
        ctx.state = state
        ctx.dims = (T, H, k)
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, pre, act, w_fc, w_proj, scale, row_src, lpo, totals, dest_rank, dest_row = ctx.saved_tensors
        state: PeerExpertParallelState = ctx.state
        T, H, k = ctx.dims
        cap = state.cap
        dy = dy.contiguous()
        dev = dy.device
        opts = dict(dtype=dy.dtype, device=dev)

        rows_grad = state.rows_grad.view(cap, H)
        _prepare(state, lpo, totals, rows_grad, row_src)
        _launch("xma_ep_dispatch_rows", dy, N.ptr(dy), N.dtype_code(dy.dtype), H, T, k, None, None, None, None, None,
                state.experts_per_rank, N.ptr(state.rows_grad.table), None, None, N.ptr(dest_rank), N.ptr(dest_row), 0)
        state.barrier()

        d_pre = torch.empty_like(pre)
        d_scale = state.d_scale.view(cap)
        d_scale.zero_()
        ops.grouped_gemm_cuda(rows_grad, w_proj, lpo, d_pre, pre, row_src, scale, d_scale, N.GEMM_NN, N.EPI_SWIGLU_BWD)
        dw_proj = torch.empty_like(w_proj)
        ops.grouped_wgrad_cuda(rows_grad, act, lpo, dw_proj)
        dw_fc = torch.empty_like(w_fc)
        ops.grouped_wgrad_cuda(d_pre, xg, lpo, dw_fc)
        ops.grouped_gemm_cuda(d_pre, w_fc, lpo, rows_grad, None, None, None, None, N.GEMM_NN, N.EPI_STORE)
        state.barrier()

        dx = torch.empty(T, H, **opts)
        _launch("xma_ep_combine_pull", dx, N.ptr(state.rows_grad.table), N.dtype_code(dy.dtype), H, N.ptr(dest_rank),
                N.ptr(dest_row), T, k, N.ptr(dx))
        d_weights = torch.empty(T * k, dtype=torch.float32, device=dev)
        _launch("xma_ep_pull_scalars", d_weights, N.ptr(state.d_scale.table), N.ptr(dest_rank), N.ptr(dest_row), T * k,
                N.ptr(d_weights))
        return dx, dw_fc, dw_proj, d_weights.view(T, k).to(dy.dtype), None, None


def peer_expert_parallel_swiglu_experts(hidden_states, w_fc_local, w_proj_local, router_weights, selected_experts,
                                        state: PeerExpertParallelState) -> torch.Tensor:
    return _PeerFusedSwigluExperts.apply(hidden_states, w_fc_local, w_proj_local, router_weights, selected_experts, state)
