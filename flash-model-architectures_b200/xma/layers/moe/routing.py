"""Routing objects of the MoE layer: router top-k/softmax and the padded expert order."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ... import _native as N
from ... import ops


@dataclass
class ExpertIndex:
    """Everything derived from `selected_experts` (no gradients flow through any of it).

    The first four fields are the reference's objects (xma/layers/moe/__init__.py:218-225), with the
    sort made stable; the rest describe the padded expert order the grouped GEMMs run on.
    """

    expert_frequency: torch.Tensor  # uint32 [E]
    expert_offsets: torch.Tensor  # int32 [E], inclusive cumulative sum
    sorted_expert_idxs: torch.Tensor  # int32 [T*k]
    sorted_scattered_idxs: torch.Tensor  # int32 [T*k]
    padded_offsets: torch.Tensor  # int32 [E+1]
    row_src: torch.Tensor  # int32 [cap]
    inv_row: torch.Tensor  # int32 [T*k]
    tile_expert: torch.Tensor | None  # int32 [cap/block_m + 1]; None unless block_m == XMA_BLOCK_M
    rows_in_use: torch.Tensor  # int32 [1], view of padded_offsets[E]
    cap: int
    num_experts: int
    top_k: int
    block_m: int


@torch.no_grad()
def build_expert_index(
    selected_experts: torch.Tensor, num_experts: int, block_m: int = N.XMA_BLOCK_M, top_k: int | None = None
) -> ExpertIndex:
    """Stable counting sort of the flattened expert ids into the padded expert order.

    `block_m=1` gives the plain (unpadded) sorted order; `top_k` overrides the fan-out recorded in the
    index (rows per source row) when `selected_experts` is already flat."""
    assert selected_experts.dtype in (torch.int32, torch.int64)
    if top_k is None:
        top_k = selected_experts.size(-1) if selected_experts.dim() > 1 else 1
    ids = selected_experts.contiguous().view(-1)
    n = ids.numel()
    device = ids.device
    cap = N.padded_capacity(n, num_experts, block_m)
    i32 = dict(dtype=torch.int32, device=device)
    padded_offsets = torch.empty(num_experts + 1, **i32)
    index = ExpertIndex(
        expert_frequency=torch.empty(num_experts, dtype=torch.uint32, device=device),
        expert_offsets=torch.empty(num_experts, **i32),
        sorted_expert_idxs=torch.empty(n, **i32),
        sorted_scattered_idxs=torch.empty(n, **i32),
        padded_offsets=padded_offsets,
        row_src=torch.empty(cap, **i32),
        inv_row=torch.empty(n, **i32),
        tile_expert=torch.empty(cap // block_m + 1, **i32) if block_m == N.XMA_BLOCK_M else None,
        rows_in_use=padded_offsets[num_experts:],
        cap=cap,
        num_experts=num_experts,
        top_k=top_k,
        block_m=block_m,
    )
    workspace = torch.empty(N.index_workspace_elems(n, num_experts), **i32)
    ops.moe_index_build_cuda(
        ids, index.expert_frequency, index.expert_offsets, index.sorted_expert_idxs, index.sorted_scattered_idxs,
        index.padded_offsets, index.row_src, index.inv_row, index.tile_expert, workspace, num_experts, block_m,
    )
    return index


class _RouterTopKSoftmax(torch.autograd.Function):
    """top-k over the logits, then softmax over the k selected values in float32
    (xma/layers/moe/__init__.py:194-201, 268-274), forward and backward in one kernel each."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, top_k: int):
        logits = logits.contiguous()
        T = logits.size(0)
        weights = torch.empty(T, top_k, dtype=logits.dtype, device=logits.device)
        probs = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
        selected = torch.empty(T, top_k, dtype=torch.int64, device=logits.device)
        ops.router_topk_softmax_cuda(logits, weights, probs, selected, top_k)
        ctx.save_for_backward(probs, selected)
        ctx.top_k = top_k
        ctx.num_experts = logits.size(1)
        ctx.mark_non_differentiable(selected)
        return weights, selected

    @staticmethod
    def backward(ctx, d_weights: torch.Tensor, _d_selected):
        probs, selected = ctx.saved_tensors
        d_weights = d_weights.contiguous()
        d_logits = torch.empty(d_weights.size(0), ctx.num_experts, dtype=d_weights.dtype, device=d_weights.device)
        ops.router_topk_softmax_backward_cuda(d_weights, probs, selected, d_logits, ctx.top_k)
        return d_logits, None


def router_topk_softmax(logits: torch.Tensor, top_k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Returns (router_weights [T,k] in logits.dtype, selected_experts [T,k] int64)."""
    return _RouterTopKSoftmax.apply(logits, top_k)


FUSED_ROUTER_MAX_EXPERTS = 256

_segment_offsets: dict = {}


def _offsets(values: tuple[int, ...], device: torch.device) -> torch.Tensor:
    """int32 device tensor of row-segment boundaries, built once per distinct layout."""
    if torch.compiler.is_compiling():  # no global state while a compiler traces this
        return torch.tensor(values, dtype=torch.int32, device=device)
    key = (device, values)
    t = _segment_offsets.get(key)
    if t is None:
        t = _segment_offsets[key] = torch.tensor(values, dtype=torch.int32, device=device)
    return t


def fused_router_supported(x: torch.Tensor, w_gate: torch.Tensor, top_k: int) -> bool:
    """Limits of xma_router_gate_topk: bf16 / fp16, one accumulator tile holds a token's logits over all
    experts (E <= 256), and the [T, E] logits are written by bulk tensor stores, whose rows must be a
    multiple of 16 bytes (E % 8 == 0). Measured on B200 against a library GEMM followed by the stand-alone
    top-k kernel: 0.139 ms against 0.161 ms at T=32768, H=7168, E=256; 0.031 against 0.028 ms at T=8192,
    H=2048, E=64; 0.047 against 0.042 ms at T=16384, H=4096, E=8 (few experts leave most of each
    accumulator tile unused, but the step is one launch and the logits never travel twice)."""
    E, H = w_gate.shape
    return (
        x.dtype in (torch.bfloat16, torch.float16)
        and w_gate.dtype == x.dtype
        and E % 8 == 0
        and E <= FUSED_ROUTER_MAX_EXPERTS
        and H % 8 == 0
        and top_k <= 8
        and top_k <= E
    )


class _FusedRouter(torch.autograd.Function):
    """self.gate(x), top-k and softmax (xma/layers/moe/__init__.py:192-201, 268-274) in one tensor-core
    kernel. Backward, all on this library's kernels: the top-k/softmax backward kernel scatters
    d(weights) into d(logits); d(x) = d(logits) @ W_g is the grouped GEMM with every token in one group;
    d(W_g) = d(logits)^T @ x is the weight-gradient GEMM with the token dimension cut into row segments
    (one per "expert" slot, float32 partial results) followed by a sum over the segments."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, w_gate: torch.Tensor, top_k: int):
        x = x.contiguous()
        w_gate = w_gate.contiguous()
        T, E = x.size(0), w_gate.size(0)
        opts = dict(device=x.device)
        logits = torch.empty(T, E, dtype=x.dtype, **opts)
        weights = torch.empty(T, top_k, dtype=x.dtype, **opts)
        probs = torch.empty(T, top_k, dtype=torch.float32, **opts)
        selected = torch.empty(T, top_k, dtype=torch.int64, **opts)
        ops.router_gate_topk_cuda(x, w_gate, logits, weights, probs, selected, top_k)
        ctx.save_for_backward(x, w_gate, probs, selected)
        ctx.top_k = top_k
        ctx.mark_non_differentiable(selected)
        return logits, weights, selected

    @staticmethod
    def backward(ctx, d_logits_in, d_weights, _d_selected):
        x, w_gate, probs, selected = ctx.saved_tensors
        T, H = x.shape
        E = w_gate.size(0)
        dev = x.device
        if T == 0:
            return (torch.zeros_like(x) if ctx.needs_input_grad[0] else None,
                    torch.zeros_like(w_gate) if ctx.needs_input_grad[1] else None, None)
        t_pad = -(-T // N.XMA_BLOCK_M) * N.XMA_BLOCK_M
        d_logits_pad = torch.empty(t_pad, E, dtype=x.dtype, device=dev)  # rows past T are never summed
        d_logits = d_logits_pad[:T]
        if d_weights is None:
            d_logits.zero_()
        else:
            ops.router_topk_softmax_backward_cuda(d_weights.contiguous(), probs, selected, d_logits, ctx.top_k)
        if d_logits_in is not None:  # e.g. an auxiliary load-balancing loss on the logits
            d_logits.add_(d_logits_in)
        dx = dw = None
        if not torch.compiler.is_compiling():
            N.profiler.prefix = "router_"  # these GEMM calls are not the expert GEMMs in a per-kernel table
        if ctx.needs_input_grad[0]:
            # rows >= T of the padded buffers belong to nobody: a row of the product depends on its own row only
            dx_pad = torch.empty(t_pad, H, dtype=x.dtype, device=dev)
            ops.grouped_gemm_cuda(d_logits_pad, w_gate.view(1, E, H), _offsets((0, t_pad), dev), dx_pad, None, None, None,
                                  None, N.GEMM_NN, N.EPI_STORE)
            dx = dx_pad[:T]
        if ctx.needs_input_grad[1]:
            # Split the T rows into segments so that about every SM pair gets a tile: tiles per segment =
            # ceil(E / 256) * ceil(H / 256).
            tiles = -(-E // 256) * -(-H // 256)
            splits = max(1, min(-(-74 * 2 // tiles), -(-T // 1024)))
            seg = -(-(-(-T // splits)) // N.XMA_BLOCK_M) * N.XMA_BLOCK_M
            splits = -(-T // seg)
            t_up = -(-T // 64) * 64
            bounds = tuple(min(i * seg, t_up) for i in range(splits + 1))
            partial = torch.empty(splits, E, H, dtype=torch.float32, device=dev)
            ops.grouped_wgrad_f32_cuda(d_logits, x, _offsets(bounds, dev), partial, False)
            dw = torch.empty_like(w_gate)
            ops.sum_partials_cuda(partial, dw)
        if not torch.compiler.is_compiling():
            N.profiler.prefix = ""
        return dx, dw, None


def fused_router(x: torch.Tensor, w_gate: torch.Tensor, top_k: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (router_logits [T,E], router_weights [T,k], selected_experts [T,k] int64)."""
    return _FusedRouter.apply(x, w_gate, top_k)
