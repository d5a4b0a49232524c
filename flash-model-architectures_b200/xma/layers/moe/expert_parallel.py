"""Expert parallelism for `MoE`: experts are sharded in contiguous blocks over the ranks of a
process group (one process per GPU), tokens stay on their home rank, and two variable-size
all-to-alls (NCCL over NVLink/NVSwitch) move rows to the experts and back.

The reference has no parallelism of any kind; the contract here is that the expert-parallel result
equals the single-GPU result of the same global batch (routing integers exactly, values within the
bf16 tolerance).

Per step and rank:
  1. route locally; stable-sort the (token, slot) rows by GLOBAL expert id (block_m = 1), which
     also groups them by destination rank because each rank owns a contiguous block of experts;
  2. gather the rows into that order: this is the send buffer;
  3. all-to-all the per-expert counts (E ints), read the split sizes on the host (one small D2H);
  4. all-to-all the rows; received rows are ordered (source rank, local expert, position);
  5. stable-sort the received rows by local expert into the padded expert order and run the fused
     grouped GEMMs without router scaling;
  6. all-to-all the result rows back and combine them on the home rank with the router weights.
The backward pass is the same path in reverse: every piece is an autograd function.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ... import _native as N
from .experts_cuda import combine_rows, fused_swiglu_experts, gather_rows
from .routing import build_expert_index


class _AllToAllRows(torch.autograd.Function):
    """out = concat over sources of the row blocks they send here; backward sends the gradients back."""

    @staticmethod
    def forward(ctx, rows: torch.Tensor, send_splits: list[int], recv_splits: list[int], group):
        rows = rows.contiguous()
        out = rows.new_empty((sum(recv_splits),) + tuple(rows.shape[1:]))
        dist.all_to_all_single(out, rows, output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)
        ctx.send_splits, ctx.recv_splits, ctx.group = send_splits, recv_splits, group
        return out

    @staticmethod
    def backward(ctx, d_out: torch.Tensor):
        d_out = d_out.contiguous()
        d_rows = d_out.new_empty((sum(ctx.send_splits),) + tuple(d_out.shape[1:]))
        dist.all_to_all_single(
            d_rows, d_out, output_split_sizes=ctx.send_splits, input_split_sizes=ctx.recv_splits, group=ctx.group
        )
        return d_rows, None, None, None


def all_to_all_rows(rows: torch.Tensor, send_splits: list[int], recv_splits: list[int], group) -> torch.Tensor:
    return _AllToAllRows.apply(rows, send_splits, recv_splits, group)


@torch.no_grad()
def exchange_counts(expert_frequency: torch.Tensor, group) -> tuple[torch.Tensor, list[int], list[int]]:
    """expert_frequency [E] (rows this rank routes to every global expert) ->
    (recv_counts [G, E_local]: rows every source rank sends to each of this rank's experts,
     send_splits [G], recv_splits [G]) with the split sizes read back to the host once."""
    world = dist.get_world_size(group)
    counts = expert_frequency.to(torch.int64).view(world, -1)
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=group)
    sums = torch.stack([counts.sum(1), recv_counts.sum(1)]).tolist()  # the one host synchronisation
    return recv_counts, [int(v) for v in sums[0]], [int(v) for v in sums[1]]


@torch.no_grad()
def local_expert_ids(recv_counts: torch.Tensor, total: int) -> torch.Tensor:
    """Local expert id of every received row: rows arrive ordered by (source rank, local expert)."""
    world, experts_local = recv_counts.shape
    ids = torch.arange(experts_local, device=recv_counts.device, dtype=torch.int32).repeat(world)
    return torch.repeat_interleave(ids, recv_counts.flatten(), output_size=total)


def expert_parallel_swiglu_experts(
    hidden_states: torch.Tensor,
    w_fc_local: torch.Tensor,
    w_proj_local: torch.Tensor,
    router_weights: torch.Tensor,
    selected_experts: torch.Tensor,
    num_experts: int,
    group,
) -> torch.Tensor:
    """The expert MLPs of one MoE layer with the experts sharded over `group`."""
    world = dist.get_world_size(group)
    assert num_experts % world == 0 and w_fc_local.size(0) == num_experts // world
    num_rows = selected_experts.numel()

    home = build_expert_index(selected_experts, num_experts, block_m=1)
    send = gather_rows(hidden_states, home, rows=num_rows)
    recv_counts, send_splits, recv_splits = exchange_counts(home.expert_frequency, group)
    recv = all_to_all_rows(send, send_splits, recv_splits, group)

    ids = local_expert_ids(recv_counts, recv.size(0))
    local = build_expert_index(ids, num_experts // world, block_m=N.XMA_BLOCK_M, top_k=1)
    out_rows = fused_swiglu_experts(recv, w_fc_local, w_proj_local, None, local)

    back = all_to_all_rows(out_rows, recv_splits, send_splits, group)
    return combine_rows(back, router_weights, home)
