"""`MoE` and `Experts`: same constructor, forward signature, parameter and buffer names as
xma/layers/moe/__init__.py:23-274, computed by the sm_100a kernels of libxma_b200.

Differences from the reference that a caller can observe:
  * only `kernel_backend=None` / `KernelBackend.cuda` are served; anything else raises;
  * the expert sort is stable and top-k ties go to the lowest expert id (the reference leaves both
    unspecified);
  * with `activation_function=xma.functional.swiglu_packed` and `is_glu=True` the whole expert MLP
    runs as fused grouped GEMMs; any other callable runs between two unfused grouped GEMMs.
"""

from __future__ import annotations

import warnings
from typing import Callable

import torch
import torch.nn as nn

from ...accelerator import KernelBackend, require_cuda_backend
from ...functional.swiglu_packed import swiglu_packed
from ...module import XMAModule
from .expert_parallel import expert_parallel_swiglu_experts
from .expert_parallel_peer import PeerExpertParallelState, peer_expert_parallel_swiglu_experts
from .experts_cuda import combine_rows, fused_swiglu_experts, gather_rows, grouped_linear
from .routing import (ExpertIndex, build_expert_index, fused_router, fused_router_supported,
                      router_topk_softmax)


class Experts(XMAModule):
    """Stacked per-expert weights `[E, out, in]` (xma/layers/moe/__init__.py:23-125)."""

    def __init__(
        self, num_experts: int, in_features: int, out_features: int, add_bias: bool = True, std: float | None = None
    ) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))
        self.bias = None
        if add_bias:
            self.bias = nn.Parameter(torch.empty(num_experts, out_features))
        self.std = std
        self.num_experts = num_experts
        self.in_features = in_features
        self.out_features = out_features
        # Unused by the kernels; kept because they are part of the reference's state_dict.
        self.register_buffer("N_array", torch.empty((num_experts,), dtype=torch.uint32))
        self.register_buffer("K_array", torch.empty((num_experts,), dtype=torch.uint32))
        self.reset_parameters()

    def forward(self, rows: torch.Tensor, index: ExpertIndex) -> torch.Tensor:
        """rows (padded expert order) -> rows @ weight[e]^T."""
        if self.bias is not None:
            raise NotImplementedError("expert biases are not supported (the reference kernel path asserts the same)")
        return grouped_linear(rows, self.weight, index)

    def extra_repr(self) -> str:
        return "num_experts={}, in_features={}, out_features={}".format(
            self.num_experts, self.in_features, self.out_features
        )

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0, std=self.std)
        if self.bias is not None:
            self.bias.zero_()
        self.N_array.fill_(self.out_features)
        self.K_array.fill_(self.in_features)


class MoE(XMAModule):
    def __init__(
        self,
        num_experts: int,
        num_experts_per_tok: int,
        hidden_size: int,
        intermediate_size: int,
        activation_function: Callable,
        is_glu: bool,
        add_bias: bool,
        std: float,
        *,
        expert_parallel_group=None,
        expert_parallel_mode: str = "peer",
    ) -> None:
        """Same positional arguments as the reference. `expert_parallel_group` (keyword-only, not in
        the reference) shards the experts in contiguous blocks over that torch.distributed group:
        this rank then holds `num_experts / world_size` experts in `c_fc` / `c_proj`.
        `expert_parallel_mode`: "peer" moves rows with kernels over NVLink peer memory (all ranks on
        one node), "nccl" with variable-size NCCL all-to-alls."""
        super().__init__()
        if expert_parallel_mode not in ("peer", "nccl"):
            raise ValueError(f"expert_parallel_mode must be 'peer' or 'nccl', got {expert_parallel_mode!r}")
        self.expert_parallel_group = expert_parallel_group
        self.expert_parallel_mode = expert_parallel_mode
        self._peer_state = None
        self.num_local_experts = num_experts
        if expert_parallel_group is not None:
            import torch.distributed as dist

            world = dist.get_world_size(expert_parallel_group)
            if num_experts % world != 0:
                raise ValueError(f"num_experts ({num_experts}) must be divisible by the group size ({world})")
            self.num_local_experts = num_experts // world
        self.num_experts = num_experts
        self.top_k = num_experts_per_tok
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.is_glu = is_glu

        self.gate = nn.Linear(in_features=hidden_size, out_features=num_experts, bias=False)
        self.c_fc = Experts(
            num_experts=self.num_local_experts,
            in_features=hidden_size,
            out_features=2 * intermediate_size if is_glu else intermediate_size,
            add_bias=add_bias,
            std=std,
        )
        self.act = activation_function
        self.c_proj = Experts(
            num_experts=self.num_local_experts, in_features=intermediate_size, out_features=hidden_size, add_bias=add_bias, std=std
        )

    def forward(
        self, hidden_states: torch.Tensor, *, kernel_backend: KernelBackend | None = None
    ) -> tuple[torch.Tensor, torch.Tensor]:
        require_cuda_backend(kernel_backend)
        original_shape = hidden_states.shape
        hidden_states = hidden_states.view(-1, self.hidden_size)
        router_logits, router_weights, selected_experts = self._compute_routing_weights(hidden_states)
        hidden_states = self._compute_experts(
            hidden_states, router_weights, selected_experts, kernel_backend=kernel_backend
        )
        return hidden_states.view(original_shape), router_logits

    def all_reduce_router_gradient(self) -> None:
        """With expert parallelism every rank routes its own tokens through a replicated router:
        `gate.weight.grad` holds this rank's share. Sums the shares over the expert-parallel group so
        the replicas stay identical (a data-parallel wrapper that already reduces it makes this call
        unnecessary). Expert weights live on one rank each and need no reduction."""
        if self.expert_parallel_group is None or self.gate.weight.grad is None:
            return
        import torch.distributed as dist

        dist.all_reduce(self.gate.weight.grad, group=self.expert_parallel_group)

    def _compute_routing_weights(self, hidden_states: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        if self.gate.bias is None and fused_router_supported(hidden_states, self.gate.weight, self.top_k):
            return fused_router(hidden_states, self.gate.weight, self.top_k)
        router_logits = self.gate(hidden_states)
        router_weights, selected_experts = router_topk_softmax(router_logits, self.top_k)
        return router_logits, router_weights, selected_experts

    def _get_topk(self, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """(values, indices) of the top_k largest logits per row, largest first
        (xma/layers/moe/__init__.py:268-274). The indices come from the routing kernel, so ties go to
        the lowest expert id, and the values are the logits at those indices."""
        _, indices = router_topk_softmax(x.detach(), self.top_k)
        return x.gather(-1, indices), indices

    def _fused_path(self) -> bool:
        return (
            self.act is swiglu_packed
            and self.is_glu
            and self.c_fc.bias is None
            and self.c_fc.weight.dtype in (torch.bfloat16, torch.float16)
            and self.intermediate_size % 128 == 0
            and self.hidden_size % 8 == 0
        )

    def _compute_experts(
        self,
        hidden_states: torch.Tensor,
        router_weights: torch.Tensor,
        selected_experts: torch.Tensor,
        *,
        kernel_backend: KernelBackend | None = None,
    ) -> torch.Tensor:
        require_cuda_backend(kernel_backend)
        if self.c_fc.bias is not None or self.c_proj.bias is not None:
            raise NotImplementedError("expert biases are not supported (the reference kernel path asserts the same)")
        router_weights = router_weights.to(hidden_states.dtype)
        if self.expert_parallel_group is not None:
            if not self._fused_path():
                raise NotImplementedError("expert parallelism is implemented for the fused swiglu path")
            if self.expert_parallel_mode == "peer" and self._peer_state is None:
                state = PeerExpertParallelState(self.expert_parallel_group, self.num_experts)
                try:
                    # Collective: either every rank maps every buffer or every rank raises.
                    state.ensure(hidden_states.size(0), self.top_k, self.hidden_size, hidden_states.dtype,
                                 hidden_states.device)
                    self._peer_state = state
                except RuntimeError as error:
                    warnings.warn(f"expert_parallel_mode='peer' is not available here ({error}); using 'nccl'")
                    self.expert_parallel_mode = "nccl"
            if self.expert_parallel_mode == "peer":
                return peer_expert_parallel_swiglu_experts(
                    hidden_states, self.c_fc.weight, self.c_proj.weight, router_weights,
                    selected_experts.to(torch.int64), self._peer_state,
                )
            return expert_parallel_swiglu_experts(
                hidden_states, self.c_fc.weight, self.c_proj.weight, router_weights, selected_experts,
                self.num_experts, self.expert_parallel_group,
            )
        index = build_expert_index(selected_experts, self.num_experts)
        if self._fused_path():
            return fused_swiglu_experts(hidden_states, self.c_fc.weight, self.c_proj.weight, router_weights, index)
        rows = gather_rows(hidden_states, index)
        rows = self.c_fc(rows, index)
        rows = self.act(rows)
        rows = self.c_proj(rows, index)
        return combine_rows(rows, router_weights, index)
