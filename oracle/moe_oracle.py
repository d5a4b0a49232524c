"""CPU oracle for the MoE hot path. TEST INFRASTRUCTURE ONLY.

A plain-PyTorch restatement of the reference's torch path (`kernel_backend=KernelBackend.torch`) of
open-lm-engine/flash-model-architectures, function by function. Only `tests/`,
`__graft_entry__.smoke()` and `bench.py` (its `cpu_baseline` / `--impl reference` legs when the copy of
the reference is absent, and its `ep_check`, which runs outside every timed region) may import it, and
only as the checker; the product package never does.

Parity is pinned: `tests/golden/*.npz` were produced by running the reference itself
(`tests/golden/make_golden.py`), and `tests/test_oracle.py` checks this file against them.

Two deliberate differences from the reference, both where the reference leaves the result
unspecified:
  * the expert sort is stable (`sort(stable=True)`; the reference calls `sort()` at
    xma/layers/moe/__init__.py:218, whose order inside one expert is arbitrary);
  * `continuous_count` is called on the torch path directly (the reference forgets to forward
    `kernel_backend` at xma/layers/moe/__init__.py:219).
Neither changes the layer's output.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def continuous_count(x: torch.Tensor, bins: int) -> torch.Tensor:
    """xma/functional/continuous_count/__init__.py:28-40 (torch branch)."""
    if bins == 1:
        return torch.tensor([x.numel()], dtype=torch.uint32, device=x.device)
    return x.bincount(minlength=bins).to(torch.uint32)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """xma/functional/swiglu/__init__.py:34-43: up * silu(gate) in float32, result in gate.dtype."""
    return (up.float() * F.silu(gate.float())).to(gate.dtype)


def swiglu_packed(x: torch.Tensor) -> torch.Tensor:
    """xma/functional/swiglu_packed.py:36-37 with xma/functional/swiglu/__init__.py:34-43:
    up = first half, gate = second half, float32 inside, result in x.dtype."""
    up, gate = x.chunk(2, dim=-1)
    return (up.float() * F.silu(gate.float())).to(x.dtype)


def get_topk(logits: torch.Tensor, top_k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """xma/layers/moe/__init__.py:268-274."""
    if top_k == 1:
        return logits.max(dim=-1, keepdim=True)
    return logits.topk(top_k, dim=-1)


def compute_routing_weights(
    hidden_states: torch.Tensor, gate_weight: torch.Tensor, top_k: int
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """xma/layers/moe/__init__.py:190-203: logits, softmax over the top-k logits in float32."""
    router_logits = F.linear(hidden_states, gate_weight)
    router_weights, selected_experts = get_topk(router_logits, top_k)
    router_weights = F.softmax(router_weights.float(), dim=-1).type_as(hidden_states)
    return router_logits, router_weights, selected_experts


def sort_experts(selected_experts: torch.Tensor, num_experts: int):
    """xma/layers/moe/__init__.py:218-225 with a stable sort.
    Returns sorted_expert_idxs, sorted_scattered_idxs, expert_frequency (uint32), expert_offsets."""
    sorted_expert_idxs, sorted_scattered_idxs = selected_experts.flatten().sort(stable=True)
    expert_frequency = continuous_count(sorted_expert_idxs, num_experts)
    expert_offsets = expert_frequency.to(torch.int64).cumsum(-1)
    return sorted_expert_idxs, sorted_scattered_idxs, expert_frequency, expert_offsets


def compute_experts(
    hidden_states: torch.Tensor,
    router_weights: torch.Tensor,
    selected_experts: torch.Tensor,
    w_fc: torch.Tensor,
    w_proj: torch.Tensor,
    activation=swiglu_packed,
) -> torch.Tensor:
    """xma/layers/moe/__init__.py:243-262 and Experts.torch_forward (:95-111): gather rows into expert
    order, one F.linear per expert, activation, second F.linear per expert, scale by the gates in
    the model dtype, index_add back to token order in the model dtype."""
    num_experts = w_fc.size(0)
    top_k = selected_experts.size(1)
    T = hidden_states.size(0)
    _, sorted_scattered_idxs, expert_frequency, _ = sort_experts(selected_experts, num_experts)
    fan_in_index = sorted_scattered_idxs // top_k
    batch_gates = router_weights.flatten()[sorted_scattered_idxs]
    h = hidden_states[fan_in_index]
    parts = h.split(expert_frequency.tolist(), dim=0)
    parts = [F.linear(parts[e], w_fc[e]) for e in range(num_experts)]
    parts = [activation(part) for part in parts]
    h = torch.cat([F.linear(parts[e], w_proj[e]) for e in range(num_experts)], dim=0)
    h = h * batch_gates.unsqueeze(-1)
    zeros = torch.zeros((T, hidden_states.size(1)), dtype=h.dtype, device=h.device)
    return zeros.index_add(0, fan_in_index, h)


def moe_forward(
    hidden_states: torch.Tensor,
    gate_weight: torch.Tensor,
    w_fc: torch.Tensor,
    w_proj: torch.Tensor,
    top_k: int,
    activation=swiglu_packed,
    selected_experts: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """MoE.forward (xma/layers/moe/__init__.py:168-188). Returns (y, router_logits, router_weights,
    selected_experts). When `selected_experts` is given, the router weights are the softmax over the
    logits gathered at those experts, so that a low-precision run and its float32 oracle cannot
    diverge in routing."""
    shape = hidden_states.shape
    x = hidden_states.reshape(-1, shape[-1])
    if selected_experts is None:
        router_logits, router_weights, selected_experts = compute_routing_weights(x, gate_weight, top_k)
    else:
        router_logits = F.linear(x, gate_weight)
        picked = router_logits.gather(1, selected_experts)
        router_weights = F.softmax(picked.float(), dim=-1).type_as(x)
    y = compute_experts(x, router_weights, selected_experts, w_fc, w_proj, activation)
    return y.view(shape), router_logits, router_weights, selected_experts


def moe_forward_backward(
    hidden_states, gate_weight, w_fc, w_proj, top_k, grad_output, activation=swiglu_packed, selected_experts=None
) -> dict[str, torch.Tensor]:
    """Forward plus autograd backward against `grad_output`, as the reference's own test does with
    `y.sum().backward()` (tests/layers/moe_test.py:124-127), generalised to any upstream gradient."""
    x = hidden_states.detach().clone().requires_grad_(True)
    gw = gate_weight.detach().clone().requires_grad_(True)
    w1 = w_fc.detach().clone().requires_grad_(True)
    w2 = w_proj.detach().clone().requires_grad_(True)
    y, logits, router_weights, selected = moe_forward(x, gw, w1, w2, top_k, activation, selected_experts)
    y.backward(grad_output)
    return {
        "y": y.detach(),
        "router_logits": logits.detach(),
        "router_weights": router_weights.detach(),
        "selected_experts": selected,
        "dx": x.grad,
        "dgate": gw.grad,
        "dw_fc": w1.grad,
        "dw_proj": w2.grad,
    }


def pack_sequence(x: torch.Tensor, cu_seqlens: torch.Tensor, padding_side: str = "left") -> torch.Tensor:
    """_PackSequence.forward_backward_torch (xma/functional/sequence_packing/__init__.py:21-38):
    padded batch [B, S, ...] -> packed tokens [total, ...]."""
    B, S = x.size()[:2]
    seqlens = (cu_seqlens[1:] - cu_seqlens[:-1]).to(torch.int64)
    batch_indices = torch.arange(B, device=x.device).repeat_interleave(seqlens)
    if padding_side == "left":
        seq_indices = torch.cat([torch.arange(int(S - sl), S, device=x.device) for sl in seqlens])
    elif padding_side == "right":
        seq_indices = torch.cat([torch.arange(int(sl), device=x.device) for sl in seqlens])
    else:
        raise ValueError(f"unexpected padding_side ({padding_side})")
    return x[batch_indices, seq_indices]


def unpack_sequence(
    x: torch.Tensor, cu_seqlens: torch.Tensor, batch_size: int, sequence_length: int, padding_side: str = "left"
) -> torch.Tensor:
    """_UnpackSequence.forward_backward_torch (xma/functional/sequence_packing/__init__.py:102-123):
    packed tokens [total, ...] -> zero-padded batch [B, S, ...]."""
    S = sequence_length
    seqlens = (cu_seqlens[1:] - cu_seqlens[:-1]).to(torch.int64)
    batch_indices = torch.arange(batch_size, device=x.device).repeat_interleave(seqlens)
    if padding_side == "left":
        seq_indices = torch.cat([torch.arange(int(S - sl), S, device=x.device) for sl in seqlens])
    elif padding_side == "right":
        seq_indices = torch.cat([torch.arange(int(sl), device=x.device) for sl in seqlens])
    else:
        raise ValueError(f"unexpected padding_side ({padding_side})")
    padded = torch.zeros(batch_size, S, *x.size()[1:], dtype=x.dtype, device=x.device)
    padded[batch_indices, seq_indices] = x
    return padded
