"""swiglu with the signature of xma/functional/swiglu/__init__.py:100-120: `up * gate * sigmoid(gate)`
for separate `gate` and `up` tensors, computed in float32 and rounded to their dtype."""

from __future__ import annotations

import torch

from ..accelerator import KernelBackend, require_cuda_backend


class _Swiglu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        from ..ops import swiglu_forward_cuda

        gate, up = gate.contiguous(), up.contiguous()
        y = torch.empty_like(gate)
        swiglu_forward_cuda(gate, up, y)
        ctx.save_for_backward(gate, up)
        return y

    @staticmethod
    def backward(ctx, dy: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        from ..ops import swiglu_backward_cuda

        gate, up = ctx.saved_tensors
        dgate, dup = torch.empty_like(gate), torch.empty_like(up)
        swiglu_backward_cuda(gate, up, dy.contiguous(), dgate, dup)
        return dgate, dup


def swiglu(gate: torch.Tensor, up: torch.Tensor, *, kernel_backend: KernelBackend | None = None) -> torch.Tensor:
    require_cuda_backend(kernel_backend)
    assert gate.size() == up.size(), "tensors gate and up should have same shape"
    assert gate.type() == up.type(), "tensors gate and up should have same dtype"
    return _Swiglu.apply(gate, up)
