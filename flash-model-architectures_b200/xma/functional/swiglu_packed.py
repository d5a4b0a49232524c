"""swiglu_packed with the signature of xma/functional/swiglu_packed.py:100-120.

`y = up * silu(gate)` with `up, gate = x.chunk(2, -1)`, computed in float32 and rounded to the
dtype of `x`. Inside `xma.layers.MoE` this callable is recognised by identity and the activation
then runs in the epilogue of the up-projection grouped GEMM; called on its own it runs as a
stand-alone sm_100a kernel.
"""

from __future__ import annotations

import torch

from ..accelerator import KernelBackend, require_cuda_backend


class _SwigluPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor) -> torch.Tensor:
        from ..ops import swiglu_packed_forward_cuda

        x = x.contiguous()
        y = torch.empty(*x.shape[:-1], x.size(-1) // 2, dtype=x.dtype, device=x.device)
        swiglu_packed_forward_cuda(x, y)
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy: torch.Tensor) -> torch.Tensor:
        from ..ops import swiglu_packed_backward_cuda

        (x,) = ctx.saved_tensors
        dx = torch.empty_like(x)
        swiglu_packed_backward_cuda(x, dy.contiguous(), dx)
        return dx


def swiglu_packed(x: torch.Tensor, *, kernel_backend: KernelBackend | None = None) -> torch.Tensor:
    require_cuda_backend(kernel_backend)
    assert x.size(-1) % 2 == 0
    original_shape = x.size()
    y = _SwigluPacked.apply(x.flatten(0, -2))
    return y.view(*original_shape[:-1], original_shape[-1] // 2)
