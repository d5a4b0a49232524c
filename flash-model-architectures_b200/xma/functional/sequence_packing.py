"""pack_sequence / unpack_sequence with the signatures of
xma/functional/sequence_packing/__init__.py:183-277, on the sm_100a copy kernels."""

from __future__ import annotations

from typing import Sequence

import torch

from ..accelerator import KernelBackend, require_cuda_backend
from ..ops import pack_unpack_sequence_cuda


class _PackSequence(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cu_seqlens, output_shape, padding_side):
        x = x.contiguous()
        cu_seqlens = cu_seqlens.contiguous()
        y = torch.empty(output_shape, device=x.device, dtype=x.dtype)
        pack_unpack_sequence_cuda(x=x, output=y, cu_seqlens=cu_seqlens, padding_side=padding_side, pack=True)
        ctx.save_for_backward(cu_seqlens)
        ctx.padding_side, ctx.x_shape = padding_side, x.size()
        return y

    @staticmethod
    def backward(ctx, dy):
        (cu_seqlens,) = ctx.saved_tensors
        dx = torch.empty(*ctx.x_shape, device=dy.device, dtype=dy.dtype)  # the kernel writes the padding zeros too
        pack_unpack_sequence_cuda(
            x=dy.contiguous(), output=dx, cu_seqlens=cu_seqlens, padding_side=ctx.padding_side, pack=False
        )
        return dx, None, None, None


class _UnpackSequence(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cu_seqlens, output_shape, padding_side):
        x = x.contiguous()
        cu_seqlens = cu_seqlens.contiguous()
        y = torch.empty(*output_shape, device=x.device, dtype=x.dtype)
        pack_unpack_sequence_cuda(x=x, output=y, cu_seqlens=cu_seqlens, padding_side=padding_side, pack=False)
        ctx.save_for_backward(cu_seqlens)
        ctx.padding_side, ctx.x_shape = padding_side, x.size()
        return y

    @staticmethod
    def backward(ctx, dy):
        (cu_seqlens,) = ctx.saved_tensors
        dx = torch.empty(*ctx.x_shape, device=dy.device, dtype=dy.dtype)
        pack_unpack_sequence_cuda(
            x=dy.contiguous(), output=dx, cu_seqlens=cu_seqlens, padding_side=ctx.padding_side, pack=True
        )
        return dx, None, None, None


def pack_sequence(
    inputs: Sequence[torch.Tensor],
    cu_seqlens: torch.Tensor,
    total_tokens: int,
    padding_side: str = "left",
    *,
    kernel_backend: KernelBackend | None = None,
) -> Sequence[torch.Tensor]:
    """Packs padded batches `[B, S, ...]` into token streams `[total_tokens, ...]`."""
    assert padding_side in ["left", "right"]
    assert isinstance(inputs, (list, tuple))
    require_cuda_backend(kernel_backend)
    outputs = []
    for x in inputs:
        assert x.dim() >= 2
        assert x.size(0) == cu_seqlens.size(0) - 1
        outputs.append(_PackSequence.apply(x, cu_seqlens, (total_tokens, *x.size()[2:]), padding_side))
    return outputs


def unpack_sequence(
    inputs: Sequence[torch.Tensor],
    cu_seqlens: torch.Tensor,
    batch_size: int,
    sequence_length: int,
    padding_side: str = "left",
    *,
    kernel_backend: KernelBackend | None = None,
) -> Sequence[torch.Tensor]:
    """Unpacks token streams `[total_tokens, ...]` into zero-padded batches `[B, S, ...]`."""
    assert padding_side in ["left", "right"]
    assert isinstance(inputs, (list, tuple))
    require_cuda_backend(kernel_backend)
    outputs = []
    for x in inputs:
        assert x.dim() >= 2
        assert cu_seqlens.size(0) - 1 == batch_size
        outputs.append(
            _UnpackSequence.apply(x, cu_seqlens, (batch_size, sequence_length, *x.size()[1:]), padding_side)
        )
    return outputs
