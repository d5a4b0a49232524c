"""continuous_count with the signature of xma/functional/continuous_count/__init__.py:11-47."""

from __future__ import annotations

import torch

from ..accelerator import KernelBackend, require_cuda_backend
from ..ops import continuous_count_cuda


@torch.no_grad()
def continuous_count(x: torch.Tensor, bins: int, *, kernel_backend: KernelBackend | None = None) -> torch.Tensor:
    """Counts the occurrences of the values 0, 1, ..., bins-1 in the 1-D int32/int64 tensor `x`.

    Returns `uint32[bins]` on `x.device`. Values outside `[0, bins)` are ignored.
    """
    if bins == 1:
        return torch.tensor([x.numel()], dtype=torch.uint32, device=x.device)

    assert x.dim() == 1, "x should be 1-dimensional"
    assert x.dtype in [torch.int32, torch.long]
    require_cuda_backend(kernel_backend)

    output = torch.empty(bins, dtype=torch.uint32, device=x.device)
    continuous_count_cuda(x=x.contiguous(), output=output, E=bins)
    return output
