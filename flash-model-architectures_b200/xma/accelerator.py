"""KernelBackend / Accelerator enums kept for signature compatibility with xma/accelerator.py:23-128.

Only `KernelBackend.cuda` (and `None`, which means the same) is served: this package has a single
sm_100a implementation and no dispatch.
"""

from __future__ import annotations

from enum import Enum

import torch


class KernelBackend(Enum):
    cuda = "cuda"
    nki = "nki"
    pallas = "pallas"
    rocm = "rocm"
    torch = "torch"
    triton = "triton"

    def get_compatible_accelerator(self) -> "Accelerator":
        return Accelerator.cuda if self == KernelBackend.cuda else None

    def verify_accelerator(self) -> bool:
        return self == KernelBackend.cuda and Accelerator.get_accelerator() == Accelerator.cuda


class Accelerator(Enum):
    cpu = "cpu"
    cuda = "cuda"

    @staticmethod
    def get_accelerator() -> "Accelerator":
        return Accelerator.cuda if torch.cuda.is_available() else Accelerator.cpu

    @staticmethod
    def get_kernel_backend() -> KernelBackend:
        return KernelBackend.cuda

    def get_current_device(self) -> int | str:
        return torch.cuda.current_device() if self == Accelerator.cuda else "cpu"


def require_cuda_backend(kernel_backend: KernelBackend | None) -> None:
    """`None` and `KernelBackend.cuda` are accepted; every other backend raises (no fallback)."""
    if kernel_backend is None or kernel_backend == KernelBackend.cuda:
        return
    raise ValueError(
        f"kernel_backend={kernel_backend} is not available: this build only has the sm_100a CUDA path"
    )
