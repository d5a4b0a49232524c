"""B200-native drop-in for the Mixture-of-Experts hot path of XMA: `MoE`, `continuous_count`,
`swiglu_packed`, `KernelBackend`. Everything runs on hand-written sm_100a kernels in
libxma_b200.so; there is no other backend and no fallback."""

import random

import numpy as np
import torch

from ._native import check_status
from .accelerator import Accelerator, KernelBackend
from .functional import continuous_count, pack_sequence, swiglu, swiglu_packed, unpack_sequence
from .layers import Experts, MoE


def set_seed(seed: int) -> None:
    """Seeds python, numpy and torch (xma/utils/random.py:11-16)."""
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
