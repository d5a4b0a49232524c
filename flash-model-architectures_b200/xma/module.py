"""Base class of the layers (xma/module.py:8-11)."""

import torch.nn as nn


class XMAModule(nn.Module):
    def extra_repr(self) -> str:
        return ""
