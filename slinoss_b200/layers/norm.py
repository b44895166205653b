"""RMSNorm that computes in the weight dtype and returns the input dtype
(reference: slinoss/layers/norm.py:10-22)."""

from __future__ import annotations

import torch
from torch import nn


class RMSNorm(nn.RMSNorm):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.weight is None or x.dtype == self.weight.dtype:
            return super().forward(x)
        return super().forward(x.to(self.weight.dtype)).to(x.dtype)


__all__ = ["RMSNorm"]
