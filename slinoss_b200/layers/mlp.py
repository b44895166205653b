"""Channel-mixing FFN of a block (library GEMMs; the activation runs on this
package's row kernel on CUDA, plain torch elsewhere).  Same constructor surface and state_dict keys as the reference's
``SLinOSSMLP`` (slinoss/layers/mlp.py:37-166)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal

import torch
from torch import nn
from torch.nn import functional as F

MLPKind = Literal["swiglu", "gelu"]


@dataclass(frozen=True, slots=True)
class SLinOSSMLPConfig:
    kind: MLPKind = "swiglu"
    hidden_dim: int | None = None
    expand: float = 8.0 / 3.0
    multiple_of: int = 128
    bias: bool = False

    def resolve_hidden_dim(self, d_model: int) -> int:
        if d_model <= 0 or self.multiple_of <= 0:
            raise ValueError("d_model and multiple_of must be positive.")
        hidden = self.hidden_dim
        if hidden is None:
            if self.expand <= 0.0:
                raise ValueError(f"expand must be positive. Got {self.expand}.")
            hidden = int(d_model * self.expand)
        if hidden <= 0:
            raise ValueError(f"hidden_dim must be positive. Got {hidden}.")
        return (int(hidden) + self.multiple_of - 1) // self.multiple_of * self.multiple_of


class SLinOSSMLP(nn.Module):
    def __init__(self, d_model: int, *, config: SLinOSSMLPConfig | None = None, device=None,
                 dtype=None, **overrides) -> None:
        super().__init__()
        if config is None:
            config = SLinOSSMLPConfig(**{k: v for k, v in overrides.items() if v is not None})
        elif any(v is not None for v in overrides.values()):
            raise ValueError("Pass either config or explicit keyword overrides, not both.")
        if config.kind not in ("swiglu", "gelu"):
            raise ValueError(f"Unsupported MLP kind: {config.kind!r}.")
        self.d_model, self.config, self.kind = int(d_model), config, config.kind
        self.hidden_dim = config.resolve_hidden_dim(self.d_model)
        width = 2 * self.hidden_dim if self.kind == "swiglu" else self.hidden_dim
        self.in_proj = nn.Linear(self.d_model, width, bias=config.bias, device=device, dtype=dtype)
        self.out_proj = nn.Linear(self.hidden_dim, self.d_model, bias=config.bias, device=device,
                                  dtype=dtype)

    @classmethod
    def from_config(cls, d_model, config, *, device=None, dtype=None) -> "SLinOSSMLP":
        return cls(d_model, config=config, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.d_model:
            raise ValueError(f"Expected last dim {self.d_model}, got {int(x.shape[-1])}.")
        h = self.in_proj(x)
        from ..ops.block import ffn_activation, ffn_activation_supported   # (ops.block imports nothing of layers)
        if ffn_activation_supported(h, self.kind):
            return self.out_proj(ffn_activation(h, self.kind))
        if self.kind == "swiglu":
            value, gate = h.chunk(2, dim=-1)
            return self.out_proj(value * F.silu(gate))
        return self.out_proj(F.gelu(h, approximate="tanh"))

    def decode_one(self, x: torch.Tensor) -> torch.Tensor:
        if x.ndim != 2 or x.shape[-1] != self.d_model:
            raise ValueError(
                f"Expected decode input shape (batch, {self.d_model}), got {tuple(x.shape)}.")
        return self.forward(x)

    step = decode_one


__all__ = ["MLPKind", "SLinOSSMLP", "SLinOSSMLPConfig"]
