"""Pre-norm residual block: ``x + mixer(norm(x))`` then ``x + ffn(norm(x))``.

Composition, parameter names and residual arithmetic (float32 add, cast back)
follow the reference block (slinoss/blocks/block.py:41-303).  On CUDA the FFN
branch runs as one rematerialising op (``ops.block.ffn_residual``) when its
conditions hold, else as plain torch.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from ..layers import RMSNorm, SLinOSSMixer
from ..layers.mlp import SLinOSSMLP
from ..ops.block import ffn_residual, ffn_residual_supported, residual_add
from .config import SLinOSSBlockConfig
from .state import SLinOSSBlockState


def make_norm(kind, d_model, *, eps, device=None, dtype=None) -> nn.Module:
    if kind == "rmsnorm":
        return RMSNorm(d_model, eps=eps, device=device, dtype=dtype)
    return nn.LayerNorm(d_model, eps=eps, device=device, dtype=dtype)


def apply_norm(norm: nn.Module, x: torch.Tensor) -> torch.Tensor:
    w = getattr(norm, "weight", None)
    return norm(x.to(dtype=w.dtype)) if isinstance(w, torch.Tensor) else norm(x)


class SLinOSSBlock(nn.Module):
    def __init__(self, config: SLinOSSBlockConfig, *, device=None, dtype=None) -> None:
        super().__init__()
        self.config, self.d_model = config, config.d_model
        self.residual_in_fp32 = bool(config.residual_in_fp32)
        self.residual_dropout = float(config.residual_dropout)
        # What the FFN branch rebuilds in the backward pass on CUDA: "full" (keeps only the branch input,
        # the reference's schedule), "rows" (keeps the projection too: no GEMM is repeated) or "none"
        # (plain autograd, the default: fastest while the activations fit in memory).
        self.ffn_remat = "none"
        kw = {"device": device, "dtype": dtype}
        self.mixer_norm = make_norm(config.norm_kind, config.d_model, eps=config.norm_eps, **kw)
        self.mixer = SLinOSSMixer(config.d_model, **config.mixer.build_kwargs(), **kw)
        if config.ffn is None:
            self.ffn_norm, self.ffn = None, None
        else:
            self.ffn_norm = make_norm(config.norm_kind, config.d_model, eps=config.norm_eps, **kw)
            self.ffn = SLinOSSMLP.from_config(config.d_model, config.ffn, **kw)

    def init_state(self, batch_size, *, device=None, dtype=None) -> SLinOSSBlockState:
        return SLinOSSBlockState(mixer=self.mixer.init_state(batch_size, device=device, dtype=dtype))

    def init_decode_state(self, batch_size, *, device=None, dtype=None) -> SLinOSSBlockState:
        return SLinOSSBlockState(
            mixer=self.mixer.init_decode_state(batch_size, device=device, dtype=dtype))

    def _drop(self, x):
        return x if self.residual_dropout <= 0.0 else F.dropout(x, self.residual_dropout, self.training)

    def _add(self, residual, branch):
        return residual_add(residual, branch, self.residual_in_fp32)

    def _ffn_residual(self, x):
        no_drop = self.residual_dropout <= 0.0 or not self.training
        if no_drop and self.ffn_remat != "none" and ffn_residual_supported(x, self.ffn_norm, self.ffn):
            return ffn_residual(x, self.ffn_norm, self.ffn, residual_in_fp32=self.residual_in_fp32,
                                remat=self.ffn_remat)
        return self._add(x, self._drop(self.ffn(apply_norm(self.ffn_norm, x))))

    def forward(self, x, *, state: SLinOSSBlockState | None = None, return_state: bool = False,
                context=None, sequence_group=None):
        if x.ndim != 3 or x.shape[-1] != self.d_model:
            raise ValueError(f"Expected x shape (batch, T, {self.d_model}), got {tuple(x.shape)}.")
        extra = {} if sequence_group is None else {"sequence_group": sequence_group}
        mixed = self.mixer(apply_norm(self.mixer_norm, x),
                           state=None if state is None else state.mixer, return_state=return_state, **extra)
        nxt = None
        if return_state:
            mixed, mixer_state = mixed
            nxt = SLinOSSBlockState(mixer=mixer_state)
        out = self._add(x, self._drop(mixed))
        if self.ffn is not None:
            out = self._ffn_residual(out)
        return (out, nxt) if return_state else out

    def step(self, x, state: SLinOSSBlockState | None = None, *, inplace=None, context=None):
        token = x
        if token.ndim == 3:
            if token.shape[1] != 1:
                raise ValueError(f"Expected time dim 1 for block.step, got {tuple(token.shape)}.")
            token = token[:, 0, :]
        if token.ndim != 2 or token.shape[-1] != self.d_model:
            raise ValueError(f"Expected x shape (batch, {self.d_model}) or "
                             f"(batch, 1, {self.d_model}), got {tuple(x.shape)}.")
        mixed, mixer_state = self.mixer.step(apply_norm(self.mixer_norm, token),
                                             None if state is None else state.mixer, inplace=inplace)
        out = self._add(token, self._drop(mixed.to(dtype=token.dtype)))
        if self.ffn is not None:
            out = self._ffn_residual(out)
        if x.ndim == 3:
            out = out.unsqueeze(1)
        return out, SLinOSSBlockState(mixer=mixer_state)


__all__ = ["SLinOSSBlock", "apply_norm", "make_norm"]
