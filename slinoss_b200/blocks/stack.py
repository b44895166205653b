"""``SLinOSSStack``: a ModuleList of blocks plus the final norm (no embeddings or
heads), with the ``forward`` / ``step`` / ``init_state`` contract of the reference
stack (slinoss/blocks/stack.py:16-250)."""

from __future__ import annotations

import torch
import torch.utils.checkpoint
from torch import nn

from .block import SLinOSSBlock, apply_norm, make_norm
from .config import SLinOSSStackConfig
from .state import SLinOSSStackState


class SLinOSSStack(nn.Module):
    def __init__(self, config: SLinOSSStackConfig, *, device=None, dtype=None) -> None:
        super().__init__()
        self.config, self.d_model = config, config.d_model
        self.blocks = nn.ModuleList(
            [SLinOSSBlock(cfg, device=device, dtype=dtype) for cfg in config.blocks])
        self.final_norm = None if config.final_norm_kind == "none" else make_norm(
            config.final_norm_kind, config.d_model, eps=config.final_norm_eps, device=device,
            dtype=dtype)

    def init_state(self, batch_size, *, device=None, dtype=None) -> SLinOSSStackState:
        return SLinOSSStackState(
            layers=[b.init_state(batch_size, device=device, dtype=dtype) for b in self.blocks])

    def init_decode_state(self, batch_size, *, device=None, dtype=None) -> SLinOSSStackState:
        return SLinOSSStackState(
            layers=[b.init_decode_state(batch_size, device=device, dtype=dtype) for b in self.blocks])

    def _final(self, x):
        return x if self.final_norm is None else apply_norm(self.final_norm, x)

    def _check_state(self, state):
        if state is not None and len(state.layers) != len(self.blocks):
            raise ValueError("State layer count must match stack depth. "
                             f"Got {len(state.layers)} state layers for {len(self.blocks)} blocks.")

    def forward(self, x, *, state: SLinOSSStackState | None = None, return_state: bool = False,
                context=None, sequence_group=None):
        """``sequence_group``: see ``SLinOSSMixer.forward`` (the time axis of ``x`` sharded over the ranks of a
        process group; norms and FFN branches are per token, only the mixers exchange anything)."""
        if x.ndim != 3 or x.shape[-1] != self.d_model:
            raise ValueError(f"Expected x shape (batch, T, {self.d_model}), got {tuple(x.shape)}.")
        hidden = x
        if sequence_group is not None:
            if state is not None or return_state or (self.config.gradient_checkpointing and self.training):
                raise ValueError("sequence_group cannot be combined with a streaming state or with "
                                 "gradient checkpointing (its exchanges are collectives).")
            for block in self.blocks:
                hidden = block(hidden, context=context, sequence_group=sequence_group)
            return self._final(hidden).to(dtype=x.dtype)
        if self.config.gradient_checkpointing and self.training:
            if state is not None or return_state:
                raise ValueError("gradient_checkpointing in SLinOSSStack requires "
                                 "state=None and return_state=False.")
            for block in self.blocks:
                hidden = torch.utils.checkpoint.checkpoint(block, hidden, use_reentrant=False)
            return self._final(hidden).to(dtype=x.dtype)
        self._check_state(state)
        layers = []
        for i, block in enumerate(self.blocks):
            out = block(hidden, state=None if state is None else state.layers[i],
                        return_state=return_state, context=context)
            if return_state:
                hidden, nxt = out
                layers.append(nxt)
            else:
                hidden = out
        out = self._final(hidden).to(dtype=x.dtype)
        return (out, SLinOSSStackState(layers=layers)) if return_state else out

    def step(self, x, state: SLinOSSStackState | None = None, *, inplace=None, context=None):
        hidden = x
        if hidden.ndim == 3:
            if hidden.shape[1] != 1:
                raise ValueError(f"Expected time dim 1 for stack.step, got {tuple(hidden.shape)}.")
            hidden = hidden[:, 0, :]
        if hidden.ndim != 2 or hidden.shape[-1] != self.d_model:
            raise ValueError(f"Expected hidden shape (batch, {self.d_model}), got {tuple(hidden.shape)}.")
        self._check_state(state)
        layers = []
        for i, block in enumerate(self.blocks):
            hidden, nxt = block.step(hidden, None if state is None else state.layers[i],
                                     inplace=inplace, context=context)
            layers.append(nxt)
        hidden = self._final(hidden).to(dtype=x.dtype)
        if x.ndim == 3:
            hidden = hidden.unsqueeze(1)
        return hidden, SLinOSSStackState(layers=layers)


__all__ = ["SLinOSSStack"]
