"""Streaming state of blocks and stacks (reference: slinoss/blocks/state.py:13-60)."""

from __future__ import annotations

from dataclasses import dataclass, field

from ..layers.state import SLinOSSMixerState


@dataclass
class SLinOSSBlockState:
    mixer: SLinOSSMixerState = field(default_factory=SLinOSSMixerState)

    def copy_(self, other):
        self.mixer.copy_(other.mixer)
        return self

    def clone(self):
        return SLinOSSBlockState(mixer=self.mixer.clone())

    def detach(self):
        return SLinOSSBlockState(mixer=self.mixer.detach())

    def to(self, *, device=None, dtype=None):
        return SLinOSSBlockState(mixer=self.mixer.to(device=device, dtype=dtype))


@dataclass
class SLinOSSStackState:
    layers: list[SLinOSSBlockState] = field(default_factory=list)

    def copy_(self, other):
        for dst, src in zip(self.layers, other.layers, strict=True):
            dst.copy_(src)
        return self

    def clone(self):
        return SLinOSSStackState(layers=[s.clone() for s in self.layers])

    def detach(self):
        return SLinOSSStackState(layers=[s.detach() for s in self.layers])

    def to(self, *, device=None, dtype=None):
        return SLinOSSStackState(layers=[s.to(device=device, dtype=dtype) for s in self.layers])


__all__ = ["SLinOSSBlockState", "SLinOSSStackState"]
