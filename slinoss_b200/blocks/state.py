"""Streaming state of blocks and stacks: thin containers over the mixers' states with the same four
operations as every state object of the package (``copy_``, ``clone``, ``detach``, ``to``).  Field names follow
the reference's state records (slinoss/blocks/state.py:13-60), because callers index them.

Both containers share one implementation: a state is a tree whose leaves are ``SLinOSSMixerState`` objects;
``_map`` rebuilds the tree with an operation applied to every leaf.
"""

from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field

from ..layers.state import SLinOSSMixerState


def _apply(node, op):
    """``op`` on every mixer state below ``node`` (a mixer state, a state container, or a list of them)."""
    if isinstance(node, SLinOSSMixerState):
        return op(node)
    if isinstance(node, list):
        return [_apply(child, op) for child in node]
    return type(node)(**{f.name: _apply(getattr(node, f.name), op) for f in dataclasses.fields(node)})


def _leaves(node):
    if isinstance(node, SLinOSSMixerState):
        yield node
    elif isinstance(node, list):
        for child in node:
            yield from _leaves(child)
    else:
        for f in dataclasses.fields(node):
            yield from _leaves(getattr(node, f.name))


class _StateTree:
    def clone(self):
        return _apply(self, lambda s: s.clone())

    def detach(self):
        return _apply(self, lambda s: s.detach())

    def to(self, *, device=None, dtype=None):
        return _apply(self, lambda s: s.to(device=device, dtype=dtype))

    def copy_(self, other):
        """In-place copy of ``other``'s tensors into this state's (same tree shape required)."""
        for dst, src in zip(_leaves(self), _leaves(other), strict=True):
            dst.copy_(src)
        return self


@dataclass
class SLinOSSBlockState(_StateTree):
    mixer: SLinOSSMixerState = field(default_factory=SLinOSSMixerState)


@dataclass
class SLinOSSStackState(_StateTree):
    layers: list[SLinOSSBlockState] = field(default_factory=list)


__all__ = ["SLinOSSBlockState", "SLinOSSStackState"]
