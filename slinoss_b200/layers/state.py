"""Streaming state containers (same fields and methods as the reference's
``ScanState`` / ``SLinOSSMixerState``, slinoss/layers/state.py:56-148)."""

from __future__ import annotations

from dataclasses import dataclass, field, fields

import torch


def _map(x, fn):
    return None if x is None else fn(x)


def _adopt(cur, new):
    """Keep ``cur``'s storage when ``new`` has the same shape/device/dtype."""
    if cur is None or new is None or cur is new:
        return new if cur is None or new is None else cur
    if cur.shape != new.shape or cur.device != new.device or cur.dtype != new.dtype:
        return new
    cur.copy_(new)
    return cur


def _to(x, device, dtype):
    if x is None:
        return None
    kw = {k: v for k, v in (("device", device), ("dtype", dtype)) if v is not None}
    return x.to(**kw) if kw else x


@dataclass
class ScanState:
    """``state (batch,heads,P,2N)``, ``b_prev (batch,groups,2N)``, ``u_prev (batch,heads,P)``."""

    state: torch.Tensor | None = None
    b_prev: torch.Tensor | None = None
    u_prev: torch.Tensor | None = None

    def _names(self):
        return [f.name for f in fields(self)]

    def copy_(self, other: "ScanState") -> "ScanState":
        for n in self._names():
            dst, src = getattr(self, n), getattr(other, n)
            if dst is not None and src is not None:
                dst.copy_(src)
        return self

    def adopt_(self, other: "ScanState") -> "ScanState":
        for n in self._names():
            setattr(self, n, _adopt(getattr(self, n), getattr(other, n)))
        return self

    def detach(self) -> "ScanState":
        return ScanState(*[_map(getattr(self, n), torch.Tensor.detach) for n in self._names()])

    def clone(self) -> "ScanState":
        return ScanState(*[_map(getattr(self, n), torch.Tensor.clone) for n in self._names()])

    def to(self, *, device=None, dtype=None) -> "ScanState":
        return ScanState(*[_to(getattr(self, n), device, dtype) for n in self._names()])


@dataclass
class SLinOSSMixerState:
    """``conv (batch, d_inner, d_conv-1)`` plus the scan state."""

    conv: torch.Tensor | None = None
    scan: ScanState = field(default_factory=ScanState)
    _engine: object | None = field(default=None, repr=False, compare=False)

    def copy_(self, other: "SLinOSSMixerState") -> "SLinOSSMixerState":
        if self.conv is not None and other.conv is not None:
            self.conv.copy_(other.conv)
        self.scan.copy_(other.scan)
        return self

    def adopt_(self, other: "SLinOSSMixerState") -> "SLinOSSMixerState":
        self.conv = _adopt(self.conv, other.conv)
        self.scan.adopt_(other.scan)
        return self

    def detach(self) -> "SLinOSSMixerState":
        return SLinOSSMixerState(conv=_map(self.conv, torch.Tensor.detach), scan=self.scan.detach())

    def clone(self) -> "SLinOSSMixerState":
        return SLinOSSMixerState(conv=_map(self.conv, torch.Tensor.clone), scan=self.scan.clone())

    def to(self, *, device=None, dtype=None) -> "SLinOSSMixerState":
        return SLinOSSMixerState(conv=_to(self.conv, device, dtype),
                                 scan=self.scan.to(device=device, dtype=dtype))


__all__ = ["ScanState", "SLinOSSMixerState"]
