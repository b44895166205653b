"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (stand-ins: the reference measures on no dataset).

Distributions: ``U ~ N(0,1)``; ``r = clamp(exp(-softplus(a)), 0.9, 0.999)`` with
``a ~ N(0,1)``; ``theta ~ U(-pi, pi)``; ``M = r e^{i theta}``;
``dt = 5e-3 + (1e-1 - 5e-3) sigmoid(N(0,1))``; ``K`` = exact first-order-hold taps
of ``(dt, r, theta)``; ``B, C ~ N(0, 1/sqrt(N))``.  Everything is drawn on the CPU
from one ``torch.Generator`` so every consumer sees identical bits.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass
class ScanCase:
    U: torch.Tensor
    M: torch.Tensor
    K: torch.Tensor
    B: torch.Tensor
    C: torch.Tensor
    dY: torch.Tensor
    initial_states: torch.Tensor | None = None
    B_prev: torch.Tensor | None = None
    U_prev: torch.Tensor | None = None

    def tensors(self):
        return (self.U, self.M, self.K, self.B, self.C)

    def to(self, device):
        mv = lambda x: None if x is None else x.to(device)
        return ScanCase(*(mv(getattr(self, f)) for f in self.__dataclass_fields__))


def foh_taps_from_polar(dt: torch.Tensor, r: torch.Tensor, theta: torch.Tensor):
    """K (...,2,2) float32 from real ``dt, r, theta`` (tap 0 = prev, 1 = curr).

    With ``z = log r + i theta`` and ``rho = e^z``: ``kappa1 = (rho-1)/z``,
    ``kappa2 = (rho (z-1) + 1)/z^2``, ``kprev = dt kappa2``,
    ``kcurr = dt kappa1 - kprev``; a cubic Taylor branch covers ``|z| < 1e-4``."""
    dt = dt.double()
    z = torch.complex(torch.log(r.double()), theta.double())
    rho = torch.exp(z)
    small = z.abs() < 1e-4
    zs = torch.where(small, torch.ones_like(z), z)
    k1 = torch.where(small, 1 + z / 2 + z * z / 6 + z ** 3 / 24, (rho - 1) / zs)
    k2 = torch.where(small, 0.5 + z / 3 + z * z / 8 + z ** 3 / 30,
                     (rho * (zs - 1) + 1) / (zs * zs))
    kp = dt * k2
    kc = dt * k1 - kp
    return torch.stack((torch.view_as_real(kp), torch.view_as_real(kc)), dim=-2).float()


def make_scan_case(batch: int, heads: int, T: int, P: int, N: int, *, groups: int | None = None,
                   dtype: torch.dtype = torch.float32, seed: int = 0, streaming: bool = False,
                   with_init: bool = False) -> ScanCase:
    """Draws one scan problem on the CPU.  ``U, B, C, dY`` are cast to ``dtype``
    after generation; ``M, K`` (and the carried state) stay float32."""
    g = torch.Generator().manual_seed(seed)
    G = heads if groups is None else groups
    rn = lambda *s: torch.randn(*s, generator=g)
    U = rn(batch, heads, T, P)
    a = rn(batch, heads, T)
    r = torch.exp(-torch.nn.functional.softplus(a)).clamp(0.9, 0.999)
    theta = (torch.rand(batch, heads, T, generator=g) * 2 - 1) * math.pi
    M = torch.stack((r * torch.cos(theta), r * torch.sin(theta)), dim=-1).contiguous()
    dt = 5e-3 + (1e-1 - 5e-3) * torch.sigmoid(rn(batch, heads, T))
    K = foh_taps_from_polar(dt, r, theta).contiguous()
    B = (rn(batch, G, T, N, 2) / math.sqrt(N)).reshape(batch, G, T, 2 * N)
    C = (rn(batch, G, T, N, 2) / math.sqrt(N)).reshape(batch, G, T, 2 * N)
    dY = rn(batch, heads, T, P)
    case = ScanCase(U.to(dtype), M, K, B.to(dtype).contiguous(), C.to(dtype).contiguous(),
                    dY.to(dtype))
    if with_init:
        case.initial_states = 0.1 * rn(batch, heads, P, 2 * N)
    if streaming:
        case.B_prev = (rn(batch, G, 2 * N) / math.sqrt(N)).to(dtype)
        case.U_prev = rn(batch, heads, P).to(dtype)
    return case


__all__ = ["ScanCase", "foh_taps_from_polar", "make_scan_case"]
