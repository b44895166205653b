"""``SLinOSSScanPrep``: owner of the per-head scan-preparation parameters.

Same parameters, buffers, bounds, initialisation schedule and ``forward`` contract
as the reference module (slinoss/layers/scanprep.py:31-429); the computation runs
on the CUDA kernels behind ``ops.scanprep``.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from .backend import B200ScanPrepBackend, ScanInputs, ScanPrepBackend, ScanPrepInputs


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _logit(p: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    p = p.clamp(min=eps, max=1.0 - eps)
    return torch.log(p) - torch.log1p(-p)


class SLinOSSScanPrep(nn.Module):
    """Maps ``(value, params, bc)`` streams to scan inputs ``(U, M, K, B, C)``."""

    param_dim: int = 3
    bc_param_rows: int = 4

    def __init__(self, *, n_heads: int, bc_groups: int | None = None, d_state: int, d_head: int,
                 backend: ScanPrepBackend | None = None, dt_min: float = 5e-3,
                 dt_max: float = 1e-1, dt_init_floor: float = 5e-3, alpha_min: float = 0.0,
                 alpha_max: float = 20.0, theta_init_min: float = 0.05,
                 theta_init_max: float = 2.0, theta_mod_scale: float = 1.0, r_min: float = 0.8,
                 r_max: float = 1.0, eps: float = 1e-8, device=None) -> None:
        super().__init__()
        groups = n_heads if bc_groups is None else int(bc_groups)
        _require(n_heads > 0, f"n_heads must be positive. Got {n_heads}.")
        _require(groups > 0, f"bc_groups must be positive. Got {groups}.")
        _require(groups <= n_heads, f"bc_groups must be <= n_heads. Got {groups}, {n_heads}.")
        _require(n_heads % groups == 0,
                 f"n_heads must be divisible by bc_groups. Got {n_heads}, {groups}.")
        _require(d_state > 0, f"d_state must be positive. Got {d_state}.")
        _require(d_head > 0, f"d_head must be positive. Got {d_head}.")
        _require(0.0 < dt_min < dt_max, f"Require 0 < dt_min < dt_max. Got {dt_min}, {dt_max}.")
        _require(0.0 < dt_init_floor <= dt_max,
                 f"Require 0 < dt_init_floor <= dt_max. Got {dt_init_floor}.")
        _require(0.0 <= alpha_min < alpha_max,
                 f"Require 0 <= alpha_min < alpha_max. Got {alpha_min}, {alpha_max}.")
        _require(0.0 < theta_init_min <= theta_init_max < math.pi,
                 "Require 0 < theta_init_min <= theta_init_max < pi. Got "
                 f"{theta_init_min}, {theta_init_max}.")
        _require(theta_mod_scale >= 0.0, f"Require theta_mod_scale >= 0. Got {theta_mod_scale}.")
        _require(0.0 < r_min <= r_max <= 1.0, f"Require 0 < r_min <= r_max <= 1. Got {r_min}, {r_max}.")

        self.n_heads, self.bc_groups = int(n_heads), groups
        self.heads_per_bc_group = self.n_heads // groups
        self.d_state, self.d_head = int(d_state), int(d_head)
        self.d_inner = self.n_heads * self.d_head
        self.backend = B200ScanPrepBackend() if backend is None else backend
        self.dt_min, self.dt_max, self.dt_init_floor = float(dt_min), float(dt_max), float(dt_init_floor)
        self.alpha_min, self.alpha_max = float(alpha_min), float(alpha_max)
        self.theta_init_min, self.theta_init_max = float(theta_init_min), float(theta_init_max)
        self.theta_mod_scale = float(theta_mod_scale)
        self.r_min, self.r_max, self.eps = float(r_min), float(r_max), float(eps)

        mk = lambda: nn.Parameter(torch.empty((self.n_heads,), device=device, dtype=torch.float32))
        self.dt_bias, self.alpha_bias, self.theta_mod_bias, self.theta_bias = mk(), mk(), mk(), mk()
        sign = torch.ones((self.n_heads,), device=device, dtype=torch.float32)
        sign[1::2] = -1.0
        self.register_buffer("theta_sign", sign, persistent=True)
        self.reset_parameters()

    # -- initialisation: heads tile a (dt, theta) log-grid in boustrophedon order and get a
    #    log-spaced radius ladder (reference: scanprep.py:148-224) -----------------------------
    def _head_init_targets(self):
        dt_lo, dt_hi = max(self.dt_min, self.dt_init_floor), self.dt_max
        _require(dt_hi > dt_lo > 0.0, f"Bad dt init bounds: {dt_lo}, {dt_hi}.")
        n_dt = max(1, int(math.floor(math.sqrt(self.n_heads))))
        n_theta = math.ceil(self.n_heads / n_dt)
        dev = self.dt_bias.device
        dt_grid = torch.logspace(math.log10(dt_lo), math.log10(dt_hi), n_dt, device=dev,
                                 dtype=torch.float32)
        th_grid = torch.logspace(math.log10(self.theta_init_min), math.log10(self.theta_init_max),
                                 n_theta, device=dev, dtype=torch.float32)
        dts, ths = [], []
        for ti in range(n_theta):
            order = range(n_dt) if ti % 2 == 0 else range(n_dt - 1, -1, -1)
            for di in order:
                dts.append(dt_grid[di])
                ths.append(th_grid[ti])
        return torch.stack(dts[: self.n_heads]), torch.stack(ths[: self.n_heads])

    def reset_parameters(self) -> None:
        dt0, theta0 = self._head_init_targets()
        dt_u0 = (dt0 - self.dt_min) / (self.dt_max - self.dt_min)
        span = self.theta_init_max - self.theta_init_min
        theta_u0 = (theta0 - self.theta_init_min) / max(span, 1.0e-6)
        dev = self.alpha_bias.device
        if math.isclose(self.r_min, self.r_max):
            alpha0 = torch.full((self.n_heads,), self.alpha_min, device=dev, dtype=torch.float32)
        else:
            r_span = self.r_max - self.r_min
            lo, hi = math.exp(-self.alpha_max), math.exp(-self.alpha_min)
            log_r0 = torch.linspace(math.log(self.r_min + r_span * lo),
                                    math.log(self.r_min + r_span * hi), self.n_heads, device=dev,
                                    dtype=torch.float64)
            ratio = ((torch.exp(log_r0) - self.r_min) / r_span).clamp(min=lo, max=hi)
            alpha0 = (-torch.log(ratio)).clamp(min=self.alpha_min, max=self.alpha_max).float()
        _require(bool(torch.isfinite(alpha0).all()), "Nonfinite alpha initialization.")
        with torch.no_grad():
            self.dt_bias.copy_(_logit(dt_u0))
            self.alpha_bias.copy_(_logit((alpha0 - self.alpha_min) / (self.alpha_max - self.alpha_min)))
            self.theta_mod_bias.zero_()
            self.theta_bias.copy_(_logit(theta_u0))

    def _validate(self, inputs: ScanPrepInputs) -> None:
        v, p, bc = inputs.value, inputs.params, inputs.bc
        _require(v.ndim == 3 and v.shape[-1] == self.d_inner,
                 f"value must be (batch, T, {self.d_inner}). Got {tuple(v.shape)}.")
        exp_p = self.n_heads * self.param_dim
        _require(p.ndim == 3 and p.shape[-1] == exp_p,
                 f"params must be (batch, T, {exp_p}). Got {tuple(p.shape)}.")
        _require(bc.ndim == 5 and tuple(bc.shape[2:]) == (self.bc_groups, self.bc_param_rows, self.d_state),
                 f"bc must be (batch, T, groups, {self.bc_param_rows}, d_state). Got {tuple(bc.shape)}.")

    def forward(self, value, params, bc) -> ScanInputs:  # type: ignore[override]
        inputs = ScanPrepInputs(value=value, params=params, bc=bc)
        self._validate(inputs)
        return self.backend(self, inputs)


__all__ = ["SLinOSSScanPrep"]
