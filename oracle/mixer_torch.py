"""torch (CPU, autograd) restatement of the mixer stages around the scan.

TEST ORACLE ONLY - never imported by the shipped package.

Stages, with the reference source each one restates:

``causal_conv_silu``   slinoss/ops/mixer/convolution.py:68-101 (depthwise causal
                       conv1d + bias + SiLU with a left state of d_conv-1 inputs)
``scan_coefficients``  slinoss/layers/scanprep.py:237-283 and
                       slinoss/ops/scanprep/reference.py:25-56 (bounded dt/alpha/
                       theta maps and the exact first-order-hold taps)
``bc_pairs``           slinoss/ops/scanprep/parameterization.py:45-107
``scanprep``           slinoss/layers/scanprep.py:385-395 (packing into U,M,K,B,C)
``gated_rmsnorm``      slinoss/ops/mixer/tail.py:63-142 (skip + SiLU gate + RMSNorm)

All functions are differentiable with autograd; gradients obtained through them
are the gradient oracle for the CUDA backward kernels.
"""

from __future__ import annotations

import math

import torch
from torch.nn import functional as F


def causal_conv_silu(x, weight, bias, conv_state=None):
    """x (B,T,C) channel-last, weight (C,W), bias (C), state (B,C,W-1) or None.

    Returns ``(silu(conv), next_state)``; next_state holds the last W-1 inputs."""
    bsz, T, C = x.shape
    W = weight.shape[1]
    xt = x.transpose(1, 2)
    left = x.new_zeros((bsz, C, W - 1)) if conv_state is None else conv_state.to(x.dtype)
    stacked = torch.cat((left, xt), dim=-1)
    out = F.conv1d(stacked, weight.unsqueeze(1), bias, groups=C)
    next_state = stacked[..., stacked.shape[-1] - (W - 1):].contiguous()
    return F.silu(out.transpose(1, 2)).contiguous(), next_state


def _wrap_angle(theta):
    return torch.remainder(theta + math.pi, 2.0 * math.pi) - math.pi


def foh_taps(dt, log_r, theta, rho, eps):
    """Exact first-order-hold taps (kprev, kcurr) as complex tensors, with the
    cubic Taylor continuation for small |z| (reference.py:25-56)."""
    z = torch.complex(log_r, theta)
    thresh = max(1.0e-4, math.sqrt(max(float(eps), 1.0e-12)))
    small = (log_r.square() + theta.square()) < thresh * thresh
    safe = torch.where(small, torch.ones_like(z), z)
    k1 = (rho - 1.0) / safe
    k2 = (rho * (safe - 1.0) + 1.0) / (safe * safe)
    z2 = z * z
    z3 = z2 * z
    k1 = torch.where(small, 1.0 + 0.5 * z + z2 / 6.0 + z3 / 24.0, k1)
    k2 = torch.where(small, 0.5 + z / 3.0 + z2 / 8.0 + z3 / 30.0, k2)
    k_prev = dt * k2
    k_curr = dt * k1 - k_prev
    return k_prev, k_curr


def scan_coefficients(params, cfg, dt_bias, alpha_bias, theta_mod_bias, theta_bias,
                      theta_sign, dtype=torch.float32):
    """params (B,T,H*3) -> M (B,H,T,2), K (B,H,T,2,2), both float32.

    ``cfg`` is a dict with dt_min, dt_max, alpha_min, alpha_max, theta_init_min,
    theta_init_max, theta_mod_scale, r_min, r_max, eps.  ``dtype`` is the arithmetic
    type: float32 is what the reference does; float64 gives the exact value of the
    same formulas (the tap quotients cancel badly in float32 for small |z|)."""
    bsz, T, _ = params.shape
    H = dt_bias.numel()
    dt_bias, alpha_bias, theta_mod_bias, theta_bias, theta_sign = (
        x.to(dtype) for x in (dt_bias, alpha_bias, theta_mod_bias, theta_bias, theta_sign))
    p = params.view(bsz, T, H, 3).permute(0, 2, 1, 3).to(dtype)
    p = p + torch.stack((dt_bias, alpha_bias, theta_mod_bias), dim=-1).view(1, H, 1, 3)
    dt = cfg["dt_min"] + (cfg["dt_max"] - cfg["dt_min"]) * torch.sigmoid(p[..., 0])
    alpha = cfg["alpha_min"] + (cfg["alpha_max"] - cfg["alpha_min"]) * torch.sigmoid(p[..., 1])
    span = cfg["theta_init_max"] - cfg["theta_init_min"]
    theta_u = torch.sigmoid(theta_bias.view(1, H, 1)
                            + cfg["theta_mod_scale"] * torch.tanh(p[..., 2]))
    theta = _wrap_angle(theta_sign.view(1, H, 1) * (cfg["theta_init_min"] + span * theta_u))
    r = cfg["r_min"] + (cfg["r_max"] - cfg["r_min"]) * torch.exp(-alpha)
    rho = torch.polar(r, theta)
    k_prev, k_curr = foh_taps(dt, torch.log(r), theta, rho, cfg["eps"])
    M = torch.view_as_real(rho).contiguous()
    K = torch.stack((torch.view_as_real(k_prev), torch.view_as_real(k_curr)), dim=-2)
    return M.to(torch.float32), K.to(torch.float32).contiguous()


def bc_pairs(bc, eps):
    """bc (B,T,G,4,N): rows (B amplitude, B phase, C amplitude, C phase) logits.

    Returns complex pairs ``(B,T,G,N,2)`` for B and C in bc's dtype:
    softplus amplitude, pi*tanh phase, divided by the RMS over N of |pair|."""
    def one(amp_row, phase_row):
        amp = F.softplus(amp_row.to(torch.float32))
        ph = math.pi * torch.tanh(phase_row.to(torch.float32))
        pair = amp.unsqueeze(-1) * torch.stack((torch.cos(ph), torch.sin(ph)), dim=-1)
        ms = pair.square().sum(dim=-1).mean(dim=-1, keepdim=True).clamp_min(float(eps))
        return pair / ms.sqrt().unsqueeze(-1)
    dtype = bc.dtype if bc.dtype in (torch.float16, torch.bfloat16, torch.float32) \
        else torch.float32
    return (one(bc[..., 0, :], bc[..., 1, :]).to(dtype),
            one(bc[..., 2, :], bc[..., 3, :]).to(dtype))


def scanprep(value, params, bc, cfg, dt_bias, alpha_bias, theta_mod_bias, theta_bias,
             theta_sign, d_head, coeff_dtype=torch.float32):
    """(value (B,T,H*P), params (B,T,3H), bc (B,T,G,4,N)) -> U, M, K, B, C."""
    bsz, T, _ = value.shape
    H = dt_bias.numel()
    G, N = bc.shape[2], bc.shape[4]
    U = value.view(bsz, T, H, d_head).permute(0, 2, 1, 3).contiguous()
    bp, cp = bc_pairs(bc, cfg["eps"])
    Bo = bp.permute(0, 2, 1, 3, 4).reshape(bsz, G, T, 2 * N).contiguous()
    Co = cp.permute(0, 2, 1, 3, 4).reshape(bsz, G, T, 2 * N).contiguous()
    M, K = scan_coefficients(params, cfg, dt_bias, alpha_bias, theta_mod_bias, theta_bias,
                             theta_sign, dtype=coeff_dtype)
    return U, M, K, Bo, Co


def gated_rmsnorm(scan_output, gate, norm_weight, eps, skip_input=None, d_skip=None):
    """``RMSNorm((Y + d_skip*U) * SiLU(gate)) * w`` -> (B,T,H*P).

    Intermediate roundings to the activation dtype follow tail.py:63-142."""
    bsz, H, T, P = scan_output.shape
    pre = scan_output
    if skip_input is not None:
        pre = (scan_output.float() + skip_input.float() * d_skip.view(1, H, 1, 1).float()
               ).to(scan_output.dtype)
    g = gate.reshape(bsz, T, H, P).permute(0, 2, 1, 3)
    gated = (pre.float() * F.silu(g.float())).to(pre.dtype)
    gated = gated.permute(0, 2, 1, 3).reshape(bsz, T, H * P)
    return F.rms_norm(gated.to(norm_weight.dtype), (H * P,), norm_weight, eps).to(gated.dtype)


__all__ = ["causal_conv_silu", "foh_taps", "scan_coefficients", "bc_pairs", "scanprep",
           "gated_rmsnorm"]
