"""Mixer tail: ``out_proj(RMSNorm((Y + d_skip*U) * SiLU(gate)))``.

The row-wise part runs in one CUDA kernel each way; ``out_proj`` stays a library
GEMM.  Mirrors ``mixer_tail`` of the reference (slinoss/ops/mixer/tail.py:477-559)
and saves the same tensors for backward: ``(scan_output, gate, skip_input)``.
"""

from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F

from ... import _C


def _dims(scan_output, gate):
    if scan_output.ndim != 4:
        raise ValueError("scan_output must be 4-D; got "
                         f"{scan_output.ndim}-D with shape {tuple(scan_output.shape)}.")
    batch, heads, T, P = map(int, scan_output.shape)
    expected = (batch, T, heads * P)
    if gate.ndim != 3 or tuple(map(int, gate.shape)) != expected:
        raise ValueError(f"gate must be {expected}; got {tuple(map(int, gate.shape))}.")
    if gate.device != scan_output.device:
        raise ValueError("gate and scan_output must be on the same device.")
    return batch, heads, T, P


class _GatedNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, scan_output, gate, skip_input, d_skip, norm_weight, eps):
        io = scan_output.dtype
        Y = scan_output.detach().contiguous()
        g = gate.detach().to(io)
        S = None if skip_input is None else skip_input.detach().to(io).contiguous()
        ds = None if d_skip is None else d_skip.detach().to(torch.float32).contiguous()
        w = norm_weight.detach().to(io).contiguous()
        normed = _C.mixer_tail_fwd(Y, g, S, ds, w, eps)
        ctx.save_for_backward(Y, g, S, ds, w)
        ctx.eps = eps
        ctx.dtypes = (gate.dtype, None if skip_input is None else skip_input.dtype,
                      None if d_skip is None else d_skip.dtype, norm_weight.dtype)
        return normed

    @staticmethod
    def backward(ctx, d_normed):
        Y, g, S, ds, w = ctx.saved_tensors
        dY, d_gate, d_skip_in, d_d_skip, d_w = _C.mixer_tail_bwd(
            Y, g, S, ds, w, ctx.eps, d_normed.to(Y.dtype))
        gd, sd, dsd, wd = ctx.dtypes
        return (dY, d_gate.to(gd), None if d_skip_in is None else d_skip_in.to(sd),
                None if d_d_skip is None else d_d_skip.to(dsd), d_w.to(wd), None)


@torch.compiler.disable
def mixer_gated_norm(scan_output, gate, norm_weight, eps, *, skip_input=None, d_skip=None):
    """Row-wise part of the tail -> ``(batch, T, heads*P)`` in scan_output's dtype."""
    _, heads, _, _ = _dims(scan_output, gate)
    if (skip_input is None) != (d_skip is None):
        raise ValueError("skip_input and d_skip must either both be provided or both be None.")
    if skip_input is not None:
        if tuple(skip_input.shape) != tuple(scan_output.shape):
            raise ValueError(f"skip_input must be {tuple(scan_output.shape)}; "
                             f"got {tuple(skip_input.shape)}.")
        if d_skip.ndim != 1 or d_skip.numel() != heads:
            raise ValueError(f"d_skip must be 1-D with length {heads}; got {tuple(d_skip.shape)}.")
    if eps is None:
        eps = float(torch.finfo(norm_weight.dtype).eps)
    return _GatedNormFn.apply(scan_output, gate, skip_input, d_skip, norm_weight, float(eps))


@torch.compiler.disable
def mixer_tail(scan_output, gate, out_norm: nn.RMSNorm, out_proj: nn.Module, *, skip_input=None,
               d_skip=None):
    """Full tail including ``out_proj`` (same call as the reference's ``mixer_tail``)."""
    if out_norm.weight is None:
        raise ValueError("mixer_tail requires an affine RMSNorm weight.")
    weight = getattr(out_proj, "weight", None)
    if not isinstance(weight, torch.Tensor):
        raise TypeError("mixer_tail requires out_proj to expose a tensor weight.")
    bias = getattr(out_proj, "bias", None)
    _, heads, _, P = _dims(scan_output, gate)
    hidden = heads * P
    if out_norm.weight.ndim != 1 or out_norm.weight.numel() != hidden:
        raise ValueError("out_norm_weight must be 1-D with length "
                         f"{hidden}; got {tuple(out_norm.weight.shape)}.")
    if weight.ndim != 2 or int(weight.shape[1]) != hidden:
        raise ValueError(f"out_proj_weight must be 2-D with shape (*, {hidden}); "
                         f"got {tuple(weight.shape)}.")
    normed = mixer_gated_norm(scan_output, gate, out_norm.weight, out_norm.eps,
                              skip_input=skip_input, d_skip=d_skip)
    return F.linear(normed, weight, bias)


__all__ = ["mixer_tail", "mixer_gated_norm"]
