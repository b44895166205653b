"""FFN branch of a block as one autograd op that rebuilds its intermediates in the backward pass.

``ffn_residual(x, ...)`` computes ``x + out_proj(act(in_proj(rmsnorm(x))))``.  Two schedules:

``remat="full"``  stores ``x`` and the parameters only; the backward pass rebuilds the normalised rows,
    the projection (one more GEMM) and the activation before it differentiates them, so none of the three
    wide intermediates (rows x d_model, rows x width, rows x hidden) of a layer stays alive between the
    passes.  This is the schedule of the reference's ``block_ffn_residual``
    (slinoss/ops/block/training.py:193-354).
``remat="rows"``  also keeps the projection, so the backward pass repeats only the two row-wise steps
    and no GEMM; it frees the normalised rows and the activation output.

The row-wise steps run on this package's CUDA kernels (``sl_rmsnorm_*``, ``sl_ffn_activation_*``), the
GEMMs on the library.
"""

from __future__ import annotations

import torch
from torch.nn import functional as F

from ... import _C


def residual_add(residual, branch, in_fp32: bool):
    """``residual + branch`` in the residual's type, summed in float32 when ``in_fp32``.  Two operands
    of one type add in float32 inside the elementwise kernel and round once, which is bit for bit the
    cast-add-cast sequence, so that case is one kernel."""
    if residual.dtype == branch.dtype:
        return residual + branch
    dt = torch.float32 if in_fp32 else residual.dtype
    return residual.to(dt).add(branch.to(dt)).to(dtype=residual.dtype)


class _FFNActivationFn(torch.autograd.Function):
    """The FFN activation on the row kernels, keeping the projection for the backward pass."""

    @staticmethod
    def forward(ctx, projected, kind):
        projected = projected.contiguous()
        ctx.save_for_backward(projected)
        ctx.kind = kind
        return _C.ffn_activation_fwd(projected, kind)

    @staticmethod
    def backward(ctx, d_hidden):
        (projected,) = ctx.saved_tensors
        return _C.ffn_activation_bwd(projected, d_hidden.contiguous(), ctx.kind), None


def ffn_activation_supported(projected, kind: str) -> bool:
    if not projected.is_cuda or projected.dtype not in _C._DTYPE_CODE or torch.is_autocast_enabled():
        return False
    width = int(projected.shape[-1])
    hidden = width // 2 if kind == "swiglu" else width
    v = 4 if projected.dtype == torch.float32 else 8
    return kind in _C.FFN_KINDS and projected.numel() > 0 and hidden % v == 0


@torch.compiler.disable
def ffn_activation(projected, kind: str):
    """``gelu(projected, tanh form)`` or ``value * silu(gate)`` of ``projected = [value | gate]`` on the CUDA
    row kernels (differentiable)."""
    return _FFNActivationFn.apply(projected, kind)


class _FFNResidualFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, norm_w, w1, b1, w2, b2, eps, kind, in_fp32, keep_projection):
        x = x.contiguous()
        normed = _C.rmsnorm_fwd(x, norm_w, eps)
        projected = F.linear(normed, w1, b1)
        del normed
        hidden = _C.ffn_activation_fwd(projected, kind)
        out = residual_add(x, F.linear(hidden, w2, b2), in_fp32)
        ctx.save_for_backward(x, norm_w, w1, b1, w2, b2, projected if keep_projection else None)
        ctx.eps, ctx.kind, ctx.in_fp32 = eps, kind, in_fp32
        return out

    @staticmethod
    def backward(ctx, d_out):
        x, norm_w, w1, b1, w2, b2, projected = ctx.saved_tensors
        need = ctx.needs_input_grad
        d_out = d_out.contiguous()
        C = x.shape[-1]
        normed = _C.rmsnorm_fwd(x, norm_w, ctx.eps)
        if projected is None:
            projected = F.linear(normed, w1, b1)
        hidden = _C.ffn_activation_fwd(projected, ctx.kind)
        d_out2 = d_out.reshape(-1, C)
        d_w2 = d_out2.t().mm(hidden.reshape(-1, hidden.shape[-1])) if need[4] else None
        d_b2 = d_out2.sum(0, dtype=torch.float32).to(b2.dtype) if (b2 is not None and need[5]) else None
        d_hidden = d_out.matmul(w2)
        del hidden
        d_projected = _C.ffn_activation_bwd(projected, d_hidden, ctx.kind)
        del projected, d_hidden
        d_proj2 = d_projected.reshape(-1, d_projected.shape[-1])
        d_w1 = d_proj2.t().mm(normed.reshape(-1, C)) if need[2] else None
        d_b1 = d_proj2.sum(0, dtype=torch.float32).to(b1.dtype) if (b1 is not None and need[3]) else None
        del normed
        d_normed = d_projected.matmul(w1)
        del d_projected
        d_x, d_nw = _C.rmsnorm_bwd(x, norm_w, ctx.eps, d_normed)
        d_x = residual_add(d_out, d_x, ctx.in_fp32) if need[0] else None
        return d_x, (d_nw.to(norm_w.dtype) if need[1] else None), d_w1, d_b1, d_w2, d_b2, None, None, None, None


def ffn_residual_supported(x, norm, ffn) -> bool:
    """True when the rematerialising op covers this call: CUDA rows in one 16-bit or float32 type shared
    by every parameter, an RMSNorm with a weight, row widths the kernels take, no autocast."""
    w = getattr(norm, "weight", None)
    if not (isinstance(norm, torch.nn.RMSNorm) and isinstance(w, torch.Tensor)):
        return False
    if not x.is_cuda or torch.is_autocast_enabled() or x.dtype not in _C._DTYPE_CODE:
        return False
    params = [w, ffn.in_proj.weight, ffn.out_proj.weight, ffn.in_proj.bias, ffn.out_proj.bias]
    if any(p is not None and (p.dtype != x.dtype or p.device != x.device) for p in params):
        return False
    v = 4 if x.dtype == torch.float32 else 8
    return _C.rmsnorm_supported(int(x.shape[-1]), x.dtype) and ffn.hidden_dim % v == 0 and x.numel() > 0


@torch.compiler.disable
def ffn_residual(x, norm, ffn, *, residual_in_fp32: bool = True, remat: str = "full"):
    """``x + ffn(norm(x))`` through the rematerialising op (see the module docstring)."""
    if remat not in ("full", "rows"):
        raise ValueError(f"remat must be 'full' or 'rows'. Got {remat!r}.")
    eps = norm.eps if norm.eps is not None else torch.finfo(x.dtype).eps
    return _FFNResidualFn.apply(x, norm.weight, ffn.in_proj.weight, ffn.in_proj.bias, ffn.out_proj.weight,
                                ffn.out_proj.bias, float(eps), ffn.kind, bool(residual_in_fp32),
                                remat == "rows")


__all__ = ["ffn_activation", "ffn_activation_supported", "ffn_residual", "ffn_residual_supported", "residual_add"]
