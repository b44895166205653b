"""RMSNorm that computes in the weight dtype and returns the input dtype
(reference: slinoss/layers/norm.py:10-22).  On CUDA the rows run on this package's
``sl_rmsnorm_fwd`` / ``sl_rmsnorm_bwd`` kernels (one pass each; the backward pass keeps
only the input and recomputes the row scale)."""

from __future__ import annotations

import torch
from torch import nn

from .. import _C


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        x = x.contiguous()
        ctx.save_for_backward(x, weight)
        ctx.eps = eps
        return _C.rmsnorm_fwd(x, weight, eps)

    @staticmethod
    def backward(ctx, d_out):
        x, weight = ctx.saved_tensors
        d_x, d_w = _C.rmsnorm_bwd(x, weight, ctx.eps, d_out.contiguous())
        return (d_x if ctx.needs_input_grad[0] else None,
                d_w.to(weight.dtype) if ctx.needs_input_grad[1] else None, None)


@torch.compiler.disable
def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last axis on the CUDA row kernels (same type for rows and weight)."""
    return _RMSNormFn.apply(x, weight, float(eps))


class RMSNorm(nn.RMSNorm):
    def _rows_kernel_ok(self, x: torch.Tensor) -> bool:
        w = self.weight
        return (w is not None and x.is_cuda and w.device == x.device and x.dtype == w.dtype and
                len(self.normalized_shape) == 1 and x.numel() > 0 and not torch.is_autocast_enabled() and
                _C.rmsnorm_supported(int(x.shape[-1]), x.dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.weight is not None and x.dtype != self.weight.dtype:
            return self.forward(x.to(self.weight.dtype)).to(x.dtype)
        if self._rows_kernel_ok(x):
            eps = self.eps if self.eps is not None else torch.finfo(x.dtype).eps
            return rmsnorm_rows(x, self.weight, eps)
        return super().forward(x)


__all__ = ["RMSNorm", "rmsnorm_rows"]
