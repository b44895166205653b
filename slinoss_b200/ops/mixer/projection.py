"""in_proj of the mixer as three row-sliced GEMMs (library calls).

Same outputs as the reference's ``split_mixer_projection``
(slinoss/ops/mixer/projection.py:31-190): ``gate`` and ``value`` are column slices
of one ``(…, 2*d_inner)`` buffer, ``params`` and ``bc`` are separate dense buffers.
The dense GEMMs stay with cuBLAS.  The backward pass writes the three row blocks of the
weight gradient straight into one buffer and accumulates the input gradient in the GEMM
epilogue, instead of letting autograd zero-fill and add a full-size weight gradient per slice.
"""

from __future__ import annotations

import torch


class _SplitProjectionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, flat, weight, gv_end, p_end):
        ctx.save_for_backward(flat, weight)
        ctx.cuts = (gv_end, p_end)
        return (torch.mm(flat, weight[:gv_end].t()), torch.mm(flat, weight[gv_end:p_end].t()),
                torch.mm(flat, weight[p_end:].t()))

    @staticmethod
    def backward(ctx, d_gv, d_params, d_bc):
        flat, weight = ctx.saved_tensors
        gv_end, p_end = ctx.cuts
        pieces = ((d_gv, 0, gv_end), (d_params, gv_end, p_end), (d_bc, p_end, weight.shape[0]))
        d_flat = d_weight = None
        if ctx.needs_input_grad[0]:
            for d, a, b in pieces:
                d_flat = torch.mm(d, weight[a:b]) if d_flat is None else d_flat.addmm_(d, weight[a:b])
        if ctx.needs_input_grad[1]:
            d_weight = torch.empty_like(weight)
            for d, a, b in pieces:
                torch.mm(d.t(), flat, out=d_weight[a:b])
        return d_flat, d_weight, None, None


def split_mixer_projection(x: torch.Tensor, weight: torch.Tensor, *, d_inner: int,
                           param_proj_dim: int):
    gv_end = 2 * int(d_inner)
    p_end = gv_end + int(param_proj_dim)
    flat = x.reshape(-1, x.shape[-1])
    lead = x.shape[:-1]
    if weight.is_contiguous() and flat.dtype == weight.dtype and not torch.is_autocast_enabled():
        gate_value, params, bc = _SplitProjectionFn.apply(flat, weight, gv_end, p_end)
    else:
        gate_value = torch.mm(flat, weight[:gv_end].t())
        params = torch.mm(flat, weight[gv_end:p_end].t())
        bc = torch.mm(flat, weight[p_end:].t())
    gate_value = gate_value.view(*lead, gv_end)
    params = params.view(*lead, p_end - gv_end)
    bc = bc.view(*lead, weight.shape[0] - p_end)
    gate, value = torch.split(gate_value, [d_inner, d_inner], dim=-1)
    return gate, value, params, bc


__all__ = ["split_mixer_projection"]
