"""in_proj of the mixer as three row-sliced GEMMs (library calls).

Same outputs as the reference's ``split_mixer_projection``
(slinoss/ops/mixer/projection.py:31-190): ``gate`` and ``value`` are column slices
of one ``(…, 2*d_inner)`` buffer, ``params`` and ``bc`` are separate dense buffers.
The dense GEMMs stay with cuBLAS; autograd differentiates the three ``mm`` calls.
"""

from __future__ import annotations

import torch


def split_mixer_projection(x: torch.Tensor, weight: torch.Tensor, *, d_inner: int,
                           param_proj_dim: int):
    gv_end = 2 * int(d_inner)
    p_end = gv_end + int(param_proj_dim)
    flat = x.reshape(-1, x.shape[-1])
    lead = x.shape[:-1]
    gate_value = torch.mm(flat, weight[:gv_end].t()).view(*lead, gv_end)
    params = torch.mm(flat, weight[gv_end:p_end].t()).view(*lead, p_end - gv_end)
    bc = torch.mm(flat, weight[p_end:].t()).view(*lead, weight.shape[0] - p_end)
    gate, value = torch.split(gate_value, [d_inner, d_inner], dim=-1)
    return gate, value, params, bc


__all__ = ["split_mixer_projection"]
