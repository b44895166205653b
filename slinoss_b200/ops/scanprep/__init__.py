"""Scan preparation (and the causal depthwise conv feeding it) on CUDA.

``conv_scanprep_b200``   value stream -> conv1d + bias + SiLU -> U, together with the
                         B/C parameterisation and the (M, K) coefficients, in one
                         C-ABI call (replaces cconv1d + scanprep_cute of the reference)
``scanprep_b200``        the same without the convolution
                         (slinoss/ops/scanprep/cute/api.py:88)
``causal_conv_silu_b200`` the convolution alone, channel-last in and out
                         (slinoss/ops/mixer/convolution.py:104-173)
"""

from __future__ import annotations

import torch

from ... import _C


def _biases(owner):
    f = lambda t: t.detach().to(torch.float32).contiguous()
    return (f(owner.dt_bias), f(owner.alpha_bias), f(owner.theta_mod_bias), f(owner.theta_bias),
            f(owner.theta_sign))


class _ConvScanPrepFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, value, params, bc, conv_weight, conv_bias, conv_state, dt_bias, alpha_bias,
                theta_mod_bias, theta_bias, owner, want_state):
        heads, P = owner.n_heads, owner.d_head
        cfg = _C.make_config(owner)
        biases = _biases(owner)
        io = value.dtype
        c = lambda x: None if x is None else x.detach().to(io)
        params_c, bc_c = c(params).contiguous(), c(bc).contiguous()
        w_c = None if conv_weight is None else c(conv_weight).contiguous()
        b_c = None if conv_bias is None else c(conv_bias).contiguous()
        st_c = None if conv_state is None else c(conv_state).contiguous()
        value_d = value.detach()
        U, M, K, Bo, Co, nstate = _C.scanprep_conv_fwd(
            value_d, w_c, b_c, st_c, params_c, bc_c, biases, cfg, heads=heads, P=P,
            want_state=want_state and w_c is not None)
        ctx.save_for_backward(value_d, params_c, bc_c, w_c, b_c, st_c, *biases)
        ctx.owner_dims = (heads, P)
        ctx.cfg = cfg
        ctx.dtypes = (params.dtype, bc.dtype,
                      None if conv_weight is None else conv_weight.dtype,
                      None if conv_bias is None else conv_bias.dtype,
                      None if conv_state is None else conv_state.dtype)
        if nstate is None:
            nstate = value.new_empty((value.shape[0], heads * P, 0))
        ctx.mark_non_differentiable(nstate)
        return U, M, K, Bo, Co, nstate

    @staticmethod
    def backward(ctx, dU, dM, dK, dBo, dCo, _dstate):
        value, params, bc, w, b, st, *biases = ctx.saved_tensors
        heads, P = ctx.owner_dims
        zeros = lambda ref, shape, dt: torch.zeros(shape, dtype=dt, device=ref.device)
        batch, T = value.shape[0], value.shape[1]
        if dU is None:
            dU = zeros(value, (batch, heads, T, P), value.dtype)
        if (dM is None) != (dK is None):
            dM = zeros(value, (batch, heads, T, 2), torch.float32) if dM is None else dM
            dK = zeros(value, (batch, heads, T, 2, 2), torch.float32) if dK is None else dK
        if (dBo is None) != (dCo is None):
            shape = (batch, bc.shape[2], T, 2 * bc.shape[4])
            dBo = zeros(value, shape, bc.dtype) if dBo is None else dBo
            dCo = zeros(value, shape, bc.dtype) if dCo is None else dCo
        f32 = lambda x: None if x is None else x.to(torch.float32)
        io = lambda x: None if x is None else x.to(value.dtype)
        g = _C.scanprep_conv_bwd(value, w, b, st, params, bc, tuple(biases), ctx.cfg, io(dU),
                                 f32(dM), f32(dK), io(dBo), io(dCo), heads=heads, P=P,
                                 want_dstate=st is not None)
        pd, bd, wd, bid, sd = ctx.dtypes
        cast = lambda x, dt: None if (x is None or dt is None) else x.to(dt)
        return (g["d_value"], cast(g["d_params"], pd), cast(g["d_bc"], bd),
                cast(g["d_conv_weight"], wd), cast(g["d_conv_bias"], bid),
                cast(g["d_conv_state"], sd), g["d_dt_bias"], g["d_alpha_bias"],
                g["d_theta_mod_bias"], g["d_theta_bias"], None, None)


@torch.compiler.disable
def conv_scanprep_b200(owner, value, params, bc, *, conv_weight=None, conv_bias=None,
                       conv_state=None, want_state=False):
    """``owner`` is the SLinOSSScanPrep module (bounds, biases, head geometry).

    ``value (batch,T,heads*P)`` may be a column slice of the in_proj output (row
    strided).  Returns ``(U, M, K, B, C, next_conv_state)``."""
    return _ConvScanPrepFn.apply(value, params, bc, conv_weight, conv_bias, conv_state,
                                 owner.dt_bias, owner.alpha_bias, owner.theta_mod_bias,
                                 owner.theta_bias, owner, want_state)


@torch.compiler.disable
def scanprep_b200(owner, value, params, bc):
    """Scan preparation without the convolution.  Returns ``(U, M, K, B, C)``."""
    return conv_scanprep_b200(owner, value, params, bc)[:5]


class _ConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, conv_state, want_state):
        C = x.shape[-1]
        io = x.dtype
        w = weight.detach().to(io).contiguous()
        b = bias.detach().to(io).contiguous()
        st = None if conv_state is None else conv_state.detach().to(io).contiguous()
        xd = x.detach()
        out = _C.scanprep_conv_fwd(xd, w, b, st, None, None, None, None, heads=1, P=C,
                                   u_layout="btc", want_state=want_state)
        y, nstate = out[0], out[5]
        ctx.save_for_backward(xd, w, b, st)
        ctx.dtypes = (weight.dtype, bias.dtype, None if conv_state is None else conv_state.dtype)
        if nstate is None:
            nstate = x.new_empty((x.shape[0], C, 0))
        ctx.mark_non_differentiable(nstate)
        return y, nstate

    @staticmethod
    def backward(ctx, dy, _dstate):
        x, w, b, st = ctx.saved_tensors
        g = _C.scanprep_conv_bwd(x, w, b, st, None, None, None, None, dy.to(x.dtype), None, None,
                                 None, None, heads=1, P=x.shape[-1], u_layout="btc",
                                 want_dstate=st is not None)
        wd, bd, sd = ctx.dtypes
        return (g["d_value"], g["d_conv_weight"].to(wd), g["d_conv_bias"].to(bd),
                None if (sd is None or g["d_conv_state"] is None) else g["d_conv_state"].to(sd),
                None)


@torch.compiler.disable
def causal_conv_silu_b200(x, weight, bias, conv_state=None, *, want_state=True):
    """``SiLU(depthwise causal conv1d(x) + bias)`` for channel-last ``x (batch,T,C)``,
    ``weight (C,d_conv)``, optional left state ``(batch,C,d_conv-1)``.
    Returns ``(y (batch,T,C), next_state)``."""
    if weight.shape[1] > 4:
        raise ValueError("the CUDA causal conv supports d_conv <= 4.")
    return _ConvFn.apply(x, weight, bias, conv_state, want_state)


__all__ = ["conv_scanprep_b200", "scanprep_b200", "causal_conv_silu_b200"]
