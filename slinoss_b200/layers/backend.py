"""The plug-in boundary of the mixer: canonical input records and backend protocols.

These are the records and call signatures ``SLinOSSMixer`` uses towards its scan,
scan-preparation, convolution and decode stages - identical to the reference's
(slinoss/layers/backend.py:26-237) so that a backend written against either
package can be injected into the other.  The concrete backends here launch the
sm_100a kernels; none of them has a CPU path.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Protocol

import torch

from ..ops.scanprep import causal_conv_silu_b200, scanprep_b200
from ..ops.v2x2ssd import v2x2ssd_cute, v2x2ssd_decode
from .state import ScanState


@dataclass(frozen=True, slots=True)
class ScanPrepInputs:
    """``value (batch,T,heads*P)``, ``params (batch,T,heads*3)``, ``bc (batch,T,groups,4,N)``."""

    value: torch.Tensor
    params: torch.Tensor
    bc: torch.Tensor


@dataclass(frozen=True, slots=True)
class ScanInputs:
    """``U (batch,heads,T,P)``, ``M (…,T,2)``, ``K (…,T,2,2)``, ``B, C (batch,groups,T,2N)``."""

    U: torch.Tensor
    M: torch.Tensor
    K: torch.Tensor
    B: torch.Tensor
    C: torch.Tensor


@dataclass(frozen=True, slots=True)
class MixerDecodeInputs:
    """Per-token ``value, gate (batch,heads,P)``, ``params (batch,heads,3)``,
    ``bc (batch,groups,4,N)``."""

    value: torch.Tensor
    params: torch.Tensor
    bc: torch.Tensor
    gate: torch.Tensor


class ScanPrepBackend(Protocol):
    def __call__(self, owner, inputs: ScanPrepInputs) -> ScanInputs: ...


class CConv1dBackend(Protocol):
    def __call__(self, owner, x: torch.Tensor, conv_state: torch.Tensor | None
                 ) -> tuple[torch.Tensor, torch.Tensor]: ...


class ScanBackend(Protocol):
    def __call__(self, inputs: ScanInputs, *, chunk_size: int, state: ScanState | None = None,
                 return_state: bool | None = None): ...


class MixerDecodeBackend(Protocol):
    def supports(self, owner, *, batch_size: int, device: torch.device, dtype: torch.dtype) -> bool: ...

    def __call__(self, owner, inputs: MixerDecodeInputs, state: ScanState
                 ) -> tuple[torch.Tensor, ScanState]: ...


class B200ScanPrepBackend:
    """Scan preparation on the CUDA kernels (``owner`` is the SLinOSSScanPrep module)."""

    def __call__(self, owner, inputs: ScanPrepInputs) -> ScanInputs:
        return ScanInputs(*scanprep_b200(owner, inputs.value, inputs.params, inputs.bc))


class B200CConv1dBackend:
    """Causal depthwise conv + SiLU on the CUDA kernel (``owner`` is the mixer)."""

    def __call__(self, owner, x, conv_state):
        if x.shape[-1] != owner.d_inner:
            raise ValueError(f"Expected conv input width {owner.d_inner}, got {int(x.shape[-1])}.")
        if conv_state is not None:
            expected = (x.shape[0], owner.d_inner, max(owner.d_conv - 1, 0))
            if tuple(conv_state.shape) != expected:
                raise ValueError(f"conv_state must be {expected}. Got {tuple(conv_state.shape)}.")
        return causal_conv_silu_b200(x, owner.dw_weight, owner.dw_bias, conv_state)


def _resolve_scan_call(inputs, state, return_state):
    """Defaults of a scan call (reference: backend.py:257-274): state is returned when
    one was passed; half inputs compute in float32 and come back in U's dtype."""
    if return_state is None:
        return_state = state is not None
    return (ScanState() if state is None else state), bool(return_state)


class B200ScanBackend:
    """The scan on the CUDA kernels.  ``path`` = "auto" | "simt" | "tc"."""

    def __init__(self, *, compute_dtype: torch.dtype | None = None, path: str = "auto") -> None:
        self.compute_dtype = compute_dtype
        self.path = path

    def __call__(self, inputs: ScanInputs, *, chunk_size: int, state: ScanState | None = None,
                 return_state: bool | None = None):
        st, return_state = _resolve_scan_call(inputs, state, return_state)
        out = v2x2ssd_cute(inputs.U, inputs.M, inputs.K, inputs.B, inputs.C,
                           chunk_size=chunk_size, initial_states=st.state, B_prev=st.b_prev,
                           U_prev=st.u_prev, compute_dtype=self.compute_dtype,
                           output_dtype=inputs.U.dtype, return_state=return_state, path=self.path)
        if not return_state:
            return out
        y, final_state, b_last, u_last = out
        return y, ScanState(state=final_state, b_prev=b_last, u_prev=u_last)


class B200MixerDecodeBackend:
    """Per-token decode on CUDA kernels (d_skip is supported, unlike the reference's fast path,
    slinoss/ops/mixer/step.py:107-122).

    ``fused_step`` is the one-launch path ``SLinOSSMixer.step`` takes outside autograd: conv update,
    scan preparation of the token, state update, skip, gate and RMSNorm in ``sl_mixer_decode_step``,
    with the mixer state updated in place.  ``__call__`` is the Protocol entry
    (slinoss/layers/backend.py:220-237): it takes the already convolved value and runs scan
    preparation, the decode kernel and the gated RMSNorm as separate launches."""

    fused = True

    def supports(self, owner, *, batch_size, device, dtype) -> bool:
        return device.type == "cuda" and dtype in (torch.float32, torch.bfloat16, torch.float16)

    @torch.compiler.disable
    def fused_step(self, owner, gate, value_raw, params, bc, state, *, normed=None, workspace=None):
        """``gate, value_raw (batch, d_inner)`` (row-strided views are fine), ``params (batch, 3H)``,
        ``bc (batch, G*4*N)``; ``state`` is the mixer's decode state (conv window, float32 scan
        state, previous b and u), all of it updated in place.  Returns ``normed (batch, d_inner)``."""
        from .. import _C
        batch = int(gate.shape[0])
        sp, scan = owner.scanprep, state.scan
        dev, dt = gate.device, gate.dtype
        if workspace is None:
            workspace = getattr(state, "_step_workspace", None)
            if workspace is None or workspace.device != dev:
                workspace = _C.mixer_decode_workspace(batch, owner.n_heads, owner.d_head, dev)
                state._step_workspace = workspace
        biases = tuple(getattr(sp, k).detach().float().contiguous()
                       for k in ("dt_bias", "alpha_bias", "theta_mod_bias", "theta_bias", "theta_sign"))
        b_out = torch.empty_like(scan.b_prev)
        normed = _C.mixer_decode_step(
            gate, value_raw, params.contiguous(), bc.contiguous().view(batch, owner.bc_groups, 4, owner.d_state),
            owner.dw_weight.detach().to(dt).contiguous(), owner.dw_bias.detach().to(dt).contiguous(),
            state.conv, biases, _C.make_config(sp), owner.d_skip.detach().float().contiguous(),
            owner.out_norm.weight.detach().to(dt).contiguous(), owner.out_norm.eps, scan.state, scan.b_prev,
            b_out, scan.u_prev, workspace, heads=owner.n_heads, P=owner.d_head, normed=normed)
        scan.b_prev = b_out
        return normed

    def __call__(self, owner, inputs: MixerDecodeInputs, state: ScanState):
        from ..ops.mixer import mixer_gated_norm

        batch = int(inputs.value.shape[0])
        value = inputs.value.reshape(batch, 1, owner.d_inner)
        params = inputs.params.reshape(batch, 1, owner.param_proj_dim)
        bc = inputs.bc.reshape(batch, 1, owner.bc_groups, owner.scanprep.bc_param_rows, owner.d_state)
        U, M, K, B, C = scanprep_b200(owner.scanprep, value, params, bc)
        st = state.state
        if st is None:
            st = torch.zeros((batch, owner.n_heads, owner.d_head, 2 * owner.d_state),
                             device=value.device, dtype=torch.float32)
        inplace = st.dtype == torch.float32 and st.is_contiguous() and not torch.is_grad_enabled()
        y, nxt, _, _ = v2x2ssd_decode(U[:, :, 0], M[:, :, 0], K[:, :, 0], B[:, :, 0], C[:, :, 0],
                                      state=st, B_prev=state.b_prev, U_prev=state.u_prev,
                                      output_dtype=value.dtype, inplace=inplace)
        gate = inputs.gate.reshape(batch, 1, owner.d_inner)
        normed = mixer_gated_norm(y.unsqueeze(2), gate, owner.out_norm.weight, owner.out_norm.eps,
                                  skip_input=U, d_skip=owner.d_skip)
        return normed[:, 0, :], ScanState(state=nxt, b_prev=B[:, :, 0].to(value.dtype),
                                          u_prev=U[:, :, 0].to(value.dtype))


__all__ = ["ScanPrepInputs", "ScanInputs", "MixerDecodeInputs", "ScanPrepBackend",
           "CConv1dBackend", "ScanBackend", "MixerDecodeBackend", "B200ScanPrepBackend",
           "B200CConv1dBackend", "B200ScanBackend", "B200MixerDecodeBackend"]
