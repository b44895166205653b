"""``SLinOSSMixer``: in_proj -> causal conv + SiLU -> scan preparation -> v2x2ssd scan
-> gated RMSNorm tail -> out_proj.

Same constructor, parameters (state_dict keys), ``forward`` / ``step`` / ``init_state``
contract as the reference mixer (slinoss/layers/mixer.py:39-410).  With the default
backends the convolution and the scan preparation run as one fused C-ABI call; an
injected backend for either stage switches to the stage-by-stage protocol path.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from ..ops.mixer import mixer_tail, split_mixer_projection
from ..ops.scanprep import conv_scanprep_b200
from .backend import (B200CConv1dBackend, B200MixerDecodeBackend, B200ScanBackend,
                      B200ScanPrepBackend, CConv1dBackend, MixerDecodeBackend, MixerDecodeInputs,
                      ScanBackend, ScanInputs, ScanPrepBackend, ScanPrepInputs)
from .norm import RMSNorm
from .scanprep import SLinOSSScanPrep, _require
from .state import ScanState, SLinOSSMixerState


class SLinOSSMixer(nn.Module):
    def __init__(self, d_model: int, *, d_state: int = 128, expand: float = 2, d_head: int = 64,
                 d_conv: int = 4, chunk_size: int = 64, bc_groups: int | None = None,
                 scanprep_backend: ScanPrepBackend | None = None,
                 cconv_backend: CConv1dBackend | None = None, dt_min: float = 5e-3,
                 dt_max: float = 1e-1, dt_init_floor: float = 5e-3, alpha_min: float = 0.0,
                 alpha_max: float = 20.0, theta_init_min: float = 0.05,
                 theta_init_max: float = 2.0, theta_mod_scale: float = 1.0, r_min: float = 0.8,
                 r_max: float = 1.0, eps: float = 1e-8, scan_backend: ScanBackend | None = None,
                 decode_backend: MixerDecodeBackend | None = None, device=None, dtype=None) -> None:
        super().__init__()
        for name, v in (("d_model", d_model), ("d_state", d_state), ("expand", expand),
                        ("d_head", d_head), ("d_conv", d_conv), ("chunk_size", chunk_size)):
            _require(v > 0, f"{name} must be positive. Got {v}.")
        if bc_groups is not None:
            _require(bc_groups > 0, f"bc_groups must be positive when provided. Got {bc_groups}.")
        self.d_model, self.d_state, self.expand = int(d_model), int(d_state), float(expand)
        self.d_head, self.d_conv, self.chunk_size = int(d_head), int(d_conv), int(chunk_size)
        self.d_inner = self._quantize_inner_dim(self.expand * self.d_model, self.d_head)
        self.n_heads = self.d_inner // self.d_head
        self.bc_groups = self.n_heads if bc_groups is None else int(bc_groups)
        _require(self.bc_groups <= self.n_heads,
                 "bc_groups must not exceed the realized head count. "
                 f"Got bc_groups={self.bc_groups}, n_heads={self.n_heads}.")
        _require(self.n_heads % self.bc_groups == 0,
                 "bc_groups must divide n_heads so the contiguous head-to-group mapping "
                 f"is well-defined. Got bc_groups={self.bc_groups}, n_heads={self.n_heads}.")
        self.heads_per_bc_group = self.n_heads // self.bc_groups

        self.scanprep = SLinOSSScanPrep(
            n_heads=self.n_heads, bc_groups=self.bc_groups, d_state=self.d_state,
            d_head=self.d_head, backend=scanprep_backend, dt_min=dt_min, dt_max=dt_max,
            dt_init_floor=dt_init_floor, alpha_min=alpha_min, alpha_max=alpha_max,
            theta_init_min=theta_init_min, theta_init_max=theta_init_max,
            theta_mod_scale=theta_mod_scale, r_min=r_min, r_max=r_max, eps=eps, device=device)
        self.scan_backend = B200ScanBackend() if scan_backend is None else scan_backend
        self.decode_backend = B200MixerDecodeBackend() if decode_backend is None else decode_backend
        self.cconv_backend = B200CConv1dBackend() if cconv_backend is None else cconv_backend

        self.param_proj_dim = self.n_heads * self.scanprep.param_dim
        self.bc_proj_dim = self.bc_groups * self.scanprep.bc_param_rows * self.d_state
        kw = {"device": device, "dtype": dtype}
        self.in_proj = nn.Linear(self.d_model, 2 * self.d_inner + self.param_proj_dim + self.bc_proj_dim,
                                 bias=False, **kw)
        self.d_skip = nn.Parameter(torch.ones((self.n_heads,), device=device, dtype=torch.float32))
        setattr(self.d_skip, "_no_weight_decay", True)
        self.dw_weight = nn.Parameter(torch.empty((self.d_inner, self.d_conv), **kw))
        self.dw_bias = nn.Parameter(torch.empty((self.d_inner,), **kw))
        self.out_proj = nn.Linear(self.d_inner, self.d_model, bias=False, **kw)
        self.out_norm = RMSNorm(self.d_inner, eps=1e-5, **kw)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        nn.init.normal_(self.d_skip)
        nn.init.kaiming_uniform_(self.dw_weight.view(self.d_inner, 1, self.d_conv), a=math.sqrt(5.0))
        bound = 1.0 / math.sqrt(float(self.d_conv))
        nn.init.uniform_(self.dw_bias, -bound, bound)
        self.scanprep.reset_parameters()

    @staticmethod
    def _quantize_inner_dim(raw_d_inner: float, d_head: int) -> int:
        """Nearest multiple of ``d_head`` (at least one head)."""
        _require(raw_d_inner > 0.0, f"raw_d_inner must be positive. Got {raw_d_inner}.")
        return max(1, int(math.floor(raw_d_inner / float(d_head) + 0.5))) * d_head

    def init_state(self, batch_size: int, *, device=None, dtype=None) -> SLinOSSMixerState:
        _require(batch_size > 0, f"batch_size must be positive. Got {batch_size}.")
        device = self.in_proj.weight.device if device is None else device
        dtype = self.in_proj.weight.dtype if dtype is None else dtype
        z = lambda *shape: torch.zeros(shape, device=device, dtype=dtype)
        return SLinOSSMixerState(
            conv=z(batch_size, self.d_inner, max(self.d_conv - 1, 0)),
            scan=ScanState(state=z(batch_size, self.n_heads, self.d_head, 2 * self.d_state),
                           b_prev=z(batch_size, self.bc_groups, 2 * self.d_state),
                           u_prev=z(batch_size, self.n_heads, self.d_head)))

    def init_decode_state(self, batch_size: int, *, device=None, dtype=None) -> SLinOSSMixerState:
        """Decode carries the scan state in float32 so the decode kernel updates it in place."""
        state = self.init_state(batch_size, device=device, dtype=dtype)
        state.scan.state = state.scan.state.to(torch.float32)
        return state

    def _fused_frontend(self) -> bool:
        # exact types: a subclass is an injected backend and gets the protocol path
        return (type(self.cconv_backend) is B200CConv1dBackend
                and type(self.scanprep.backend) is B200ScanPrepBackend and self.d_conv <= 4)

    def _frontend(self, value_proj, params, bc, conv_state, want_state):
        if self._fused_frontend():
            self.scanprep._validate(ScanPrepInputs(value=value_proj, params=params, bc=bc))
            if conv_state is not None:
                expected = (value_proj.shape[0], self.d_inner, self.d_conv - 1)
                _require(tuple(conv_state.shape) == expected,
                         f"conv_state must be {expected}. Got {tuple(conv_state.shape)}.")
            U, M, K, B, C, nstate = conv_scanprep_b200(
                self.scanprep, value_proj, params, bc, conv_weight=self.dw_weight,
                conv_bias=self.dw_bias, conv_state=conv_state, want_state=want_state)
            return ScanInputs(U, M, K, B, C), nstate
        value, nstate = self.cconv_backend(self, value_proj, conv_state)
        return self.scanprep(value, params, bc), nstate

    def forward(self, x: torch.Tensor, *, state: SLinOSSMixerState | None = None,
                return_state: bool = False, sequence_group=None):
        """``sequence_group`` (not part of the reference's signature): a ``torch.distributed`` process group
        over whose ranks the TIME axis of ``x`` is sharded in rank order.  Each rank passes its slice and gets
        its slice of the output; the causal conv takes its left context from the previous rank and the scan
        runs as ``v2x2ssd_sequence_parallel``.  Streaming state is not combined with it."""
        _require(x.ndim == 3 and x.shape[-1] == self.d_model,
                 f"Expected x shape (batch, T, {self.d_model}), got {tuple(x.shape)}.")
        if sequence_group is not None:
            _require(state is None and not return_state,
                     "sequence_group cannot be combined with a streaming state.")
            return self._forward_sequence_parallel(x, sequence_group)
        batch, T, _ = map(int, x.shape)
        if T == 0:
            empty = x.new_empty((batch, 0, self.d_model))
            nxt = SLinOSSMixerState() if state is None else state
            return (empty, nxt) if return_state else empty
        gate, value_proj, params, bc_flat = split_mixer_projection(
            x, self.in_proj.weight, d_inner=self.d_inner, param_proj_dim=self.param_proj_dim)
        bc = bc_flat.view(batch, T, self.bc_groups, self.scanprep.bc_param_rows, self.d_state)
        scan_inputs, conv_state = self._frontend(
            value_proj, params, bc, None if state is None else state.conv, return_state)
        result = self.scan_backend(scan_inputs, chunk_size=self.chunk_size,
                                   state=None if state is None else state.scan,
                                   return_state=return_state)
        scan_output, scan_state = result if return_state else (result, None)
        out = mixer_tail(scan_output, gate, self.out_norm, self.out_proj,
                         skip_input=scan_inputs.U, d_skip=self.d_skip)
        if scan_state is None:
            return out
        return out, SLinOSSMixerState(conv=conv_state, scan=scan_state)

    def _forward_sequence_parallel(self, x: torch.Tensor, group):
        from ..ops.v2x2ssd.sequence_parallel import previous_rank_value, v2x2ssd_sequence_parallel
        batch, T, _ = map(int, x.shape)
        halo = self.d_conv - 1
        _require(T >= max(halo, 1), f"every rank needs at least {max(halo, 1)} tokens of the sequence.")
        gate, value_proj, params, bc_flat = split_mixer_projection(
            x, self.in_proj.weight, d_inner=self.d_inner, param_proj_dim=self.param_proj_dim)
        bc = bc_flat.view(batch, T, self.bc_groups, self.scanprep.bc_param_rows, self.d_state)
        conv_state = None
        if halo > 0:   # the last inputs of the previous rank's slice are this slice's left context
            conv_state = previous_rank_value(value_proj[:, T - halo:, :], group).transpose(1, 2).contiguous()
        s, _ = self._frontend(value_proj, params, bc, conv_state, False)
        Y, _, _, _ = v2x2ssd_sequence_parallel(s.U, s.M, s.K, s.B, s.C, chunk_size=self.chunk_size, group=group)
        return mixer_tail(Y, gate, self.out_norm, self.out_proj, skip_input=s.U, d_skip=self.d_skip)

    def step(self, x: torch.Tensor, state: SLinOSSMixerState | None = None, *,
             inplace: bool | None = None):
        """One decode token.  ``x (batch, d_model)`` or ``(batch, 1, d_model)``."""
        squeeze = x.ndim == 2
        if squeeze:
            x = x.unsqueeze(1)
        _require(x.ndim == 3 and x.shape[1] == 1 and x.shape[-1] == self.d_model,
                 f"Expected x shape (batch, d_model) or (batch, 1, {self.d_model}), got {tuple(x.shape)}.")
        if inplace is None:
            inplace = not torch.is_grad_enabled()
        if torch.is_grad_enabled():
            _require(not inplace, "In-place decode is unsupported when gradients are enabled.")
            y, nxt = self.forward(x, state=state, return_state=True)
        else:
            token = x[:, 0, :]
            batch = int(token.shape[0])
            nxt = (self.init_decode_state(batch, device=token.device, dtype=token.dtype)
                   if state is None else (state if inplace else state.clone()))
            y = self._decode_token(token, nxt).unsqueeze(1)
        return (y[:, 0, :], nxt) if squeeze else (y, nxt)

    def _fused_decode_ready(self, state: SLinOSSMixerState, token: torch.Tensor) -> bool:
        """The one-launch decode step needs a complete in-place state in the kernel's layouts."""
        sc = state.scan
        return (getattr(self.decode_backend, "fused", False)
                and self.decode_backend.supports(self, batch_size=int(token.shape[0]), device=token.device,
                                                 dtype=token.dtype)
                and self.d_conv <= 4 and state.conv is not None and state.conv.dtype == token.dtype
                and state.conv.is_contiguous() and sc.state is not None and sc.state.dtype == torch.float32
                and sc.state.is_contiguous() and sc.b_prev is not None and sc.u_prev is not None
                and sc.b_prev.dtype == token.dtype and sc.u_prev.dtype == token.dtype
                and sc.b_prev.is_contiguous() and sc.u_prev.is_contiguous())

    def _decode_token(self, token: torch.Tensor, state: SLinOSSMixerState) -> torch.Tensor:
        batch = int(token.shape[0])
        gate, value_proj, params, bc = split_mixer_projection(
            token, self.in_proj.weight, d_inner=self.d_inner, param_proj_dim=self.param_proj_dim)
        if self._fused_decode_ready(state, token):
            normed = self.decode_backend.fused_step(self, gate, value_proj, params, bc, state)
            return self.out_proj(normed)
        value, conv_state = self.cconv_backend(self, value_proj.unsqueeze(1), state.conv)
        state.conv = conv_state if state.conv is None or state.conv.shape != conv_state.shape \
            else state.conv.copy_(conv_state)
        inputs = MixerDecodeInputs(
            value=value.reshape(batch, self.n_heads, self.d_head),
            params=params.reshape(batch, self.n_heads, self.scanprep.param_dim),
            bc=bc.reshape(batch, self.bc_groups, self.scanprep.bc_param_rows, self.d_state),
            gate=gate.reshape(batch, self.n_heads, self.d_head))
        out, scan_state = self.decode_backend(self, inputs, state.scan)
        state.scan.adopt_(scan_state)
        return self.out_proj(out)


__all__ = ["SLinOSSMixer"]
