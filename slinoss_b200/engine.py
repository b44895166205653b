"""CUDA-graph decode engine for ``SLinOSSMixer``: one captured graph per token.

A decode token of the mixer is in_proj (library GEMM) -> ``sl_mixer_decode_step`` (one launch: conv
update, scan preparation, state update, skip, gate, RMSNorm) -> out_proj (library GEMM).  Launching
these three from Python costs more host time than the GPU needs at small batch; the engine captures
them once over static buffers and replays the graph per token.  The reference has the same idea for
its whole model (scripts/perf/_training_model.py:120-200); here it is part of the package because
the fused step exists to be replayed.
"""

from __future__ import annotations

import torch

from .layers.state import SLinOSSMixerState
from .ops.mixer.projection import split_mixer_projection


class MixerDecodeEngine:
    """Holds a mixer's decode state in static buffers and advances it one token per ``step``.

    ``step(x)`` takes ``x (batch, d_model)`` and returns ``y (batch, d_model)`` (a view of the engine's
    output buffer: copy it if it must outlive the next step).  ``reset()`` zeroes the carried state.
    The mixer's parameters are read at replay time, so weight updates are seen; changing their
    shapes, dtype or device needs a new engine."""

    def __init__(self, mixer, batch_size: int, *, device=None, dtype=None, use_graph: bool = True):
        p = next(mixer.parameters())
        self.mixer = mixer
        self.device = torch.device(device) if device is not None else p.device
        self.dtype = dtype or p.dtype
        if self.device.type != "cuda":
            raise ValueError("MixerDecodeEngine needs a CUDA device: the kernels have no CPU path.")
        from . import _C
        self.batch = int(batch_size)
        self.state: SLinOSSMixerState = mixer.init_decode_state(self.batch, device=self.device, dtype=self.dtype)
        kw = dict(device=self.device, dtype=self.dtype)
        self.x = torch.zeros((self.batch, mixer.d_model), **kw)
        self.y = torch.zeros((self.batch, mixer.d_model), **kw)
        self._normed = torch.empty((self.batch, mixer.d_inner), **kw)
        self._b_next = torch.empty_like(self.state.scan.b_prev)
        self._workspace = _C.mixer_decode_workspace(self.batch, mixer.n_heads, mixer.d_head, self.device)
        self._graph = None
        if use_graph:
            self._capture()

    # one token over the static buffers (everything in place: the graph sees fixed addresses)
    def _token(self):
        from . import _C
        m, st = self.mixer, self.state
        gate, value, params, bc = split_mixer_projection(
            self.x, m.in_proj.weight, d_inner=m.d_inner, param_proj_dim=m.param_proj_dim)
        sp = m.scanprep
        biases = tuple(getattr(sp, k).detach().float() for k in
                       ("dt_bias", "alpha_bias", "theta_mod_bias", "theta_bias", "theta_sign"))
        _C.mixer_decode_step(
            gate, value, params, bc.view(self.batch, m.bc_groups, 4, m.d_state), m.dw_weight.detach(),
            m.dw_bias.detach(), st.conv, biases, _C.make_config(sp), m.d_skip.detach().float(),
            m.out_norm.weight.detach(), m.out_norm.eps, st.scan.state, st.scan.b_prev, self._b_next,
            st.scan.u_prev, self._workspace, heads=m.n_heads, P=m.d_head, normed=self._normed)
        st.scan.b_prev.copy_(self._b_next)
        torch.mm(self._normed, m.out_proj.weight.detach().t(), out=self.y)

    def _capture(self):
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side), torch.no_grad():      # warm-up outside the capture
            self._token()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self.reset()
        self._graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self._graph):
            self._token()
        torch.cuda.synchronize(self.device)
        self.reset()

    def reset(self):
        st = self.state
        for t in (st.conv, st.scan.state, st.scan.b_prev, st.scan.u_prev):
            t.zero_()

    @torch.no_grad()
    def step(self, x: torch.Tensor) -> torch.Tensor:
        if tuple(x.shape) != tuple(self.x.shape):
            raise ValueError(f"Expected x shape {tuple(self.x.shape)}, got {tuple(x.shape)}.")
        self.x.copy_(x)
        if self._graph is not None:
            self._graph.replay()
        else:
            self._token()
        return self.y


__all__ = ["MixerDecodeEngine"]
