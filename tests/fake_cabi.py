"""CPU stand-ins for the tensor-level launchers of ``slinoss_b200._C``.

The reference's own tests exercise its Python boundary on GPU-less machines by
monkeypatching the kernel entry point with a recording fake
(tests/test_cute_backend.py:42-160 there).  This does the same one level lower:
each launcher of ``_C`` is replaced by a function with the same signature that
computes its result with the oracle on CPU tensors and records the call.  Only
tests use this module; the package itself has no CPU path.
"""

from __future__ import annotations

import numpy as np
import torch

from oracle import mixer_torch as mt
from oracle import scan_np


def _n(x):
    return None if x is None else x.detach().to(torch.float64).cpu().numpy()


def _t(x, dtype):
    return torch.from_numpy(np.ascontiguousarray(x)).to(dtype)


class FakeCABI:
    def __init__(self):
        self.calls = []

    def install(self, monkeypatch):
        from slinoss_b200 import _C
        for name in ("scan_fwd", "scan_bwd", "scan_decode", "scanprep_conv_fwd",
                     "scanprep_conv_bwd", "mixer_tail_fwd", "mixer_tail_bwd"):
            monkeypatch.setattr(_C, name, getattr(self, name))
        monkeypatch.setattr(_C, "require_cuda", lambda *a: None)
        monkeypatch.setattr(_C, "make_config", lambda owner: {
            k: getattr(owner, k) for k in ("dt_min", "dt_max", "alpha_min", "alpha_max",
                                           "theta_init_min", "theta_init_max", "theta_mod_scale",
                                           "r_min", "r_max", "eps")})
        return self

    # ---- scan ---------------------------------------------------------------------------
    def scan_fwd(self, U, M, K, B, C, z0, B_prev, U_prev, *, chunk_size, y_dtype, want_final,
                 path="auto", save_states=False):
        self.calls.append(("scan_fwd", dict(chunk_size=chunk_size, path=path, io=U.dtype,
                                            shapes=[tuple(t.shape) for t in (U, M, K, B, C)],
                                            has_state=z0 is not None, has_prev=B_prev is not None)))
        assert M.dtype == K.dtype == torch.float32 and B.dtype == C.dtype == U.dtype
        Y, fin, _, _ = scan_np.v2x2ssd(_n(U), _n(M), _n(K), _n(B), _n(C), chunk_size=chunk_size,
                                       initial_states=_n(z0), B_prev=_n(B_prev), U_prev=_n(U_prev))
        out = (_t(Y, y_dtype), (_t(fin, torch.float32) if want_final else None))
        return out + (None,) if save_states else out

    def scan_bwd(self, U, M, K, B, C, z0, B_prev, U_prev, dY, d_final, *, chunk_size, path="auto",
                 saved=None):
        self.calls.append(("scan_bwd", dict(chunk_size=chunk_size, path=path)))
        dYn = _n(dY) if dY is not None else np.zeros(U.shape)
        g = scan_np.v2x2ssd_bwd(_n(U), _n(M), _n(K), _n(B), _n(C), dYn, d_final_state=_n(d_final),
                                initial_states=_n(z0), B_prev=_n(B_prev), U_prev=_n(U_prev))
        f32 = torch.float32
        return (_t(g["U"], U.dtype), _t(g["M"], f32), _t(g["K"], f32), _t(g["B"], B.dtype),
                _t(g["C"], C.dtype), _t(g["initial_states"], f32) if z0 is not None else None,
                _t(g["B_prev"], B.dtype) if B_prev is not None else None,
                _t(g["U_prev"], U.dtype) if U_prev is not None else None)

    def scan_decode(self, U, M, K, B, C, state, B_prev, U_prev, *, y_dtype, state_out=None):
        self.calls.append(("scan_decode", dict(inplace=state_out is state)))
        u = lambda x: None if x is None else x.unsqueeze(2)
        Y, fin, _, _ = scan_np.v2x2ssm(_n(u(U)), _n(u(M)), _n(u(K)), _n(u(B)), _n(u(C)),
                                       initial_states=_n(state), B_prev=_n(B_prev), U_prev=_n(U_prev))
        fin = _t(fin, torch.float32)
        if state_out is not None:
            state_out.copy_(fin)
            fin = state_out
        return _t(Y[:, :, 0], y_dtype), fin

    # ---- scan preparation / conv -------------------------------------------------------------
    def _prep_graph(self, value, w, b, st, params, bc, biases, cfg, heads, P, u_layout):
        """Differentiable oracle graph of the fused front end."""
        outs = {}
        if value is not None:
            v = value
            if w is not None:
                v, outs["state"] = mt.causal_conv_silu(value, w, b, st)
            bsz, T, _ = v.shape
            outs["U"] = v.view(bsz, T, heads, P).permute(0, 2, 1, 3).contiguous() \
                if u_layout == "bhtp" else v.contiguous()
        if bc is not None:
            bp, cp = mt.bc_pairs(bc, cfg["eps"])
            bsz, T, G, N = bc.shape[0], bc.shape[1], bc.shape[2], bc.shape[4]
            outs["B"] = bp.permute(0, 2, 1, 3, 4).reshape(bsz, G, T, 2 * N).contiguous()
            outs["C"] = cp.permute(0, 2, 1, 3, 4).reshape(bsz, G, T, 2 * N).contiguous()
        if params is not None:
            outs["M"], outs["K"] = mt.scan_coefficients(params.float(), cfg, *biases)
        return outs

    def scanprep_conv_fwd(self, value, conv_weight, conv_bias, conv_state, params, bc, biases, cfg,
                          *, heads, P, u_layout="bhtp", want_state=False):
        self.calls.append(("scanprep_conv_fwd", dict(fused_conv=conv_weight is not None,
                                                     u_layout=u_layout, want_state=want_state)))
        with torch.no_grad():
            o = self._prep_graph(value, conv_weight, conv_bias, conv_state, params, bc, biases, cfg,
                                 heads, P, u_layout)
        return (o.get("U"), o.get("M"), o.get("K"), o.get("B"), o.get("C"),
                o.get("state") if want_state else None)

    def scanprep_conv_bwd(self, value, conv_weight, conv_bias, conv_state, params, bc, biases, cfg,
                          dU, dM, dK, dBo, dCo, *, heads, P, u_layout="bhtp", want_dstate=False):
        self.calls.append(("scanprep_conv_bwd", {}))
        leaf = lambda x: None if x is None else x.detach().clone().requires_grad_(True)
        v, w, b, st, p_, bc_ = map(leaf, (value, conv_weight, conv_bias, conv_state, params, bc))
        bl = None if biases is None else [leaf(x) for x in biases[:4]] + [biases[4]]
        with torch.enable_grad():
            o = self._prep_graph(v, w, b, st, p_, bc_, bl, cfg, heads, P, u_layout)
            pairs = [(o[k], g) for k, g in (("U", dU), ("M", dM), ("K", dK), ("B", dBo), ("C", dCo))
                     if k in o and g is not None]
            wrt = [x for x in (v, w, b, st, p_, bc_) if x is not None] + (bl[:4] if bl and p_ is not None else [])
            grads = torch.autograd.grad([a for a, _ in pairs], wrt, [g.to(a.dtype) for a, g in pairs],
                                        allow_unused=True)
        it = iter(grads)
        take = lambda x: None if x is None else next(it)
        out = dict(d_value=take(v), d_conv_weight=take(w), d_conv_bias=take(b), d_conv_state=take(st),
                   d_params=take(p_), d_bc=take(bc_))
        for k in ("d_dt_bias", "d_alpha_bias", "d_theta_mod_bias", "d_theta_bias"):
            out[k] = next(it) if (bl and p_ is not None) else None
        for k in ("d_conv_weight", "d_conv_bias"):
            if out[k] is not None:
                out[k] = out[k].float()
        return out

    # ---- tail -----------------------------------------------------------------------------
    def mixer_tail_fwd(self, Y, gate, skip, d_skip, norm_weight, eps):
        self.calls.append(("mixer_tail_fwd", {}))
        with torch.no_grad():
            return mt.gated_rmsnorm(Y, gate, norm_weight, eps, skip, d_skip)

    def mixer_tail_bwd(self, Y, gate, skip, d_skip, norm_weight, eps, d_normed):
        self.calls.append(("mixer_tail_bwd", {}))
        leaf = lambda x: None if x is None else x.detach().clone().requires_grad_(True)
        y, g, s, ds, w = map(leaf, (Y, gate, skip, d_skip, norm_weight))
        with torch.enable_grad():
            out = mt.gated_rmsnorm(y, g, w, eps, s, ds)
            wrt = [x for x in (y, g, s, ds, w) if x is not None]
            grads = torch.autograd.grad(out, wrt, d_normed.to(out.dtype))
        it = iter(grads)
        take = lambda x: None if x is None else next(it)
        dy, dg, dsi, dds, dw = take(y), take(g), take(s), take(ds), take(w)
        return dy, dg, dsi, None if dds is None else dds.float(), dw.float()
