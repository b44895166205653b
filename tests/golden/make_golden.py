"""Generates the golden vectors under tests/golden/ by running the REFERENCE
implementation (b-vitamins/slinoss) on the CPU.

Usage (only where the reference checkout exists; the fixtures are committed):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

Every fixture stores its inputs (or, for the large config-0 case, the seed and a
checksum of the regenerated inputs) next to the reference's outputs, so the tests
never need the reference at run time.
"""

from __future__ import annotations

import math
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent


def _np(x):
    return None if x is None else x.detach().to(torch.float32).cpu().numpy() \
        if x.dtype != torch.float64 else x.detach().cpu().numpy()


def checksum(*tensors) -> float:
    """Order-sensitive float64 checksum of the regenerated inputs."""
    acc = 0.0
    for i, t in enumerate(tensors):
        v = t.detach().double().flatten()
        w = torch.cos(torch.arange(v.numel(), dtype=torch.float64) * 0.37 + i)
        acc += float((v * w).sum())
    return acc


def golden_scan_c0(ref):
    """Config 0: batch 2, heads 4, T 256, P 64, N 32, chunk 64, float32, seed 0."""
    sys.path.insert(0, str(REPO))
    from slinoss_b200.synthetic import make_scan_case
    case = make_scan_case(2, 4, 256, 64, 32, seed=0)
    Y, fin, _, _ = ref.v2x2ssd(case.U, case.M, case.K, case.B, case.C, chunk_size=64)
    Y64, fin64, _, _ = ref.v2x2ssm(case.U.double(), case.M.double(), case.K.double(),
                                   case.B.double(), case.C.double())
    np.savez_compressed(HERE / "scan_c0.npz", Y=_np(Y), final_state=_np(fin),
                        Y_seq_fp64=_np(Y64.float()), input_checksum=checksum(*case.tensors()),
                        shape=np.array([2, 4, 256, 64, 32, 64]))


def golden_scan_grad(ref):
    """Small grouped, streaming, ragged case with gradients by autograd through the
    reference's chunked scan (float64)."""
    g = torch.Generator().manual_seed(1)
    b, h, G, T, P, N, L = 2, 4, 2, 43, 16, 8, 16
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    radius = 0.6 + 0.35 * torch.rand(b, h, T, generator=g, dtype=torch.float64)
    angle = (2 * torch.rand(b, h, T, generator=g, dtype=torch.float64) - 1) * math.pi
    M = torch.stack((radius * torch.cos(angle), radius * torch.sin(angle)), -1)
    K = 0.1 * rn(b, h, T, 2, 2)
    U = rn(b, h, T, P)
    B, C = 0.3 * rn(b, G, T, 2 * N), 0.3 * rn(b, G, T, 2 * N)
    z0, Bp, Up = 0.1 * rn(b, h, P, 2 * N), 0.3 * rn(b, G, 2 * N), rn(b, h, P)
    ins = [U, M, K, B, C, z0, Bp, Up]
    for x in ins:
        x.requires_grad_(True)
    Y, fin, Bl, Ul = ref.v2x2ssd(U, M, K, B, C, chunk_size=L, initial_states=z0, B_prev=Bp, U_prev=Up)
    dY, dF = rn(*Y.shape), rn(*fin.shape)
    grads = torch.autograd.grad([Y, fin], ins, [dY, dF])
    names = ["U", "M", "K", "B", "C", "initial_states", "B_prev", "U_prev"]
    out = {n: _np(x) for n, x in zip(names, ins)}
    out.update({"d" + n: _np(gr) for n, gr in zip(names, grads)})
    out.update(Y=_np(Y), final_state=_np(fin), dY=_np(dY), d_final_state=_np(dF),
               chunk=np.array(L))
    np.savez_compressed(HERE / "scan_grad.npz", **out)


def _mixer_module(slinoss, seed=0, **kw):
    torch.manual_seed(seed)
    m = slinoss.layers.SLinOSSMixer(32, d_state=8, expand=2, d_head=16, d_conv=4, chunk_size=8, **kw)
    with torch.no_grad():  # move the scanprep biases off their init so every path is exercised
        for p in m.scanprep.parameters():
            p.add_(0.3 * torch.randn_like(p))
    return m


def golden_scanprep(slinoss):
    m = _mixer_module(slinoss, bc_groups=2)
    sp = m.scanprep
    g = torch.Generator().manual_seed(2)
    b, T = 2, 12
    value = torch.randn(b, T, m.d_inner, generator=g, requires_grad=True)
    params = torch.randn(b, T, m.param_proj_dim, generator=g, requires_grad=True)
    bc = torch.randn(b, T, m.bc_groups, 4, m.d_state, generator=g, requires_grad=True)
    from slinoss.layers.backend import ScanPrepInputs
    si = sp._prepare_inputs_reference(ScanPrepInputs(value=value, params=params, bc=bc))
    outs = [si.U, si.M, si.K, si.B, si.C]
    cots = [torch.randn(o.shape, generator=g) for o in outs]
    wrt = [value, params, bc, sp.dt_bias, sp.alpha_bias, sp.theta_mod_bias, sp.theta_bias]
    grads = torch.autograd.grad(outs, wrt, cots)
    d = dict(value=_np(value), params=_np(params), bc=_np(bc))
    d.update({k: _np(getattr(sp, k)) for k in ("dt_bias", "alpha_bias", "theta_mod_bias",
                                               "theta_bias", "theta_sign")})
    d.update({k: _np(o) for k, o in zip(("U", "M", "K", "B", "C"), outs)})
    d.update({"cot_" + k: _np(o) for k, o in zip(("U", "M", "K", "B", "C"), cots)})
    d.update({"d_" + k: _np(gr) for k, gr in zip(("value", "params", "bc", "dt_bias", "alpha_bias",
                                                  "theta_mod_bias", "theta_bias"), grads)})
    d["dims"] = np.array([m.n_heads, m.bc_groups, m.d_state, m.d_head])
    # known-answer: r = 1, theta = 0 gives kprev = kcurr = dt / 2 (tests/test_scanprep.py:150-161)
    from slinoss.ops.scanprep.reference import foh_taps_from_polar
    dt = torch.tensor([0.01, 0.05, 0.1])
    kp, kc = foh_taps_from_polar(dt, torch.ones(3), torch.zeros(3), eps=1e-8)
    d["kat_dt"], d["kat_kprev"], d["kat_kcurr"] = _np(dt), _np(kp), _np(kc)
    np.savez_compressed(HERE / "scanprep.npz", **d)


def golden_conv(slinoss):
    from slinoss.ops.mixer.convolution import apply_reference_causal_depthwise_conv
    m = _mixer_module(slinoss)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 11, m.d_inner, generator=g, requires_grad=True)
    st = torch.randn(2, m.d_inner, 3, generator=g, requires_grad=True)
    y, nxt = apply_reference_causal_depthwise_conv(m, x, st)
    cot = torch.randn(y.shape, generator=g)
    gx, gst, gw, gb = torch.autograd.grad(y, [x, st, m.dw_weight, m.dw_bias], cot)
    y0, nxt0 = apply_reference_causal_depthwise_conv(m, x, None)
    np.savez_compressed(HERE / "conv.npz", x=_np(x), state=_np(st), weight=_np(m.dw_weight),
                        bias=_np(m.dw_bias), y=_np(y), next_state=_np(nxt), cot=_np(cot),
                        d_x=_np(gx), d_state=_np(gst), d_weight=_np(gw), d_bias=_np(gb),
                        y_nostate=_np(y0), next_state_nostate=_np(nxt0))


def golden_tail(slinoss):
    from slinoss.ops.mixer.tail import _mixer_tail_forward
    m = _mixer_module(slinoss)
    g = torch.Generator().manual_seed(4)
    b, T = 2, 9
    Y = torch.randn(b, m.n_heads, T, m.d_head, generator=g, requires_grad=True)
    U = torch.randn(b, m.n_heads, T, m.d_head, generator=g, requires_grad=True)
    gate = torch.randn(b, T, m.d_inner, generator=g, requires_grad=True)
    with torch.no_grad():
        m.out_norm.weight.add_(0.2 * torch.randn(m.d_inner, generator=g))
    out = _mixer_tail_forward(Y, gate, m.out_norm.weight, m.out_norm.eps, m.out_proj.weight, None,
                              skip_input=U, d_skip=m.d_skip)
    cot = torch.randn(out.shape, generator=g)
    wrt = [Y, gate, U, m.d_skip, m.out_norm.weight, m.out_proj.weight]
    grads = torch.autograd.grad(out, wrt, cot)
    d = dict(Y=_np(Y), U=_np(U), gate=_np(gate), d_skip=_np(m.d_skip),
             norm_weight=_np(m.out_norm.weight), proj_weight=_np(m.out_proj.weight),
             eps=np.array(m.out_norm.eps), out=_np(out), cot=_np(cot))
    d.update({"d_" + k: _np(gr) for k, gr in zip(("Y", "gate", "U", "d_skip", "norm_weight",
                                                  "proj_weight"), grads)})
    np.savez_compressed(HERE / "tail.npz", **d)


def golden_mixer(slinoss):
    """Whole mixer forward+backward, a two-segment streaming pass and 3 decode steps."""
    m = _mixer_module(slinoss, bc_groups=2)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 21, 32, generator=g, requires_grad=True)
    out = m(x)
    cot = torch.randn(out.shape, generator=g)
    names = [n for n, _ in m.named_parameters()]
    grads = torch.autograd.grad(out, [x, *m.parameters()], cot)
    d = {"sd_" + k: _np(v) for k, v in m.state_dict().items()}
    d.update(x=_np(x), out=_np(out), cot=_np(cot), d_x=_np(grads[0]))
    d.update({"dp_" + n: _np(gr) for n, gr in zip(names, grads[1:])})
    with torch.no_grad():
        o1, st = m(x[:, :13], return_state=True)
        o2, st2 = m(x[:, 13:], state=st, return_state=True)
        d["out_segmented"] = _np(torch.cat([o1, o2], 1))
        d["seg_state"] = _np(st2.scan.state)
        d["seg_conv"] = _np(st2.conv)
        state = None
        steps = []
        for t in range(3):
            y, state = m.step(x[:, t], state)
            steps.append(y)
        d["out_steps"] = _np(torch.stack(steps, 1))
    np.savez_compressed(HERE / "mixer.npz", **d)


def golden_scanprep_fp64(slinoss):
    """The reference's scan preparation evaluated in float64 (module and inputs cast to double):
    the exact value of the same formulas, which the float32 evaluation reaches only to its own
    round-off (the tap quotients cancel for small |z|)."""
    # The reference's coefficient code casts to float32 in two helpers (principal_angle and
    # _pack_complex, slinoss/ops/scanprep/reference.py:11-22); they are replaced here, for this call
    # only, by the same two formulas without the cast, so that its own code runs in float64 throughout.
    import slinoss.layers.scanprep as lsp
    import slinoss.ops.scanprep.reference as osr
    two_pi = 2.0 * math.pi
    keep = (lsp.principal_angle, osr._pack_complex, lsp._pack_complex)
    lsp.principal_angle = lambda th: torch.remainder(th + math.pi, two_pi) - math.pi
    osr._pack_complex = lsp._pack_complex = lambda x: torch.view_as_real(x).contiguous()
    try:
        _golden_scanprep_fp64(slinoss)
    finally:
        lsp.principal_angle, osr._pack_complex, lsp._pack_complex = keep


def _golden_scanprep_fp64(slinoss):
    m = _mixer_module(slinoss, bc_groups=2).double()
    sp = m.scanprep
    g = torch.Generator().manual_seed(2)
    b, T = 2, 12
    value = torch.randn(b, T, m.d_inner, generator=g).double().requires_grad_(True)
    params = torch.randn(b, T, m.param_proj_dim, generator=g).double().requires_grad_(True)
    bc = torch.randn(b, T, m.bc_groups, 4, m.d_state, generator=g).double().requires_grad_(True)
    from slinoss.layers.backend import ScanPrepInputs
    si = sp._prepare_inputs_reference(ScanPrepInputs(value=value, params=params, bc=bc))
    outs = [si.U, si.M, si.K, si.B, si.C]
    assert all(o.dtype == torch.float64 for o in (si.M, si.K)), [o.dtype for o in outs]
    cots = [torch.randn(o.shape, generator=g).double() for o in outs]
    wrt = [value, params, bc, sp.dt_bias, sp.alpha_bias, sp.theta_mod_bias, sp.theta_bias]
    grads = torch.autograd.grad(outs, wrt, cots)
    d = dict(value=_np(value), params=_np(params), bc=_np(bc))
    d.update({k: _np(getattr(sp, k)) for k in ("dt_bias", "alpha_bias", "theta_mod_bias",
                                               "theta_bias", "theta_sign")})
    d.update({k: _np(o) for k, o in zip(("U", "M", "K", "B", "C"), outs)})
    d.update({"cot_" + k: _np(o) for k, o in zip(("U", "M", "K", "B", "C"), cots)})
    d.update({"d_" + k: _np(gr) for k, gr in zip(("value", "params", "bc", "dt_bias", "alpha_bias",
                                                  "theta_mod_bias", "theta_bias"), grads)})
    d["dims"] = np.array([m.n_heads, m.bc_groups, m.d_state, m.d_head])
    np.savez_compressed(HERE / "scanprep_fp64.npz", **d)


def golden_tail_fp64(slinoss):
    """The reference's mixer tail in float64 on the inputs of the float32 fixture."""
    from slinoss.ops.mixer.tail import _mixer_tail_forward
    t = dict(np.load(HERE / "tail.npz"))
    leaf = lambda k: torch.from_numpy(t[k]).double().requires_grad_(True)
    Y, U, gate, d_skip, nw, pw = (leaf(k) for k in ("Y", "U", "gate", "d_skip", "norm_weight",
                                                    "proj_weight"))
    out = _mixer_tail_forward(Y, gate, nw, float(t["eps"]), pw, None, skip_input=U, d_skip=d_skip)
    grads = torch.autograd.grad(out, [Y, gate, U, d_skip, nw, pw], torch.from_numpy(t["cot"]).double())
    d = {"out": _np(out)}
    d.update({"d_" + k: _np(gr) for k, gr in zip(("Y", "gate", "U", "d_skip", "norm_weight",
                                                  "proj_weight"), grads)})
    np.savez_compressed(HERE / "tail_fp64.npz", **d)


def golden_stack(slinoss):
    """Two-block stack (mixer + gelu FFN, final norm): forward, gradients and three decode steps."""
    import slinoss.blocks as rb
    torch.manual_seed(7)
    cfg = rb.SLinOSSStackConfig.uniform(
        rb.SLinOSSBlockConfig(d_model=32, mixer=rb.SLinOSSMixerConfig(d_state=8, d_head=16, chunk_size=8),
                              ffn=rb.SLinOSSMLPConfig(kind="gelu", expand=2.0, multiple_of=8)), n_layers=2)
    stack = rb.SLinOSSStack(cfg)
    with torch.no_grad():
        for n, p in stack.named_parameters():
            if "scanprep" in n or "norm" in n:
                p.add_(0.2 * torch.randn_like(p))
    g = torch.Generator().manual_seed(8)
    x = torch.randn(2, 19, 32, generator=g, requires_grad=True)
    out = stack(x)
    cot = torch.randn(out.shape, generator=g)
    names = [n for n, _ in stack.named_parameters()]
    grads = torch.autograd.grad(out, [x, *stack.parameters()], cot)
    d = {"sd_" + k: _np(v) for k, v in stack.state_dict().items()}
    d.update(x=_np(x), out=_np(out), cot=_np(cot), d_x=_np(grads[0]))
    d.update({"dp_" + n: _np(gr) for n, gr in zip(names, grads[1:])})
    with torch.no_grad():
        state, steps = None, []
        for t in range(3):
            y, state = stack.step(x[:, t], state)
            steps.append(y)
        d["out_steps"] = _np(torch.stack(steps, 1))
    np.savez_compressed(HERE / "stack.npz", **d)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of a checkout of the reference (slinoss)>")
    ref_root = sys.argv[1]
    sys.dont_write_bytecode = True
    sys.path.insert(0, ref_root)
    import slinoss
    import slinoss.layers  # noqa: F401
    from slinoss.ops.v2x2ssd import reference as ref
    torch.set_num_threads(8)
    golden_scan_c0(ref)
    golden_scan_grad(ref)
    golden_scanprep(slinoss)
    golden_conv(slinoss)
    golden_tail(slinoss)
    golden_mixer(slinoss)
    golden_scanprep_fp64(slinoss)
    golden_tail_fp64(slinoss)
    golden_stack(slinoss)
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)


if __name__ == "__main__":
    main()
