"""Pins the oracle (oracle/) against golden vectors produced by the reference itself.

Runs on the CPU.  Tolerances: the float64 restatement must agree with the
reference's float64 results to 1e-10 and with its float32 results to the float32
round-off of the reference (2e-5 absolute, the bound the reference's own tests use,
tests/test_v2x2ssd_reference.py:92-207 there).
"""

import numpy as np
import pytest
import torch

from oracle import mixer_torch as mt
from oracle import scan_np
from slinoss_b200.synthetic import make_scan_case
from tests.golden.make_golden import checksum


def rel(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


def test_scan_config0_forward(golden):
    g = golden("scan_c0")
    case = make_scan_case(2, 4, 256, 64, 32, seed=0)
    if abs(checksum(*case.tensors()) - float(g["input_checksum"])) > 1e-6 * abs(float(g["input_checksum"])):
        pytest.skip("torch's CPU generator no longer reproduces the fixture inputs")
    n = lambda x: x.numpy()
    args = [n(t) for t in case.tensors()]
    Y64, fin64, _, _ = scan_np.v2x2ssm(*args, dtype=np.float64)
    assert rel(Y64, g["Y_seq_fp64"]) < 1e-6          # fixture is stored in float32
    assert rel(Y64, g["Y"]) < 1e-5                   # reference chunked float32 vs exact
    Yc, finc, _, _ = scan_np.v2x2ssd(*args, chunk_size=64, dtype=np.float64)
    assert rel(Yc, Y64) < 1e-10 and rel(finc, fin64) < 1e-10
    assert rel(finc, g["final_state"]) < 1e-5
    Yf, finf, _, _ = scan_np.v2x2ssd(*args, chunk_size=64, dtype=np.float32)
    assert rel(Yf, g["Y"]) < 1e-5 and rel(finf, g["final_state"]) < 1e-5


def test_scan_grouped_streaming_forward_and_gradients(golden):
    g = golden("scan_grad")
    kw = dict(initial_states=g["initial_states"], B_prev=g["B_prev"], U_prev=g["U_prev"])
    ins = [g[k] for k in "UMKBC"]
    L = int(g["chunk"])
    for fn, extra in ((scan_np.v2x2ssm, {}), (scan_np.v2x2ssd, {"chunk_size": L})):
        Y, fin, Bl, Ul = fn(*ins, **kw, **extra)
        assert rel(Y, g["Y"]) < 1e-10 and rel(fin, g["final_state"]) < 1e-10
        assert np.array_equal(Bl, g["B"][:, :, -1]) and np.array_equal(Ul, g["U"][:, :, -1])
    grads = scan_np.v2x2ssd_bwd(*ins, g["dY"], d_final_state=g["d_final_state"], **kw)
    for name, got in grads.items():
        assert rel(got, g["d" + name]) < 1e-10, name


def test_scan_chunk_size_is_a_numerical_noop():
    case = make_scan_case(1, 2, 37, 8, 4, seed=3, streaming=True, with_init=True)
    n = lambda x: None if x is None else x.numpy()
    kw = dict(initial_states=n(case.initial_states), B_prev=n(case.B_prev), U_prev=n(case.U_prev))
    base = scan_np.v2x2ssm(*[n(t) for t in case.tensors()], **kw)
    for L in (1, 5, 16, 64):
        out = scan_np.v2x2ssd(*[n(t) for t in case.tensors()], chunk_size=L, **kw)
        assert rel(out[0], base[0]) < 1e-10 and rel(out[1], base[1]) < 1e-10


def test_scan_zero_length_passes_state_through():
    case = make_scan_case(2, 2, 0, 4, 3, seed=1, streaming=True, with_init=True)
    n = lambda x: x.numpy()
    Y, fin, Bl, Ul = scan_np.v2x2ssd(*[n(t) for t in case.tensors()], chunk_size=8,
                                     initial_states=n(case.initial_states), B_prev=n(case.B_prev),
                                     U_prev=n(case.U_prev))
    assert Y.shape == (2, 2, 0, 4)
    assert np.allclose(fin, n(case.initial_states)) and np.allclose(Bl, n(case.B_prev))


def test_scan_rejects_zero_transition_in_chunked_path():
    case = make_scan_case(1, 1, 8, 4, 2, seed=0)
    M = case.M.numpy().copy()
    M[0, 0, 3] = 0.0
    with pytest.raises(ValueError, match="strictly nonzero"):
        scan_np.v2x2ssd(case.U.numpy(), M, case.K.numpy(), case.B.numpy(), case.C.numpy(), chunk_size=4)


def _cfg():
    return dict(dt_min=5e-3, dt_max=1e-1, alpha_min=0.0, alpha_max=20.0, theta_init_min=0.05,
                theta_init_max=2.0, theta_mod_scale=1.0, r_min=0.8, r_max=1.0, eps=1e-8)


def test_scanprep_forward_and_gradients(golden):
    g = golden("scanprep")
    t = lambda k, rg=False: torch.from_numpy(g[k]).requires_grad_(rg)
    H, G, N, P = map(int, g["dims"])
    value, params, bc = t("value", True), t("params", True), t("bc", True)
    biases = [t(k, True) for k in ("dt_bias", "alpha_bias", "theta_mod_bias", "theta_bias")]
    outs = mt.scanprep(value, params, bc, _cfg(), *biases, t("theta_sign"), P)
    for name, o in zip("UMKBC", outs):
        assert rel(o.detach().numpy(), g[name]) < 1e-6, name
    grads = torch.autograd.grad(outs, [value, params, bc, *biases], [t("cot_" + k) for k in "UMKBC"])
    for name, gr in zip(("value", "params", "bc", "dt_bias", "alpha_bias", "theta_mod_bias",
                         "theta_bias"), grads):
        assert rel(gr.numpy(), g["d_" + name]) < 1e-5, name


def test_foh_taps_known_answer(golden):
    g = golden("scanprep")
    dt = torch.from_numpy(g["kat_dt"])
    z = torch.zeros(3)
    kp, kc = mt.foh_taps(dt, z, z, torch.polar(torch.ones(3), z), 1e-8)
    assert torch.allclose(kp.real, dt / 2, atol=1e-7) and torch.allclose(kc.real, dt / 2, atol=1e-7)
    assert np.allclose(torch.view_as_real(kp).numpy(), g["kat_kprev"], atol=1e-7)
    assert np.allclose(torch.view_as_real(kc).numpy(), g["kat_kcurr"], atol=1e-7)


def test_bc_pairs_have_unit_rms():
    bc = torch.randn(2, 5, 3, 4, 16)
    b, c = mt.bc_pairs(bc, 1e-8)
    for pairs in (b, c):
        ms = pairs.square().sum(-1).mean(-1)
        assert torch.allclose(ms, torch.ones_like(ms), atol=1e-5)


def test_conv_forward_and_gradients(golden):
    g = golden("conv")
    t = lambda k: torch.from_numpy(g[k]).requires_grad_(True)
    x, st, w, b = t("x"), t("state"), t("weight"), t("bias")
    y, nxt = mt.causal_conv_silu(x, w, b, st)
    assert rel(y.detach().numpy(), g["y"]) < 1e-6 and rel(nxt.detach().numpy(), g["next_state"]) < 1e-7
    grads = torch.autograd.grad(y, [x, st, w, b], torch.from_numpy(g["cot"]))
    for name, gr in zip(("x", "state", "weight", "bias"), grads):
        assert rel(gr.numpy(), g["d_" + name]) < 1e-5, name
    y0, n0 = mt.causal_conv_silu(x, w, b, None)
    assert rel(y0.detach().numpy(), g["y_nostate"]) < 1e-6
    assert rel(n0.detach().numpy(), g["next_state_nostate"]) < 1e-7


def test_tail_forward_and_gradients(golden):
    g = golden("tail")
    t = lambda k: torch.from_numpy(g[k]).requires_grad_(True)
    Y, U, gate, ds, nw, pw = t("Y"), t("U"), t("gate"), t("d_skip"), t("norm_weight"), t("proj_weight")
    out = torch.nn.functional.linear(mt.gated_rmsnorm(Y, gate, nw, float(g["eps"]), U, ds), pw)
    assert rel(out.detach().numpy(), g["out"]) < 1e-6
    grads = torch.autograd.grad(out, [Y, gate, U, ds, nw, pw], torch.from_numpy(g["cot"]))
    for name, gr in zip(("Y", "gate", "U", "d_skip", "norm_weight", "proj_weight"), grads):
        assert rel(gr.numpy(), g["d_" + name]) < 1e-5, name


def test_scanprep_float64_branch_is_the_reference_in_float64(golden):
    """The float64 evaluation of scan preparation (``coeff_dtype=float64``) against the reference's
    own code run in float64: this is what the CUDA kernels' float64 tap arithmetic is held to."""
    g = golden("scanprep_fp64")
    t = lambda k, rg=False: torch.from_numpy(g[k]).double().requires_grad_(rg)
    H, G, N, P = map(int, g["dims"])
    value, params, bc = t("value", True), t("params", True), t("bc", True)
    biases = [t(k, True) for k in ("dt_bias", "alpha_bias", "theta_mod_bias", "theta_bias")]
    # M and K as float64 straight from the coefficient stage (the packing casts them to float32)
    bsz, T, _ = params.shape
    p4 = params.view(bsz, T, H, 3).permute(0, 2, 1, 3) + torch.stack(biases[:3], -1).view(1, H, 1, 3)
    cfg = _cfg()
    dt = cfg["dt_min"] + (cfg["dt_max"] - cfg["dt_min"]) * torch.sigmoid(p4[..., 0])
    alpha = cfg["alpha_min"] + (cfg["alpha_max"] - cfg["alpha_min"]) * torch.sigmoid(p4[..., 1])
    span = cfg["theta_init_max"] - cfg["theta_init_min"]
    theta_u = torch.sigmoid(biases[3].view(1, H, 1) + cfg["theta_mod_scale"] * torch.tanh(p4[..., 2]))
    theta = mt._wrap_angle(t("theta_sign").view(1, H, 1) * (cfg["theta_init_min"] + span * theta_u))
    r = cfg["r_min"] + (cfg["r_max"] - cfg["r_min"]) * torch.exp(-alpha)
    rho = torch.polar(r, theta)
    kp, kc = mt.foh_taps(dt, torch.log(r), theta, rho, cfg["eps"])
    M = torch.view_as_real(rho)
    K = torch.stack((torch.view_as_real(kp), torch.view_as_real(kc)), dim=-2)
    assert rel(M.detach().numpy(), g["M"]) < 1e-12 and rel(K.detach().numpy(), g["K"]) < 1e-12
    grads = torch.autograd.grad([M, K], [params, *biases], [t("cot_M"), t("cot_K")])
    for name, gr in zip(("params", "dt_bias", "alpha_bias", "theta_mod_bias", "theta_bias"), grads):
        # (the reference rounds the params gradient to float32 on its way back through its input cast)
        assert rel(gr.numpy(), g["d_" + name]) < (1e-7 if name == "params" else 1e-10), name
    # ... and the packed call agrees with it to the float32 rounding of its outputs
    outs = mt.scanprep(value.float(), params.float(), bc.float(), cfg, *[b.float() for b in biases],
                       t("theta_sign").float(), P, coeff_dtype=torch.float64)
    assert rel(outs[1].detach().numpy(), g["M"]) < 1e-7 and rel(outs[2].detach().numpy(), g["K"]) < 1e-7


def test_tail_float64_against_the_reference_in_float64(golden):
    g, g64 = golden("tail"), golden("tail_fp64")
    t = lambda k: torch.from_numpy(g[k]).double().requires_grad_(True)
    Y, U, gate, ds, nw, pw = t("Y"), t("U"), t("gate"), t("d_skip"), t("norm_weight"), t("proj_weight")
    out = torch.nn.functional.linear(mt.gated_rmsnorm(Y, gate, nw, float(g["eps"]), U, ds), pw)
    assert rel(out.detach().numpy(), g64["out"]) < 1e-12
    grads = torch.autograd.grad(out, [Y, gate, U, ds, nw, pw], torch.from_numpy(g["cot"]).double())
    for name, gr in zip(("Y", "gate", "U", "d_skip", "norm_weight", "proj_weight"), grads):
        assert rel(gr.numpy(), g64["d_" + name]) < 1e-10, name


@pytest.mark.parametrize("shape", [(1, 2, 2, 70, 64, 64, True, True), (2, 4, 2, 43, 16, 8, True, True),
                                   (1, 3, 3, 130, 8, 5, False, False)])
def test_c_port_of_the_scan_matches_the_numpy_oracle(shape, golden):
    """oracle/csrc/v2x2ssd_cpu.c is what ``bench.py --impl reference`` and ``cpu_baseline`` time."""
    from oracle import scan_c
    b, h, g_, T, P, N, streaming, init = shape
    case = make_scan_case(b, h, T, P, N, groups=g_, seed=5 * T, streaming=streaming, with_init=init)
    n = lambda x: None if x is None else x.numpy()
    args = [n(x) for x in case.tensors()]
    kw = dict(initial_states=n(case.initial_states), B_prev=n(case.B_prev), U_prev=n(case.U_prev))
    wY, wfin, _, _ = scan_np.v2x2ssm(*args, **kw)
    Y, fin = scan_c.forward(*args, **kw)
    assert rel(Y, wY) < 1e-5 and rel(fin, wfin) < 1e-5
    dfin = np.random.default_rng(0).standard_normal(wfin.shape).astype(np.float32)
    want = scan_np.v2x2ssd_bwd(*args, n(case.dY), d_final_state=dfin, **kw)
    got = scan_c.backward(*args, n(case.dY), d_final_state=dfin, **kw)
    for name in want:
        assert rel(got[name], want[name]) < 2e-5, name
    # the reference's own golden (grouped, streaming, ragged, float64 autograd)
    gg = golden("scan_grad")
    kw = dict(initial_states=gg["initial_states"], B_prev=gg["B_prev"], U_prev=gg["U_prev"])
    ins = [gg[k] for k in "UMKBC"]
    Y, fin = scan_c.forward(*ins, **kw)
    assert rel(Y, gg["Y"]) < 1e-5 and rel(fin, gg["final_state"]) < 1e-5
    got = scan_c.backward(*ins, gg["dY"], d_final_state=gg["d_final_state"], **kw)
    for name, val in got.items():
        assert rel(val, gg["d" + name]) < 2e-5, name
