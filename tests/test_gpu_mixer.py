"""Parity of the CUDA scan-preparation / conv / tail kernels and of the whole mixer
with the oracle and with golden vectors of the reference (through the C ABI)."""

from pathlib import Path

import numpy as np
import pytest
import torch

import slinoss_b200 as sb
from oracle import mixer_torch as mt
from slinoss_b200.ops.mixer import mixer_gated_norm
from slinoss_b200.ops.scanprep import causal_conv_silu_b200, conv_scanprep_b200, scanprep_b200
from tests.util import rel, tol

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cfg(sp):
    return {k: getattr(sp, k) for k in ("dt_min", "dt_max", "alpha_min", "alpha_max",
                                        "theta_init_min", "theta_init_max", "theta_mod_scale",
                                        "r_min", "r_max", "eps")}


def _scanprep_module(heads, groups, N, P, seed=0):
    torch.manual_seed(seed)
    sp = sb.SLinOSSScanPrep(n_heads=heads, bc_groups=groups, d_state=N, d_head=P)
    with torch.no_grad():
        for p in sp.parameters():
            p.add_(0.3 * torch.randn_like(p))
    return sp


def _oracle_prep(sp_cpu, value, params, bc, w=None, b=None, st=None):
    v = value
    nstate = None
    if w is not None:
        v, nstate = mt.causal_conv_silu(value, w, b, st)
    # The tap quotients lose up to ~1e-4 relative accuracy in float32 (the reference's
    # own arithmetic); the kernels evaluate them in float64, so they are held to 1e-5
    # against the float64 evaluation of the same formulas.
    out = mt.scanprep(v, params, bc, _cfg(sp_cpu), sp_cpu.dt_bias, sp_cpu.alpha_bias,
                      sp_cpu.theta_mod_bias, sp_cpu.theta_bias, sp_cpu.theta_sign, sp_cpu.d_head,
                      coeff_dtype=torch.float64)
    return (*out, nstate)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dims", [(4, 2, 8, 16, 2, 12), (3, 3, 5, 8, 1, 37), (32, 32, 64, 64, 2, 70)])
def test_scanprep_forward_backward(dims, dtype):
    H, G, N, P, bsz, T = dims
    sp_cpu = _scanprep_module(H, G, N, P)
    sp = _scanprep_module(H, G, N, P).to(DEV)
    gen = torch.Generator().manual_seed(1)
    mk = lambda *s: torch.randn(*s, generator=gen).to(dtype)
    value, params, bc = mk(bsz, T, H * P), mk(bsz, T, 3 * H), mk(bsz, T, G, 4, N)
    cots = [mk(bsz, H, T, P), mk(bsz, H, T, 2).float(), mk(bsz, H, T, 2, 2).float(),
            mk(bsz, G, T, 2 * N), mk(bsz, G, T, 2 * N)]
    # oracle in float32 on the same (rounded) inputs
    lv = lambda x: x.float().clone().requires_grad_(True)
    ov, op_, obc = lv(value), lv(params), lv(bc)
    want = _oracle_prep(sp_cpu, ov, op_, obc)[:5]
    obias = [sp_cpu.dt_bias, sp_cpu.alpha_bias, sp_cpu.theta_mod_bias, sp_cpu.theta_bias]
    wgrads = torch.autograd.grad(want, [ov, op_, obc, *obias], [c.float() for c in cots])
    gv, gp, gbc = (x.to(DEV).requires_grad_(True) for x in (value, params, bc))
    got = scanprep_b200(sp, gv, gp, gbc)
    for name, a, w_ in zip("UMKBC", got, want):
        t = 1e-5 if name in "MK" else tol(dtype)
        assert rel(a, w_) <= t, (name, rel(a, w_))
    gbias = [sp.dt_bias, sp.alpha_bias, sp.theta_mod_bias, sp.theta_bias]
    ggrads = torch.autograd.grad(got, [gv, gp, gbc, *gbias], [c.to(DEV) for c in cots])
    for name, a, w_ in zip(("value", "params", "bc", "dt_bias", "alpha_bias", "theta_mod_bias",
                            "theta_bias"), ggrads, wgrads):
        t = tol(dtype) if name in ("value", "params", "bc") else max(tol(dtype), 1e-4)
        assert rel(a, w_) <= t, (name, rel(a, w_))


def test_scanprep_against_reference_golden(golden):
    g = golden("scanprep")
    H, G, N, P = map(int, g["dims"])
    sp = sb.SLinOSSScanPrep(n_heads=H, bc_groups=G, d_state=N, d_head=P).to(DEV)
    with torch.no_grad():
        for k in ("dt_bias", "alpha_bias", "theta_mod_bias", "theta_bias"):
            getattr(sp, k).copy_(torch.from_numpy(g[k]))
    t = lambda k: torch.from_numpy(g[k]).to(DEV).requires_grad_(True)
    value, params, bc = t("value"), t("params"), t("bc")
    out = sp(value, params, bc)
    for name in "UMKBC":
        # K: the golden holds the reference's float32 taps, exact only to ~1e-4
        assert rel(getattr(out, name), g[name]) <= (1e-4 if name == "K" else 1e-5), name
    grads = torch.autograd.grad([out.U, out.M, out.K, out.B, out.C],
                                [value, params, bc, sp.dt_bias, sp.alpha_bias, sp.theta_mod_bias,
                                 sp.theta_bias],
                                [torch.from_numpy(g["cot_" + k]).to(DEV) for k in "UMKBC"])
    for name, gr in zip(("value", "params", "bc", "dt_bias", "alpha_bias", "theta_mod_bias",
                         "theta_bias"), grads):
        # The golden gradients come from float32 autograd through the cancelling tap
        # quotients (exact to ~1e-3) and, for heads whose dt sigmoid is saturated at
        # initialisation, through sigma*(1-sigma) evaluated in float32 (exact to ~1e-2).
        # The kernels evaluate both in float64; the strict check is the float64 oracle in
        # test_scanprep_forward_backward.
        assert rel(gr, g["d_" + name]) <= (5e-2 if "bias" in name else 1e-3 if name == "params" else 1e-4), \
            (name, rel(gr, g["d_" + name]))


def test_scanprep_against_the_reference_evaluated_in_float64(golden):
    """The strict bar for the coefficient kernels: the reference's own scan preparation run in
    float64 (tests/golden/make_golden.py, golden_scanprep_fp64).  M, K and the gradients that flow
    through the taps and the saturating sigmoids agree to 1e-5; the looser bounds against the
    float32 golden above are the reference's float32 round-off, not the kernels'."""
    g = golden("scanprep_fp64")
    H, G, N, P = map(int, g["dims"])
    sp = sb.SLinOSSScanPrep(n_heads=H, bc_groups=G, d_state=N, d_head=P).to(DEV)
    with torch.no_grad():
        for k in ("dt_bias", "alpha_bias", "theta_mod_bias", "theta_bias"):
            getattr(sp, k).copy_(torch.from_numpy(g[k]).float())
    t = lambda k: torch.from_numpy(g[k]).float().to(DEV).requires_grad_(True)
    value, params, bc = t("value"), t("params"), t("bc")
    out = sp(value, params, bc)
    for name in "UMKBC":
        assert rel(getattr(out, name), g[name]) <= 1e-5, (name, rel(getattr(out, name), g[name]))
    grads = torch.autograd.grad([out.U, out.M, out.K, out.B, out.C],
                                [value, params, bc, sp.dt_bias, sp.alpha_bias, sp.theta_mod_bias,
                                 sp.theta_bias],
                                [torch.from_numpy(g["cot_" + k]).float().to(DEV) for k in "UMKBC"])
    for name, gr in zip(("value", "params", "bc", "dt_bias", "alpha_bias", "theta_mod_bias",
                         "theta_bias"), grads):
        assert rel(gr, g["d_" + name]) <= 1e-5, (name, rel(gr, g["d_" + name]))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dims", [(2, 11, 64, 4, True), (1, 2, 40, 4, True), (3, 70, 96, 3, False),
                                  (2, 33, 8, 2, True), (1, 5, 16, 1, False)])
def test_conv_forward_backward(dims, dtype):
    bsz, T, C, W, with_state = dims
    gen = torch.Generator().manual_seed(3)
    mk = lambda *s: torch.randn(*s, generator=gen).to(dtype)
    x, w, b = mk(bsz, T, C), 0.5 * mk(C, W), mk(C)
    st = mk(bsz, C, W - 1) if with_state and W > 1 else None
    cot = mk(bsz, T, C)
    lv = lambda v: None if v is None else v.float().clone().requires_grad_(True)
    ox, ow, ob, ost = lv(x), lv(w), lv(b), lv(st)
    wy, wn = mt.causal_conv_silu(ox, ow, ob, ost)
    wl = [v for v in (ox, ow, ob, ost) if v is not None]
    wg = torch.autograd.grad(wy, wl, cot.float())
    gl = lambda v: None if v is None else v.to(DEV).requires_grad_(True)
    gx, gw, gb, gst = gl(x), gl(w), gl(b), gl(st)
    y, nxt = causal_conv_silu_b200(gx, gw, gb, gst)
    assert rel(y, wy) <= tol(dtype) and rel(nxt, wn) <= 1e-6
    gg = torch.autograd.grad(y, [v for v in (gx, gw, gb, gst) if v is not None], cot.to(DEV))
    for a, w_ in zip(gg, wg):
        assert rel(a, w_) <= tol(dtype), rel(a, w_)


def test_conv_on_a_column_slice_and_reference_golden(golden):
    g = golden("conv")
    t = lambda k: torch.from_numpy(g[k]).to(DEV)
    wide = torch.cat([torch.zeros_like(t("x")), t("x")], dim=-1)      # value is a column slice
    x = wide[..., wide.shape[-1] // 2:].requires_grad_(True)
    w, b, st = (t(k).requires_grad_(True) for k in ("weight", "bias", "state"))
    y, nxt = causal_conv_silu_b200(x, w, b, st)
    assert rel(y, g["y"]) <= 1e-5 and rel(nxt, g["next_state"]) <= 1e-6
    grads = torch.autograd.grad(y, [x, st, w, b], t("cot"))
    for name, gr in zip(("x", "state", "weight", "bias"), grads):
        assert rel(gr, g["d_" + name]) <= 1e-5, name
    y0, n0 = causal_conv_silu_b200(x, w, b, None)
    assert rel(y0, g["y_nostate"]) <= 1e-5 and rel(n0, g["next_state_nostate"]) <= 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dims", [(2, 4, 9, 16), (1, 32, 70, 64), (2, 3, 5, 24)])
def test_tail_forward_backward(dims, dtype):
    bsz, H, T, P = dims
    gen = torch.Generator().manual_seed(4)
    mk = lambda *s: torch.randn(*s, generator=gen).to(dtype)
    Y, U, gate = mk(bsz, H, T, P), mk(bsz, H, T, P), mk(bsz, T, H * P)
    ds, nw = torch.randn(H, generator=gen), (1 + 0.2 * torch.randn(H * P, generator=gen)).to(dtype)
    cot = mk(bsz, T, H * P)
    # float32 inputs: the oracle runs in float64 (its own float32 evaluation is exact to ~1e-4 only)
    odt = torch.float64 if dtype == torch.float32 else dtype
    lv = lambda v: v.to(odt if v.dtype == dtype or v.dtype == torch.float32 else v.dtype).clone().requires_grad_(True)
    oY, oU, og, ods, onw = lv(Y), lv(U), lv(gate), lv(ds), lv(nw)
    want = mt.gated_rmsnorm(oY, og, onw, 1e-5, oU, ods)
    wg = torch.autograd.grad(want, [oY, og, oU, ods, onw], cot.to(want.dtype))
    gl = lambda v: v.to(DEV).requires_grad_(True)
    gY, gU, gg, gds, gnw = gl(Y), gl(U), gl(gate), gl(ds), gl(nw)
    got = mixer_gated_norm(gY, gg, gnw, 1e-5, skip_input=gU, d_skip=gds)
    assert rel(got, want) <= tol(dtype)
    ggr = torch.autograd.grad(got, [gY, gg, gU, gds, gnw], cot.to(DEV))
    for name, a, w_ in zip(("Y", "gate", "U", "d_skip", "norm_weight"), ggr, wg):
        assert rel(a, w_) <= tol(dtype), (name, rel(a, w_))


def test_tail_against_the_reference_evaluated_in_float64(golden):
    g, g64 = golden("tail"), golden("tail_fp64")
    t = lambda k: torch.from_numpy(g[k]).to(DEV).requires_grad_(True)
    Y, U, gate, ds, nw, pw = t("Y"), t("U"), t("gate"), t("d_skip"), t("norm_weight"), t("proj_weight")
    out = torch.nn.functional.linear(mixer_gated_norm(Y, gate, nw, float(g["eps"]), skip_input=U, d_skip=ds), pw)
    assert rel(out, g64["out"]) <= 1e-5
    grads = torch.autograd.grad(out, [Y, gate, U, ds, nw, pw], torch.from_numpy(g["cot"]).to(DEV))
    for name, gr in zip(("Y", "gate", "U", "d_skip", "norm_weight", "proj_weight"), grads):
        assert rel(gr, g64["d_" + name]) <= 1e-5, (name, rel(gr, g64["d_" + name]))


def _load_mixer(g, dtype=torch.float32, **kw):
    m = sb.SLinOSSMixer(32, d_state=8, expand=2, d_head=16, d_conv=4, chunk_size=8, bc_groups=2, **kw)
    m.load_state_dict({k[3:]: torch.from_numpy(v) for k, v in g.items() if k.startswith("sd_")})
    return m.to(DEV)


def test_mixer_against_reference_golden(golden):
    g = golden("mixer")
    m = _load_mixer(g)
    x = torch.from_numpy(g["x"]).to(DEV).requires_grad_(True)
    out = m(x)
    assert rel(out, g["out"]) <= 5e-5
    grads = torch.autograd.grad(out, [x, *m.parameters()], torch.from_numpy(g["cot"]).to(DEV))
    assert rel(grads[0], g["d_x"]) <= 1e-4
    for (name, _), gr in zip(m.named_parameters(), grads[1:]):
        # scanprep bias gradients of the golden are float32-autograd values through saturated
        # sigmoids and cancelling tap quotients (see test_scanprep_against_reference_golden)
        t = 5e-2 if name.startswith("scanprep.") else 1e-4
        assert rel(gr, g["dp_" + name]) <= t, (name, rel(gr, g["dp_" + name]))
    with torch.no_grad():
        o1, st = m(x[:, :13], return_state=True)
        o2, st2 = m(x[:, 13:], state=st, return_state=True)
        assert rel(torch.cat([o1, o2], 1), g["out_segmented"]) <= 5e-5
        assert rel(st2.scan.state, g["seg_state"]) <= 5e-5 and rel(st2.conv, g["seg_conv"]) <= 1e-6
        state, ys = None, []
        for t in range(3):
            y, state = m.step(x[:, t], state)
            ys.append(y)
        assert rel(torch.stack(ys, 1), g["out_steps"]) <= 5e-5


def test_stack_against_reference_golden(golden):
    """Two blocks (mixer + gelu FFN, final norm) with the reference's weights: forward, every
    gradient and three decode steps against the reference's own float32 results.  The bounds are
    those of the mixer golden: the GEMMs run in cuBLAS here and in the CPU BLAS there (different
    summation order), and the scan-preparation bias gradients of the golden carry the reference's
    float32 round-off."""
    g = golden("stack")
    cfg = sb.SLinOSSStackConfig.uniform(
        sb.SLinOSSBlockConfig(d_model=32, mixer=sb.SLinOSSMixerConfig(d_state=8, d_head=16, chunk_size=8),
                              ffn=sb.SLinOSSMLPConfig(kind="gelu", expand=2.0, multiple_of=8)), n_layers=2)
    stack = sb.SLinOSSStack(cfg)
    stack.load_state_dict({k[3:]: torch.from_numpy(v) for k, v in g.items() if k.startswith("sd_")})
    stack = stack.to(DEV)
    x = torch.from_numpy(g["x"]).to(DEV).requires_grad_(True)
    out = stack(x)
    assert rel(out, g["out"]) <= 5e-5, rel(out, g["out"])
    grads = torch.autograd.grad(out, [x, *stack.parameters()], torch.from_numpy(g["cot"]).to(DEV))
    assert rel(grads[0], g["d_x"]) <= 1e-4
    for (name, _), gr in zip(stack.named_parameters(), grads[1:]):
        t = 5e-2 if ".scanprep." in name else 2e-4
        assert rel(gr, g["dp_" + name]) <= t, (name, rel(gr, g["dp_" + name]))
    with torch.no_grad():
        state, ys = None, []
        for t in range(3):
            y, state = stack.step(x[:, t], state)
            ys.append(y)
        assert rel(torch.stack(ys, 1), g["out_steps"]) <= 5e-5


def test_fused_decode_step_and_graph_engine_follow_the_forward_pass():
    """``SLinOSSMixer.step`` (one launch per token between the two GEMMs) and the CUDA-graph engine
    against the reference's own step outputs and against a forward pass over the same tokens."""
    from slinoss_b200.engine import MixerDecodeEngine
    g = dict(np.load(Path(__file__).resolve().parent / "golden" / "mixer.npz"))
    m = _load_mixer(g)
    x = torch.from_numpy(g["x"]).to(DEV)
    with torch.no_grad():
        full = m(x)
        state, ys = None, []
        for t in range(x.shape[1]):
            y, state = m.step(x[:, t], state)
            ys.append(y)
        ys = torch.stack(ys, 1)
        assert rel(ys[:, :3], g["out_steps"]) <= 5e-5          # the reference's decode steps
        assert rel(ys, full) <= 5e-5                            # token by token == forward pass
        for use_graph in (False, True):
            eng = MixerDecodeEngine(m, x.shape[0], use_graph=use_graph)
            for rep in range(2):                                # reset() brings the engine back to token 0
                eng.reset()
                es = torch.stack([eng.step(x[:, t]).clone() for t in range(x.shape[1])], 1)
                assert rel(es, full) <= 5e-5, (use_graph, rep, rel(es, full))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_decode_step_at_the_benchmark_shape(dtype):
    """d_model 1024, 32 heads x 64, N 64 (the N = 64 fast path of the state update), bf16 and float32:
    the one-launch step against the separate-kernel backend call on the same state."""
    torch.manual_seed(3)
    m = sb.SLinOSSMixer(1024, d_state=64, expand=2, d_head=64, d_conv=4, chunk_size=64).to(DEV).to(dtype)
    x = torch.randn(3, 7, 1024, device=DEV, dtype=dtype)
    with torch.no_grad():
        full = m(x)
        state, ys = None, []
        for t in range(7):
            y, state = m.step(x[:, t], state)
            ys.append(y)
        assert rel(torch.stack(ys, 1), full) <= (5e-5 if dtype == torch.float32 else 2e-2)
        # the Protocol path (separate launches) from the same starting state gives the same token
        m2 = sb.SLinOSSMixer(1024, d_state=64, expand=2, d_head=64, d_conv=4, chunk_size=64).to(DEV).to(dtype)
        m2.load_state_dict(m.state_dict())
        m2.decode_backend.fused = False
        state2, ys2 = None, []
        for t in range(7):
            y, state2 = m2.step(x[:, t], state2)
            ys2.append(y)
        assert rel(torch.stack(ys2, 1), torch.stack(ys, 1)) <= (1e-5 if dtype == torch.float32 else 2e-2)
        assert rel(state2.scan.state, state.scan.state) <= (1e-5 if dtype == torch.float32 else 2e-2)


def test_mixer_bf16_close_to_float32():
    torch.manual_seed(0)
    m32 = sb.SLinOSSMixer(256, d_state=64, expand=2, d_head=64, chunk_size=64).to(DEV)
    m16 = sb.SLinOSSMixer(256, d_state=64, expand=2, d_head=64, chunk_size=64).to(DEV)
    m16.load_state_dict(m32.state_dict())
    m16 = m16.to(torch.bfloat16)
    x = torch.randn(2, 130, 256, device=DEV)
    a = m32(x)
    b = m16(x.to(torch.bfloat16))
    assert b.dtype == torch.bfloat16 and rel(b, a) <= 5e-2
    b.float().square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in m16.parameters())


def test_stack_trains_one_step():
    torch.manual_seed(0)
    cfg = sb.SLinOSSStackConfig.uniform(
        sb.SLinOSSBlockConfig(d_model=128, mixer=sb.SLinOSSMixerConfig(d_state=64, expand=1.0, d_head=64),
                              ffn=sb.SLinOSSMLPConfig(kind="gelu", expand=4.0)), n_layers=2)
    stack = sb.SLinOSSStack(cfg).to(DEV)
    opt = torch.optim.AdamW(stack.parameters(), lr=1e-3)
    x = torch.randn(2, 96, 128, device=DEV)
    losses = []
    for _ in range(3):
        loss = stack(x).square().mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert all(np.isfinite(losses)) and losses[-1] < losses[0]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixer_with_its_default_state_width_of_128(dtype):
    """``SLinOSSMixer``'s default ``d_state`` is 128: the two-pass tensor-core scan (16-bit) or the exact scan
    (float32) in the forward and backward pass, the generic loops of the fused decode step; token by token ==
    forward pass, and the 16-bit run against the same module in float32 on the exact kernels."""
    torch.manual_seed(11)
    m = sb.SLinOSSMixer(256, d_head=64, d_conv=4, chunk_size=64).to(DEV).to(dtype)     # d_state = 128, expand = 2
    assert m.d_state == 128
    x = torch.randn(2, 70, 256, device=DEV, dtype=dtype, requires_grad=True)
    out = m(x)
    (gx,) = torch.autograd.grad(out.float().square().sum(), x)
    with torch.no_grad():
        state, ys = None, []
        for t in range(6):
            y, state = m.step(x[:, t], state)
            ys.append(y)
    t_step = 5e-5 if dtype == torch.float32 else 2e-2
    assert rel(torch.stack(ys, 1), out[:, :6]) <= t_step
    # the same module in float32 on the exact kernels is the yardstick for the 16-bit run
    if dtype != torch.float32:
        m32 = sb.SLinOSSMixer(256, d_head=64, d_conv=4, chunk_size=64).to(DEV)
        m32.load_state_dict({k: v.float() for k, v in m.state_dict().items()})
        x32 = x.detach().float().requires_grad_()
        out32 = m32(x32)
        (gx32,) = torch.autograd.grad(out32.square().sum(), x32)
        assert rel(out, out32) <= 3e-2 and rel(gx, gx32) <= 6e-2
