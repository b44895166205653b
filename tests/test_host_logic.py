"""Host-side logic of the package on a GPU-less machine.

The tensor-level launchers of ``slinoss_b200._C`` are replaced by oracle-backed
fakes (tests/fake_cabi.py), so what is under test is everything above the C ABI:
validation and error messages, dtype policy, autograd wiring, state threading
and the composition of the mixer - checked against golden vectors of the
reference's own mixer.
"""

import numpy as np
import pytest
import torch

import slinoss_b200 as sb
from slinoss_b200.ops.v2x2ssd import v2x2ssd, v2x2ssd_cute, v2x2ssd_decode
from slinoss_b200.synthetic import make_scan_case
from tests.fake_cabi import FakeCABI


@pytest.fixture
def fake(monkeypatch):
    return FakeCABI().install(monkeypatch)


def rel(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def test_cpu_tensors_are_rejected_without_fake():
    case = make_scan_case(1, 1, 4, 2, 2)
    with pytest.raises(ValueError, match="require CUDA tensors"):
        v2x2ssd(*case.tensors(), chunk_size=4)


def test_validation_messages(fake):
    c = make_scan_case(1, 2, 4, 2, 2)
    with pytest.raises(ValueError, match=r"U must be \(batch,heads,T,P\)"):
        v2x2ssd(c.U[0], c.M, c.K, c.B, c.C)
    with pytest.raises(ValueError, match="must be contiguous"):
        v2x2ssd(c.U.transpose(2, 3), c.M, c.K, c.B, c.C)
    with pytest.raises(ValueError, match="passed together"):
        v2x2ssd(*c.tensors(), B_prev=torch.zeros(1, 2, 4))
    with pytest.raises(ValueError, match="chunk_size must be positive"):
        v2x2ssd(*c.tensors(), chunk_size=0)
    with pytest.raises(ValueError, match="only float32 compute"):
        v2x2ssd(*c.tensors(), compute_dtype=torch.float64)
    with pytest.raises(ValueError, match="group dimension must divide heads"):
        v2x2ssd(c.U, c.M, c.K, torch.zeros(1, 3, 4, 4), torch.zeros(1, 3, 4, 4))
    with pytest.raises(ValueError, match="initial_states must be"):
        v2x2ssd(*c.tensors(), initial_states=torch.zeros(1, 2, 2, 2))
    assert not fake.calls  # nothing was launched


def test_zero_length_returns_carried_state(fake):
    c = make_scan_case(2, 2, 0, 4, 3, streaming=True, with_init=True)
    Y, fin, Bl, Ul = v2x2ssd(*c.tensors(), initial_states=c.initial_states, B_prev=c.B_prev,
                             U_prev=c.U_prev)
    assert Y.shape == (2, 2, 0, 4) and torch.equal(fin, c.initial_states)
    assert torch.equal(Bl, c.B_prev) and torch.equal(Ul, c.U_prev) and not fake.calls


def test_dtype_policy_and_launch_arguments(fake):
    c = make_scan_case(1, 4, 9, 4, 2, groups=2, dtype=torch.bfloat16)
    Y = v2x2ssd_cute(c.U, c.M, c.K, c.B, c.C, chunk_size=4)
    assert Y.dtype == torch.bfloat16
    name, info = fake.calls[-1]
    assert name == "scan_fwd" and info["io"] == torch.bfloat16 and info["chunk_size"] == 4
    assert info["shapes"][3] == (1, 2, 9, 4)
    out = v2x2ssd(*c.tensors(), output_dtype=torch.float32)
    assert out[0].dtype == out[1].dtype == out[2].dtype == torch.float32


def test_autograd_matches_reference_gradients(fake, golden):
    g = golden("scan_grad")
    t = lambda k: torch.from_numpy(g[k]).float().requires_grad_(True)
    ins = {k: t(k) for k in ("U", "M", "K", "B", "C", "initial_states", "B_prev", "U_prev")}
    Y, fin, Bl, Ul = v2x2ssd(ins["U"], ins["M"], ins["K"], ins["B"], ins["C"],
                             chunk_size=int(g["chunk"]), initial_states=ins["initial_states"],
                             B_prev=ins["B_prev"], U_prev=ins["U_prev"])
    assert rel(Y.detach(), g["Y"]) < 1e-5
    dBl, dUl = torch.randn_like(Bl), torch.randn_like(Ul)
    grads = torch.autograd.grad([Y, fin, Bl, Ul], list(ins.values()),
                                [torch.from_numpy(g["dY"]).float(),
                                 torch.from_numpy(g["d_final_state"]).float(), dBl, dUl])
    for (name, _), gr in zip(ins.items(), grads):
        want = g["d" + name].copy()
        if name == "B":
            want[:, :, -1] += dBl.numpy()   # gradients of B_last / U_last land on the last row
        if name == "U":
            want[:, :, -1] += dUl.numpy()
        assert rel(gr, want) < 1e-5, name


def test_decode_equals_forward_tokenwise(fake):
    c = make_scan_case(2, 2, 5, 4, 3, streaming=True, with_init=True)
    Y, fin, _, _ = v2x2ssd(*c.tensors(), chunk_size=4, initial_states=c.initial_states,
                           B_prev=c.B_prev, U_prev=c.U_prev)
    state, bp, up = c.initial_states.clone(), c.B_prev, c.U_prev
    for t in range(5):
        y, state, bp, up = v2x2ssd_decode(c.U[:, :, t], c.M[:, :, t], c.K[:, :, t], c.B[:, :, t],
                                          c.C[:, :, t], state=state, B_prev=bp, U_prev=up,
                                          inplace=True)
        assert rel(y, Y[:, :, t]) < 1e-5
    assert rel(state, fin) < 1e-5


def _load_mixer(g, **kw):
    m = sb.SLinOSSMixer(32, d_state=8, expand=2, d_head=16, d_conv=4, chunk_size=8, bc_groups=2, **kw)
    sd = {k[3:]: torch.from_numpy(v) for k, v in g.items() if k.startswith("sd_")}
    assert set(sd) == set(m.state_dict())       # same state_dict keys as the reference mixer
    m.load_state_dict(sd)
    return m


def test_mixer_forward_backward_matches_reference_golden(fake, golden):
    g = golden("mixer")
    m = _load_mixer(g)
    x = torch.from_numpy(g["x"]).requires_grad_(True)
    out = m(x)
    assert rel(out.detach(), g["out"]) < 2e-5
    grads = torch.autograd.grad(out, [x, *m.parameters()], torch.from_numpy(g["cot"]))
    assert rel(grads[0], g["d_x"]) < 1e-4
    for (name, _), gr in zip(m.named_parameters(), grads[1:]):
        assert rel(gr, g["dp_" + name]) < 1e-4, name
    launched = [n for n, _ in fake.calls]
    assert launched.count("scanprep_conv_fwd") == 1   # conv + scanprep went out as ONE fused call
    assert fake.calls[0][1]["fused_conv"]


def test_mixer_streaming_and_decode_match_reference_golden(fake, golden):
    g = golden("mixer")
    m = _load_mixer(g)
    x = torch.from_numpy(g["x"])
    with torch.no_grad():
        o1, st = m(x[:, :13], return_state=True)
        o2, st2 = m(x[:, 13:], state=st, return_state=True)
        assert rel(torch.cat([o1, o2], 1), g["out_segmented"]) < 2e-5
        assert rel(st2.scan.state, g["seg_state"]) < 2e-5 and rel(st2.conv, g["seg_conv"]) < 1e-6
        state, ys = None, []
        for t in range(3):
            y, state = m.step(x[:, t], state)
            ys.append(y)
        assert rel(torch.stack(ys, 1), g["out_steps"]) < 2e-5
        assert state.scan.state.dtype == torch.float32


def test_injected_backends_use_the_protocol_path(fake, golden):
    from slinoss_b200.layers import B200CConv1dBackend, ScanInputs

    seen = {}

    class SpyScan:
        def __call__(self, inputs: ScanInputs, *, chunk_size, state=None, return_state=None):
            seen["shapes"] = {k: tuple(getattr(inputs, k).shape) for k in "UMKBC"}
            seen["chunk"] = chunk_size
            return torch.zeros_like(inputs.U)

    class SpyConv(B200CConv1dBackend):
        def __call__(self, owner, x, conv_state):
            seen["conv_in"] = tuple(x.shape)
            return super().__call__(owner, x, conv_state)

    m = _load_mixer(golden("mixer"), scan_backend=SpyScan(), cconv_backend=SpyConv())
    m(torch.randn(2, 6, 32))
    assert seen["conv_in"] == (2, 6, 64) and seen["chunk"] == 8
    assert seen["shapes"] == {"U": (2, 4, 6, 16), "M": (2, 4, 6, 2), "K": (2, 4, 6, 2, 2),
                              "B": (2, 2, 6, 16), "C": (2, 2, 6, 16)}
    kinds = [(n, i.get("fused_conv")) for n, i in fake.calls if n == "scanprep_conv_fwd"]
    assert kinds == [("scanprep_conv_fwd", True), ("scanprep_conv_fwd", False)]


def test_stack_forward_and_step_agree(fake):
    torch.manual_seed(0)
    cfg = sb.SLinOSSStackConfig.uniform(
        sb.SLinOSSBlockConfig(d_model=32, mixer=sb.SLinOSSMixerConfig(d_state=4, d_head=8, chunk_size=4),
                              ffn=sb.SLinOSSMLPConfig(kind="gelu", expand=2.0, multiple_of=8)), n_layers=2)
    stack = sb.SLinOSSStack(cfg).eval()
    x = torch.randn(2, 5, 32)
    with torch.no_grad():
        full = stack(x)
        state, ys = None, []
        for t in range(5):
            y, state = stack.step(x[:, t], state)
            ys.append(y)
    assert rel(torch.stack(ys, 1), full) < 1e-4


def test_measure_module_imports_without_a_gpu_and_refuses_to_run(monkeypatch):
    from slinoss_b200 import measure
    assert measure.nbytes(torch.zeros(3, 4), None, torch.zeros(2, dtype=torch.bfloat16)) == 48 + 4
    peak, kind = measure.hbm_peak()
    assert peak > 1000 and kind in ("measured", "fallback")
    monkeypatch.setattr("sys.argv", ["measure"])
    with pytest.raises(SystemExit, match="no CPU path"):
        measure.main()


def test_transition_product_matches_the_running_complex_product():
    import torch
    from slinoss_b200.ops.v2x2ssd.sequence_parallel import _scale_state, transition_product
    g = torch.Generator().manual_seed(0)
    r = 0.8 + 0.2 * torch.rand(2, 3, 500, generator=g, dtype=torch.float64)
    th = (2 * torch.rand(2, 3, 500, generator=g, dtype=torch.float64) - 1) * torch.pi
    M = torch.stack((r * torch.cos(th), r * torch.sin(th)), -1)
    want = torch.view_as_complex(M.contiguous()).prod(-1)            # 0.9^500 ~ 1e-23: still a normal float64
    got = torch.view_as_complex(transition_product(M.float()).double())
    assert ((got - want).abs() / want.abs()).max() < 1e-4             # float32 inputs, float64 accumulation
    # complex scalar times interleaved state
    z = torch.randn(2, 3, 4, 10, generator=g)
    pi = torch.view_as_complex(torch.randn(2, 3, 2, generator=g))
    out = _scale_state(pi, z)
    ref = torch.view_as_real(torch.view_as_complex(z.reshape(2, 3, 4, 5, 2)) * pi[..., None, None]).reshape(z.shape)
    assert torch.equal(out, ref)
