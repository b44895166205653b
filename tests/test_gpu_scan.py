"""Parity of the CUDA scan (forward, backward, decode) with the oracle.

Every case runs through the public op, i.e. through the C ABI.  The oracle is
evaluated in float64 on the very same (already rounded) inputs; the bar is
``max|got-want| / max|want| <= 1e-5`` for float32 and ``<= 2e-2`` for bf16/fp16,
per tensor, outputs and gradients alike.
"""

import numpy as np
import pytest
import torch

from oracle import scan_np
from slinoss_b200.ops.v2x2ssd import v2x2ssd, v2x2ssd_cute, v2x2ssd_decode
from slinoss_b200.synthetic import make_scan_case
from tests.util import n64, rel, tol

pytestmark = pytest.mark.gpu

DEV = "cuda"

# (batch, heads, groups, T, P, N, chunk, streaming, init)
SHAPES = [
    (2, 4, 4, 256, 64, 32, 64, False, False),   # config 0
    (2, 4, 2, 43, 16, 8, 16, True, True),       # grouped, ragged, streaming
    (1, 2, 2, 1, 5, 3, 4, True, True),          # single token, odd sizes
    (2, 2, 1, 17, 33, 5, 8, False, True),       # P not a multiple of 32, N odd
    (1, 2, 2, 70, 64, 128, 64, True, False),    # N = 128 (the mixer default d_state)
    (1, 3, 3, 33, 130, 8, 32, True, True),      # P > 64: several P tiles per head
    (1, 2, 2, 63, 64, 64, 64, False, False),    # chunk - 1
    (1, 2, 2, 64, 64, 64, 64, False, False),    # chunk
    (1, 2, 2, 65, 64, 64, 64, True, True),      # chunk + 1
]


def _oracle_fwd(case):
    return scan_np.v2x2ssm(*[n64(t) for t in case.tensors()], initial_states=n64(case.initial_states),
                           B_prev=n64(case.B_prev), U_prev=n64(case.U_prev))


def _run(case, chunk, path, **kw):
    c = case.to(DEV)
    return v2x2ssd(*c.tensors(), chunk_size=chunk, initial_states=c.initial_states,
                   B_prev=c.B_prev, U_prev=c.U_prev, path=path, **kw)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_forward_simt(shape, dtype):
    b, h, g, T, P, N, L, streaming, init = shape
    case = make_scan_case(b, h, T, P, N, groups=g, dtype=dtype, seed=T + P, streaming=streaming,
                          with_init=init)
    Y, fin, Bl, Ul = _run(case, L, "simt")
    wY, wfin, _, _ = _oracle_fwd(case)
    assert Y.dtype == dtype and fin.dtype == dtype
    assert rel(Y, wY) <= tol(dtype), rel(Y, wY)
    assert rel(fin, wfin) <= tol(dtype)
    assert torch.equal(Bl.cpu(), case.B[:, :, -1]) and torch.equal(Ul.cpu(), case.U[:, :, -1])


def test_forward_config0_against_reference_golden(golden):
    g = golden("scan_c0")
    case = make_scan_case(2, 4, 256, 64, 32, seed=0)
    Y, fin, _, _ = _run(case, 64, "simt")
    assert rel(Y, g["Y"]) <= 1e-5 and rel(fin, g["final_state"]) <= 1e-5
    assert rel(Y, g["Y_seq_fp64"]) <= 1e-5


def test_float32_state_output_on_request():
    case = make_scan_case(1, 2, 20, 8, 4, dtype=torch.bfloat16)
    out = _run(case, 8, "simt", output_dtype=torch.float32)
    assert all(t.dtype == torch.float32 for t in out)


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_backward_simt(shape, dtype):
    b, h, g, T, P, N, L, streaming, init = shape
    case = make_scan_case(b, h, T, P, N, groups=g, dtype=dtype, seed=7 * T + N, streaming=streaming,
                          with_init=init)
    c = case.to(DEV)
    names = ["U", "M", "K", "B", "C"] + (["initial_states"] if init else []) \
        + (["B_prev", "U_prev"] if streaming else [])
    leaves = {k: getattr(c, k).clone().requires_grad_(True) for k in names}
    out = v2x2ssd(leaves["U"], leaves["M"], leaves["K"], leaves["B"], leaves["C"], chunk_size=L,
                  initial_states=leaves.get("initial_states"), B_prev=leaves.get("B_prev"),
                  U_prev=leaves.get("U_prev"), path="simt")
    gen = torch.Generator().manual_seed(5)
    d_final = torch.randn(out[1].shape, generator=gen).to(dtype)
    grads = torch.autograd.grad([out[0], out[1]], list(leaves.values()), [c.dY, d_final.to(DEV)])
    want = scan_np.v2x2ssd_bwd(*[n64(t) for t in case.tensors()], n64(case.dY),
                               d_final_state=n64(d_final), initial_states=n64(case.initial_states),
                               B_prev=n64(case.B_prev), U_prev=n64(case.U_prev))
    for name, gr in zip(names, grads):
        assert gr.dtype == leaves[name].dtype
        assert rel(gr, want[name]) <= tol(dtype), (name, rel(gr, want[name]))


def test_backward_against_reference_golden(golden):
    g = golden("scan_grad")
    t = lambda k: torch.from_numpy(g[k]).float().to(DEV).requires_grad_(True)
    names = ("U", "M", "K", "B", "C", "initial_states", "B_prev", "U_prev")
    ins = {k: t(k) for k in names}
    Y, fin, _, _ = v2x2ssd(ins["U"], ins["M"], ins["K"], ins["B"], ins["C"], chunk_size=int(g["chunk"]),
                           initial_states=ins["initial_states"], B_prev=ins["B_prev"],
                           U_prev=ins["U_prev"], path="simt")
    assert rel(Y, g["Y"]) <= 1e-5 and rel(fin, g["final_state"]) <= 1e-5
    grads = torch.autograd.grad([Y, fin], list(ins.values()),
                                [torch.from_numpy(g["dY"]).float().to(DEV),
                                 torch.from_numpy(g["d_final_state"]).float().to(DEV)])
    for name, gr in zip(names, grads):
        assert rel(gr, g["d" + name]) <= 1e-5, (name, rel(gr, g["d" + name]))


def test_gradients_of_b_last_and_u_last_reach_the_last_row():
    case = make_scan_case(1, 2, 9, 4, 3).to(DEV)
    U, B = case.U.clone().requires_grad_(True), case.B.clone().requires_grad_(True)
    out = v2x2ssd(U, case.M, case.K, B, case.C, chunk_size=4, path="simt")
    gU, gB = torch.autograd.grad([out[2].sum() + out[3].sum()], [U, B])
    assert torch.all(gU[:, :, -1] == 1) and torch.all(gU[:, :, :-1] == 0)
    assert torch.all(gB[:, :, -1] == 1) and torch.all(gB[:, :, :-1] == 0)


def test_forward_is_deterministic_and_leaves_inputs_untouched():
    case = make_scan_case(2, 4, 100, 64, 64, dtype=torch.bfloat16).to(DEV)
    before = [t.clone() for t in case.tensors()]
    a = v2x2ssd(*case.tensors(), chunk_size=64, path="simt")
    b = v2x2ssd(*case.tensors(), chunk_size=64, path="simt")
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert all(torch.equal(x, y) for x, y in zip(before, case.tensors()))


def test_segmented_equals_full_pass():
    case = make_scan_case(2, 2, 150, 64, 64, seed=9, streaming=True, with_init=True).to(DEV)
    kw = dict(chunk_size=64, path="simt")
    Y, fin, _, _ = v2x2ssd(*case.tensors(), initial_states=case.initial_states, B_prev=case.B_prev,
                           U_prev=case.U_prev, **kw)
    cut = 77
    sl = lambda t, a, b: t[:, :, a:b].contiguous()
    Y1, f1, b1, u1 = v2x2ssd(*[sl(t, 0, cut) for t in case.tensors()],
                             initial_states=case.initial_states, B_prev=case.B_prev,
                             U_prev=case.U_prev, **kw)
    Y2, f2, _, _ = v2x2ssd(*[sl(t, cut, 150) for t in case.tensors()], initial_states=f1, B_prev=b1,
                           U_prev=u1, **kw)
    assert rel(torch.cat([Y1, Y2], 2), Y) <= 1e-5 and rel(f2, fin) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("N", [64, 128])           # one / two float4 of a state row per lane
def test_decode_equals_forward_tokenwise(dtype, N):
    case = make_scan_case(3, 4, 6, 64, N, groups=2, dtype=dtype, streaming=True, with_init=True)
    wY, wfin, _, _ = _oracle_fwd(case)
    c = case.to(DEV)
    state, bp, up = c.initial_states.clone(), c.B_prev, c.U_prev
    for t in range(6):
        y, state, bp, up = v2x2ssd_decode(c.U[:, :, t], c.M[:, :, t], c.K[:, :, t], c.B[:, :, t],
                                          c.C[:, :, t], state=state, B_prev=bp, U_prev=up,
                                          inplace=(t % 2 == 0))
        assert rel(y, wY[:, :, t]) <= tol(dtype)
    assert state.dtype == torch.float32 and rel(state, wfin) <= 1e-5


def test_decode_odd_sizes():
    case = make_scan_case(2, 3, 1, 5, 3, streaming=True, with_init=True)
    wY, wfin, _, _ = _oracle_fwd(case)
    c = case.to(DEV)
    y, st, _, _ = v2x2ssd_decode(c.U[:, :, 0], c.M[:, :, 0], c.K[:, :, 0], c.B[:, :, 0], c.C[:, :, 0],
                                 state=c.initial_states, B_prev=c.B_prev, U_prev=c.U_prev)
    assert rel(y, wY[:, :, 0]) <= 1e-5 and rel(st, wfin) <= 1e-5


def test_full_size_config1_properties():
    """Config 1 (batch 8, heads 16, T 4096, P 64, N 64, bf16): too large for the CPU
    oracle, so it is checked through size-independent properties: a slice of streams
    against the oracle, exact homogeneity in U, and the segmented == full identity."""
    case = make_scan_case(8, 16, 4096, 64, 64, dtype=torch.bfloat16, seed=0).to(DEV)
    Y, fin, _, _ = v2x2ssd(*case.tensors(), chunk_size=64, output_dtype=torch.float32)
    assert torch.isfinite(Y).all() and torch.isfinite(fin).all()
    # one (batch, head) stream, first 512 tokens, against the float64 oracle
    sl = lambda t: t[3:4, 5:6, :512].contiguous()
    wY, _, _, _ = scan_np.v2x2ssm(*[n64(sl(t)) for t in case.tensors()])
    assert rel(Y[3:4, 5:6, :512], wY) <= 2e-2
    # doubling U doubles Y exactly (power-of-two scaling commutes with every rounding)
    Y2, fin2, _, _ = v2x2ssd(case.U * 2, case.M, case.K, case.B, case.C, chunk_size=64,
                             output_dtype=torch.float32)
    assert torch.equal(Y2, Y * 2) and torch.equal(fin2, fin * 2)
    # two segments with the carried state reproduce the single pass
    cut = 2048 + 64
    s1 = [t[:, :, :cut].contiguous() for t in case.tensors()]
    s2 = [t[:, :, cut:].contiguous() for t in case.tensors()]
    Ya, fa, ba, ua = v2x2ssd(*s1, chunk_size=64, output_dtype=torch.float32)
    Yb, fb, _, _ = v2x2ssd(*s2, chunk_size=64, initial_states=fa, B_prev=ba.to(torch.bfloat16),
                           U_prev=ua.to(torch.bfloat16), output_dtype=torch.float32)
    assert rel(torch.cat([Ya, Yb], 2), Y) <= 2e-2 and rel(fb, fin) <= 2e-2


def test_full_size_config1_forward_and_backward_of_whole_streams():
    """The configuration the benchmark times (batch 8, heads 16, T 4096, bf16, 128 CTAs x 64 chunks):
    Y and all five gradients of three whole (batch, head) streams from different batch entries
    against the float64 oracle, which handles single streams of that length in seconds."""
    case = make_scan_case(8, 16, 4096, 64, 64, dtype=torch.bfloat16, seed=0)
    c = case.to(DEV)
    leaves = [t.clone().requires_grad_(True) for t in c.tensors()]
    Y = v2x2ssd_cute(*leaves, chunk_size=64)
    grads = torch.autograd.grad(Y, leaves, c.dY)
    from slinoss_b200 import _C
    assert _C.device_status() == 0
    for (b, h) in ((0, 0), (3, 5), (7, 15)):
        sl = lambda t: t[b:b + 1, h:h + 1].contiguous()
        args = [n64(sl(t)) for t in case.tensors()]
        wY = scan_np.v2x2ssm(*args)[0]
        want = scan_np.v2x2ssd_bwd(*args, n64(sl(case.dY)))
        assert rel(sl(Y), wY) <= 2e-2, (b, h, rel(sl(Y), wY))
        for name, gr in zip("UMKBC", grads):
            assert torch.isfinite(sl(gr)).all(), (b, h, name)
            assert rel(sl(gr), want[name]) <= 2e-2, (b, h, name, rel(sl(gr), want[name]))


# ---- tensor-core (tcgen05) path: P = 64, N = 64 or 128, 16-bit operands -------------------------------
TC_SHAPES = [
    (1, 1, 1, 64, False, False),
    (2, 4, 2, 1, True, True),
    (1, 2, 2, 63, False, True),
    (1, 2, 2, 65, True, False),
    (2, 4, 4, 200, True, True),
    (1, 4, 1, 333, False, False),
    (2, 2, 2, 1024, True, True),
]


@pytest.mark.parametrize("N", [64, 128])           # 128: two passes over the column blocks of B and C
@pytest.mark.parametrize("shape", TC_SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_forward_tensor_core_path(shape, dtype, N):
    from slinoss_b200 import _C
    b, h, g, T, streaming, init = shape
    case = make_scan_case(b, h, T, 64, N, groups=g, dtype=dtype, seed=3 * T + b, streaming=streaming,
                          with_init=init)
    Y, fin, _, _ = _run(case, 64, "tc", output_dtype=torch.float32)
    wY, wfin, _, _ = _oracle_fwd(case)
    assert _C.device_status() == 0
    assert rel(Y, wY) <= 2e-2, rel(Y, wY)
    assert rel(fin, wfin) <= 2e-2, rel(fin, wfin)
    Yh = _run(case, 64, "tc")[0]
    assert Yh.dtype == dtype and rel(Yh, wY) <= 2e-2


def test_tensor_core_path_agrees_with_exact_path_on_reference_test_distribution():
    """|m| in [0.6, 0.95] (the reference's own test generator): strong decay inside a chunk."""
    import math
    gen = torch.Generator().manual_seed(0)
    b, h, T = 2, 3, 300
    radius = 0.6 + 0.35 * torch.rand(b, h, T, generator=gen)
    angle = (2 * torch.rand(b, h, T, generator=gen) - 1) * math.pi
    M = torch.stack((radius * torch.cos(angle), radius * torch.sin(angle)), -1).to(DEV)
    K = (0.1 * torch.randn(b, h, T, 2, 2, generator=gen)).to(DEV)
    U = torch.randn(b, h, T, 64, generator=gen).to(torch.bfloat16).to(DEV)
    B = (0.1 * torch.randn(b, h, T, 128, generator=gen)).to(torch.bfloat16).to(DEV)
    C = (0.1 * torch.randn(b, h, T, 128, generator=gen)).to(torch.bfloat16).to(DEV)
    a = v2x2ssd(U, M, K, B, C, chunk_size=64, path="tc", output_dtype=torch.float32)
    e = v2x2ssd(U, M, K, B, C, chunk_size=64, path="simt", output_dtype=torch.float32)
    assert rel(a[0], e[0]) <= 2e-2 and rel(a[1], e[1]) <= 2e-2
    wY, wfin, _, _ = scan_np.v2x2ssm(*[n64(t) for t in (U, M, K, B, C)])
    assert rel(a[0], wY) <= 2e-2 and rel(a[1], wfin) <= 2e-2


def test_auto_path_prefers_tensor_cores_and_falls_back_for_float32():
    from slinoss_b200 import _C
    assert _C.workspace_bytes(_C.WS_SCAN_FWD, 1, 1, 1, 64, 64, 64, 64, torch.bfloat16, "auto") == 0
    assert _C.workspace_bytes(_C.WS_SCAN_FWD, 1, 1, 1, 64, 64, 128, 64, torch.bfloat16, "auto") > 0
    odd = make_scan_case(1, 1, 70, 64, 96, dtype=torch.bfloat16)      # neither 64 nor 128 state columns
    with pytest.raises(RuntimeError, match="unsupported"):
        _run(odd, 64, "tc")
    assert rel(_run(odd, 64, "auto", output_dtype=torch.float32)[0], _oracle_fwd(odd)[0]) <= 2e-2
    case = make_scan_case(1, 2, 70, 64, 64, dtype=torch.float32)
    with pytest.raises(RuntimeError, match="unsupported"):
        _run(case, 64, "tc")
    Y = _run(case, 64, "auto")[0]
    assert rel(Y, _oracle_fwd(case)[0]) <= 1e-5


# (batch, heads, T, initial state, gradient of the final state, groups of B/C, carried B_prev / U_prev)
TC_BWD_SHAPES = [
    (1, 1, 64, False, False, 1, False),
    (1, 2, 1, True, True, 2, False),
    (2, 2, 63, False, True, 2, False),
    (1, 3, 65, True, True, 3, False),
    (2, 4, 200, True, False, 4, False),
    (1, 2, 333, False, False, 2, False),
    (1, 2, 1024, True, True, 2, False),
    (2, 4, 200, True, True, 2, False),      # grouped B/C: two heads share a row of B and C
    (1, 4, 333, False, False, 1, False),    # one group for all heads
    (1, 6, 130, True, True, 3, False),
    (1, 2, 1, True, True, 2, True),         # carried taps: the token before the sequence
    (2, 2, 65, False, False, 2, True),
    (2, 4, 200, True, True, 2, True),       # ... grouped as well
    (1, 3, 333, True, False, 1, True),
]


@pytest.mark.parametrize("N", [64, 128])
@pytest.mark.parametrize("shape", TC_BWD_SHAPES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_backward_tensor_core_path(shape, dtype, N):
    from slinoss_b200 import _C
    b, h, T, init, with_dfinal, g, streaming = shape
    case = make_scan_case(b, h, T, 64, N, groups=g, dtype=dtype, seed=11 * T + h, with_init=init,
                          streaming=streaming)
    c = case.to(DEV)
    names = ["U", "M", "K", "B", "C"] + (["initial_states"] if init else []) \
        + (["B_prev", "U_prev"] if streaming else [])
    leaves = {k: getattr(c, k).clone().requires_grad_(True) for k in names}
    out = v2x2ssd(leaves["U"], leaves["M"], leaves["K"], leaves["B"], leaves["C"], chunk_size=64,
                  initial_states=leaves.get("initial_states"), B_prev=leaves.get("B_prev"),
                  U_prev=leaves.get("U_prev"), path="tc")
    gen = torch.Generator().manual_seed(5)
    d_final = torch.randn(out[1].shape, generator=gen).to(dtype) if with_dfinal else None
    outs, cots = [out[0]], [c.dY]
    if with_dfinal:
        outs.append(out[1]); cots.append(d_final.to(DEV))
    grads = torch.autograd.grad(outs, list(leaves.values()), cots)
    assert _C.device_status() == 0
    want = scan_np.v2x2ssd_bwd(*[n64(t) for t in case.tensors()], n64(case.dY),
                               d_final_state=n64(d_final), initial_states=n64(case.initial_states),
                               B_prev=n64(case.B_prev), U_prev=n64(case.U_prev))
    for name, gr in zip(names, grads):
        assert torch.isfinite(gr).all(), name
        assert rel(gr, want[name]) <= 2e-2, (name, rel(gr, want[name]))


def test_segmented_training_on_the_tensor_core_path_matches_the_single_pass():
    """Two segments chained through (final_state, B_last, U_last): the gradients that flow back through
    the carried state and the carried taps must add up to those of the single pass."""
    case = make_scan_case(2, 4, 333, 64, 64, groups=2, dtype=torch.bfloat16, seed=17).to(DEV)
    cut = 150

    def run(segmented):
        lv = [t.clone().requires_grad_(True) for t in case.tensors()]
        if not segmented:
            Y = v2x2ssd_cute(*lv, chunk_size=64, path="tc")
        else:
            a = [t[:, :, :cut].contiguous() for t in lv]
            b = [t[:, :, cut:].contiguous() for t in lv]
            Ya, fa, ba, ua = v2x2ssd_cute(*a, chunk_size=64, path="tc", return_state=True,
                                          output_dtype=torch.float32)
            Yb = v2x2ssd_cute(*b, chunk_size=64, path="tc", initial_states=fa,
                              B_prev=ba.to(torch.bfloat16), U_prev=ua.to(torch.bfloat16),
                              output_dtype=torch.float32)
            Y = torch.cat([Ya, Yb], 2)
        return Y, torch.autograd.grad(Y, lv, case.dY.to(Y.dtype))

    Yf, gf = run(False)
    Ys, gs = run(True)
    assert rel(Ys, Yf) <= 2e-2
    for name, a, b in zip("UMKBC", gs, gf):
        assert rel(a, b) <= 2e-2, (name, rel(a, b))
    want = scan_np.v2x2ssd_bwd(*[n64(t) for t in case.tensors()], n64(case.dY))
    for name, a in zip("UMKBC", gs):
        assert rel(a, want[name]) <= 2e-2, (name, rel(a, want[name]))


def test_backward_tensor_core_agrees_with_exact_path_at_strong_decay():
    import math
    gen = torch.Generator().manual_seed(1)
    b, h, T = 1, 2, 300
    radius = 0.6 + 0.35 * torch.rand(b, h, T, generator=gen)
    angle = (2 * torch.rand(b, h, T, generator=gen) - 1) * math.pi
    M = torch.stack((radius * torch.cos(angle), radius * torch.sin(angle)), -1).to(DEV)
    K = (0.1 * torch.randn(b, h, T, 2, 2, generator=gen)).to(DEV)
    mk = lambda *s: torch.randn(*s, generator=gen).to(torch.bfloat16).to(DEV)
    U, B, C, dY = mk(b, h, T, 64), 0.1 * mk(b, h, T, 128), 0.1 * mk(b, h, T, 128), mk(b, h, T, 64)
    res = {}
    for path in ("tc", "simt"):
        lv = [x.clone().requires_grad_(True) for x in (U, M, K, B, C)]
        Y = v2x2ssd_cute(*lv, chunk_size=64, path=path)
        res[path] = torch.autograd.grad(Y, lv, dY)
    for name, a, e in zip("UMKBC", res["tc"], res["simt"]):
        assert rel(a, e) <= 2e-2, (name, rel(a, e))
    want = scan_np.v2x2ssd_bwd(*[n64(t) for t in (U, M, K, B, C)], n64(dY))
    for name, a in zip("UMKBC", res["tc"]):
        assert rel(a, want[name]) <= 2e-2, (name, rel(a, want[name]))


@pytest.mark.parametrize("N", [64, 128])
def test_saved_chunk_states_and_recompute_give_the_same_gradients(N):
    case = make_scan_case(2, 2, 300, 64, N, dtype=torch.bfloat16, seed=2, with_init=True).to(DEV)
    res = []
    for keep in (True, False):
        lv = [x.clone().requires_grad_(True) for x in (*case.tensors(), case.initial_states)]
        Y = v2x2ssd_cute(*lv[:5], chunk_size=64, initial_states=lv[5], path="tc", save_chunk_states=keep)
        res.append(torch.autograd.grad(Y, lv, case.dY))
    for a, b in zip(*res):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype,lo,hi,bar_dm", [(torch.bfloat16, 0.3, 0.6, 2e-2), (torch.float16, 0.05, 0.3, 2e-2),
                                                (torch.bfloat16, 0.05, 0.3, 1e-1), (torch.float16, 0.01, 0.1, 5e-2)])
def test_tensor_core_path_at_small_transition_radius(dtype, lo, hi, bar_dm):
    """Far below the model's operating region (|m| >= r_min = 0.8 by default): everything stays finite, Y and
    the gradients of U, K, B, C keep the 16-bit bar; dM = S / conj(m) amplifies the operands' rounding by 1/|m|,
    so with bfloat16 operands its bar holds down to |m| of about 0.3 and loosens below (float16 keeps it)."""
    import math
    gen = torch.Generator().manual_seed(1)
    b, h, T = 1, 2, 300
    radius = lo + (hi - lo) * torch.rand(b, h, T, generator=gen)
    angle = (2 * torch.rand(b, h, T, generator=gen) - 1) * math.pi
    M = torch.stack((radius * torch.cos(angle), radius * torch.sin(angle)), -1).to(DEV)
    K = (0.1 * torch.randn(b, h, T, 2, 2, generator=gen)).to(DEV)
    mk = lambda *s: torch.randn(*s, generator=gen).to(dtype).to(DEV)
    U, B, C, dY = mk(b, h, T, 64), 0.1 * mk(b, h, T, 128), 0.1 * mk(b, h, T, 128), mk(b, h, T, 64)
    lv = [x.clone().requires_grad_(True) for x in (U, M, K, B, C)]
    Y = v2x2ssd_cute(*lv, chunk_size=64, path="tc")
    grads = torch.autograd.grad(Y, lv, dY)
    wY = scan_np.v2x2ssm(*[n64(t) for t in (U, M, K, B, C)])[0]
    want = scan_np.v2x2ssd_bwd(*[n64(t) for t in (U, M, K, B, C)], n64(dY))
    assert rel(Y, wY) <= 2e-2
    for name, g in zip("UMKBC", grads):
        assert torch.isfinite(g).all(), name
        assert rel(g, want[name]) <= (bar_dm if name == "M" else 2e-2), (name, rel(g, want[name]))
