"""The C-ABI calls inside CUDA-graph capture.

The reference promises that its ops can be captured after one warm call (their launchers
use torch's current stream and allocate nothing that outlives the call).  The library's
entry points allocate nothing at all and take the stream as an argument, so the Python
launchers can be captured with ``torch.cuda.graph``: output and workspace tensors then
come from the graph's private pool.  Each test captures one call sequence, overwrites
the static input tensors with a second problem, replays, and compares with eager calls
on that second problem (bit-exact: the same kernels run on the same bits).
"""

import pytest
import torch

from slinoss_b200 import _C
from slinoss_b200.synthetic import make_scan_case
from tests.util import rel

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _capture(fn):
    """One warm call on a side stream, then the capture of a second call."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = fn()
    return graph, outs


def _refill(dst_case, src_case):
    for name in ("U", "M", "K", "B", "C", "dY", "initial_states"):
        d, s = getattr(dst_case, name), getattr(src_case, name)
        if d is not None:
            d.copy_(s)


@pytest.mark.parametrize("path,dtype,shape", [
    ("tc", torch.bfloat16, (2, 3, 300, 64, 64)),      # tensor-core kernels, ragged last chunk
    ("tc", torch.bfloat16, (2, 2, 200, 64, 128)),     # two column blocks: strided device copies inside the capture
    ("simt", torch.float32, (2, 2, 130, 32, 16)),     # float32-exact kernels
])
def test_scan_forward_and_backward_replay_from_a_graph(path, dtype, shape):
    static = make_scan_case(*shape, dtype=dtype, seed=1, with_init=True).to(DEV)
    other = make_scan_case(*shape, dtype=dtype, seed=2, with_init=True).to(DEV)

    def step(c):
        Y, fin, st = _C.scan_fwd(c.U, c.M, c.K, c.B, c.C, c.initial_states, None, None, chunk_size=64,
                                 y_dtype=dtype, want_final=True, path=path, save_states=True)
        grads = _C.scan_bwd(c.U, c.M, c.K, c.B, c.C, c.initial_states, None, None, c.dY, None,
                            chunk_size=64, path=path, saved=(st, fin))
        return (Y, fin) + tuple(g for g in grads if g is not None)

    graph, outs = _capture(lambda: step(static))
    _refill(static, other)
    for o in outs:
        o.fill_(float("nan"))
    graph.replay()
    graph.replay()            # a second replay over the first one's workspaces
    torch.cuda.synchronize()
    want = step(other)
    torch.cuda.synchronize()
    assert len(outs) == len(want)
    for i, (g, w) in enumerate(zip(outs, want)):
        assert torch.isfinite(g.float()).all(), i
        # the same kernels on the same bits; float atomics (grouped or wide-P sums) may reorder
        assert torch.equal(g, w) or rel(g, w) <= 1e-6, (i, rel(g, w))
    assert _C.device_status() == 0


def test_decode_steps_replay_from_a_graph_and_update_the_state_in_place():
    b, h, P, N, steps = 4, 8, 64, 64, 3
    g = torch.Generator().manual_seed(5)
    r = lambda *s: torch.randn(*s, generator=g)

    def tokens():
        rad = torch.exp(-torch.nn.functional.softplus(r(steps, b, h))).clamp(0.9, 0.999)
        th = (torch.rand(steps, b, h, generator=g) * 2 - 1) * torch.pi
        return dict(U=r(steps, b, h, P).to(torch.bfloat16).to(DEV),
                    B=(r(steps, b, h, 2 * N) / N ** 0.5).to(torch.bfloat16).to(DEV),
                    C=(r(steps, b, h, 2 * N) / N ** 0.5).to(torch.bfloat16).to(DEV),
                    M=torch.stack([rad * torch.cos(th), rad * torch.sin(th)], -1).contiguous().to(DEV),
                    K=(0.05 * r(steps, b, h, 2, 2)).to(DEV))

    static, other = tokens(), tokens()
    state0 = (0.1 * r(b, h, P, 2 * N)).to(DEV)
    state = state0.clone()

    def run(tok, st):
        """``steps`` tokens, state updated in place; B_prev / U_prev are the previous token's rows."""
        ys = []
        Bp, Up = torch.zeros_like(tok["B"][0]), torch.zeros_like(tok["U"][0])
        for s in range(steps):
            y, _ = _C.scan_decode(tok["U"][s], tok["M"][s], tok["K"][s], tok["B"][s], tok["C"][s], st,
                                  Bp, Up, y_dtype=torch.bfloat16, state_out=st)
            ys.append(y)
            Bp, Up = tok["B"][s], tok["U"][s]
        return torch.stack(ys)

    graph, ys = _capture(lambda: run(static, state))
    for k in static:
        static[k].copy_(other[k])
    state.copy_(state0)
    graph.replay()
    torch.cuda.synchronize()
    eager_state = state0.clone()
    want = run(other, eager_state)
    torch.cuda.synchronize()
    assert torch.equal(ys, want)
    assert torch.equal(state, eager_state)
    assert not torch.equal(state, state0)


def test_mixer_forward_with_forked_row_kernels_replays_from_a_graph():
    """A sequence-sized mixer forward launches the three scan-preparation kernels on side streams between a
    fork and a join; inside a capture those become edges of the graph."""
    import slinoss_b200 as sb
    torch.manual_seed(0)
    m = sb.SLinOSSMixer(256, d_state=64, expand=2, d_head=64, d_conv=4, chunk_size=64).to(DEV).to(torch.bfloat16)
    x = torch.randn(2, 2048, 256, device=DEV, dtype=torch.bfloat16)      # batch * T >= the fork threshold
    other = torch.randn_like(x)
    with torch.no_grad():
        graph, out = _capture(lambda: m(x))
        x.copy_(other)
        graph.replay()
        torch.cuda.synchronize()
        want = m(other)
    assert torch.equal(out, want)
