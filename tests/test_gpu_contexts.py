"""The mixer under the execution contexts the reference supports for its CUDA path (no_grad,
inference_mode, autocast, torch.compile with the custom ops kept out of the traced graph)."""

import pytest
import torch

import slinoss_b200 as sb
from tests.util import rel

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _mixer(dtype):
    torch.manual_seed(0)
    return sb.SLinOSSMixer(256, d_state=64, expand=2, d_head=64, d_conv=4, chunk_size=64, device=DEV, dtype=dtype)


def test_no_grad_and_inference_mode_equal_the_training_forward():
    m = _mixer(torch.bfloat16)
    x = torch.randn(2, 130, 256, device=DEV, dtype=torch.bfloat16)
    want = m(x)
    with torch.no_grad():
        a = m(x)
    with torch.inference_mode():
        b = m(x)
        out, state = m(x, return_state=True)
        y1, state = m.step(x[:, 0], m.init_decode_state(2, device=DEV, dtype=torch.bfloat16))
    assert torch.equal(a, want) and torch.equal(b, want) and torch.equal(out, want)
    assert rel(y1, want[:, 0]) <= 2e-2


def test_autocast_runs_the_16_bit_kernels_on_float32_parameters():
    m32 = _mixer(torch.float32)
    m16 = _mixer(torch.bfloat16)
    m16.load_state_dict(m32.state_dict())
    x = torch.randn(2, 130, 256, device=DEV, requires_grad=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = m32(x)
    assert y.dtype == torch.bfloat16
    y.float().square().mean().backward()
    x16 = x.detach().to(torch.bfloat16).requires_grad_()
    y16 = m16(x16)
    y16.float().square().mean().backward()
    assert rel(y, y16) <= 3e-2
    assert rel(x.grad, x16.grad) <= 5e-2
    for (n, p), q in zip(m32.named_parameters(), m16.parameters()):
        assert p.grad is not None and p.grad.dtype == torch.float32, n
        assert rel(p.grad, q.grad) <= 6e-2, (n, rel(p.grad, q.grad))


def test_torch_compile_keeps_the_custom_ops_out_of_the_graph():
    m = _mixer(torch.bfloat16)
    x = torch.randn(2, 96, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    want = m(x)
    (gw,) = torch.autograd.grad(want.float().sum(), x)
    compiled = torch.compile(m, backend="eager")      # traces the module; no code generation involved
    got = compiled(x)
    (gg,) = torch.autograd.grad(got.float().sum(), x)
    assert rel(got, want) <= 1e-6 and rel(gg, gw) <= 1e-6


def test_torch_compile_of_a_block_with_the_ffn_branch():
    torch.manual_seed(1)
    cfg = sb.SLinOSSBlockConfig(d_model=256, mixer=sb.SLinOSSMixerConfig(d_state=64, d_head=64, expand=1.0),
                                ffn=sb.SLinOSSMLPConfig(kind="gelu", expand=2.0, multiple_of=64))
    blk = sb.SLinOSSBlock(cfg, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(2, 70, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    want = blk(x)
    (gw,) = torch.autograd.grad(want.float().sum(), x)
    for remat in ("none", "full"):
        blk.ffn_remat = remat
        got = torch.compile(blk, backend="eager")(x)
        (gg,) = torch.autograd.grad(got.float().sum(), x)
        assert rel(got, want) <= 1e-2 and rel(gg, gw) <= 2e-2, remat


def test_gradient_checkpointing_of_the_stack_gives_the_same_gradients():
    torch.manual_seed(2)
    blk = sb.SLinOSSBlockConfig(d_model=256, mixer=sb.SLinOSSMixerConfig(d_state=64, d_head=64, expand=1.0),
                                ffn=sb.SLinOSSMLPConfig(kind="gelu", expand=2.0, multiple_of=64))
    res = []
    for ckpt in (False, True):
        torch.manual_seed(3)
        stack = sb.SLinOSSStack(sb.SLinOSSStackConfig.uniform(blk, n_layers=2, gradient_checkpointing=ckpt),
                                device=DEV, dtype=torch.bfloat16).train()
        x = torch.randn(2, 100, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        out = stack(x)
        out.float().square().mean().backward()
        res.append((out.detach(), x.grad, [p.grad.clone() for p in stack.parameters()]))
    (o0, g0, p0), (o1, g1, p1) = res
    assert torch.equal(o0, o1) and torch.equal(g0, g1)        # deterministic kernels: recomputation is bit-equal
    for a, b in zip(p0, p1):
        assert rel(a, b) <= 1e-3                               # (weight gradients sum float atomics in another order)
