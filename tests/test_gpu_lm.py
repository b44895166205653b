"""The stacked-LM training step on one GPU: its shortcuts (clipping folded into the fused optimizer,
the head GEMM without the last position, the projection's own backward pass) against the plain
formulation of the same step."""

import copy

import pytest
import torch
import torch.nn.functional as F

from slinoss_b200.lm import DataParallelTrainer, SLinOSSLM, lm_stack_config
from slinoss_b200.ops.mixer import split_mixer_projection
from tests.util import rel

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _model(dtype=torch.float32):
    torch.manual_seed(0)
    return SLinOSSLM(512, lm_stack_config(256, 2), device=DEV, dtype=dtype)


def test_loss_drops_the_last_position_before_the_head():
    m = _model()
    ids = torch.randint(0, 512, (2, 96), device=DEV)
    logits = m(ids)
    want = F.cross_entropy(logits[:, :-1].reshape(-1, 512).float(), ids[:, 1:].reshape(-1))
    assert rel(m.loss(ids), want) <= 1e-6


@pytest.mark.parametrize("clip", [1e-3, 1e3])        # one that clips, one that does not
def test_clipping_inside_the_fused_optimizer_equals_clip_then_step(clip):
    a = _model()
    b = copy.deepcopy(a)
    ids = torch.randint(0, 512, (2, 128), device=DEV)
    ta = DataParallelTrainer(a, grad_clip=clip, reduce=False)
    tb = DataParallelTrainer(b, grad_clip=0.0, reduce=False)
    for _ in range(2):
        ta.step(ids)
        # the plain formulation: scale the gradients, then step
        tb.opt.zero_grad(set_to_none=True)
        b.loss(ids).backward()
        norm = torch.nn.utils.clip_grad_norm_(b.parameters(), clip)
        tb.opt.step()
        assert rel(ta.last_grad_norm, norm) <= 1e-5
    for (n, pa), pb in zip(a.named_parameters(), b.parameters()):
        assert rel(pa, pb) <= 1e-5, n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_projection_backward_equals_autograd_of_the_three_gemms(dtype):
    torch.manual_seed(1)
    x = torch.randn(3, 50, 128, device=DEV).to(dtype).requires_grad_()
    w = (0.1 * torch.randn(2 * 96 + 12 + 64, 128, device=DEV)).to(dtype).requires_grad_()
    outs = split_mixer_projection(x, w, d_inner=96, param_proj_dim=12)
    gs = [torch.randn_like(o) for o in outs]
    torch.autograd.backward(outs, gs)
    x2, w2 = x.detach().double().requires_grad_(), w.detach().double().requires_grad_()
    full = F.linear(x2, w2)
    want = torch.split(full, [96, 96, 12, 64], dim=-1)
    torch.autograd.backward(want, [g.double() for g in gs])
    t = 1e-5 if dtype == torch.float32 else 2e-2
    for o, o2 in zip(outs, want):
        assert rel(o, o2) <= t
    assert rel(x.grad, x2.grad) <= t and rel(w.grad, w2.grad) <= t
