"""Row-wise kernels of the block's FFN branch and the rematerialising op built on them, against plain
torch evaluated in float64 on the same inputs (the reference's FFN branch is the same torch expression:
slinoss/blocks/block.py, slinoss/layers/mlp.py)."""

import pytest
import torch
import torch.nn.functional as F

import slinoss_b200 as sb
from slinoss_b200 import _C
from slinoss_b200.blocks import block as block_mod
from tests.util import rel

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 3e-3}


def _rms64(x, w, eps):
    x = x.double()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,C", [(1, 8), (37, 256), (130, 512), (33, 1024), (19, 2048), (5000, 512)])
def test_rmsnorm_forward_and_backward(dtype, rows, C):
    if dtype == torch.float32 and C > 1024:
        pytest.skip("float32 rows go up to 1024 channels")
    torch.manual_seed(rows + C)
    x = torch.randn(rows, C, device=DEV).to(dtype)
    w = (1 + 0.3 * torch.randn(C, device=DEV)).to(dtype)
    dy = torch.randn(rows, C, device=DEV).to(dtype)
    eps = 1e-5
    out = _C.rmsnorm_fwd(x, w, eps)
    x64, w64 = x.double().requires_grad_(), w.double().requires_grad_()
    want = _rms64(x64, w64, eps)
    want.backward(dy.double())
    assert rel(out, want) <= TOL[dtype]
    dx, dw = _C.rmsnorm_bwd(x, w, eps, dy)
    assert dw.dtype == torch.float32
    assert rel(dx, x64.grad) <= TOL[dtype]
    assert rel(dw, w64.grad) <= 1e-5      # float32 accumulation whatever the row type


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["gelu", "swiglu"])
@pytest.mark.parametrize("rows,H", [(3, 8), (257, 384), (64, 2048)])
def test_activation_forward_and_backward(dtype, kind, rows, H):
    torch.manual_seed(rows + H)
    W = 2 * H if kind == "swiglu" else H
    proj = (2.0 * torch.randn(rows, W, device=DEV)).to(dtype)
    dh = torch.randn(rows, H, device=DEV).to(dtype)
    p64 = proj.double().requires_grad_()
    if kind == "gelu":
        want = F.gelu(p64, approximate="tanh")
    else:
        v, g = p64.chunk(2, dim=-1)
        want = v * F.silu(g)
    want.backward(dh.double())
    hidden = _C.ffn_activation_fwd(proj, kind)
    dproj = _C.ffn_activation_bwd(proj, dh, kind)
    assert hidden.shape == (rows, H) and dproj.shape == proj.shape
    assert rel(hidden, want) <= TOL[dtype]
    assert rel(dproj, p64.grad) <= TOL[dtype]


def _block(kind, bias, dtype, d_model=256, remat="full"):
    torch.manual_seed(3)
    cfg = sb.SLinOSSBlockConfig(
        d_model=d_model,
        mixer=sb.SLinOSSMixerConfig(d_state=16, d_head=32, expand=1.0),
        ffn=sb.SLinOSSMLPConfig(kind=kind, expand=2.0, multiple_of=64, bias=bias))
    blk = sb.SLinOSSBlock(cfg, device=DEV, dtype=dtype)
    assert blk.ffn_remat == "none"
    blk.ffn_remat = remat
    with torch.no_grad():
        blk.ffn_norm.weight.add_(0.2 * torch.randn_like(blk.ffn_norm.weight))
        if bias:
            blk.ffn.in_proj.bias.normal_(0, 0.2)
            blk.ffn.out_proj.bias.normal_(0, 0.2)
    return blk


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("remat", ["full", "rows"])
@pytest.mark.parametrize("kind,bias", [("gelu", True), ("gelu", False), ("swiglu", True)])
def test_ffn_branch_of_the_block_rematerialised_against_plain_autograd(dtype, kind, bias, remat):
    blk = _block(kind, bias, dtype, remat=remat)
    x = torch.randn(3, 70, 256, device=DEV).to(dtype)
    dy = torch.randn_like(x)
    names = [n for n, _ in blk.named_parameters() if n.startswith("ffn")]

    def run(fused):
        blk.ffn_remat = remat if fused else "none"
        blk.zero_grad(set_to_none=True)
        xi = x.clone().requires_grad_()
        out = blk._ffn_residual(xi)
        out.backward(dy)
        return out.detach(), xi.grad, {n: p.grad.clone() for n, p in blk.named_parameters() if n in names}

    launches = _C.kernel_launches()
    out_f, dx_f, g_f = run(True)
    assert _C.kernel_launches() - launches == 6      # norm, act; norm, act, act', norm'
    out_p, dx_p, g_p = run(False)
    assert _C.kernel_launches() - launches == 6 + 4  # the plain path: norm and activation, forward and backward

    # float64 evaluation of the same expression
    blk64 = _block(kind, bias, dtype, remat="none").double()
    blk64.load_state_dict({k: v.double() for k, v in blk.state_dict().items()})
    x64 = x.double().requires_grad_()
    out64 = blk64._ffn_residual(x64)
    out64.backward(dy.double())
    g64 = {n: p.grad for n, p in blk64.named_parameters() if n in names}
    t = TOL[dtype]
    assert rel(out_f, out64) <= t and rel(dx_f, x64.grad) <= t
    for n in names:
        # the plain path's own distance from float64 bounds what 16-bit rounding allows
        allowed = max(t, 2.0 * rel(g_p[n], g64[n]))
        assert rel(g_f[n], g64[n]) <= allowed, n
    assert rel(out_f, out_p) <= t and rel(dx_f, dx_p) <= 2 * t


@pytest.mark.parametrize("remat,kept", [("full", 0), ("rows", 1)])
def test_ffn_branch_keeps_only_its_input_between_the_passes(remat, kept):
    blk = _block("gelu", True, torch.bfloat16, d_model=512, remat=remat)
    x = torch.randn(8, 512, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    out = blk._ffn_residual(x)
    saved = {t.data_ptr() for t in out.grad_fn.saved_tensors if t is not None}
    assert x.data_ptr() in saved
    big = [t for t in out.grad_fn.saved_tensors if t is not None and t.numel() >= x.numel() and
           t.data_ptr() != x.data_ptr()]
    assert len(big) == kept                      # "rows" keeps the projection, "full" nothing wide


def test_plain_path_is_kept_for_layernorm_dropout_and_autocast():
    blk = _block("gelu", True, torch.float32)
    x = torch.randn(2, 5, 256, device=DEV)
    n0 = _C.kernel_launches()
    blk.ffn_remat = "none"
    blk._ffn_residual(x)
    assert _C.kernel_launches() == n0 + 2        # the norm and the activation
    blk.ffn_remat = "full"
    assert block_mod.ffn_residual_supported(x, blk.ffn_norm, blk.ffn)
    assert not block_mod.ffn_residual_supported(x.bfloat16(), blk.ffn_norm, blk.ffn)
    assert not block_mod.ffn_residual_supported(x, torch.nn.LayerNorm(256, device=DEV), blk.ffn)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        assert not block_mod.ffn_residual_supported(x, blk.ffn_norm, blk.ffn)
    blk.residual_dropout = 0.5
    blk.train()
    n0 = _C.kernel_launches()
    blk._ffn_residual(x)
    assert _C.kernel_launches() == n0 + 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_module_runs_on_the_row_kernels_and_matches_torch(dtype):
    torch.manual_seed(5)
    norm = sb.RMSNorm(512, eps=1e-5, device=DEV, dtype=dtype)
    with torch.no_grad():
        norm.weight.add_(0.3 * torch.randn_like(norm.weight))
    x = torch.randn(4, 33, 512, device=DEV).to(dtype).requires_grad_()
    dy = torch.randn_like(x)
    n0 = _C.kernel_launches()
    out = norm(x)
    out.backward(dy)
    assert _C.kernel_launches() - n0 == 2
    x64 = x.detach().double().requires_grad_()
    w64 = norm.weight.detach().double().requires_grad_()
    want = F.rms_norm(x64, (512,), w64, 1e-5)
    want.backward(dy.double())
    assert rel(out, want) <= TOL[dtype] and rel(x.grad, x64.grad) <= TOL[dtype]
    assert rel(norm.weight.grad, w64.grad) <= TOL[dtype]
    # rows in another type than the weight: computed in the weight's type, returned in the rows'
    assert norm(x.detach().double()).dtype == torch.float64


@pytest.mark.parametrize("kind", ["gelu", "swiglu"])
def test_mlp_module_runs_its_activation_on_the_row_kernel(kind):
    torch.manual_seed(7)
    mlp = sb.SLinOSSMLP(256, kind=kind, expand=2.0, multiple_of=64, bias=True, device=DEV, dtype=torch.float32)
    x = torch.randn(3, 17, 256, device=DEV, requires_grad=True)
    dy = torch.randn(3, 17, 256, device=DEV)
    n0 = _C.kernel_launches()
    out = mlp(x)
    out.backward(dy)
    assert _C.kernel_launches() - n0 == 2
    m64 = sb.SLinOSSMLP(256, kind=kind, expand=2.0, multiple_of=64, bias=True, device=DEV, dtype=torch.float64)
    m64.load_state_dict({k: v.double() for k, v in mlp.state_dict().items()})
    x64 = x.detach().double().requires_grad_()
    out64 = m64(x64)
    out64.backward(dy.double())
    assert rel(out, out64) <= 1e-5 and rel(x.grad, x64.grad) <= 1e-5
    for (n, p), q in zip(mlp.named_parameters(), m64.parameters()):
        assert rel(p.grad, q.grad) <= 1e-5, n
