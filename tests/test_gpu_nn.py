"""Norm / activation / embedding / cross-entropy / optimizer kernels against fp32 PyTorch."""
import pytest
import torch

from elfa_b200 import native, ops
from elfa_b200.native import lib, stream_ptr

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", [ops.LAYERNORM, ops.RMSNORM])
@pytest.mark.parametrize("rows,D", [(64, 128), (1000, 1024), (513, 4096), (96, 8192)])
@pytest.mark.parametrize("with_res", [False, True])
def test_norm_fwd_bwd(cuda_device, kind, rows, D, with_res):
    torch.manual_seed(rows + D)
    dev = cuda_device
    x = torch.randn(rows, D, device=dev).to(torch.bfloat16).requires_grad_(True)
    r = torch.randn(rows, D, device=dev).to(torch.bfloat16).requires_grad_(True) if with_res else None
    w = (1 + 0.1 * torch.randn(D, device=dev)).to(torch.bfloat16).requires_grad_(True)
    b = (0.1 * torch.randn(D, device=dev)).to(torch.bfloat16).requires_grad_(True) if kind == ops.LAYERNORM else None
    eps = 1e-5 if kind == ops.LAYERNORM else 1e-6
    y, s = ops.norm(x, w, b, eps=eps, kind=kind, residual=r)
    gy = torch.randn_like(y)
    gs = torch.randn_like(y) if with_res else None
    if with_res:
        torch.autograd.backward([y, s], [gy, gs])
    else:
        y.backward(gy)
    # fp32 reference on CPU-style formula
    xr = x.detach().float().requires_grad_(True)
    rr = r.detach().float().requires_grad_(True) if with_res else None
    wr = w.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True) if b is not None else None
    sin = (xr + rr).to(torch.bfloat16).float() + 0 * (xr + rr) if with_res else xr
    if with_res:  # keep the rounding of the stored sum but a differentiable path
        sin = xr + rr + ((xr + rr).to(torch.bfloat16).float() - (xr + rr)).detach()
    if kind == ops.RMSNORM:
        yr = sin * torch.rsqrt((sin * sin).mean(-1, keepdim=True) + eps) * wr
    else:
        yr = torch.nn.functional.layer_norm(sin, (D,), wr, br, eps)
    if with_res:
        torch.autograd.backward([yr, sin], [gy.float(), gs.float()])
    else:
        yr.backward(gy.float())
    assert (y.float() - yr).abs().max() < 0.06
    assert (x.grad.float() - xr.grad).abs().max() < 0.08
    if with_res:
        assert (r.grad.float() - rr.grad).abs().max() < 0.08
    tol_w = 0.02 * (rows ** 0.5) + 0.1
    assert (w.grad.float() - wr.grad).abs().max() < tol_w
    if b is not None:
        assert (b.grad.float() - br.grad).abs().max() < tol_w
    assert native.status() == 0


@pytest.mark.parametrize("name", ["gelu", "silu", "relu", "gelu_erf"])
def test_activation(cuda_device, name):
    x = torch.randn(1000, 333, device=cuda_device).to(torch.bfloat16).requires_grad_(True)
    y = ops.activation(x, name)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    fn = {"gelu": lambda t: torch.nn.functional.gelu(t, approximate="tanh"), "silu": torch.nn.functional.silu,
          "relu": torch.relu, "gelu_erf": torch.nn.functional.gelu}[name]
    yr = fn(xr)
    yr.backward(g.float())
    assert (y.float() - yr).abs().max() < 0.03
    assert (x.grad.float() - xr.grad).abs().max() < 0.05


@pytest.mark.parametrize("rows,V", [(64, 4096), (300, 32000), (17, 1000)])
@pytest.mark.parametrize("smoothing", [0.0, 0.1])
def test_cross_entropy(cuda_device, rows, V, smoothing):
    torch.manual_seed(V)
    logits = (3 * torch.randn(rows, V, device=cuda_device)).to(torch.bfloat16)
    targets = torch.randint(0, V, (rows,), device=cuda_device)
    targets[0] = -100
    lr = logits.detach().float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, targets, label_smoothing=smoothing, reduction="sum", ignore_index=-100) / rows
    ref.backward()
    lg = logits.clone().requires_grad_(True)
    loss = ops.cross_entropy(lg * 1.0, targets, smoothing)   # "* 1.0": a non-leaf the op may overwrite
    loss.backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * max(1.0, abs(ref.item()))
    assert (lg.grad.float() - lr.grad).abs().max() < 2e-3 / rows * 50 + 1e-4
    assert native.status() == 0


def test_cross_entropy_bad_target_sets_status(cuda_device):
    logits = torch.randn(8, 256, device=cuda_device).to(torch.bfloat16)
    targets = torch.full((8,), 999, device=cuda_device)
    ops.cross_entropy(logits, targets)
    assert native.status() & native.ST_BAD_TARGET
    assert native.status() == 0


def test_embedding(cuda_device):
    torch.manual_seed(1)
    V, D, B, T = 512, 256, 3, 40
    tok = torch.randn(V, D, device=cuda_device).to(torch.bfloat16).requires_grad_(True)
    pos = torch.randn(64, D, device=cuda_device).to(torch.bfloat16).requires_grad_(True)
    ids = torch.randint(0, V, (B, T), device=cuda_device)
    out = ops.embedding(ids, tok, pos)
    ref = (tok.detach().float()[ids] + pos.detach().float()[:T]).to(torch.bfloat16)
    assert torch.equal(out, ref)
    g = torch.randn_like(out)
    out.backward(g)
    dtok = torch.zeros(V, D, device=cuda_device)
    dtok.index_add_(0, ids.view(-1), g.float().view(-1, D))
    assert (tok.grad.float() - dtok).abs().max() < 0.05
    assert (pos.grad.float()[:T] - g.float().sum(0)).abs().max() < 0.05
    # vocabulary-parallel halves sum to the full embedding
    lo = ops.embedding(ids, tok.detach()[:256], pos.detach(), 0, 0).float()
    hi = ops.embedding(ids, tok.detach()[256:], pos.detach(), 0, 256).float()
    assert (lo + hi - ref.float()).abs().max() < 0.02


def test_adamw_and_clip(cuda_device):
    torch.manual_seed(2)
    n = 1_000_003
    dev = cuda_device
    master = torch.randn(n, device=dev)
    grad = torch.randn(n, device=dev) * 3
    m = torch.zeros(n, device=dev)
    v = torch.zeros(n, device=dev)
    param = torch.empty(n, dtype=torch.bfloat16, device=dev)
    p_ref = master.clone().requires_grad_(True)
    opt = torch.optim.AdamW([p_ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    scal = torch.zeros(4, dtype=torch.float32, device=dev)
    part = torch.empty(2048, dtype=torch.float32, device=dev)
    st = stream_ptr(master)
    for step in (1, 2, 3):
        g = grad * step
        lib.call("elfa_sumsq", g, 0, n, part, scal, 0, st)
        lib.call("elfa_clip_coef", scal, 1.0, 1.0, st)
        lib.call("elfa_adamw", param, 1, master, m, v, g, 0, n, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, scal, st)
        p_ref.grad = g.clone()
        norm = torch.nn.utils.clip_grad_norm_([p_ref], 1.0)
        opt.step()
        assert abs(scal[2].item() - norm.item()) < 1e-3 * norm.item()
    assert (master - p_ref.detach()).abs().max() < 1e-5
    assert torch.equal(param, master.to(torch.bfloat16))
    # non-finite gradient: state untouched, status flag raised
    before = master.clone()
    g = grad.clone()
    g[5] = float("inf")
    lib.call("elfa_sumsq", g, 0, n, part, scal, 0, st)
    lib.call("elfa_clip_coef", scal, 1.0, 1.0, st)
    lib.call("elfa_adamw", param, 1, master, m, v, g, 0, n, 1e-2, 0.9, 0.95, 1e-8, 0.1, 4, scal, st)
    assert torch.equal(before, master)
    assert native.status() & native.ST_NONFINITE


@pytest.mark.parametrize("rows,cols", [(7, 33), (64, 1000), (300, 4096), (5, 32000)])
def test_softmax_rows(cuda_device, rows, cols):
    from elfa_b200.ops import nn as nnops
    x = (torch.randn(rows, cols, device=cuda_device) * 3).bfloat16()
    y = nnops.softmax(x, 0.7)
    ref = torch.softmax(x.float() * 0.7, dim=-1)
    assert (y.float() - ref).abs().max() <= 2 ** -8 * ref.max() + 1e-4
    assert (y.float().sum(-1) - 1).abs().max() < 0.02


def test_newton_schulz_on_the_gemm_matches_fp32(cuda_device):
    """Muon's orthogonalisation on the tcgen05 GEMM (``3I -`` and the 0.5 folded into epilogues) against the fp32 loop,
    for the right (tall) and the left (wide) form."""
    from elfa_b200.optim.optimizers import newton_schulz
    g = torch.Generator().manual_seed(4)
    for rows, cols in ((512, 256), (256, 768)):
        m = torch.randn(rows, cols, generator=g)
        m = (m / m.norm()).to(torch.bfloat16)
        got = newton_schulz(m.to(cuda_device), 3).float().cpu()
        ref = newton_schulz(m.float(), 3).float()
        assert (got - ref).abs().max().item() < 0.02 * ref.abs().max().item() + 1e-3
    torch.cuda.synchronize()
    assert native.status() == 0


def test_muon_handles_dimensions_that_are_not_multiples_of_eight(cuda_device):
    """A 2-D parameter whose sides are not multiples of 8 is orthogonalised on the GPU too (zero padding, exact), not on the host."""
    from elfa_b200.optim import FlatParams
    from elfa_b200.optim.optimizers import Muon, newton_schulz
    g = torch.Generator().manual_seed(5)
    w = torch.nn.Parameter((torch.randn(100, 36, generator=g) * 0.1).to(torch.bfloat16).to(cuda_device))
    flat = FlatParams([("w", w)])
    opt = Muon(flat, lr=0.1, momentum=0.0, iterations=3, max_grad_norm=0.0)
    grad = torch.randn(100, 36, generator=g).to(cuda_device)
    w.main_grad.copy_(grad)
    before = opt.master.clone()                  # fp32 master weights: the update itself, without the bf16 rounding of w
    opt.step(0.1)
    torch.cuda.synchronize()
    assert native.status() == 0
    ref = newton_schulz((grad / grad.norm()).float().cpu(), 3)
    step = ((before - opt.master)[:w.numel()].view(100, 36)).cpu() / 0.1
    assert (step - ref).abs().max().item() < 0.03 * ref.abs().max().item() + 2e-3
