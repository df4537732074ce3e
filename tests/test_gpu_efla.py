"""EFLA scan, ShortConv and the EFLA/PRISM model family on the GPU against the fp32 references."""
import pytest
import torch

from elfa_b200 import native
from elfa_b200.ops import efla as eops

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,T,H,d,chunk", [(1, 16, 1, 32, 16), (2, 50, 2, 64, 16), (1, 40, 2, 128, 8), (1, 70, 1, 96, 16), (2, 100, 2, 64, 32),
                                           (1, 2048, 2, 64, 16), (1, 4096, 1, 128, 16)])     # long sequences: fp32 state drift would show
@pytest.mark.parametrize("with_state", [False, True])
def test_efla_scan_forward_backward(cuda_device, B, T, H, d, chunk, with_state):
    torch.manual_seed(d + T)
    dev = cuda_device
    k = (torch.randn(B, T, H, d, device=dev) * (0.7 / d ** 0.5 * 3)).to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(B, T, H, d, device=dev).to(torch.bfloat16).requires_grad_(True)
    beta = torch.tensor([0.8], device=dev, requires_grad=True)
    s0 = (0.1 * torch.randn(B, H, d, d, device=dev)).requires_grad_(True) if with_state else None
    o, s = eops.efla_scan(k, v, beta, s0, chunk)
    go = torch.randn_like(o)
    gs = 0.1 * torch.randn_like(s)
    torch.autograd.backward([o, s], [go, gs])
    torch.cuda.synchronize()
    assert native.status() == 0
    kr = k.detach().float().requires_grad_(True)
    vr = v.detach().float().requires_grad_(True)
    br = beta.detach().clone().requires_grad_(True)
    sr = s0.detach().clone().requires_grad_(True) if with_state else None
    o_ref, s_ref = (eops.efla_scan_ref if T <= 256 else eops.efla_scan_chunked_ref)(kr, vr, br, sr)
    torch.autograd.backward([o_ref, s_ref], [go.float(), gs])
    assert (o.float() - o_ref).abs().max() < 0.05
    assert (s - s_ref).abs().max() < 0.02
    gk = kr.grad.abs().max().item()
    assert (k.grad.float() - kr.grad).abs().max() < 0.03 * max(gk, 1.0)
    assert (v.grad.float() - vr.grad).abs().max() < 0.03 * max(vr.grad.abs().max().item(), 1.0)
    assert abs(beta.grad.item() - br.grad.item()) < 0.03 * max(abs(br.grad.item()), 1.0)
    if with_state:
        assert (s0.grad - sr.grad).abs().max() < 0.03 * max(sr.grad.abs().max().item(), 1.0)


def test_efla_chunks_compose_as_affine_maps(cuda_device):
    torch.manual_seed(0)
    k = torch.randn(1, 24, 2, 32, device=cuda_device) * 0.3
    v = torch.randn(1, 24, 2, 32, device=cuda_device)
    beta = torch.tensor(1.0, device=cuda_device)
    _, s_full = eops.efla_scan_ref(k, v, beta)
    a1, b1 = eops.chunk_affine_map(k[:, :10], v[:, :10], beta)
    a2, b2 = eops.chunk_affine_map(k[:, 10:], v[:, 10:], beta)
    a, b = eops.compose_affine(a1, b1, a2, b2)
    assert (b - s_full).abs().max() < 1e-4           # zero initial state: S_end = B
    s0 = torch.randn(1, 2, 32, 32, device=cuda_device)
    _, s_from = eops.efla_scan_ref(k, v, beta, s0)
    assert (a @ s0 + b - s_from).abs().max() < 1e-3


@pytest.mark.parametrize("B,T,C,W", [(2, 33, 64, 4), (1, 100, 256, 16)])
def test_shortconv(cuda_device, B, T, C, W):
    torch.manual_seed(W)
    dev = cuda_device
    x = torch.randn(B, T, C, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(C, W, device=dev) * 0.3).to(torch.bfloat16).requires_grad_(True)
    b = (torch.randn(C, device=dev) * 0.1).to(torch.bfloat16).requires_grad_(True)
    y = eops.shortconv(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = eops.shortconv_ref(xr, wr, br)
    yr.backward(g.float())
    assert (y.float() - yr).abs().max() < 0.05
    assert (x.grad.float() - xr.grad).abs().max() < 0.05
    assert (w.grad.float() - wr.grad).abs().max() < 0.02 * (B * T) ** 0.5 + 0.1
    assert (b.grad.float() - br.grad).abs().max() < 0.02 * (B * T) ** 0.5 + 0.1
    assert native.status() == 0


def test_efla_model_trains_on_gpu(cuda_device):
    import os
    import warnings
    warnings.simplefilter("ignore")
    from elfa_b200.config import Config
    from elfa_b200.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    losses = {}
    for name, dev, dt in (("gpu", cuda_device, "bf16"), ("cpu", torch.device("cpu"), "fp32")):
        cfg = Config.from_file(os.path.join(root, "configs", "smoke.yaml"), env_override=False)
        cfg.model.dtype = dt
        cfg.checkpoint.dir = ""
        cfg.telemetry.log_file = ""
        cfg.bench.synthetic = "uniform"
        cfg.data.seq_len = 32
        cfg.training.mixed_precision = False
        tr = Trainer(cfg, device=dev, telemetry=False)
        losses[name] = tr.run(max_steps=3)
    assert native.status() == 0
    for a, b in zip(losses["gpu"], losses["cpu"]):
        assert abs(a - b) < 0.08 * abs(b), losses


def test_lion_muon_update_replayed_from_a_cuda_graph_equals_eager(cuda_device, monkeypatch):
    """The Lion + Muon update is captured into a CUDA graph at the second step and replayed afterwards (learning rate through the
    device scalars, so the schedule is followed): same losses and weights as launching every kernel eagerly."""
    import os
    import warnings
    warnings.simplefilter("ignore")
    from elfa_b200.config import Config
    from elfa_b200.trainer import Trainer
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run(graph):
        monkeypatch.setenv("ELFA_OPT_GRAPH", "1" if graph else "0")
        cfg = Config.from_file(os.path.join(root, "configs", "smoke.yaml"), env_override=False)
        cfg.model.dtype = "bf16"
        cfg.checkpoint.dir = ""
        cfg.telemetry.log_file = ""
        cfg.bench.synthetic = "uniform"
        cfg.data.seq_len = 32
        cfg.training.lr_schedule = "linear_warmup_cosine"       # the learning rate changes every step
        cfg.training.warmup_steps = 2
        cfg.training.total_steps = 6
        tr = Trainer(cfg, device=cuda_device, telemetry=False)
        losses = tr.run(max_steps=5)
        assert (tr.optimizer._graph is not None) == graph
        return losses, tr.flat.flat.float().clone()
    la, wa = run(True)
    lb, wb = run(False)
    assert native.status() == 0
    assert la == lb, (la, lb)
    assert torch.equal(wa, wb)


def test_prism_refine_kernel_matches_reference(cuda_device):
    from elfa_b200.ops import efla as eops
    torch.manual_seed(0)
    B, T, G, d, L = 2, 64, 8, 64, 3
    u = (torch.randn(B, T, G * d, device=cuda_device) * 0.5).bfloat16().requires_grad_(True)
    v = (torch.randn(B, T, G * d, device=cuda_device) * 0.5).bfloat16().requires_grad_(True)
    ps = [torch.sigmoid(torch.randn(B, T, d, device=cuda_device)).bfloat16().requires_grad_(True) for _ in range(L)]
    go = torch.randn(B, T, G * d, device=cuda_device).bfloat16()
    y = eops.prism_refine(u, v, ps, d)
    y.backward(go)
    got = [y.detach().float(), u.grad.float(), v.grad.float()] + [p.grad.float() for p in ps]
    u2, v2 = u.detach().float().requires_grad_(True), v.detach().float().requires_grad_(True)
    ps2 = [p.detach().float().requires_grad_(True) for p in ps]
    y2 = eops.prism_refine_ref(u2, v2, ps2, d)
    y2.backward(go.float())
    want = [y2.detach(), u2.grad, v2.grad] + [p.grad for p in ps2]
    for a, b in zip(got, want):
        assert (a - b).abs().max() <= 0.02 * b.abs().max() + 0.02, ((a - b).abs().max(), b.abs().max())
