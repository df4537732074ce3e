"""tcgen05 GEMM against an fp32 PyTorch reference: layouts, tails, epilogues."""
import pytest
import torch

from elfa_b200 import native, ops

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    """fp64 product of the bf16 operands, returned in fp32: the exact value up to the final rounding."""
    af = (a.t() if a_mn else a).double()
    bf = (b if b_mn else b.t()).double()
    return (af @ bf).float()


def _mk(M, N, K, a_mn, b_mn, dev, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randn((K, M) if a_mn else (M, K), generator=g).to(torch.bfloat16).to(dev)
    b = torch.randn((K, N) if b_mn else (N, K), generator=g).to(torch.bfloat16).to(dev)
    return a, b


def _close(out, ref, K):
    """Relative bound: one bf16 rounding of the output (2^-9 of its magnitude) plus fp32 accumulation, i.e. 2^-8 of the largest
    reference magnitude; a wrong rounding mode, a dropped K slice or a misplaced tile all exceed it."""
    err = (out.float() - ref).abs().max().item()
    tol = 2.0 ** -8 * ref.abs().max().item()
    assert err <= tol, f"max err {err} > {tol} (K = {K})"


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 1376, 512), (200, 96, 136), (4096, 4096, 1024)])
def test_gemm_layouts(cuda_device, M, N, K, a_mn, b_mn):
    if a_mn and M % 8:
        pytest.skip("MN-major A needs M % 8 == 0")
    a, b = _mk(M, N, K, a_mn, b_mn, cuda_device)
    out = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    assert native.status() == 0
    _close(out, _ref(a, b, a_mn, b_mn), K)


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_tile_widths(cuda_device, bn):
    a, b = _mk(512, 768, 320, False, True, cuda_device, seed=1)
    out = ops.gemm(a, b, b_mn=True, force_bn=bn)
    _close(out, _ref(a, b, False, True), 320)
    assert native.status() == 0


def test_gemm_epilogues(cuda_device):
    M, N, K = 512, 1024, 256
    a, b = _mk(M, N, K, False, True, cuda_device, seed=2)
    bias = torch.randn(N, device=cuda_device).to(torch.bfloat16)
    aux = torch.randn(M, N, device=cuda_device).to(torch.bfloat16)
    base = _ref(a, b, False, True) + bias.float()
    pre = torch.empty(M, N, dtype=torch.bfloat16, device=cuda_device)
    out = ops.gemm(a, b, b_mn=True, bias=bias, gelu=True, preact=pre)
    _close(pre, base, K)
    _close(out, ops.gelu_tanh_ref(base), K)
    out = ops.gemm(a, b, b_mn=True, aux=aux, dgelu_aux=True)
    _close(out, _ref(a, b, False, True) * ops.dgelu_tanh_ref(aux.float()), K)
    out = ops.gemm(a, b, b_mn=True, aux=aux, add_aux=True)
    _close(out, _ref(a, b, False, True) + aux.float(), K)
    acc = torch.randn(M, N, device=cuda_device)
    acc0 = acc.clone()
    ops.gemm(a, b, b_mn=True, out=acc, accumulate=True)
    _close(acc, _ref(a, b, False, True) + acc0, K)
    o32 = ops.gemm(a, b, b_mn=True, out_dtype=torch.float32, alpha=0.5)
    assert o32.dtype == torch.float32
    _close(o32, 0.5 * _ref(a, b, False, True), K)
    assert native.status() == 0


def test_gemm_many_tiles_persistent(cuda_device):
    # more tiles than SMs and a CTA cap: every CTA loops over several tiles and both accumulator buffers
    a, b = _mk(2048, 2048, 512, False, False, cuda_device, seed=3)
    out = ops.gemm(a, b, max_ctas=7)
    _close(out, _ref(a, b, False, False), 512)
    out2 = ops.gemm(a, b)
    assert torch.equal(out, out2), "result must not depend on the tile-to-CTA assignment"
    assert native.status() == 0


def test_linear_autograd(cuda_device):
    torch.manual_seed(0)
    x = torch.randn(4, 64, 256, device=cuda_device).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(256, 512, device=cuda_device) * 0.05).to(torch.bfloat16).requires_grad_(True)
    y = ops.linear(x, w, None, "gelu")
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    yr = torch.nn.functional.gelu(xr @ wr, approximate="tanh")
    yr.backward(g.float())
    assert (y.float() - yr).abs().max() < 0.05
    assert (x.grad.float() - xr.grad).abs().max() < 0.1
    assert (w.grad.float() - wr.grad).abs().max() < 0.02 * (256 ** 0.5) + 0.3


@pytest.mark.parametrize("M,N,K", [(512, 4096, 16384), (4096, 1536, 8192), (1376, 4096, 4096)])
def test_weight_gradient_split_k_accumulate(cuda_device, M, N, K):
    # fp32 accumulate output with few tiles: the kernel splits K over several CTAs and adds atomically
    a, b = _mk(M, N, K, True, True, cuda_device, seed=5)
    acc = torch.randn(M, N, device=cuda_device)
    acc0 = acc.clone()
    ops.gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True)
    ref = _ref(a, b, True, True) + acc0
    err = (acc - ref).abs().max().item()
    assert err < 0.01 * (K ** 0.5) + 0.05, err
    assert native.status() == 0


def test_staged_epilogue_tails_and_bias_gelu(cuda_device):
    # plain bf16 outputs go through the shared-memory + TMA-store epilogue: odd M / N tails, bias, GELU
    for (M, N, K) in [(200, 96, 136), (130, 1376, 64), (1000, 264, 512)]:
        a, b = _mk(M, N, K, False, True, cuda_device, seed=6)
        bias = torch.randn(N, device=cuda_device).to(torch.bfloat16)
        out = torch.full((M + 8, N), 7.0, dtype=torch.bfloat16, device=cuda_device)   # guard rows must stay untouched
        ops.gemm(a, b, b_mn=True, out=out[:M], bias=bias, gelu=True)
        ref = ops.gelu_tanh_ref(_ref(a, b, False, True) + bias.float())
        _close(out[:M], ref, K)
        assert torch.all(out[M:] == 7.0)
    assert native.status() == 0


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 320), (200, 96, 136), (1000, 1376, 512), (2048, 2304, 1024)])
def test_gemm_cta_pair_tiles(cuda_device, M, N, K, a_mn, b_mn):
    """256 x 256 tiles computed by CTA pairs (cta_group::2), forced on shapes with row / column / K tails."""
    a, b = _mk(M, N, K, a_mn, b_mn, cuda_device, seed=5)
    out = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, force_bn=512)
    torch.cuda.synchronize()
    assert native.status() == 0
    _close(out, _ref(a, b, a_mn, b_mn), K)


def test_gemm_cta_pair_epilogues_and_persistence(cuda_device):
    M, N, K = 1024, 1536, 512
    a, b = _mk(M, N, K, True, True, cuda_device, seed=6)
    ref = _ref(a, b, True, True)
    acc = torch.randn(M, N, device=cuda_device)
    acc0 = acc.clone()
    ops.gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True, force_bn=512)       # staged fp32 reduce-add epilogue
    _close(acc, ref + acc0, K)
    few = ops.gemm(a, b, a_mn=True, b_mn=True, force_bn=512, max_ctas=6)                # 3 pairs loop over 24 tiles
    full = ops.gemm(a, b, a_mn=True, b_mn=True, force_bn=512)
    _close(full, ref, K)
    assert torch.equal(few, full)
    x, w = _mk(M, N, K, False, True, cuda_device, seed=7)
    bias = torch.randn(N, device=cuda_device).to(torch.bfloat16)
    pre = torch.empty(M, N, dtype=torch.bfloat16, device=cuda_device)
    out = ops.gemm(x, w, b_mn=True, bias=bias, gelu=True, preact=pre, force_bn=512)
    base = _ref(x, w, False, True) + bias.float()
    _close(pre, base, K)
    _close(out, ops.gelu_tanh_ref(base), K)
    assert native.status() == 0
