"""Block-scaled MXFP8 tensor-core GEMM against an fp32 PyTorch product of the dequantised operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g)
    # very different magnitudes per 32-block and per row, so a wrong scale lookup cannot hide
    x = x * torch.pow(2.0, torch.randint(-6, 7, (M, K // 32), device="cuda", generator=g).float()).repeat_interleave(32, 1)
    w = w * torch.pow(2.0, torch.randint(-6, 7, (N, K // 32), device="cuda", generator=g).float()).repeat_interleave(32, 1)
    return x.bfloat16(), w.bfloat16()


@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 128, 0), (256, 384, 512, 0), (256, 384, 512, 128), (300, 200, 160, 0),
                                      (1024, 1536, 4096, 0), (2048, 4096, 1024, 128), (384, 1000, 2048, 192),
                                      (256, 192, 128, 384), (300, 200, 160, 384), (1024, 1536, 4096, 384), (4096, 4096, 2048, 0),
                                      (2000, 1000, 512, 384)])
def test_mxfp8_gemm_matches_dequantised_product(M, N, K, bn):
    from elfa_b200 import native
    from elfa_b200.ops import gemm_mxfp8 as q
    x, w = _operands(M, N, K, M + N + K)
    xq, xdeq = q.quantize_mxfp8(x, dequantized=True)
    wq, _ = q.quantize_mxfp8(w, right=True)
    y = q.gemm_mxfp8(xq, wq, force_bn=bn)
    torch.cuda.synchronize()
    native.check_status()
    xf, wf = q.dequantize_ref(xq), q.dequantize_ref(wq)
    assert torch.equal(xdeq.float(), xf.bfloat16().float())            # the bf16 copy is the dequantised operand
    ref = xf.double() @ wf.double().t()
    err = (y.double() - ref).abs().max().item()
    bound = 2 ** -8 * ref.abs().max().item() + 1e-3                    # bf16 rounding of the output
    assert err <= bound, (err, bound)


def test_mxfp8_quantiser_matches_fake_quant():
    from elfa_b200.ops import gemm_mxfp8 as q
    from elfa_b200.quant.qat import QuantSpec, fake_quant
    x, _ = _operands(512, 64, 1024, 7)
    _, deq = q.quantize_mxfp8(x, dequantized=True)
    spec = QuantSpec(fmt="mxfp8")
    assert torch.equal(deq, fake_quant(x, spec))


def test_mxfp8_gemm_epilogue():
    from elfa_b200.ops import gemm_mxfp8 as q
    from elfa_b200.ops.gemm import gelu_tanh_ref
    x, w = _operands(256, 512, 256, 3)
    x, w = x * 0.05, w * 0.05
    bias = torch.randn(512, device="cuda").bfloat16()
    xq, _ = q.quantize_mxfp8(x)
    wq, _ = q.quantize_mxfp8(w, right=True)
    pre = torch.empty(256, 512, device="cuda", dtype=torch.bfloat16)
    y = q.gemm_mxfp8(xq, wq, bias=bias, gelu=True, preact=pre)
    ref_pre = q.dequantize_ref(xq) @ q.dequantize_ref(wq).t() + bias.float()
    assert (pre.float() - ref_pre).abs().max() <= 2 ** -7 * ref_pre.abs().max() + 1e-3
    assert (y.float() - gelu_tanh_ref(ref_pre)).abs().max() <= 2 ** -7 * ref_pre.abs().max() + 1e-3


@pytest.mark.parametrize("act", [None, "gelu"])
def test_quant_linear_block_scaled_path_equals_fake_quant_path(act):
    from elfa_b200.parallel.mesh import ParallelContext
    from elfa_b200.parallel.tp import column_parallel_linear
    from elfa_b200.quant.qat import QuantSpec, new_weight_epoch
    torch.manual_seed(0)
    x = (torch.randn(4, 96, 256, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(256, 512, device="cuda") * 0.05).bfloat16()
    dy = torch.randn(4, 96, 512, device="cuda").bfloat16()
    outs = []
    for hw in (True, False):
        new_weight_epoch()
        xi, wi = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
        y = column_parallel_linear(xi, wi, ParallelContext(), act, QuantSpec(fmt="mxfp8", block_scaled_gemm=hw))
        y.backward(dy)
        outs.append((y.detach().float(), xi.grad.float(), wi.grad.float()))
    (y1, dx1, dw1), (y0, dx0, dw0) = outs
    assert (y1 - y0).abs().max() <= 2 ** -7 * y0.abs().max()
    assert (dx1 - dx0).abs().max() <= 2 ** -6 * dx0.abs().max()      # GELU' of a pre-activation that differs in the last bf16 bit
    assert (dw1 - dw0).abs().max() <= 2 ** -6 * dw0.abs().max()


@pytest.mark.parametrize("rows,cols,right", [(128, 128, False), (300, 160, False), (1024, 4096, False), (200, 512, True),
                                             (1536, 1024, True)])
def test_mxfp8_dequantise_kernel_is_exact(rows, cols, right):
    """The native dequantiser returns exactly the bf16 copy the quantiser wrote and the PyTorch decode."""
    from elfa_b200 import native
    from elfa_b200.ops import gemm_mxfp8 as q
    x, _ = _operands(rows, 128, cols, rows + cols)
    op, deq = q.quantize_mxfp8(x, dequantized=True, right=right)
    out = q.dequantize_mxfp8(op)
    torch.cuda.synchronize()
    assert native.status() == 0
    assert torch.equal(out, deq)
    assert torch.equal(out.float(), q.dequantize_ref(op))
