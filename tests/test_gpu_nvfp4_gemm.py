"""Block-scaled NVFP4 tensor-core GEMM against an fp32 PyTorch product of the dequantised operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(M, K, device="cuda", generator=g)
    w = torch.randn(N, K, device="cuda", generator=g)
    # different magnitudes per 16-block, so a wrong scale lookup cannot hide
    x = x * torch.pow(2.0, torch.randint(-3, 4, (M, K // 16), device="cuda", generator=g).float()).repeat_interleave(16, 1)
    w = w * torch.pow(2.0, torch.randint(-3, 4, (N, K // 16), device="cuda", generator=g).float()).repeat_interleave(16, 1)
    return x.bfloat16(), w.bfloat16()


@pytest.mark.parametrize("M,N,K,bn", [(128, 128, 256, 0), (256, 384, 512, 0), (256, 384, 512, 128), (300, 200, 160, 0),
                                      (1024, 1536, 4096, 0), (2048, 4096, 1024, 128), (384, 1000, 2048, 0)])
def test_nvfp4_gemm_matches_dequantised_product(M, N, K, bn):
    from elfa_b200 import native
    from elfa_b200.ops import gemm_nvfp4 as q
    x, w = _operands(M, N, K, M + N + K)
    xq, xdeq = q.quantize_nvfp4(x, dequantized=True)
    wq, _ = q.quantize_nvfp4(w, right=True)
    y = q.gemm_nvfp4(xq, wq, force_bn=bn)
    torch.cuda.synchronize()
    native.check_status()
    xf, wf = q.dequantize_ref(xq), q.dequantize_ref(wq)
    assert torch.equal(xdeq.float(), xf.bfloat16().float())            # the bf16 copy is the (rounded) dequantised operand
    ref = xf.double() @ wf.double().t()
    err = (y.double() - ref).abs().max().item()
    bound = 2 ** -8 * ref.abs().max().item() + 1e-3                    # bf16 rounding of the output
    assert err <= bound, (err, bound)


def test_nvfp4_quantiser_matches_fake_quant():
    from elfa_b200.ops import gemm_nvfp4 as q
    from elfa_b200.quant.qat import QuantSpec, fake_quant
    x, _ = _operands(512, 64, 1024, 7)
    _, deq = q.quantize_nvfp4(x, dequantized=True)
    assert torch.equal(deq, fake_quant(x, QuantSpec(fmt="nvfp4")))


def test_nvfp4_gemm_epilogue():
    from elfa_b200.ops import gemm_nvfp4 as q
    from elfa_b200.ops.gemm import gelu_tanh_ref
    x, w = _operands(256, 512, 256, 3)
    x, w = x * 0.05, w * 0.05
    bias = torch.randn(512, device="cuda").bfloat16()
    xq, _ = q.quantize_nvfp4(x)
    wq, _ = q.quantize_nvfp4(w, right=True)
    pre = torch.empty(256, 512, device="cuda", dtype=torch.bfloat16)
    y = q.gemm_nvfp4(xq, wq, bias=bias, gelu=True, preact=pre)
    ref_pre = q.dequantize_ref(xq) @ q.dequantize_ref(wq).t() + bias.float()
    assert (pre.float() - ref_pre).abs().max() <= 2 ** -7 * ref_pre.abs().max() + 1e-3
    assert (y.float() - gelu_tanh_ref(ref_pre)).abs().max() <= 2 ** -7 * ref_pre.abs().max() + 1e-3


def test_quant_linear_nvfp4_tensor_core_path_close_to_fake_quant_path():
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
        y = column_parallel_linear(xi, wi, ParallelContext(), None, QuantSpec(fmt="nvfp4", block_scaled_gemm=hw))
        y.backward(dy)
        outs.append((y.detach().float(), xi.grad.float(), wi.grad.float()))
    (y1, dx1, dw1), (y0, dx0, dw0) = outs
    assert (y1 - y0).abs().max() <= 2 ** -6 * y0.abs().max()      # bf16 rounding of the fake-quantised operands
    assert torch.equal(dx1, dx0) and torch.equal(dw1, dw0)         # backward uses the same fake-quantised tensors
