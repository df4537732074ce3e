"""tcgen05 attention kernels against the fp32 PyTorch formula."""
import pytest
import torch

from elfa_b200 import native, ops

pytestmark = pytest.mark.gpu


def _qkv(S, B, H, hd, dev, seq_first=True, seed=0):
    g = torch.Generator().manual_seed(seed)
    shape = (S, B, 3, H, hd) if seq_first else (B, S, 3, H, hd)
    return torch.randn(shape, generator=g).to(torch.bfloat16).to(dev)


@pytest.mark.parametrize("S,B,H,hd", [(128, 1, 1, 64), (256, 2, 2, 128), (384, 1, 3, 128), (200, 2, 2, 32), (1024, 1, 4, 64),
                                      (2048, 1, 2, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_forward(cuda_device, S, B, H, hd, causal):
    qkv = _qkv(S, B, H, hd, cuda_device)
    with torch.no_grad():
        out = ops.attention(qkv, causal=causal)
    torch.cuda.synchronize()
    assert native.status() == 0
    ref = ops.attention_ref(qkv.float(), causal=causal)
    err = (out.float() - ref).abs().max().item()
    assert err < 0.03, f"max err {err}"


def test_attention_forward_batch_first(cuda_device):
    qkv = _qkv(256, 2, 2, 64, cuda_device, seq_first=False, seed=3)
    with torch.no_grad():
        out = ops.attention(qkv, causal=True, seq_first=False)
    ref = ops.attention_ref(qkv.float(), causal=True, seq_first=False)
    assert (out.float() - ref).abs().max() < 0.03
    assert native.status() == 0


@pytest.mark.parametrize("S,B,H,hd", [(128, 1, 1, 64), (256, 1, 2, 128), (384, 2, 2, 128), (200, 1, 2, 32), (1024, 1, 2, 64)])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_backward(cuda_device, S, B, H, hd, causal):
    qkv = _qkv(S, B, H, hd, cuda_device, seed=7).requires_grad_(True)
    out = ops.attention(qkv, causal=causal)
    g = torch.randn_like(out)
    out.backward(g)
    torch.cuda.synchronize()
    assert native.status() == 0
    ref_in = qkv.detach().float().requires_grad_(True)
    ref = ops.attention_ref(ref_in, causal=causal)
    ref.backward(g.float())
    err = (qkv.grad.float() - ref_in.grad).abs()
    scale = ref_in.grad.abs().max().item()
    for name, i in (("dq", 0), ("dk", 1), ("dv", 2)):
        e = err[:, :, i].max().item()
        assert e < 0.02 * max(scale, 1.0) + 0.02, f"{name}: max err {e} (grad scale {scale})"


@pytest.mark.parametrize("S,B,H,hd,world", [(512, 1, 2, 128, 4), (768, 2, 2, 64, 3), (256, 1, 1, 128, 2)])
def test_ring_attention_blocks_on_one_gpu(cuda_device, S, B, H, hd, world):
    """The block kernels of ring attention (unmasked blocks, log-sum-exp merge, backward with the global
    log-sum-exp) for every rank of a ring, run one after the other on this GPU, against fp32 attention
    over the whole sequence."""
    from elfa_b200.parallel.ring_attention import ring_attention_emulated
    qkv = _qkv(S, B, H, hd, cuda_device, seed=11)
    g = torch.randn(S, B, H * hd, device=cuda_device, dtype=torch.bfloat16)
    out, dqkv = ring_attention_emulated(qkv, world, causal=True, dout=g)
    torch.cuda.synchronize()
    assert native.status() == 0
    ref_in = qkv.float().requires_grad_(True)
    ref = ops.attention_ref(ref_in, causal=True)
    ref.backward(g.float())
    assert (out.float() - ref).abs().max().item() < 0.03
    scale = ref_in.grad.abs().max().item()
    e = (dqkv.float() - ref_in.grad).abs().max().item()
    assert e < 0.03 * max(scale, 1.0) + 0.03, f"max gradient err {e} (grad scale {scale})"


def _doc_starts(B, S, dev, seed):
    """Random document boundaries: ``doc_start[b, s]`` = first position of the document that holds token s."""
    g = torch.Generator().manual_seed(seed)
    ds = torch.zeros(B, S, dtype=torch.int32)
    for b in range(B):
        cuts = sorted(set(torch.randint(1, S, (max(1, S // 150),), generator=g).tolist()))
        for c in cuts:
            ds[b, c:] = c
    return ds.to(dev)


@pytest.mark.parametrize("S,B,H,Hkv,hd", [(256, 2, 4, 2, 64), (384, 1, 8, 2, 128), (200, 1, 4, 1, 32), (1024, 1, 4, 4, 128)])
@pytest.mark.parametrize("packed", [False, True])
def test_grouped_query_and_packed_attention(cuda_device, S, B, H, Hkv, hd, packed):
    """Grouped-query attention (H query heads on Hkv key / value heads) and packed sequences (per-document causal mask
    with block skipping), forward and backward, against the fp32 formula with repeated key heads / an explicit mask."""
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn((S, B, H + 2 * Hkv, hd), generator=g).to(torch.bfloat16).to(cuda_device).requires_grad_(True)
    ds = _doc_starts(B, S, cuda_device, 9) if packed else None
    out = ops.attention(qkv, causal=True, num_heads=H, doc_start=ds)
    go = torch.randn_like(out)
    out.backward(go)
    torch.cuda.synchronize()
    assert native.status() == 0
    ref_in = qkv.detach().float().requires_grad_(True)
    ref = ops.attention_ref(ref_in, causal=True, num_heads=H, doc_start=ds)
    ref.backward(go.float())
    assert (out.float() - ref).abs().max().item() < 0.03
    scale = ref_in.grad.abs().max().item()
    e = (qkv.grad.float() - ref_in.grad).abs().max().item()
    assert e < 0.02 * max(scale, 1.0) + 0.02, f"max gradient err {e} (grad scale {scale})"
