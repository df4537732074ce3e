"""Number formats, QAT, optimizers, schedules, clipping, sharding arithmetic, models, eval (CPU)."""
import math
import os
import warnings

import pytest
import torch

from elfa_b200 import ops
from elfa_b200.config import Config
from elfa_b200.eval import Generator, generate_needle_case, generate_summary_case, lcs_length, rouge_l, rouge_n, sample_top_p, score_summary
from elfa_b200.ops import efla as eops
from elfa_b200.optim import AdamW, FlatParams, GradientClipper, Lion, LionMuon, LossScaler, LRScheduler
from elfa_b200.optim.optimizers import newton_schulz
from elfa_b200.parallel import tp as tpl
from elfa_b200.parallel.mesh import global_rank, mesh_coords
from elfa_b200.quant import (ScaleFactor, bf16_round, e2m1_round, e4m3_round, e5m2_round, mxfp8_fake_quant_ref, nvfp4_fake_quant_ref,
                             pack_fp4, unpack_fp4)
from elfa_b200.quant.qat import QuantSpec, fake_quant, fake_quant_ste

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ------------------------------------------------------------------------------------------- formats
def test_e4m3_edge_values():
    x = torch.tensor([0.0, 2.0 ** -9, 2.0 ** -10 * 1.01, 448.0, 500.0, -1000.0, 1.0625, 1.1875, 0.0009765625])
    y = e4m3_round(x)
    assert y[1] == 2.0 ** -9                    # smallest subnormal survives
    assert y[3] == 448.0 and y[4] == 448.0 and y[5] == -448.0      # saturates, never inf
    assert y[6] == 1.0 and y[7] == 1.25         # ties to even mantissa (1.0625 -> 1.0, 1.1875 -> 1.25)
    assert torch.isnan(e4m3_round(torch.tensor([float("nan")]))).all()


def test_e5m2_bf16_and_fp4_codecs():
    assert e5m2_round(torch.tensor([57344.0]))[0] == 57344.0 and torch.isinf(e5m2_round(torch.tensor([70000.0]))[0])
    assert bf16_round(torch.tensor([1.00390625]))[0] == 1.0 and bf16_round(torch.tensor([1.01171875]))[0] == 1.015625
    x = torch.tensor([0.24, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -2.5])
    assert e2m1_round(x).tolist() == [0.0, 0.0, 0.5, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -2.0]
    vals = torch.tensor([0.5, -6.0, 3.0, 1.5, 0.0, -0.5])
    packed = pack_fp4(vals)
    assert packed.tolist() == [1 | (15 << 4), 5 | (3 << 4), 0 | (9 << 4)]     # low nibble = even element
    assert unpack_fp4(packed).tolist() == vals.tolist()


def test_block_formats_and_delayed_scaling():
    torch.manual_seed(0)
    x = torch.randn(8, 96) * torch.logspace(-3, 3, 96)
    q = mxfp8_fake_quant_ref(x)
    blocks = x.reshape(8, 3, 32)
    amax = blocks.abs().amax(-1, keepdim=True)
    step = torch.pow(2.0, torch.floor(torch.log2(amax)) - 8) * 32       # coarsest e4m3 step in the top binade
    assert ((q.reshape(8, 3, 32) - blocks).abs() <= step * 2.01).all()  # <= half a step except the saturating band
    assert torch.equal(mxfp8_fake_quant_ref(q), q)                      # idempotent
    assert torch.equal(mxfp8_fake_quant_ref(torch.zeros(2, 32)), torch.zeros(2, 32))
    w = torch.randn(64, 8)
    assert torch.allclose(mxfp8_fake_quant_ref(w, axis=0), mxfp8_fake_quant_ref(w.t().contiguous(), axis=1).t())
    n4 = nvfp4_fake_quant_ref(torch.randn(4, 64))
    assert n4.unique().numel() < 4 * 64 and torch.equal(nvfp4_fake_quant_ref(torch.zeros(1, 16)), torch.zeros(1, 16))
    sf = ScaleFactor(history_len=3)
    for a in (2.0, 8.0, 1.0, 1.0):
        sf.update(a)
    assert sf.scale == 448.0 / 8.0
    sf.update(1.0)
    assert sf.scale == 448.0 / 1.0


def test_qat_surrogates():
    x = torch.linspace(-2, 2, 41).reshape(1, 41).repeat(2, 1).requires_grad_(True)
    for sur, check in (("straight_through", lambda g: torch.all(g == 1)),
                       ("piecewise_linear", lambda g: g[0, 0] == pytest.approx(0.1) and g[0, 20] == 1),
                       ("sigmoid_tempered", lambda g: g[0, 20] == pytest.approx(2.5) and g[0, 0] < 1e-6)):
        spec = QuantSpec("int_affine", bits=4, surrogate=sur)
        x.grad = None
        y = fake_quant_ste(x, spec)
        y.sum().backward()
        assert check(x.grad), sur
    q = fake_quant(x.detach(), QuantSpec("int_affine", bits=4))
    assert q.unique().numel() <= 16
    assert (fake_quant(x.detach(), QuantSpec("fp8_tensor")) - x.detach()).abs().max() < 0.1


# ------------------------------------------------------------------------------------------ optimisers
def _flat(shapes, dtype=torch.float32):
    ps = [torch.nn.Parameter(torch.randn(*s, dtype=dtype)) for s in shapes]
    return FlatParams([(f"p{i}", p) for i, p in enumerate(ps)]), ps


def test_flat_buffers_alias_parameters_and_segments():
    flat, ps = _flat([(8, 8), (8,), (4, 4)])
    assert all(p.data.data_ptr() >= flat.flat.data_ptr() for p in ps)
    ps[0].main_grad.fill_(2.0)
    o = flat.offsets[flat.params.index(ps[0])]
    assert flat.grads[o] == 2.0
    runs = flat.wd_ranges()
    assert runs[0][2] is True and runs[-1][2] is False and runs[0][0] == 0 and runs[-1][1] == flat.numel
    flat.zero_grad()
    assert flat.grads.abs().sum() == 0


def test_adamw_and_lion_match_reference_formulas():
    torch.manual_seed(0)
    flat, ps = _flat([(16, 16), (16,)])
    ref = [p.detach().clone().requires_grad_(True) for p in flat.params]
    opt = AdamW(flat, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, max_grad_norm=0.0)
    topt = torch.optim.AdamW([{"params": [ref[0]], "weight_decay": 0.1}, {"params": [ref[1]], "weight_decay": 0.0}], lr=1e-2,
                             betas=(0.9, 0.95), eps=1e-8)
    for _ in range(3):
        for p, r in zip(flat.params, ref):
            g = torch.randn_like(p)
            p.main_grad.copy_(g)
            r.grad = g.clone()
        opt.step()
        topt.step()
        opt.zero_grad()
    for p, r in zip(flat.params, ref):
        assert torch.allclose(p.data, r.data, atol=1e-6)
    flat2, _ = _flat([(4, 4)])
    p = flat2.params[0]
    before = p.data.clone()
    lion = Lion(flat2, lr=0.1, betas=(0.9, 0.99), weight_decay=0.0, max_grad_norm=0.0)
    p.main_grad.fill_(3.0)
    lion.step()
    assert torch.allclose(p.data, before - 0.1)            # sign update, magnitude independent of |g|
    assert torch.allclose(lion.m[:16], torch.full((16,), 0.03))     # the rest of the flat buffer is padding


def test_newton_schulz_orthogonalises_and_lion_muon_routes_by_rank():
    torch.manual_seed(1)
    m = torch.randn(32, 16)
    y = newton_schulz(m / m.norm(), 30)
    assert torch.allclose(y.t() @ y, torch.eye(16), atol=1e-3)
    flat, ps = _flat([(8, 8), (8,)])
    opt = LionMuon(flat, lr=0.1, max_grad_norm=0.0)
    for p in flat.params:
        p.main_grad.copy_(torch.randn_like(p))
    before = [p.data.clone() for p in flat.params]
    opt.step()
    i2 = [i for i, p in enumerate(flat.params) if p.dim() == 2][0]
    i1 = 1 - i2
    assert torch.allclose((flat.params[i1].data - before[i1]).abs(), torch.full((8,), 0.1), atol=1e-6)    # Lion: +-lr
    assert not torch.allclose(flat.params[i2].data, before[i2])


def test_clipping_loss_scaling_and_nonfinite_skip():
    g = [torch.full((25,), 2.0), torch.full((100,), 1.0)]
    c = GradientClipper("norm", 5.0)
    n = c.clip(g)
    assert n == pytest.approx(math.sqrt(200.0)) and GradientClipper.global_norm(g) == pytest.approx(5.0)
    assert GradientClipper("value", 0.5).clip([torch.tensor([2.0, -3.0])]) == pytest.approx(math.sqrt(13))
    flat, _ = _flat([(4, 4)])
    opt = AdamW(flat, lr=0.1, max_grad_norm=1.0)
    before = flat.flat.clone()
    flat.params[0].main_grad.fill_(float("inf"))
    opt.step()
    assert opt.skipped() and torch.equal(flat.flat, before)
    s = LossScaler(1024.0, dynamic=True, growth_interval=2)
    s.update(True)
    assert s.scale == 512.0
    s.update(False)
    s.update(False)
    assert s.scale == 1024.0


def test_lr_schedules():
    s = LRScheduler("linear_warmup_cosine", 1e-3, 1e-4, warmup_steps=10, total_steps=110)
    assert s.lr_at(0) == pytest.approx(1e-4) and s.lr_at(5) == pytest.approx(5e-4) and s.lr_at(10) == pytest.approx(1e-3)
    assert s.lr_at(60) == pytest.approx(5.5e-4) and s.lr_at(110) == pytest.approx(1e-4) and s.lr_at(500) == pytest.approx(1e-4)
    assert LRScheduler("constant", 3e-4).lr_at(77) == 3e-4
    assert LRScheduler("cosine", 1.0, 0.0, 0, 100).lr_at(50) == pytest.approx(0.5)
    assert LRScheduler("linear", 1.0, 0.0, 0, 100).lr_at(25) == pytest.approx(0.75)
    assert LRScheduler("polynomial", 1.0, 0.0, 0, 100).lr_at(50) == pytest.approx(0.25)


# -------------------------------------------------------------------------------------------- sharding
def test_rank_layout_and_param_sharding_roundtrip():
    assert global_rank(1, 2, 4) == 6 and mesh_coords(6, 4, 2) == (1, 2)
    assert [global_rank(0, t, 4) for t in range(4)] == [0, 1, 2, 3]          # TP ranks are contiguous
    full = torch.arange(8 * 24, dtype=torch.float32).reshape(8, 24)
    for kind in ("col", "row", "col_qkv", "col_gated", "vocab"):
        shards = [tpl.shard_param(full, kind, 4, r).clone() for r in range(4)]
        assert torch.equal(tpl.unshard_param(shards, kind), full), kind
    q = tpl.shard_param(full, "col_qkv", 4, 1)
    assert q.shape == (8, 6) and q[0].tolist() == [2, 3, 10, 11, 18, 19]      # heads 1 of Q, K and V


# ---------------------------------------------------------------------------------------------- models
def _cfg(name):
    warnings.simplefilter("ignore")
    c = Config.from_file(os.path.join(ROOT, "configs", name), env_override=False)
    c.checkpoint.dir = ""
    c.telemetry.log_file = ""
    return c


def test_gpt_matches_plain_pytorch_reimplementation():
    from elfa_b200.models.gpt import GPTModel
    cfg = _cfg("bench/smoke_cpu.yaml")
    m = GPTModel(cfg, device=torch.device("cpu"))
    assert m.count_parameters() == sum(p.numel() for _, p in m.named_checkpoint_parameters())
    names = [n for n, _ in m.named_checkpoint_parameters()]
    assert names[0] == "embed_tokens.weight" and "blocks.1.mlp_down.weight" in names and len(set(names)) == len(names)
    ids = torch.randint(0, 4096, (2, 32))
    tgt = torch.randint(0, 4096, (2, 32))
    loss = m(ids, tgt)
    F = torch.nn.functional
    x = m.embed_tokens[ids] + m.pos_embed[:32]
    for b in m.blocks:
        h = F.layer_norm(x, (128,), b.ln1.weight, b.ln1.bias, 1e-5)
        qkv = (h @ b.attn.w_qkv).view(2, 32, 3, 4, 32)
        q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(2, 32, 128)
        x = x + a @ b.attn.w_o
        h = F.layer_norm(x, (128,), b.ln2.weight, b.ln2.bias, 1e-5)
        x = x + F.gelu(h @ b.mlp.up, approximate="tanh") @ b.mlp.down
    logits = F.layer_norm(x, (128,), m.final_norm.weight, m.final_norm.bias, 1e-5) @ m.embed_tokens.t()
    ref = F.cross_entropy(logits.reshape(-1, 4096), tgt.reshape(-1))
    assert abs(loss.item() - ref.item()) < 1e-4
    assert torch.allclose(m(ids), logits, atol=1e-4)


def test_cpu_smoke_golden_curve_and_resume(tmp_path):
    from elfa_b200.trainer import Trainer
    cfg = _cfg("bench/smoke_cpu.yaml")
    cfg.checkpoint.dir = str(tmp_path / "ck")
    cfg.checkpoint.save_interval = 2
    t = Trainer(cfg, device=torch.device("cpu"), telemetry=False)
    losses = t.run(max_steps=4)
    assert abs(losses[0] - math.log(4096)) < 0.1 and all(math.isfinite(x) for x in losses)
    t2 = Trainer(cfg, device=torch.device("cpu"), telemetry=False)
    t2.resume(os.path.join(cfg.checkpoint.dir, "step_00000002"))
    cont = t2.run(max_steps=2)
    assert cont == pytest.approx(losses[2:], abs=1e-5)
    # a second run from scratch reproduces the curve bit for bit
    t3 = Trainer(cfg, device=torch.device("cpu"), telemetry=False)
    assert t3.run(max_steps=2) == losses[:2]


def test_efla_math_and_model_family():
    b = torch.tensor(1.0)
    assert eops.stable_coefficient(b, torch.tensor(0.0)).item() == pytest.approx(1.0)          # c(lam -> 0) = beta
    assert eops.stable_coefficient(b, torch.tensor(1.0)).item() == pytest.approx(1 - math.exp(-1))
    k = torch.tensor([[[[1.0, 0.0]]]])
    v = torch.tensor([[[[2.0, 3.0]]]])
    o, s = eops.efla_scan_ref(k, v, b)
    c = 1 - math.exp(-1)
    assert torch.allclose(s[0, 0], torch.tensor([[2 * c, 3 * c], [0.0, 0.0]])) and torch.allclose(o[0, 0, 0], torch.tensor([2 * c, 3 * c]))
    x = torch.randn(1, 10, 4)
    w = torch.randn(4, 3)
    y = eops.shortconv_ref(x, w)
    assert y.shape == x.shape and torch.allclose(y[0, 0], x[0, 0] * w[:, 0]) and torch.allclose(y[0, 2], x[0, 2] * w[:, 0] + x[0, 1] * w[:, 1] + x[0, 0] * w[:, 2])
    from elfa_b200.models.efla_model import EflaModel
    cfg = _cfg("smoke.yaml")
    cfg.model.dtype = "fp32"
    m = EflaModel(cfg, device=torch.device("cpu"))
    names = [n for n, _ in m.named_checkpoint_parameters()]
    assert names[:5] == ["embed_tokens.weight", "blocks.0.ln1.weight", "blocks.0.efla.w_k", "blocks.0.efla.w_v", "blocks.0.efla.w_o"]
    assert "blocks.0.prism.w_p.1" in names and "blocks.1.prism.shortconv.weight" in names and names[-1] == "final_norm.weight"
    assert m.count_parameters() == sum(p.numel() for p in m.parameters())
    assert dict(m.named_checkpoint_parameters())["blocks.0.efla.beta_param"].dtype == torch.float32


# ------------------------------------------------------------------------------------------------ eval
def test_sampling_rouge_and_generators():
    logits = torch.tensor([0.0, 10.0, 0.0, 9.0])
    assert sample_top_p(logits, temperature=0.0) == 1
    g = torch.Generator().manual_seed(0)
    draws = {sample_top_p(logits, 1.0, 0.9, g) for _ in range(50)}
    assert draws <= {1, 3}
    assert lcs_length([1, 2, 3, 4], [2, 4, 5]) == 2
    assert rouge_n([1, 2, 3], [1, 2, 4], 1)["f1"] == pytest.approx(2 / 3) and rouge_l([1, 2, 3], [1, 2, 3])["f1"] == 1.0
    c = generate_needle_case(200, 1000, 7)
    assert c.tokens[c.position] == 1 and c.tokens[c.position + 3:c.position + 7] == c.answer and c.tokens[-3] == 1
    s = generate_summary_case(300, 1000, 3)
    assert score_summary(s, s.reference)["coverage"] == 1.0
    from elfa_b200.models.gpt import GPTModel
    m = GPTModel(_cfg("bench/smoke_cpu.yaml"), device=torch.device("cpu"))
    out = Generator(m).generate_greedy([5, 6, 7], 4)
    assert len(out) == 7 and out[:3] == [5, 6, 7]


def test_fused_collective_oracles_equal_the_unsharded_computation():
    """N simulated ranks: all-gather->GEMM, GEMM->reduce-scatter, reduce-scatter + AdamW + all-gather and the ZeRO-3
    gather in front of a GEMM give what one rank computes on the whole tensors."""
    from elfa_b200.ref import collectives as C
    g = torch.Generator().manual_seed(0)
    n, M, K, N = 4, 32, 24, 40
    x = torch.randn(M, K, generator=g, dtype=torch.float64)
    w = torch.randn(K, N, generator=g, dtype=torch.float64)
    ys = C.ag_gemm(list(x.chunk(n, 0)), list(w.chunk(n, 1)))                  # column parallel
    assert torch.allclose(torch.cat(ys, 1), x @ w)
    outs = C.gemm_rs(list(x.chunk(n, 1)), list(w.chunk(n, 0)))                # row parallel
    assert torch.allclose(torch.cat(outs, 0), x @ w)
    ys3 = C.zero3_gather_gemm([x, 2 * x], list(w.reshape(-1).chunk(n, 0)), (K, N))
    assert torch.allclose(ys3[1], 2 * (x @ w))
    # ZeRO-1/2 step against single-rank AdamW on the averaged, clipped gradient
    P = 64
    p0 = torch.randn(P, generator=g)
    grads = [torch.randn(P, generator=g) * 8.0 for _ in range(n)]             # "loss-scaled" by 8
    master = [c.clone() for c in p0.chunk(n, 0)]
    m = [torch.zeros(P // n) for _ in range(n)]
    v = [torch.zeros(P // n) for _ in range(n)]
    got, norm = C.rs_adamw_ag(grads, master, m, v, step=1, lr=1e-2, loss_scale=8.0, max_norm=0.5, param_dtype=torch.float32)
    g_avg = sum(grads) / (n * 8.0)
    ref_norm = float(g_avg.norm())
    assert abs(norm - ref_norm) < 1e-5 and norm > 0.5
    p_ref, m_ref, v_ref = p0.clone(), torch.zeros(P), torch.zeros(P)
    C.adamw_update(p_ref, g_avg * (0.5 / (ref_norm + 1e-6)), m_ref, v_ref, 1, 1e-2, 0.9, 0.95, 1e-8, 0.1)
    assert all(torch.allclose(t, p_ref, atol=1e-6) for t in got)
    # the oracle's AdamW is torch's (which the framework's optimizer is tested against above)
    q = torch.randn(16, generator=g).requires_grad_(True)
    q2, mq, vq = q.detach().clone(), torch.zeros(16), torch.zeros(16)
    topt = torch.optim.AdamW([q], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in (1, 2, 3):
        gr = torch.randn(16, generator=g)
        q.grad = gr.clone()
        topt.step()
        C.adamw_update(q2, gr, mq, vq, step, 1e-2, 0.9, 0.95, 1e-8, 0.1)
    assert torch.allclose(q.detach(), q2, atol=1e-6)


@pytest.mark.parametrize("B,T,H,d,C,with_state", [(2, 50, 2, 16, 16, True), (1, 128, 2, 32, 64, False), (1, 37, 1, 8, 64, True)])
def test_efla_chunk_parallel_form_equals_the_sequential_recurrence(B, T, H, d, C, with_state):
    """WY / chunk-parallel restatement (triangular solve per chunk, T / C sequential steps) against the token-by-token
    oracle: outputs, final state and every gradient (keys, values, beta, initial state)."""
    from elfa_b200.ops.efla import efla_scan_chunked_ref, efla_scan_ref
    torch.manual_seed(T)
    k = (torch.randn(B, T, H, d) * 0.5).requires_grad_(True)
    v = torch.randn(B, T, H, d).requires_grad_(True)
    beta = torch.tensor(0.8, requires_grad=True)
    s0 = (0.1 * torch.randn(B, H, d, d)).requires_grad_(True) if with_state else None
    ins = [k, v, beta] + ([s0] if with_state else [])
    o, s = efla_scan_ref(k, v, beta, s0)
    go, gs = torch.randn_like(o), torch.randn_like(s)
    g_ref = torch.autograd.grad([o, s], ins, [go, gs])
    o2, s2 = efla_scan_chunked_ref(k, v, beta, s0, C)
    g_chk = torch.autograd.grad([o2, s2], ins, [go, gs])
    assert o2.shape == o.shape and (o - o2).abs().max() < 1e-4 and (s - s2).abs().max() < 1e-4
    for a, b in zip(g_ref, g_chk):
        assert (a - b).abs().max() < 1e-4 * max(1.0, a.abs().max().item())


def test_packed_rows_equal_separate_documents_and_gqa_shapes():
    """A row of two packed documents (doc_start) gives each document the logits it gets on its own; grouped-query
    attention trains and checkpoints with its [query | key | value] projection."""
    import os
    from elfa_b200.config import Config
    from elfa_b200.models.gpt import GPTModel
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = Config.from_file(os.path.join(root, "configs", "bench", "smoke_cpu.yaml"), env_override=False)
    cfg.model.dtype = "fp32"
    cfg.model.num_kv_heads = 2
    m = GPTModel(cfg, device=torch.device("cpu"))
    assert m.blocks[0].attn.w_qkv.shape[1] == (cfg.model.num_heads + 2 * 2) * cfg.model.head_dim
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.model.vocab_size, (1, 48), generator=g)
    doc = torch.zeros(1, 48, dtype=torch.int32)
    doc[:, 20:] = 20
    with torch.no_grad():
        packed = m.hidden_states(ids, doc_start=doc)
        first = m.hidden_states(ids[:, :20])
        second = m.hidden_states(ids[:, 20:])
    assert torch.allclose(packed[:20], first, atol=1e-5) and torch.allclose(packed[20:], second, atol=1e-5)
    from elfa_b200.data.packing import document_starts
    import numpy as np
    ends = np.zeros((1, 8), dtype=bool)
    ends[0, 2] = ends[0, 5] = True
    assert document_starts(ends).tolist() == [[0, 0, 0, 3, 3, 3, 6, 6]]
