"""Descriptors, RNGs, layout helpers, optimizer-state quantisation, offload, sequence-parallel helpers (CPU)."""
import os
import subprocess
import sys

import pytest
import torch

from elfa_b200.parallel.descriptors import ParallelConfig, SequenceParallelConfig, ShardSpec, TensorParallelConfig, ZeroConfig, split_sizes
from elfa_b200.quant import optstate
from elfa_b200.runtime.offload import HostOffloader, NvmeStore
from elfa_b200.utils.layout import HostMemoryPool, PaddingStrategy, TensorCoreTiles
from elfa_b200.utils.rng import DeterministicRng, DistributedRng, PhiloxRng

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_arithmetic():
    assert ShardSpec(0, 4, 1).local_shape((128, 7)) == (32, 7)
    assert SequenceParallelConfig(4, 1).local_range(1000) == (250, 250)
    assert split_sizes(10, 4) == [3, 3, 2, 2] and ShardSpec(0, 4, 2).offset(10) == 6
    z = ZeroConfig(stage=2, partitions=4, rank=1)
    assert z.owner_of(0) == 0 and z.owner_of(1 << 20) == 1 and z.owner_of(5 << 20) == 1 and z.owns((1 << 20) + 5)
    assert z.should_shard_optimizer() and z.should_shard_gradients() and not z.should_shard_params()
    assert z.flat_range(4096) == (1024, 2048)
    assert TensorParallelConfig(8, 3).spec(1).local_size(4096) == 512
    p = ParallelConfig(dp_size=2, tp_size=4, dp_rank=1, tp_rank=2)
    assert p.global_rank() == 6 and p.world_size() == 8
    q = ParallelConfig.from_global_rank(6, dp=2, tp=4)
    assert (q.dp_rank, q.tp_rank) == (1, 2)


def test_rngs_are_deterministic_and_rank_streams_differ():
    a, b = DeterministicRng(42), DeterministicRng(42)
    assert [a.next_u32() for _ in range(5)] == [b.next_u32() for _ in range(5)]
    assert DeterministicRng(1).next_u32() != DeterministicRng(2).next_u32()
    r = DeterministicRng(7)
    assert all(0 <= r.range(10) < 10 for _ in range(100)) and all(0.0 <= r.uniform() < 1.0 for _ in range(100))
    xs = [r.normal() for _ in range(4000)]
    m = sum(xs) / len(xs)
    assert abs(m) < 0.1 and abs(sum((x - m) ** 2 for x in xs) / len(xs) - 1.0) < 0.15
    items = list(range(20))
    DeterministicRng(3).shuffle(items)
    assert sorted(items) == list(range(20)) and items != list(range(20))
    d0, d1 = DistributedRng(5, 0), DistributedRng(5, 1)
    assert d0["data"].next_u32() != d1["data"].next_u32() and d0["init"].next_u32() != d0["dropout"].next_u32()
    ph = PhiloxRng(123)
    assert ph.at(9) == PhiloxRng(123).at(9) and ph.at(9) != ph.at(10)


def test_layout_helpers_and_host_pool():
    assert PaddingStrategy(128).padded_bytes(130) == 256 and PaddingStrategy(128).optimal_leading_dimension(1000, 2) == 1024
    assert TensorCoreTiles().block_m == 128 and TensorCoreTiles().tmem_columns == 512
    pool = HostMemoryPool(4096, 128)
    a, b, c = pool.alloc(1000), pool.alloc(1000), pool.alloc(1000)
    assert (a, b, c) == (0, 1024, 2048) and pool.bytes_in_use() == 3072
    pool.release(b)
    assert pool.alloc(512) == 1024                     # best fit reuses the hole
    pool.release(a)
    pool.release(c)
    with pytest.raises(MemoryError):
        pool.alloc(4096)
    pool.release(1024)
    assert pool.free == [(0, 4096)]                    # fully coalesced


def test_optimizer_state_quantisation_bounds():
    torch.manual_seed(0)
    x = torch.randn(1000) * 3
    q, s = optstate.quantize_int8_absmax(x)
    assert (optstate.dequantize_int8_absmax(q, s) - x).abs().max() <= s * 0.5 + 1e-6
    for bits in (8, 4):
        codes, scale, zp, n = optstate.quantize_blockwise(x, bits, 128)
        back = optstate.dequantize_blockwise(codes, scale, zp, n, bits, 128)
        assert back.shape == x.shape and (back - x).abs().max() <= scale.max() * 0.5 + 1e-5
        assert codes.numel() == (1024 if bits == 8 else 512)
    assert optstate.fake_quantize_state(x, 32) is x and optstate.fake_quantize_state(x, 8).unique().numel() <= 255
    u, s8, lo = optstate.quantize_dynamic_u8(x)
    assert (optstate.dequantize_dynamic_u8(u, s8, lo) - x).abs().max() <= s8 * 0.5 + 1e-5


def test_offload_roundtrips(tmp_path):
    off = HostOffloader(torch.device("cpu"))
    t = torch.randn(64, 32).to(torch.bfloat16)
    off.offload("m", t)
    out = torch.empty_like(t)
    off.prefetch("m", out)
    off.wait("m")
    assert torch.equal(out, t)
    from elfa_b200.runtime.offload import PinnedPool
    pool = PinnedPool(4096, pin=False)
    a = pool.alloc((10, 3), torch.float32)
    b = pool.alloc((7,), torch.bfloat16)
    assert a.shape == (10, 3) and b.dtype == torch.bfloat16 and a.data_ptr() % 256 == pool.slab.data_ptr() % 256
    assert b.data_ptr() - a.data_ptr() == 256 and pool.bytes_free() == 4096 - 256 - 14
    a.fill_(1.0)
    b.fill_(2.0)
    assert float(a.sum()) == 30.0                       # the views do not overlap
    with pytest.raises(MemoryError):
        pool.alloc((5000,), torch.uint8)
    pool.reset()
    assert pool.bytes_free() == 4096 and pool.peak == 256 + 14
    store = NvmeStore(str(tmp_path / "nvme"))
    store.write("m", off.mirrors["m"]).wait()
    back = torch.empty_like(t)
    store.read("m", back).wait()
    store.flush()
    store.close()
    assert torch.equal(back, t)


def test_sequence_parallel_helpers_over_gloo():
    code = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, %r)
from elfa_b200.parallel import sp
from elfa_b200.ops import efla as eops
dist.init_process_group("gloo")
r, w = dist.get_rank(), dist.get_world_size()
torch.manual_seed(0)
x = torch.arange(2 * 10 * 3, dtype=torch.float32).reshape(2, 10, 3)
loc = sp.split_sequence(x, r, w)
assert torch.equal(sp.gather_sequence(loc), x)
got = sp.ring_exchange(torch.full((2,), float(r)), 1)
assert got[0].item() == (r - 1) %% w
halo = sp.halo_from_left(loc, 2)
want = torch.zeros(2, 2, 3) if r == 0 else x[:, sum(sp.ShardSpec(1, w, i).local_size(10) for i in range(r)) - 2:][:, :2]
assert torch.equal(halo, want)
k = torch.randn(1, 12, 2, 8) * 0.4; v = torch.randn(1, 12, 2, 8); beta = torch.tensor(0.9)
kl, vl = sp.split_sequence(k, r, w), sp.split_sequence(v, r, w)
s_in = sp.efla_cross_rank_state(kl, vl, beta)
o_loc, _ = eops.efla_scan_ref(kl, vl, beta, s_in)
o_full, _ = eops.efla_scan_ref(k, v, beta)
assert (o_loc - sp.split_sequence(o_full, r, w)).abs().max() < 1e-4
g = torch.ones(4 * w, 3) * (r + 1)
assert torch.equal(sp.reduce_scatter_gradients(g), torch.full((4, 3), float(sum(range(1, w + 1)))))
if r == 0: print("SP_OK")
''' % ROOT
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29631", "-c", code]
    # torch.distributed.run needs a script path: write it out
    path = os.path.join("/tmp", "elfa_sp_worker.py")
    with open(path, "w") as f:
        f.write(code)
    cmd = cmd[:-2] + [path]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0 and "SP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_loss_history_moving_average_early_stop_manifest(tmp_path):
    import json
    from elfa_b200.utils.history import LossHistory
    h = LossHistory()
    for i, x in enumerate([5.0, 4.0, 3.0, 2.5, float("nan"), 2.4]):
        h.record(i + 1, x)
    assert h.best() == 2.4 and abs(h.moving_average(3) - (2.5 + 2.4) / 2) < 1e-9
    assert not h.should_stop_early(patience=2)
    for i in range(4):
        h.record(10 + i, 2.45)
    assert h.should_stop_early(patience=3) and not h.should_stop_early(patience=3, min_delta=-1.0)
    h.record_eval(12, perplexity=11.0)
    doc = json.load(open(h.write_manifest(str(tmp_path / "run"), {"config_hash": "abc"})))
    assert doc["num_steps"] == 10 and doc["best_loss"] == 2.4 and doc["evals"][0]["perplexity"] == 11.0 and doc["config_hash"] == "abc"


def test_entropy_tokenizer_roundtrip_merges_and_file(tmp_path):
    from elfa_b200.data.entropy_tokenizer import BOS, EOD, EOS, EntropyTokenizer
    tok = EntropyTokenizer(400)
    texts = ["the cat sat on the mat.", "the dog sat, the cat ran!", "that is the end"]
    plain = tok.encode(texts[0])
    assert plain[0] == BOS and plain[-1] == EOS and all(6 <= t < 262 for t in plain[1:-1])
    tok.train(texts, 20)
    ids = tok.encode(texts[0])
    assert len(ids) < len(plain) and tok.decode(ids) == texts[0].encode()
    assert tok.decode(tok.encode("zebra: ünïcode")) == "zebra: ünïcode".encode()
    p = str(tmp_path / "tok.bin")
    tok.save(p)
    tok2 = EntropyTokenizer(400)
    tok2.load(p)
    assert tok2.encode(texts[1]) == tok.encode(texts[1]) and tok2.eod_token() == EOD
    b = tok.batch(ids, 8)
    assert b.tokens == ids[:8] and b.targets == ids[1:9]


def test_hash_helpers(tmp_path):
    from elfa_b200.utils import hashing as H
    assert H.sha256_hex(b"abc") == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"
    p = tmp_path / "f.bin"
    p.write_bytes(b"x" * 3_000_000)
    assert H.sha256_file(str(p)) == H.sha256_bytes(b"x" * 3_000_000) and H.verify_sha256(b"abc", H.sha256_bytes(b"abc"))
    # XXH64 reference vectors (seed 0): empty input and "a"
    assert H.xxh64(b"") == 0xEF46DB3751D8E999 and H.xxh64(b"a") == 0xD24EC4F1A98C6E5B
    assert H.xxh64(b"a" * 100) != H.xxh64(b"a" * 101) and H.hash_string("k") == H.xxh64(b"k")
    assert H.combine(1, 2) != H.combine(2, 1) and H.hash_fields([1, "a", 2.5]) != H.hash_fields([1, "a", 2.0])


def test_native_header_parses_and_library_exports_every_prototype():
    """Every prototype of the C header maps to ctypes types, and the built library (when present) exports it."""
    import ctypes
    from elfa_b200 import native
    protos = native._parse_header(native._HEADER.read_text())
    assert len(protos) > 40 and "elfa_gemm_bf16" in protos and "elfa_p2p_send" in protos
    if native._LIB_PATH.exists():
        dll = ctypes.CDLL(str(native._LIB_PATH))
        missing = [n for n in protos if not hasattr(dll, n)]
        assert not missing, missing


def test_efla_model_sequence_parallel_forward_matches_single_rank(tmp_path):
    """Halo + affine-state hand-off per layer: every rank's logits equal its slice of the whole-sequence forward."""
    code = r'''
import sys, torch, torch.distributed as dist
sys.path.insert(0, %r)
from elfa_b200.config import Config
from elfa_b200.models.efla_model import EflaModel
from elfa_b200.parallel import sp
dist.init_process_group("gloo")
r, w = dist.get_rank(), dist.get_world_size()
cfg = Config.from_file(%r, env_override=False)
cfg.model.dtype = "fp32"
cfg.model.num_layers = 2
m = EflaModel(cfg, device=torch.device("cpu")).eval()
torch.manual_seed(1)
ids = torch.randint(0, cfg.model.vocab_size, (2, 96))
with torch.no_grad():
    full = m(ids)
    loc = m.forward_sequence_parallel(sp.split_sequence(ids, r, w))
    naive = m(sp.split_sequence(ids, r, w))
want = sp.split_sequence(full, r, w)
assert (loc - want).abs().max() < 1e-3 * want.abs().max() + 1e-4
assert r == 0 or (naive - want).abs().max() > 0.1          # without the hand-off the later blocks are wrong
dist.barrier()
if r == 0: print("SP_MODEL_OK")
''' % (ROOT, os.path.join(ROOT, "configs", "smoke.yaml"))
    path = str(tmp_path / "sp_model_worker.py")
    with open(path, "w") as f:
        f.write(code)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29672", path]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0 and "SP_MODEL_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_efla_model_sequence_parallel_training_matches_single_rank(tmp_path):
    """Sequence-parallel training of the EFLA family: the loss and every parameter gradient (summed over the ranks) equal
    the single-rank run on the whole sequence - the state hand-off and the ShortConv halo are differentiated through."""
    code = r'''
import sys, torch, torch.distributed as dist
sys.path.insert(0, %r)
from elfa_b200.config import Config
from elfa_b200.models.efla_model import EflaModel
from elfa_b200.parallel import sp
dist.init_process_group("gloo")
r, w = dist.get_rank(), dist.get_world_size()
cfg = Config.from_file(%r, env_override=False)
cfg.model.dtype = "fp32"
cfg.model.num_layers = 2
cfg.bench.init_std = 0.005      # small keys: with the default init |k|^2 saturates the delta rule (o_t = v_t) and dL/dk is noise
m = EflaModel(cfg, device=torch.device("cpu"))
torch.manual_seed(1)
ids = torch.randint(0, cfg.model.vocab_size, (2, 97))
inp, tgt = ids[:, :96], ids[:, 1:]
denom = float(tgt.numel())
loss_full = m(inp, tgt, loss_denominator=denom)
loss_full.backward()
ref = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
m.zero_grad()
loss_loc = m(sp.split_sequence(inp, r, w), sp.split_sequence(tgt, r, w), loss_denominator=denom, sp_group=dist.group.WORLD)
loss_loc.backward()
tot = loss_loc.detach().clone()
dist.all_reduce(tot)
assert abs(float(tot) - float(loss_full)) < 1e-4 * abs(float(loss_full)), (float(tot), float(loss_full))
worst = 0.0
scale = max(v.abs().max().item() for v in ref.values())
for n, p in m.named_parameters():
    if n not in ref:
        continue
    g = p.grad.clone() if p.grad is not None else torch.zeros_like(p)
    dist.all_reduce(g)
    e = (g - ref[n]).abs().max().item() / (ref[n].abs().max().item() + 1e-6 * scale)
    worst = max(worst, e)
    assert e < 2e-3, (n, e)
dist.barrier()
if r == 0: print("SP_TRAIN_OK", worst)
''' % (ROOT, os.path.join(ROOT, "configs", "smoke.yaml"))
    path = str(tmp_path / "sp_train_worker.py")
    with open(path, "w") as f:
        f.write(code)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29673", path]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2", CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0 and "SP_TRAIN_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_launcher_runs_a_command_and_resolves_latest_checkpoint(tmp_path):
    from elfa_b200 import launch
    r = subprocess.run([sys.executable, "-m", "elfa_b200.launch", "--gpus", "1", "version"], capture_output=True, text=True, timeout=300,
                       cwd=ROOT, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0 and "elfa" in (r.stdout + r.stderr).lower()
    assert launch.resolve_resume(["train", "--config", "x.yaml"]) == ["train", "--config", "x.yaml"]
    ck = tmp_path / "ck"
    (ck / "step_3").mkdir(parents=True)
    (ck / "step_12").mkdir()
    try:
        out = launch.resolve_resume(["train", "--checkpoint-dir", str(ck), "--resume", "latest"])
        assert out[-1].endswith("step_12")
    except (FileNotFoundError, ValueError, SystemExit):
        pass          # directories without a manifest are not checkpoints for the resolver: that refusal is fine too


def test_flag_protocol_models_with_threads_as_ranks():
    """The slot / counter rules of the fused all-gather and of the neighbour mailbox, run with one thread per
    rank and random delays: two slots are safe, one slot is not, a missing signal ends in a timeout status."""
    from elfa_b200.runtime.protocol_model import TIMEOUT, MailboxModel, PushGatherModel
    for seed in range(3):
        ranks = PushGatherModel(4, ring=2, seed=seed).run(40)
        assert all(r.status == 0 and not r.errors for r in ranks), [r.errors[:2] for r in ranks]
    broken = 0
    for seed in range(20):           # negative control: a single slot is overwritten before slow ranks have read it
        ranks = PushGatherModel(4, ring=1, seed=seed).run(60)
        broken += any(r.errors for r in ranks)
        if broken:
            break
    assert broken > 0
    ranks = PushGatherModel(3, ring=2, seed=1, wait_limit_s=0.3, skip_signal=(1, 2)).run(6)
    assert any(r.status == TIMEOUT for r in ranks)           # bounded: every thread returned
    ranks = MailboxModel(4, seed=2).run(50)
    assert all(r.status == 0 and not r.errors for r in ranks), [r.errors[:2] for r in ranks]
    from elfa_b200.runtime.protocol_model import BarrierModel
    ranks = BarrierModel(4, seed=3).run(40)
    assert all(r.status == 0 and not r.errors for r in ranks), [r.errors[:2] for r in ranks]
    ranks = BarrierModel(3, seed=4, wait_limit_s=0.3, absent=(2, 5)).run(8)       # a rank leaves before barrier 5
    assert ranks[0].status == TIMEOUT and ranks[1].status == TIMEOUT and not any(r.errors for r in ranks)


def test_phase_timer_and_chrome_trace(tmp_path):
    import json
    import torch
    from elfa_b200.utils.tracing import PhaseTimer, nvtx_range
    t = PhaseTimer(torch.device("cpu"), active=True)
    for _ in range(3):
        with t.phase("forward"):
            with nvtx_range("inner"):
                torch.randn(64, 64) @ torch.randn(64, 64)
        with t.phase("backward"):
            pass
    s = t.summary()
    assert s["forward"]["calls"] == 3 and s["backward"]["calls"] == 3 and s["forward"]["ms"] >= 0.0
    t.write_chrome_trace(str(tmp_path / "trace.json"))
    ev = json.load(open(tmp_path / "trace.json"))["traceEvents"]
    assert len(ev) == 6 and ev[0]["name"] == "forward" and ev[0]["ph"] == "X"
    off = PhaseTimer(torch.device("cpu"), active=False)
    with off.phase("x"):
        pass
    assert off.summary() == {}


def test_error_codes_finite_checks_and_overrides():
    import math
    import torch
    from elfa_b200.config import Config
    from elfa_b200.utils.errors import NotFiniteError, TrainingError, apply_overrides, check_finite, parse_key_value
    check_finite(1.0)
    check_finite(torch.zeros(4, 4))
    with pytest.raises(NotFiniteError) as e:
        check_finite(math.nan)
    assert e.value.code == "NaN" and e.value.area == "training"
    with pytest.raises(NotFiniteError) as e:
        check_finite(torch.tensor([1.0, float("inf")]), "loss")
    assert e.value.code == "Inf" and "loss" in str(e.value)
    err = TrainingError("CheckpointCorrupted", "sha256 mismatch")
    assert err.area == "checkpoint" and "CheckpointCorrupted: sha256 mismatch" in str(err) and err.file.endswith("test_cpu_misc.py")
    with pytest.raises(ValueError):
        TrainingError("NoSuchCode")
    assert parse_key_value("a=b, c.d = e ,junk,x=1=2") == {"a": "b", "c.d": "e", "x": "1=2"}
    cfg = Config.from_file(os.path.join(ROOT, "configs", "smoke.yaml"), env_override=False)
    apply_overrides(cfg, parse_key_value("training.learning_rate=1e-4,runtime.zero_stage=1,runtime.sequence_parallel=false,model.name=x"))
    assert cfg.training.learning_rate == 1e-4 and cfg.runtime.zero_stage == 1 and cfg.runtime.sequence_parallel is False
    assert cfg.model.name == "x"
    with pytest.raises(TrainingError):
        apply_overrides(cfg, {"training.no_such_key": "1"})
    with pytest.raises(TrainingError):
        apply_overrides(cfg, {"runtime.zero_stage": "many"})


def test_trainer_reports_phase_times_when_tracing_is_on():
    from elfa_b200.config import Config
    from elfa_b200.trainer import Trainer
    from elfa_b200.utils import tracing
    cfg = Config.from_file(os.path.join(ROOT, "configs", "bench", "smoke_cpu.yaml"), env_override=False)
    cfg.checkpoint.dir = ""
    cfg.telemetry.log_file = ""
    tracing.enable(True)
    try:
        tr = Trainer(cfg, device=torch.device("cpu"), telemetry=False)
        tr.run(max_steps=2)
        s = tr.tracer.summary()
    finally:
        tracing.enable(False)
    assert set(s) == {"forward", "backward", "optimizer"}
    assert s["optimizer"]["calls"] == 2 and s["forward"]["calls"] == s["backward"]["calls"] >= 2
    assert all(v["ms"] > 0 for v in s.values())


def test_gpt_incremental_decoding_matches_full_forward():
    """Key / value cache: prompt in one call, then token by token - the logits equal those of a forward pass over
    the whole sequence, and greedy generation gives the same tokens with and without the cache."""
    from elfa_b200.config import Config
    from elfa_b200.eval.evaluator import Generator
    from elfa_b200.models.gpt import GPTModel
    cfg = Config.from_file(os.path.join(ROOT, "configs", "bench", "smoke_cpu.yaml"), env_override=False)
    model = GPTModel(cfg, None, torch.device("cpu"))
    model.reset_parameters(3)
    model.eval()
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.model.vocab_size, (2, 24), generator=g)
    with torch.no_grad():
        full = model(ids)                                            # [B, S, V]
        logits, st = model.forward_with_states(ids[:, :10])
        parts = [logits]
        for t in range(10, 20):
            logits, st = model.forward_with_states(ids[:, t:t + 1], st)
            parts.append(logits)
        logits, st = model.forward_with_states(ids[:, 20:24], st)   # several new tokens at once
        parts.append(logits)
    inc = torch.cat(parts, 1)
    assert st["pos"] == 24 and inc.shape == full.shape
    assert (inc - full).abs().max().item() < 2e-4
    gen = Generator(model, device=torch.device("cpu"))
    with_cache = gen.generate_greedy([5, 6, 7], 12)
    model_max = cfg.model.max_seq_len
    try:
        cfg.model.max_seq_len = 8        # positions "run out": the generator takes the windowed path (positions stay valid: 15 <= real table)
        windowed = gen.generate_greedy([5, 6, 7], 12)
    finally:
        cfg.model.max_seq_len = model_max
    assert with_cache == windowed and len(with_cache) == 15


def test_ring_attention_block_schedule_covers_the_causal_triangle_evenly():
    from elfa_b200.parallel.ring_attention import block_schedule, zigzag_slices
    for world in (2, 3, 8):
        # contiguous split: rank r computes r full blocks and one masked one
        for r in range(world):
            sched = [block_schedule(r, j, True, False) for j in range(world)]
            assert sum(len(s) for s in sched) == r + 1 and sched[r] == [(0, 0, True)]
        # zig-zag split: every (query chunk, key chunk) pair of the 2N-chunk causal triangle appears exactly once ...
        seen = set()
        work = []
        for r in range(world):
            chunk_of = lambda rank, part: rank if part == 0 else 2 * world - 1 - rank
            w = 0.0
            for j in range(world):
                for qi, ki, masked in block_schedule(r, j, True, True):
                    qc, kc = chunk_of(r, qi), chunk_of(j, ki)
                    assert (qc, kc) not in seen and (kc < qc or (kc == qc and masked)) and (masked == (kc == qc))
                    seen.add((qc, kc))
                    w += 0.5 if masked else 1.0
            work.append(w)
        n2 = 2 * world
        assert seen == {(q, k) for q in range(n2) for k in range(q + 1)}
        assert len(set(work)) == 1                      # ... and every rank has the same amount of work
        (a0, a1), (b0, b1) = zigzag_slices(64 * n2, 1, world)
        assert (a0, a1) == (64, 128) and (b0, b1) == (64 * (n2 - 2), 64 * (n2 - 1))


def test_ncu_summary_reads_raw_csv():
    from elfa_b200.utils import ncu_summary
    text = "\n".join([
        "==PROF== noise that is not CSV",
        '"ID","Kernel Name","gpu__time_duration.sum","launch__grid_size","smsp__average_warps_issue_stalled_wait_per_issue_active.ratio",'
        '"smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio","smsp__average_warps_issue_stalled_selected_per_issue_active.ratio"',
        '"","","us","","inst","inst","inst"',
        '"0","my_kernel<64>(const float *)","12.5","148","1.25","0.5","1.0"',
    ])
    launches = ncu_summary.parse(text)
    assert len(launches) == 1 and launches[0]["gpu__time_duration.sum"] == "12.5 us"
    md = ncu_summary.summarise(launches[0])
    assert "my_kernel<64>" in md and "| duration | 12.5 us |" in md and "| grid | 148 |" in md
    assert "wait 1.25, barrier 0.50" in md and "selected" not in md


@pytest.mark.parametrize("nvme", [False, True])
def test_optimizer_state_offload_between_steps(tmp_path, nvme):
    """runtime.cpu_offload / nvme_offload: the moments leave the device after every step and come back for the next;
    the loss curve and a save / resume are the same as without offload."""
    from elfa_b200.config import Config
    from elfa_b200.trainer import Trainer

    def run(offload, ckpt_dir=""):
        cfg = Config.from_file(os.path.join(ROOT, "configs", "bench", "smoke_cpu.yaml"), env_override=False)
        cfg.checkpoint.dir = ckpt_dir
        cfg.checkpoint.save_interval = 0
        cfg.telemetry.log_file = ""
        cfg.runtime.cpu_offload = offload and not nvme
        cfg.runtime.nvme_offload = offload and nvme
        cfg.runtime.nvme_path = str(tmp_path / "nvme")
        return Trainer(cfg, device=torch.device("cpu"), telemetry=False)

    base = run(False)
    ref = base.run(max_steps=4)
    tr = run(True, str(tmp_path / "ck"))
    assert tr.offload is not None and tr.offload.device_bytes() == 0 and len(tr.offload.tensors) >= 2
    got = tr.run(max_steps=2)
    assert tr.offload.device_bytes() == 0                 # evicted again after the step
    path = tr.save_checkpoint()
    tr.close()
    tr2 = run(True, str(tmp_path / "ck"))
    tr2.resume(path)
    got += tr2.run(max_steps=2)
    tr2.close()
    assert got == pytest.approx(ref, abs=1e-5)


def test_launcher_restarts_a_failed_job_from_its_newest_checkpoint(tmp_path):
    """A rank leaves between steps on the first start (host-side fault plan); the launcher starts the job again, which
    resumes from the last checkpoint and finishes."""
    ck = str(tmp_path / "ck")
    launch = [sys.executable, "-m", "elfa_b200.launch", "--gpus", "1"]
    train = ["train", "--config", os.path.join(ROOT, "configs", "bench", "smoke_cpu.yaml"), "--checkpoint-dir", ck,
             "--set", "checkpoint.save_interval=2,training.total_steps=6,telemetry.log_file="]
    cmd = launch + ["--max-restarts", "1"] + train
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", ELFA_FAULT="kill_rank:step=3,attempt=0,code=17")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0, out[-3000:]
    assert "exit code 17: restart 1 of 1" in out and "resumed from step 2" in out and "finished at step 6" in out
    # without restarts the same fault ends the job with the rank's exit code
    r = subprocess.run(launch + train, capture_output=True, text=True, timeout=600, cwd=ROOT,
                       env=dict(env, ELFA_FAULT="kill_rank:step=1,code=17"))
    assert r.returncode == 17


def test_bench_reference_arm_reports_unavailable_as_json():
    import json
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1"], capture_output=True,
                       text=True, timeout=300, cwd=ROOT, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and len(line["unavailable"]) > 10
    # argument checks that need no GPU: the twin is a single-process aid, N ranks need the distributed launcher
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", WORLD_SIZE="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--twin", "4", "--gpus", "2"], capture_output=True, text=True,
                       timeout=300, cwd=ROOT, env=env)
    assert r.returncode == 2 and "--twin" in r.stderr
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], capture_output=True, text=True, timeout=300,
                       cwd=ROOT, env=env)
    assert r.returncode == 2 and "WORLD_SIZE" in r.stderr


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_bench_takes_the_headline_branch_at_every_world_size(world, monkeypatch):
    """The launcher's WORLD_SIZE must not change which branch of bench.py a configuration file selects."""
    import importlib.util
    from elfa_b200.config import Config
    spec = importlib.util.spec_from_file_location("elfa_bench_script", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    monkeypatch.setenv("WORLD_SIZE", str(world))
    monkeypatch.setenv("RANK", "0")
    path = os.path.join(ROOT, "configs", "bench", "gpt7b_tp8_mxfp8.yaml")
    cfg = Config.from_file(path, env_override=False)
    assert (cfg.runtime.tensor_parallel_size, cfg.runtime.world_size) == (8, 8)
    cfg.runtime.world_size = world
    mb, scaling, metric = bench.plan_run(cfg, 8, 8, world)
    assert mb == 4 and scaling == "strong" and metric == bench.METRIC
    assert cfg.runtime.tensor_parallel_size == world and cfg.training.global_batch_size == 32
    # a data-parallel file keeps its micro-batch per GPU (weak scaling)
    cfg = Config.from_file(os.path.join(ROOT, "configs", "bench", "gpt350m_zero1.yaml"), env_override=False)
    ytp, yw = cfg.runtime.tensor_parallel_size, cfg.runtime.world_size
    cfg.runtime.world_size = world
    mb, scaling, _ = bench.plan_run(cfg, ytp, yw, world)
    assert scaling == "weak" and cfg.training.global_batch_size == mb * world and cfg.runtime.tensor_parallel_size == 1


def test_build_object_keys_follow_contents(tmp_path):
    """An object is rebuilt when its source, a header or the flags change - and only then (contents, not file times)."""
    from elfa_b200.build import object_keys
    (tmp_path / "a.cu").write_text("// a\n")
    (tmp_path / "runtime.cu").write_text("// r\n")
    (tmp_path / "c.cuh").write_text("// h\n")
    k0 = object_keys(tmp_path, (), "d0")
    assert set(k0) == {"a", "runtime"} and k0 == object_keys(tmp_path, (), "d0")
    (tmp_path / "a.cu").write_text("// a2\n")
    k1 = object_keys(tmp_path, (), "d0")
    assert k1["a"] != k0["a"] and k1["runtime"] == k0["runtime"]
    assert object_keys(tmp_path, (), "d1")["runtime"] != k1["runtime"] and object_keys(tmp_path, (), "d1")["a"] == k1["a"]
    (tmp_path / "c.cuh").write_text("// h2\n")
    k2 = object_keys(tmp_path, (), "d0")
    assert k2["a"] != k1["a"] and k2["runtime"] != k1["runtime"]
    k3 = object_keys(tmp_path, ("-DELFA_BOUNDS",), "d0")
    assert k3["a"] != k2["a"] and k3["runtime"] != k2["runtime"]


def test_deferred_signal_push_protocol_model():
    """The push role as it runs now: asynchronous stores that land in any order, peers served without draining the pipeline, a
    peer's counter raised one peer late after the older stores are known to have landed. Safe with the wait; the negative
    control (counter raised without it) lets a consumer read pieces that have not landed."""
    from elfa_b200.runtime.protocol_model import DeferredSignalPushModel
    for seed in range(2):
        ranks = DeferredSignalPushModel(4, pieces=3, seed=seed).run(16)
        assert all(r.status == 0 and not r.errors for r in ranks), [r.errors[:2] for r in ranks]
    broken = 0
    for seed in range(20):
        ranks = DeferredSignalPushModel(4, pieces=3, seed=seed, wait_for_completion=False).run(16)
        broken += any(r.errors for r in ranks)
        if broken:
            break
    assert broken > 0
