"""Config schema, dataset / tokenizer / checkpoint formats, telemetry (CPU)."""
import json
import os
import struct
import warnings

import numpy as np
import pytest
import torch

from elfa_b200.checkpoint import (CheckpointManager, CheckpointMetadata, convert_checkpoint, list_checkpoints, read_tensors,
                                  validate_checkpoint, write_tensors)
from elfa_b200.checkpoint.manager import parse_step
from elfa_b200.config import Config, ConfigError, default_1t
from elfa_b200.data import (BinaryDataset, DataLoader, DatasetBuilder, StreamingPacker, SyntheticDataset, Tokenizer, pack_sequences,
                            write_token_file)
from elfa_b200.telemetry import StepMetrics, Telemetry, TrainingStats, check_nan_inf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_configs_parse_with_reference_values():
    s = Config.from_file(os.path.join(ROOT, "configs", "smoke.yaml"), env_override=False)
    assert (s.model.vocab_size, s.model.hidden_dim, s.model.num_heads, s.model.head_dim) == (8192, 256, 4, 64)
    assert s.model.norm_type == "rmsnorm" and s.training.optimizer == "lion_muon" and s.training.total_steps == 10
    assert s.model.efla.chunk_size == 128 and s.model.prism.shortconv_window == 16 and s.checkpoint.keep_last_n == 2
    t = Config.from_file(os.path.join(ROOT, "configs", "train.yaml"), env_override=False)
    assert t.model.max_seq_len == 50_000_000 and t.model.target_params == 10 ** 12 and t.runtime.zero_stage == 2
    assert t.runtime.tensor_parallel_size == 8 and t.training.lr_schedule == "linear_warmup_cosine"
    s.validate()


def test_partial_yaml_takes_defaults_and_missing_section_is_an_error():
    y = "model:\n  hidden_dim: 512\n  num_heads: 8\n  head_dim: 64\ntraining: {}\nruntime: {}\ndata: {}\ncheckpoint: {}\ntelemetry: {}\n"
    c = Config.from_yaml(y, env_override=False)
    d = default_1t()
    assert c.model.hidden_dim == 512 and c.model.vocab_size == d.model.vocab_size == 65536
    assert c.training.learning_rate == 1e-4 and c.runtime.seed == 42 and c.data.seq_len == 8192
    with pytest.raises(ConfigError):
        Config.from_yaml("model: {}\ntraining: {}\n", env_override=False)


def test_unknown_keys_and_bad_enums_warn_and_floats_without_dot_parse():
    y = ("model:\n  norm_type: batchnorm\n  bogus: 1\ntraining:\n  learning_rate: 1e-4\n  min_learning_rate: 3\nruntime: {}\ndata: {}\n"
         "checkpoint: {}\ntelemetry: {}\n")
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        c = Config.from_yaml(y, env_override=False)
    msgs = " ".join(str(x.message) for x in w)
    assert "bogus" in msgs and "norm_type" in msgs
    assert c.model.norm_type == "rmsnorm" and c.training.learning_rate == 1e-4 and c.training.min_learning_rate == 3.0


def test_validation_rules():
    c = default_1t()
    c.model.hidden_dim = 100
    with pytest.raises(ConfigError):
        c.validate()
    c = default_1t()
    c.runtime.pipeline_parallel_size = 2
    with pytest.raises(ConfigError):
        c.validate()
    c = default_1t()
    c.training.global_batch_size, c.training.micro_batch_size = 10, 3
    with pytest.raises(ConfigError):
        c.validate()
    assert len(default_1t().config_hash()) == 64


def test_bench_configs_match_baseline_shapes():
    want = {"gpt350m_zero1": (24, 1024, 16, 4096, 32000, 2048), "gpt1p3b_zero3": (24, 2048, 16, 8192, 32000, 2048),
            "gpt7b_tp8_mxfp8": (32, 4096, 32, 11008, 32000, 4096), "gpt13b_tp4dp2_nvfp4": (40, 5120, 40, 13824, 32000, 4096),
            "smoke_cpu": (2, 128, 4, 512, 4096, 128)}
    for name, (L, D, H, F, V, S) in want.items():
        c = Config.from_file(os.path.join(ROOT, "configs", "bench", name + ".yaml"), env_override=False)
        m = c.model
        assert (m.num_layers, m.hidden_dim, m.num_heads, m.intermediate_dim, m.vocab_size, c.data.seq_len) == (L, D, H, F, V, S)
        assert c.mixer() == "attention" and m.norm_type == "layernorm" and m.tie_embeddings
    c = Config.from_file(os.path.join(ROOT, "configs", "bench", "gpt13b_tp4dp2_nvfp4.yaml"), env_override=False)
    assert c.quant.mlp == "nvfp4" and c.quant.attention == "mxfp8" and c.runtime.data_parallel_size == 2


# ---------------------------------------------------------------------------------------------- data
def test_dataset_format_roundtrip_and_header_layout(tmp_path):
    tok = np.arange(1000, dtype=np.uint32) % 97
    p = str(tmp_path / "d.bin")
    write_token_file(p, tok, [("shard_000000.bin", 1000, b"\x11" * 32)])
    raw = open(p, "rb").read()
    magic, ver, n, ns = struct.unpack_from("<IIQI", raw, 0)
    assert (magic, ver, n, ns) == (0xEF1AD001, 1, 1000, 1)
    ds = BinaryDataset.open(p)
    assert ds.offset == 20 + 4 + len("shard_000000.bin") + 8 + 32
    assert np.array_equal(ds.get_tokens(10, 5), tok[10:15])
    with pytest.raises(IndexError):
        ds.get_tokens(999, 5)
    ld = DataLoader(ds, 2, 100, shuffle=False, pin_memory=False)
    b = ld.next()
    assert b.input.shape == (2, 100) and torch.equal(b.input[0, 1:], b.target[0, :-1])
    assert ld.num_samples == 9 and ld.num_batches() == 4       # the 10th window has no look-ahead token


def test_loader_shuffle_is_seeded_dp_ranks_are_disjoint_and_skip_resumes():
    ds = SyntheticDataset(100, 64 * 20 + 1, "uniform", 0)
    a = DataLoader(ds, 2, 64, shuffle=True, seed=3, pin_memory=False)
    b = DataLoader(ds, 2, 64, shuffle=True, seed=3, pin_memory=False)
    assert torch.equal(a.next().input, b.next().input)
    r0 = DataLoader(ds, 1, 64, shuffle=True, seed=3, dp_rank=0, dp_size=2, pin_memory=False)
    r1 = DataLoader(ds, 1, 64, shuffle=True, seed=3, dp_rank=1, dp_size=2, pin_memory=False)
    assert set(r0._order.tolist()).isdisjoint(r1._order.tolist())
    c = DataLoader(ds, 2, 64, shuffle=True, seed=3, pin_memory=False)
    for _ in range(3):
        want = c.next_cycling()
    d = DataLoader(ds, 2, 64, shuffle=True, seed=3, pin_memory=False)
    d.skip(2)
    assert torch.equal(d.next_cycling().input, want.input)


def test_zipf_generator_is_heavy_tailed_and_seeded():
    a = SyntheticDataset(32000, 200000, "zipf", 1, 1.1)
    b = SyntheticDataset(32000, 200000, "zipf", 1, 1.1)
    assert np.array_equal(a.tokens, b.tokens) and a.tokens.max() < 32000
    counts = np.sort(np.bincount(a.tokens, minlength=32000))[::-1]
    assert counts[0] > 20 * counts[1000]


def test_dataset_builder_and_packing(tmp_path):
    b = DatasetBuilder(str(tmp_path), "ds", shard_tokens=100)
    b.add(np.arange(250))
    merged = b.finish()
    assert len(b.records) == 3 and os.path.getsize(tmp_path / "shard_000000.bin") == 64 + 400
    assert len(BinaryDataset.open(merged)) == 250 and os.path.exists(tmp_path / "ds.index")
    tokens, pos, sid, cu = pack_sequences([[1, 2, 3], [4, 5], [6, 7, 8, 9]])
    assert len(tokens) == 9 and cu.tolist() == [0, 3, 5, 9] and pos.tolist() == [0, 1, 2, 0, 1, 0, 1, 2, 3]
    sp = StreamingPacker(4, eod_token=4)
    sp.add_document([10, 11, 12])
    sp.add_document([13, 14])
    rows = sp.finish()
    assert rows.shape == (2, 4) and rows[0].tolist() == [10, 11, 12, 4]


def test_bpe_roundtrip_specials_atomic_and_file_format(tmp_path):
    text = "low lower lowest newer newest wider widest " * 20
    tok = Tokenizer.train_from_text(text, 300)
    assert tok.vocab_size > 260 and tok.merges[0][2] == 260
    s = "lowest <eos> newer<bos>wider"
    ids = tok.encode(s)
    assert tok.decode(ids) == s and ids.count(259) == 1 and ids.count(258) == 1
    p = str(tmp_path / "tok.bin")
    tok.save(p)
    raw = open(p, "rb").read()
    assert struct.unpack_from("<IIII", raw, 0) == (0x544B5A31, tok.vocab_size, 4, len(tok.merges))
    assert Tokenizer.load(p).encode(s) == ids
    src = tmp_path / "c.txt"
    src.write_text("lower newest")
    n = tok.encode_file(str(src), str(tmp_path / "c.tok"))
    out = open(tmp_path / "c.tok", "rb").read()
    assert struct.unpack_from("<Q", out, 0)[0] == n and len(out) == 8 + 4 * n
    # deterministic tie-break: two equally frequent pairs -> the lexicographically smaller one merges first
    t2 = Tokenizer.train(b"abab cdcd", 261)
    assert t2.merges[0][:2] == (ord("a"), ord("b"))


# ----------------------------------------------------------------------------------------- checkpoint
def test_tensor_file_layout_and_integrity(tmp_path):
    p = str(tmp_path / "tensors.bin")
    a = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    b = torch.randn(5).to(torch.bfloat16)
    write_tensors(p, [("a.weight", a), ("b", b)])
    raw = open(p, "rb").read()
    assert raw[:8] == b"EFLATNS1" and struct.unpack_from("<II", raw, 8) == (1, 2)
    first = 16 + (4 + 8 + 4 + 16 + 4 + 8 + 8 + 32) + (4 + 1 + 4 + 8 + 4 + 8 + 8 + 32)
    nl = struct.unpack_from("<I", raw, 16)[0]
    off = 16 + 4 + nl + 4 + 16
    dtype_code, offset, size = struct.unpack_from("<IQQ", raw, off)
    assert (dtype_code, offset, size) == (0, first, 24)
    t = read_tensors(p)
    assert torch.equal(t["a.weight"], a) and torch.equal(t["b"], b) and t["b"].dtype == torch.bfloat16
    corrupted = bytearray(raw)
    corrupted[first + 3] ^= 0xFF
    open(p, "wb").write(bytes(corrupted))
    with pytest.raises(ValueError, match="SHA-256"):
        read_tensors(p)
    with pytest.raises(ValueError):
        write_tensors(p, [("x", a), ("x", a)])


def test_manager_atomic_save_keep_last_n_metadata_and_convert(tmp_path):
    d = str(tmp_path / "ck")
    m = CheckpointManager(d, keep_last_n=2, compression=True, async_save=True)
    w = torch.randn(4, 4)
    for step in (1, 2, 3):
        meta = CheckpointMetadata(step=step, epoch=0, tokens_seen=step * 10, loss=1.5, learning_rate=1e-3, timestamp=1,
                                  config_hash="a" * 64)
        m.save(step, [("w", w * step)], meta, optimizer_state={"m": torch.ones(3)}, rng_state=b"xyz", config_yaml="model: {}\n")
    m.wait()
    assert [s for s, _ in list_checkpoints(d)] == [2, 3]
    assert not [n for n in os.listdir(d) if n.startswith(".tmp") or n.endswith(".bak")]
    meta, tensors, opt, rng, cfg = m.load_full()
    assert meta.step == 3 and torch.equal(tensors["w"], w * 3) and torch.equal(opt["m"], torch.ones(3)) and rng == b"xyz"
    assert json.loads(open(os.path.join(d, "step_00000003", "metadata.json")).read())["tokens_seen"] == 30
    assert validate_checkpoint(os.path.join(d, "step_00000003")).step == 3
    with pytest.raises(ValueError):
        m.load(expected={"w": ((4, 5), torch.float32)})
    with pytest.raises(KeyError):
        m.load(expected={"missing": ((1,), torch.float32)})
    convert_checkpoint(os.path.join(d, "step_00000003"), str(tmp_path / "pt"), "pytorch")
    assert torch.equal(torch.load(tmp_path / "pt" / "model.pt")["w"], w * 3)
    convert_checkpoint(os.path.join(d, "step_00000003"), str(tmp_path / "st"), "safetensors")
    raw = open(tmp_path / "st" / "model.safetensors", "rb").read()
    hl = struct.unpack_from("<Q", raw, 0)[0]
    assert json.loads(raw[8:8 + hl])["w"]["shape"] == [4, 4]
    assert parse_step("step_00001000") == 1000 and parse_step("step_1") is None
    with pytest.raises(ValueError):
        CheckpointMetadata.from_json('{"step": 1, "extra": 2}')
    with pytest.raises(ValueError):
        CheckpointMetadata.from_json('{"step": 1, "config_hash": "xyz"}')


# ------------------------------------------------------------------------------------------ telemetry
def test_telemetry_jsonl_schema_and_prometheus(tmp_path):
    log = str(tmp_path / "t.log")
    t = Telemetry(rank=0, log_file=log, log_level="warn")
    t.log_metrics(StepMetrics(3, 1536, 8.25, 3e-4, 1.5, 1234.5, 10, 20, 99, {"mfu": 0.5}))
    t.close()
    rec = json.loads(open(log + ".jsonl").read().strip())
    assert list(rec)[:9] == ["step", "tokens", "loss", "lr", "grad_norm", "throughput", "memory_used", "memory_total", "timestamp"]
    assert rec["step"] == 3 and rec["mfu"] == 0.5
    assert "step=3 loss=8.2500" in open(log).read()
    prom = t.export_prometheus()
    assert "efla_training_step 3" in prom and "efla_training_loss 8.25" in prom and "efla_training_throughput 1234.50" in prom
    assert "efla_training_lr 0.0003" in prom and "efla_training_grad_norm 1.5" in prom and "efla_training_mfu 0.5" in prom
    assert "efla_memory_used_bytes 10" in prom and "efla_training_tokens 1536" in prom
    assert check_nan_inf([1.0, 2.0]) and not check_nan_inf(torch.tensor([1.0, float("nan")]))
    s = TrainingStats(window=2)
    s.update(1.0, 10)
    s.update(3.0, 10)
    s.update(5.0, 10)
    assert s.average_loss() == 4.0 and s.tokens == 30


def test_prefetch_loader_keeps_order_epochs_and_resume_position():
    from elfa_b200.data.dataset import DataLoader, PrefetchLoader, SyntheticDataset
    ds = SyntheticDataset(1000, 16 * 10 + 1, "uniform", 0, 1.1)
    plain = DataLoader(ds, 2, 16, shuffle=True, seed=3, pin_memory=False)
    want = [(plain.next_cycling(), plain.epoch) for _ in range(12)]          # 5 batches per epoch: rolls over twice
    pre = PrefetchLoader(DataLoader(ds, 2, 16, shuffle=True, seed=3, pin_memory=False), depth=3)
    for b, ep in want:
        got = pre.next_cycling()
        assert torch.equal(got.input, b.input) and torch.equal(got.target, b.target) and pre.epoch == ep
    pre.close()
    resumed = PrefetchLoader(DataLoader(ds, 2, 16, shuffle=True, seed=3, pin_memory=False), depth=2)
    resumed.skip(7)
    assert resumed.epoch == 1
    got = resumed.next_cycling()
    assert torch.equal(got.input, want[7][0].input)
    resumed.close()


def test_dataset_cli_synth_pack_info(tmp_path, capsys):
    from elfa_b200 import cli
    from elfa_b200.data.dataset import BinaryDataset
    from elfa_b200.data.tokenizer import EOS, PAD, Tokenizer
    out = str(tmp_path / "smoke.bin")
    assert cli.main(["dataset", "synth", "--output", out, "--tokens", "1000", "--vocab-size", "8192", "--seed", "42"]) == 0
    ds = BinaryDataset.open(out)
    assert len(ds) == 1000 and int(ds.get_tokens(0, 1000).max()) < 8192
    assert cli.main(["dataset", "synth", "--output", str(tmp_path / "again.bin"), "--tokens", "1000"]) == 0
    assert np.array_equal(BinaryDataset.open(str(tmp_path / "again.bin")).get_tokens(0, 1000), ds.get_tokens(0, 1000))   # seeded
    tok = Tokenizer.train_from_text("the quick brown fox jumps over the lazy dog " * 20, 300)
    tok.save(str(tmp_path / "tok.bin"))
    docs = tmp_path / "docs.jsonl"
    docs.write_text("\n".join(json.dumps({"text": t}) for t in ["the quick fox", "lazy dog", "brown fox jumps over"]) + "\n")
    packed = str(tmp_path / "packed.bin")
    assert cli.main(["dataset", "pack", "--input", str(docs), "--tokenizer", str(tmp_path / "tok.bin"), "--output", packed,
                     "--seq-len", "8", "--jsonl"]) == 0
    p = BinaryDataset.open(packed)
    toks = p.get_tokens(0, len(p)).tolist()
    assert len(p) % 8 == 0 and toks.count(EOS) == 3 and (toks[-1] == PAD or toks[-1] == EOS)
    first_doc = toks[:toks.index(EOS)]
    assert tok.decode(first_doc) == "the quick fox"
    assert cli.main(["dataset", "info", packed]) == 0
    assert f"{len(p)} tokens" in capsys.readouterr().out


def test_health_probe_against_a_stand_in_nvml():
    from types import SimpleNamespace
    from elfa_b200.telemetry import health

    class FakeNvml:
        def __init__(self, temp=55, used=10, total=100, reasons=0, ecc=0, dead=False):
            self.temp, self.used, self.total, self.reasons, self.ecc, self.dead = temp, used, total, reasons, ecc, dead
            self.calls = []

        def nvmlInit(self):
            self.calls.append("init")

        def nvmlShutdown(self):
            self.calls.append("shutdown")

        def nvmlDeviceGetHandleByIndex(self, i):
            if self.dead:
                raise RuntimeError("GPU is lost")
            return i

        def nvmlDeviceGetTemperature(self, dev, sensor):
            return self.temp

        def nvmlDeviceGetMemoryInfo(self, dev):
            return SimpleNamespace(used=self.used, total=self.total)

        def nvmlDeviceGetCurrentClocksEventReasons(self, dev):
            return self.reasons

        def nvmlDeviceGetTotalEccErrors(self, dev, kind, counter):
            return self.ecc

    fake = FakeNvml()
    h, r = health.probe(0, fake)
    assert h.ok() and r["temperature_c"] == 55 and fake.calls == ["init", "shutdown"]       # only reads, and it closes NVML
    h, _ = health.probe(0, FakeNvml(reasons=health.SW_POWER_CAP))
    assert h.ok()                                                                            # a power cap is not a fault
    h, _ = health.probe(0, FakeNvml(temp=95))
    assert not h.temperature_ok and h.gpu_healthy
    h, _ = health.probe(0, FakeNvml(reasons=health.HW_THERMAL_SLOWDOWN))
    assert not h.temperature_ok
    h, _ = health.probe(0, FakeNvml(reasons=health.HW_SLOWDOWN))
    assert not h.gpu_healthy
    h, _ = health.probe(0, FakeNvml(ecc=2))
    assert not h.gpu_healthy
    h, _ = health.probe(0, FakeNvml(used=99, total=100))
    assert not h.memory_healthy
    h, _ = health.probe(0, FakeNvml(dead=True))
    assert not h.gpu_healthy
    assert health.describe(health.SW_POWER_CAP | health.HW_SLOWDOWN) == "sw_power_cap,hw_slowdown" and health.describe(0) == "none"


def test_cli_evaluate_perplexity_long_context_needle_summary(tmp_path, capsys):
    """evaluate on a freshly saved checkpoint of the small GPT: perplexity, a context-length sweep and the synthetic tasks."""
    from elfa_b200 import cli
    from elfa_b200.config import Config
    from elfa_b200.trainer import Trainer
    cfg = Config.from_file(os.path.join(ROOT, "configs", "bench", "smoke_cpu.yaml"), env_override=False)
    cfg.checkpoint.dir = str(tmp_path / "ck")
    cfg.telemetry.log_file = ""
    tr = Trainer(cfg, device=torch.device("cpu"), telemetry=False)
    tr.run(max_steps=1)
    path = tr.save_checkpoint()
    tr.close()
    data = str(tmp_path / "eval.bin")
    assert cli.main(["dataset", "synth", "--output", data, "--tokens", "2000", "--vocab-size", str(cfg.model.vocab_size)]) == 0
    capsys.readouterr()
    rc = cli.main(["evaluate", "--checkpoint", path, "--data", data, "--max-tokens", "512", "--long-context", "32,64",
                   "--needle", "2", "--summary", "1", "--haystack-len", "40"])
    out = capsys.readouterr().out
    assert rc == 0, out
    assert "perplexity=" in out and "context=32" in out and "context=64" in out
    assert "needle cases=2 length=40" in out and "needle accuracy by depth decile:" in out and "rouge1=" in out
