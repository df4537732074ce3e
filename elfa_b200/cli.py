"""Command line interface: ``python -m elfa_b200 <command>``.

Same surface as the reference binary (reference: ``src/main.zig:15-26`` commands, ``:107-539``
handlers)::

    train --config F [--resume P] [--data P] [--checkpoint-dir D]
    evaluate --checkpoint P --data P [--config F] [--max-tokens N]
    generate --checkpoint P [--prompt S] [--max-tokens 256] [--temperature 1.0] [--top-p 0.9] [--config F]
    smoke-test [--config configs/smoke.yaml]
    checkpoint list [--dir checkpoints] | validate --path P | convert --input P --output P [--format efla_native|safetensors|pytorch]
    tokenizer train --corpus F [--output tokenizer.bin] [--vocab-size 65536] [--type bpe]
              | encode --tokenizer F (--text S | --input F --output F) | decode --tokenizer F --tokens "1,2,3"
    validate --config F
    profile | version | help

Unknown flags are errors. Multi-GPU runs are launched with ``python -m torch.distributed.run`` (one
process per GPU); rank and world size come from the launcher's environment.
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List, Optional

VERSION = "elfa_b200 0.1.0 (NVIDIA Blackwell sm_100a, PyTorch + native tcgen05 kernels)"


def _load_cfg(path: str):
    from .config import Config
    return Config.from_file(path)


def _device():
    import torch
    if torch.cuda.is_available():
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        return torch.device("cuda", local)
    return torch.device("cpu")


def cmd_train(a) -> int:
    from .trainer import Trainer
    cfg = _load_cfg(a.config)
    if a.set:
        from .utils.errors import apply_overrides, parse_key_value
        for text in a.set:                       # --set training.learning_rate=1e-4,runtime.zero_stage=1
            apply_overrides(cfg, parse_key_value(text))
        cfg.validate()
    if a.checkpoint_dir:
        cfg.checkpoint.dir = a.checkpoint_dir
    if a.data:
        cfg.data.path = a.data
        cfg.bench.synthetic = "none"
    tr = Trainer(cfg, device=_device())
    if a.resume:
        meta = tr.resume(a.resume)
        print(f"resumed from step {meta.step}")
    losses = tr.run(a.data)
    tr.close()
    if losses:
        print(f"finished at step {tr.step}: loss {losses[-1]:.4f}")
    return 0


def _load_for_inference(ckpt: str, config: Optional[str]):
    import torch
    from .checkpoint.manager import resolve_checkpoint
    from .config import Config
    from .trainer import Trainer
    path = resolve_checkpoint(ckpt)
    cfg_path = config or os.path.join(path, "config.yaml")
    if not os.path.exists(cfg_path):
        raise SystemExit(f"no config: pass --config or put config.yaml into {path}")
    cfg = Config.from_file(cfg_path, env_override=False)
    cfg.runtime.world_size, cfg.runtime.tensor_parallel_size, cfg.runtime.zero_stage = 1, 1, 0
    cfg.checkpoint.dir = ""
    cfg.telemetry.log_file = ""
    tr = Trainer(cfg, device=_device(), telemetry=False)
    tr.resume(path)
    tr.model.eval()
    return tr, cfg


def cmd_evaluate(a) -> int:
    from .eval import Evaluator
    tr, cfg = _load_for_inference(a.checkpoint, a.config)
    ev = Evaluator(tr.model, cfg, tr.device)
    if a.data:
        r = ev.evaluate_perplexity(a.data, max_tokens=a.max_tokens)
        print(f"tokens={r['tokens']} loss={r['loss']:.6f} perplexity={r['perplexity']:.4f}")
        if a.long_context:
            from .data.dataset import BinaryDataset
            lengths = [int(x) for x in a.long_context.split(",") if x.strip()]
            for row in ev.evaluate_long_context(BinaryDataset.open(a.data), lengths):
                print(f"context={row['context']} loss={row['loss']:.6f} perplexity={row['perplexity']:.4f}")
    if a.needle or a.summary:
        from .eval.harness import EvalHarness
        from .eval.needle import depth_accuracy, generate_needle_case
        from .eval.summary import generate_summary_case
        h = EvalHarness(tr.model, tr.device)
        length = a.haystack_len or min(cfg.data.seq_len, cfg.model.max_seq_len) // 2
        if a.needle:
            cases = [generate_needle_case(length, cfg.model.vocab_size, seed=i) for i in range(a.needle)]
            r = h.needle_recall(cases)
            print(f"needle cases={r['cases']} length={length} recall={r['recall']:.4f} precision={r['precision']:.4f}")
            per_case = [(c.depth, h.needle_recall([c])["recall"] == 1.0) for c in cases]
            print("needle accuracy by depth decile: " + " ".join("-" if x != x else f"{x:.2f}" for x in depth_accuracy(per_case)))
        if a.summary:
            cases = [generate_summary_case(length, cfg.model.vocab_size, seed=i) for i in range(a.summary)]
            r = h.summary_rouge(cases, max_new_tokens=32)
            print(f"summary cases={a.summary} rouge1={r['rouge1']:.4f} rouge2={r['rouge2']:.4f} rougeL={r['rougeL']:.4f}")
    if not (a.data or a.needle or a.summary):
        raise SystemExit("evaluate needs --data and / or --needle N / --summary N")
    return 0


def cmd_generate(a) -> int:
    from .data.tokenizer import Tokenizer
    from .eval import Generator
    tr, cfg = _load_for_inference(a.checkpoint, a.config)
    tok = Tokenizer.load(cfg.data.tokenizer_path) if os.path.exists(cfg.data.tokenizer_path) else None
    g = Generator(tr.model, tok, tr.device)
    if tok is not None:
        print(g.generate(a.prompt, a.max_tokens, a.temperature, a.top_p))
    else:
        ids = [min(b, cfg.model.vocab_size - 1) for b in a.prompt.encode()]
        out = g.generate_ids(ids, a.max_tokens, a.temperature, a.top_p)
        print(",".join(str(i) for i in out))
    return 0


def cmd_smoke(a) -> int:
    from .trainer import Trainer
    cfg = _load_cfg(a.config)
    cfg.runtime.world_size, cfg.runtime.tensor_parallel_size, cfg.runtime.zero_stage = 1, 1, 0
    cfg.checkpoint.dir = ""
    cfg.telemetry.log_file = ""
    dev = _device()
    if dev.type == "cpu":
        cfg.model.dtype = "fp32"
    tr = Trainer(cfg, device=dev, telemetry=False)
    losses = tr.smoke_test(3)
    print("smoke test passed: losses " + ", ".join(f"{x:.4f}" for x in losses))
    return 0


def cmd_checkpoint(a) -> int:
    from .checkpoint import convert_checkpoint, list_checkpoints, validate_checkpoint
    if a.action == "list":
        for step, path in list_checkpoints(a.dir):
            print(f"{step:10d}  {path}")
        return 0
    if a.action == "validate":
        meta = validate_checkpoint(a.path)
        print(f"valid: step={meta.step} tokens_seen={meta.tokens_seen} loss={meta.loss:.6f}")
        return 0
    convert_checkpoint(a.input, a.output, a.format)
    print(f"converted {a.input} -> {a.output} ({a.format})")
    return 0


def cmd_tokenizer(a) -> int:
    from .data.tokenizer import Tokenizer
    if a.action == "train":
        if a.type != "bpe":
            raise SystemExit(f"tokenizer type '{a.type}' is not supported (only bpe)")
        with open(a.corpus, "rb") as f:
            tok = Tokenizer.train(f.read(), a.vocab_size)
        tok.save(a.output)
        print(f"trained {tok.vocab_size} tokens ({len(tok.merges)} merges) -> {a.output}")
        return 0
    tok = Tokenizer.load(a.tokenizer)
    if a.action == "encode":
        if a.text is not None:
            print(",".join(str(i) for i in tok.encode(a.text)))
        else:
            if not a.input or not a.output:
                raise SystemExit("encode needs --text or --input and --output")
            n = tok.encode_file(a.input, a.output)
            print(f"{n} tokens -> {a.output}")
        return 0
    ids = [int(x) for x in a.tokens.split(",") if x.strip()]
    print(tok.decode(ids))
    return 0


def cmd_dataset(a) -> int:
    """Token files in the binary dataset format: ``synth`` (seeded random tokens, what the reference's smoke script
    generates with an inline Python snippet), ``pack`` (one document per line or per JSONL ``text`` field, tokenised and
    packed into rows of ``--seq-len`` with end-of-document separators), ``info`` (header and size).
    reference: ``scripts/run_local_smoke.sh:29-52``, ``src/data_packer.zig:5-240``."""
    import json
    import numpy as np
    from .data.dataset import BinaryDataset, write_token_file
    if a.action == "synth":
        toks = np.random.default_rng(a.seed).integers(0, a.vocab_size, size=a.tokens, dtype=np.int64)
        write_token_file(a.output, toks)
        print(f"{a.tokens} random tokens < {a.vocab_size} (seed {a.seed}) -> {a.output}")
        return 0
    if a.action == "info":
        ds = BinaryDataset.open(a.path)
        n = len(ds)
        head = ds.get_tokens(0, min(n, 8)).tolist()
        print(f"{a.path}: {n} tokens, {os.path.getsize(a.path)} bytes, first tokens {head}")
        return 0
    from .data.packing import StreamingPacker
    from .data.tokenizer import Tokenizer
    tok = Tokenizer.load(a.tokenizer)
    packer = StreamingPacker(a.seq_len, eod_token=a.eod_token, shuffle=a.shuffle, seed=a.seed)
    docs = 0
    with open(a.input, "r", encoding="utf-8") as f:
        for line in f:
            line = line.rstrip("\n")
            if not line:
                continue
            if a.jsonl:
                line = json.loads(line).get(a.field, "")
            packer.add_document(tok.encode(line))
            docs += 1
    rows = packer.finish(pad_token=a.pad_token)
    write_token_file(a.output, rows.reshape(-1))
    print(f"{docs} documents -> {rows.shape[0]} rows of {a.seq_len} tokens -> {a.output}")
    return 0


def cmd_validate(a) -> int:
    cfg = _load_cfg(a.config)
    cfg.validate()
    est = cfg.model.estimate_parameters()
    mem = cfg.estimate_memory_bytes()
    print(f"config ok: ~{est:,} parameters (estimate), ~{mem / 2 ** 30:.1f} GiB per GPU over {cfg.runtime.world_size} GPUs")
    tgt = cfg.model.target_params
    if tgt and abs(est - tgt) > 0.05 * tgt:
        print(f"warning: estimate is more than 5% off target_params={tgt:,}")
    return 0


def cmd_profile(a) -> int:
    print("Profiling recipes (run on a GPU machine):\n"
          "  ncu --set full --clock-control none -k regex:gemm_bf16_kernel -c 3 -o prof python bench.py --layers 2 --steps 1 --warmup 1\n"
          "  ncu --metrics gpu__time_duration.sum --clock-control none --csv --log-file launches.csv python bench.py --steps 1 --warmup 1\n"
          "  python -m elfa_b200.utils.ncu_summary prof.ncu-rep        # roofline counters + top stall reasons as a table (no GPU needed)\n"
          "  python -m elfa_b200.utils.microbench gemm|attn_fwd|efla|...   # one kernel, device-timed, for a small capture\n"
          "  ELFA_TRACE=1 adds NVTX ranges and per-phase device times (trainer.tracer.summary())\n"
          "  python bench.py --twin 8    # per-rank compute time of an 8-rank job without communication, on one GPU\n"
          "  ELFA_FLAG_TIMEOUT_MS=500 shortens every device-side wait; the status word reports a timeout\n"
          "  python -m elfa_b200.build --bounds; ELFA_BOUNDS=1 ...   # checked build: index tests inside the pipelined kernels (status bit 4)\n"
          "  torchrun --nproc-per-node N baseline/link_probe.py      # peer-memory copy mechanisms apart from any GEMM\n"
          "  torchrun --nproc-per-node N baseline/fused_vs_nccl.py   # fused kernels against NCCL collective + GEMM, per op")
    return 0


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="elfa_b200", description="Blackwell-native LLM pre-training framework", allow_abbrev=False)
    sub = p.add_subparsers(dest="command")
    t = sub.add_parser("train", allow_abbrev=False)
    t.add_argument("--config", required=True)
    t.add_argument("--resume")
    t.add_argument("--data")
    t.add_argument("--checkpoint-dir")
    t.add_argument("--set", action="append", default=[], metavar="SECTION.KEY=VALUE[,...]",
                   help="configuration overrides applied after the file is read")
    t.set_defaults(fn=cmd_train)
    e = sub.add_parser("evaluate", allow_abbrev=False)
    e.add_argument("--checkpoint", required=True)
    e.add_argument("--data", help="token file: perplexity (token-weighted mean loss)")
    e.add_argument("--config")
    e.add_argument("--max-tokens", type=int)
    e.add_argument("--long-context", metavar="N1,N2,...", help="with --data: perplexity at these context lengths")
    e.add_argument("--needle", type=int, default=0, metavar="CASES", help="synthetic needle-in-a-haystack recall / precision")
    e.add_argument("--summary", type=int, default=0, metavar="CASES", help="synthetic long-form summary ROUGE-1/2/L")
    e.add_argument("--haystack-len", type=int, default=0, help="tokens per synthetic case (default: half the context)")
    e.set_defaults(fn=cmd_evaluate)
    g = sub.add_parser("generate", allow_abbrev=False)
    g.add_argument("--checkpoint", required=True)
    g.add_argument("--prompt", default="")
    g.add_argument("--max-tokens", type=int, default=256)
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--top-p", type=float, default=0.9)
    g.add_argument("--config")
    g.set_defaults(fn=cmd_generate)
    s = sub.add_parser("smoke-test", allow_abbrev=False)
    s.add_argument("--config", default="configs/smoke.yaml")
    s.set_defaults(fn=cmd_smoke)
    c = sub.add_parser("checkpoint", allow_abbrev=False)
    cs = c.add_subparsers(dest="action", required=True)
    cl = cs.add_parser("list", allow_abbrev=False)
    cl.add_argument("--dir", default="checkpoints")
    cv = cs.add_parser("validate", allow_abbrev=False)
    cv.add_argument("--path", required=True)
    cc = cs.add_parser("convert", allow_abbrev=False)
    cc.add_argument("--input", required=True)
    cc.add_argument("--output", required=True)
    cc.add_argument("--format", default="efla_native", choices=["efla_native", "safetensors", "pytorch"])
    c.set_defaults(fn=cmd_checkpoint)
    d = sub.add_parser("dataset", allow_abbrev=False)
    dsub = d.add_subparsers(dest="action", required=True)
    dsy = dsub.add_parser("synth", allow_abbrev=False)
    dsy.add_argument("--output", required=True)
    dsy.add_argument("--tokens", type=int, default=10000)
    dsy.add_argument("--vocab-size", type=int, default=8192)
    dsy.add_argument("--seed", type=int, default=42)
    dpk = dsub.add_parser("pack", allow_abbrev=False)
    dpk.add_argument("--input", required=True)
    dpk.add_argument("--tokenizer", required=True)
    dpk.add_argument("--output", required=True)
    dpk.add_argument("--seq-len", type=int, required=True)
    dpk.add_argument("--jsonl", action="store_true", help="every line is a JSON object; the document is its --field")
    dpk.add_argument("--field", default="text")
    dpk.add_argument("--eod-token", type=int, default=259, help="separator appended to every document (259 = <eos> of the BPE tokenizer)")
    dpk.add_argument("--pad-token", type=int, default=256)
    dpk.add_argument("--shuffle", action="store_true")
    dpk.add_argument("--seed", type=int, default=0)
    din = dsub.add_parser("info", allow_abbrev=False)
    din.add_argument("path")
    d.set_defaults(fn=cmd_dataset)
    k = sub.add_parser("tokenizer", allow_abbrev=False)
    ks = k.add_subparsers(dest="action", required=True)
    kt = ks.add_parser("train", allow_abbrev=False)
    kt.add_argument("--corpus", required=True)
    kt.add_argument("--output", default="tokenizer.bin")
    kt.add_argument("--vocab-size", type=int, default=65536)
    kt.add_argument("--type", default="bpe", choices=["bpe", "unigram", "word"])
    ke = ks.add_parser("encode", allow_abbrev=False)
    ke.add_argument("--tokenizer", required=True)
    ke.add_argument("--text")
    ke.add_argument("--input")
    ke.add_argument("--output")
    kd = ks.add_parser("decode", allow_abbrev=False)
    kd.add_argument("--tokenizer", required=True)
    kd.add_argument("--tokens", required=True)
    k.set_defaults(fn=cmd_tokenizer)
    v = sub.add_parser("validate", allow_abbrev=False)
    v.add_argument("--config", required=True)
    v.set_defaults(fn=cmd_validate)
    sub.add_parser("profile", allow_abbrev=False).set_defaults(fn=cmd_profile)
    sub.add_parser("version", allow_abbrev=False).set_defaults(fn=lambda a: print(VERSION) or 0)
    sub.add_parser("help", allow_abbrev=False).set_defaults(fn=lambda a: p.print_help() or 0)
    return p


def main(argv: Optional[List[str]] = None) -> int:
    p = build_parser()
    a = p.parse_args(argv)
    if not getattr(a, "fn", None):
        p.print_help()
        return 1
    return int(a.fn(a) or 0)


if __name__ == "__main__":
    sys.exit(main())
