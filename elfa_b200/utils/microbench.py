"""Single-kernel micro-benchmarks (device timing with CUDA events, L2 flushed between iterations).

    python -m elfa_b200.utils.microbench gemm --m 8192 --n 8192 --k 8192 [--layout nn|nt|tn] [--iters 10]
    python -m elfa_b200.utils.microbench attn_fwd --seq 4096 --heads 32 --hd 128 --batch 1
    python -m elfa_b200.utils.microbench attn_bwd --seq 4096 --heads 32 --hd 128 --batch 1
    python -m elfa_b200.utils.microbench norm --rows 16384 --dim 4096
    python -m elfa_b200.utils.microbench xent --rows 8192 --vocab 32000
    python -m elfa_b200.utils.microbench adamw --n 268435456
    python -m elfa_b200.utils.microbench mxfp8 --rows 16384 --dim 4096
    python -m elfa_b200.utils.microbench gemm_nvfp4 --m 8192 --n 8192 --k 8192
    python -m elfa_b200.utils.microbench gelu | softmax | embedding | efla
    python -m elfa_b200.utils.microbench suite --iters 2      # every bandwidth-bound kernel once, small sizes (the ncu capture)

Prints one line with the achieved rate and its fraction of the measured peak
(``MEASURED_PEAKS.json`` at the repository root when present). These are the commands the ncu
summaries under ``profiles/`` were captured with.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["hbm_gbs"] * 1e9, p["bf16_tflops"] * 1e12, "measured"
    except (OSError, KeyError):
        return 6.65e12, 1.59e15, "fallback"


def timed(fn, iters, warm=3, flush=True):
    dev = torch.device("cuda")
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if flush else None
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if scrub is not None:
            scrub.zero_()                     # 256 MB write: evicts the 126 MB L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("kernel", choices=["gemm", "attn_fwd", "attn_bwd", "norm", "norm_bwd", "xent", "adamw", "mxfp8", "gemm_mxfp8",
                                      "gemm_nvfp4", "gelu", "softmax", "embedding", "efla", "shortconv", "suite"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--layout", default="nn", choices=["nn", "nt", "tn"])
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--hd", type=int, default=128)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--window", type=int, default=16, help="shortconv: taps per channel")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--compare", action="store_true", help="also time the PyTorch / library op")
    ap.add_argument("--bn", type=int, default=0, help="gemm: force the tile width (64 / 128 / 256, 512 = CTA pairs; 0 = automatic)")
    a = ap.parse_args(argv)
    if a.kernel == "suite":
        # inputs larger than the 126 MB L2, about 1 GB on the device at most
        rc = 0
        for sub in (["norm", "--rows", "16384"], ["norm_bwd", "--rows", "16384"], ["gelu", "--rows", "16384"],
                    ["softmax", "--rows", "16384"], ["embedding", "--rows", "16384"], ["xent", "--rows", "4096"],
                    ["mxfp8", "--rows", "16384"], ["adamw", "--n", str(1 << 26)]):
            rc |= main(sub + ["--iters", str(a.iters)])
        return rc
    from .. import native, ops
    from ..native import lib, stream_ptr
    native.lib.load()
    dev = torch.device("cuda")
    hbm, flops_peak, src = peaks()
    bf = torch.bfloat16
    if a.kernel == "gemm":
        M, N, K = a.m, a.n, a.k
        if a.layout == "nn":      # x[M,K] @ W[K,N]
            A, B, kw = torch.randn(M, K, device=dev).to(bf), torch.randn(K, N, device=dev).to(bf), dict(b_mn=True)
        elif a.layout == "nt":    # dy[M,K] @ W[N,K]^T
            A, B, kw = torch.randn(M, K, device=dev).to(bf), torch.randn(N, K, device=dev).to(bf), {}
        else:                     # x[K,M]^T @ dy[K,N]
            A, B, kw = torch.randn(K, M, device=dev).to(bf), torch.randn(K, N, device=dev).to(bf), dict(a_mn=True, b_mn=True)
        out = torch.empty(M, N, dtype=bf, device=dev)
        ms = timed(lambda: ops.gemm(A, B, out=out, force_bn=a.bn, **kw), a.iters)
        fl = 2.0 * M * N * K
        line = f"gemm {a.layout} {M}x{N}x{K}: {ms:.4f} ms  {fl / ms / 1e9:.1f} TFLOP/s  {fl / ms / 1e-3 / flops_peak:.3f} of {src} cuBLAS bf16 peak"
        if a.compare:
            ref = {"nn": lambda: torch.matmul(A, B, out=out), "nt": lambda: torch.matmul(A, B.t(), out=out),
                   "tn": lambda: torch.matmul(A.t(), B, out=out)}[a.layout]
            ms2 = timed(ref, a.iters)
            line += f" | torch.matmul {ms2:.4f} ms {fl / ms2 / 1e9:.1f} TFLOP/s"
        print(line)
    elif a.kernel == "gemm_mxfp8":
        from ..ops import gemm_mxfp8 as q8
        M, N, K = a.m, a.n, a.k
        xq, _ = q8.quantize_mxfp8(torch.randn(M, K, device=dev).to(bf))
        wq, _ = q8.quantize_mxfp8(torch.randn(N, K, device=dev).to(bf), right=True)
        out = torch.empty(M, N, dtype=bf, device=dev)
        ms = timed(lambda: q8.gemm_mxfp8(xq, wq, out=out, force_bn=a.bn), a.iters)
        fl = 2.0 * M * N * K
        print(f"gemm_mxfp8 {M}x{N}x{K}: {ms:.4f} ms  {fl / ms / 1e9:.1f} TFLOP/s  {fl / ms / 1e-3 / flops_peak:.3f} of {src} cuBLAS bf16 peak "
              f"(block-scaled e4m3, nominal fp8 peak is 2x bf16)")
        x = torch.randn(M, K, device=dev).to(bf)
        ms = timed(lambda: q8.quantize_mxfp8(x, dequantized=True), a.iters)
        by = M * K * (2 + 1 + 2)
        print(f"mxfp8 quantise (payload + scales + bf16 copy) {M}x{K}: {ms:.4f} ms  {by / ms / 1e6:.1f} GB/s  {by / ms / 1e-3 / hbm:.3f} of {src} copy bandwidth")
    elif a.kernel == "gemm_nvfp4":
        from ..ops import gemm_nvfp4 as q4
        M, N, K = a.m, a.n, a.k
        xq, _ = q4.quantize_nvfp4(torch.randn(M, K, device=dev).to(bf))
        wq, _ = q4.quantize_nvfp4(torch.randn(N, K, device=dev).to(bf), right=True)
        out = torch.empty(M, N, dtype=bf, device=dev)
        ms = timed(lambda: q4.gemm_nvfp4(xq, wq, out=out, force_bn=a.bn), a.iters)
        fl = 2.0 * M * N * K
        print(f"gemm_nvfp4 {M}x{N}x{K}: {ms:.4f} ms  {fl / ms / 1e9:.1f} TFLOP/s  {fl / ms / 1e-3 / flops_peak:.3f} of {src} cuBLAS bf16 peak "
              f"(block-scaled e2m1, nominal fp4 peak is 4x bf16)")
        x = torch.randn(M, K, device=dev).to(bf)
        amax = x.abs().max().float().reshape(1)
        ms = timed(lambda: q4.quantize_nvfp4(x, dequantized=True, amax=amax), a.iters)
        by = M * K * (2 + 0.5 + 2)
        print(f"nvfp4 quantise (payload + scales + bf16 copy) {M}x{K}: {ms:.4f} ms  {by / ms / 1e6:.1f} GB/s  {by / ms / 1e-3 / hbm:.3f} of {src} copy bandwidth")
    elif a.kernel in ("gelu", "softmax", "embedding"):
        R, D = a.rows, a.dim
        if a.kernel == "embedding":
            tok = torch.randn(a.vocab, D, device=dev).to(bf)
            ids = torch.randint(0, a.vocab, (R // 4096 if R >= 4096 else 1, min(R, 4096)), device=dev)
            with torch.no_grad():
                ms = timed(lambda: ops.embedding(ids, tok), a.iters)
            by = 2.0 * ids.numel() * D * 2
        else:
            x = torch.randn(R, D, device=dev).to(bf)
            from ..ops.nn import softmax as _softmax
            fn = ops.gelu if a.kernel == "gelu" else _softmax
            with torch.no_grad():
                ms = timed(lambda: fn(x), a.iters)
            by = 2.0 * R * D * 2
        print(f"{a.kernel} {R}x{D}: {ms:.4f} ms  {by / ms / 1e6:.1f} GB/s  {by / ms / 1e-3 / hbm:.3f} of {src} copy bandwidth")
    elif a.kernel == "shortconv":
        from ..ops.efla import shortconv
        B, T, C, W = a.batch, a.seq, a.dim, a.window
        x = torch.randn(B, T, C, device=dev).to(bf).requires_grad_(True)
        w = (0.1 * torch.randn(C, W, device=dev)).to(bf).requires_grad_(True)
        b = torch.zeros(C, device=dev, dtype=bf, requires_grad=True)
        with torch.no_grad():
            ms = timed(lambda: shortconv(x, w, b), a.iters)
        y = shortconv(x, w, b)
        g = torch.randn_like(y)
        ms_b = timed(lambda: torch.autograd.grad(y, (x, w, b), g, retain_graph=True), a.iters)
        by = 2.0 * B * T * C * 2
        print(f"shortconv B{B} T{T} C{C} W{W}: forward {ms:.4f} ms ({by / ms / 1e-3 / hbm:.3f} of {src} copy bandwidth), "
              f"backward (dx + dw + db) {ms_b:.4f} ms")
    elif a.kernel == "efla":
        from ..ops.efla import efla_scan
        B, T, H, hd = a.batch, a.seq, a.heads, a.hd
        k = torch.nn.functional.normalize(torch.randn(B, T, H, hd, device=dev), dim=-1).to(bf).requires_grad_(True)
        v = torch.randn(B, T, H, hd, device=dev).to(bf).requires_grad_(True)
        beta = torch.tensor(0.5, device=dev, requires_grad=True)
        with torch.no_grad():
            ms = timed(lambda: efla_scan(k, v, beta), a.iters)
        o, _ = efla_scan(k, v, beta)
        g = torch.randn_like(o)
        ms_b = timed(lambda: torch.autograd.grad(o, (k, v, beta), g, retain_graph=True), a.iters)
        print(f"efla scan B{B} T{T} H{H} d{hd}: forward {ms:.3f} ms ({B * T / ms / 1e3:.2f} M tokens/s), backward {ms_b:.3f} ms")
    elif a.kernel in ("attn_fwd", "attn_bwd"):
        S, B, H, hd = a.seq, a.batch, a.heads, a.hd
        qkv = torch.randn(S, B, 3, H, hd, device=dev).to(bf)
        fwd_fl = 4.0 * S * S * hd * H * B / 2
        if a.kernel == "attn_fwd":
            with torch.no_grad():
                ms = timed(lambda: ops.attention(qkv), a.iters)
            print(f"attention fwd causal S{S} B{B} H{H} hd{hd}: {ms:.4f} ms  {fwd_fl / ms / 1e9:.1f} TFLOP/s  "
                  f"{fwd_fl / ms / 1e-3 / flops_peak:.3f} of {src} cuBLAS bf16 peak")
        else:
            q = qkv.clone().requires_grad_(True)
            o = ops.attention(q)
            g = torch.randn_like(o)
            ms = timed(lambda: torch.autograd.grad(o, q, g, retain_graph=True), a.iters)
            fl = 2.5 * fwd_fl
            print(f"attention bwd causal S{S} B{B} H{H} hd{hd}: {ms:.4f} ms  {fl / ms / 1e9:.1f} TFLOP/s (2.5x forward FLOPs)  "
                  f"{fl / ms / 1e-3 / flops_peak:.3f} of {src} cuBLAS bf16 peak")
    elif a.kernel in ("norm", "norm_bwd"):
        R, D = a.rows, a.dim
        x = torch.randn(R, D, device=dev).to(bf).requires_grad_(a.kernel == "norm_bwd")
        w = torch.ones(D, device=dev).to(bf).requires_grad_(a.kernel == "norm_bwd")
        b = torch.zeros(D, device=dev).to(bf).requires_grad_(a.kernel == "norm_bwd")
        if a.kernel == "norm":
            with torch.no_grad():
                ms = timed(lambda: ops.layer_norm(x, w, b), a.iters)
            by = 2.0 * R * D * 2
        else:
            y, _ = ops.layer_norm(x, w, b)
            g = torch.randn_like(y)
            ms = timed(lambda: torch.autograd.grad(y, (x, w, b), g, retain_graph=True), a.iters)
            by = 3.0 * R * D * 2
        print(f"layernorm {'bwd' if a.kernel == 'norm_bwd' else 'fwd'} {R}x{D}: {ms:.4f} ms  {by / ms / 1e6:.1f} GB/s  "
              f"{by / ms / 1e-3 / hbm:.3f} of {src} copy bandwidth")
    elif a.kernel == "xent":
        R, V = a.rows, a.vocab
        base = (torch.randn(R, V, device=dev) * 2).to(bf)
        tgt = torch.randint(0, V, (R,), device=dev)
        work = base.clone()

        def run():
            work.copy_(base)
            ops.cross_entropy(work, tgt)
        copy_ms = timed(lambda: work.copy_(base), a.iters)
        ms = timed(run, a.iters) - copy_ms
        by = 3.0 * R * V * 2      # read twice (second pass mostly from L2), write once
        print(f"cross-entropy fwd+grad {R}x{V}: {ms:.4f} ms  {by / ms / 1e6:.1f} GB/s (3 passes over the logits)  "
              f"{by / ms / 1e-3 / hbm:.3f} of {src} copy bandwidth")
    elif a.kernel == "adamw":
        n = a.n if a.n != 8192 else 1 << 28
        master, m, v = (torch.zeros(n, device=dev) for _ in range(3))
        grad = torch.randn(n, device=dev)
        param = torch.empty(n, dtype=bf, device=dev)
        ms = timed(lambda: lib.call("elfa_adamw", param, 1, master, m, v, grad, 0, n, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, None,
                                    stream_ptr(master)), a.iters, flush=False)
        by = n * (4 * 4 + 3 * 4 + 2.0)
        print(f"adamw {n} elements: {ms:.4f} ms  {by / ms / 1e6:.1f} GB/s  {by / ms / 1e-3 / hbm:.3f} of {src} copy bandwidth")
    elif a.kernel == "mxfp8":
        R, D = a.rows, a.dim
        x = torch.randn(R, D, device=dev).to(bf)
        out = torch.empty_like(x)
        ms = timed(lambda: lib.call("elfa_mxfp8_fake_quant", x, out, R, D, 1, stream_ptr(x)), a.iters)
        by = 2.0 * R * D * 2
        print(f"mxfp8 fake-quant {R}x{D}: {ms:.4f} ms  {by / ms / 1e6:.1f} GB/s  {by / ms / 1e-3 / hbm:.3f} of {src} copy bandwidth")
    st = native.status()
    if st:
        print(f"device status 0x{st:x}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
