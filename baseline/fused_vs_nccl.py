"""Times the two tensor-parallel hot paths - all-gather→GEMM and GEMM→reduce-scatter - with the
library baseline (NCCL collective + GEMM as separate kernels) and with the fused peer-memory
kernels, on the per-rank shapes of the 7B TP configuration (tokens x 4096 hidden).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29560 \
        baseline/fused_vs_nccl.py [--tokens 16384]

Device timing (CUDA events), max over ranks. The roofline of a fused op is the slower of
FLOPs / measured GEMM peak and bytes over NVLink / 770 GB/s per direction (measured peer copy).
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from elfa_b200.parallel import tp as tpl  # noqa: E402
from elfa_b200.parallel.mesh import build_context, init_distributed  # noqa: E402
from elfa_b200.runtime.symm import SymmetricArena  # noqa: E402


def timed(fn, iters=20, warm=5):
    for _ in range(warm):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=11008)
    a = ap.parse_args()
    world = init_distributed("nccl")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    pc = build_context(world, True, "nccl")
    pc.symm = SymmetricArena.for_group(pc.tp_group, dev, 4 << 30)
    peak = 1.4e15
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            peak = json.load(f)["bf16_tflops"] * 1e12
    except OSError:
        pass
    link = 770e9
    M, D, F = a.tokens, a.hidden, a.ffn
    rows = []
    for name, kind, K, N in [("qkv (AG->GEMM)", "ag", D, 3 * D // world), ("mlp_up (AG->GEMM)", "ag", D, F // world),
                             ("attn_out (GEMM->RS)", "rs", D // world, D), ("mlp_down (GEMM->RS)", "rs", F // world, D)]:
        w = (torch.randn(K, N, device=dev) * 0.02).to(torch.bfloat16)
        res = {}
        for backend in ("nccl", "fused"):
            pc.comm_backend = backend
            if kind == "ag":
                x = torch.randn(M // world, K, device=dev).to(torch.bfloat16)
                res[backend] = timed(lambda: tpl.ag_gemm(x, w, pc, b_mn=True))
            else:
                x = torch.randn(M, K, device=dev).to(torch.bfloat16)
                res[backend] = timed(lambda: tpl.gemm_rs(x, w, pc, b_mn=True))
        # the parts of the library path on their own: collective only, GEMM only
        from elfa_b200.ops.gemm import gemm
        if kind == "ag":
            full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
            coll = timed(lambda: dist.all_gather_into_tensor(full, x, group=pc.tp_group))
            mm = timed(lambda: gemm(full, w, b_mn=True))
        else:
            y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            out = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)
            coll = timed(lambda: dist.reduce_scatter_tensor(out, y, group=pc.tp_group))
            mm = timed(lambda: gemm(x, w, b_mn=True, out=y))
        flops = 2.0 * M * K * N
        wire = (world - 1) / world * M * (K if kind == "ag" else N) * 2
        floor_ms = max(flops / peak, wire / link) * 1e3
        rows.append((name, M, N, K, res["nccl"], res["fused"], floor_ms, coll, mm))
        if kind == "rs" and N % 256 == 0:
            # the same kernel with row-major receive slots (TMA tensor stores of 128-byte row segments)
            os.environ["ELFA_RS_CHUNK_MAJOR"] = "0"
            pc.comm_backend = "fused"
            t_row = timed(lambda: tpl.gemm_rs(x, w, pc, b_mn=True))
            os.environ["ELFA_RS_CHUNK_MAJOR"] = "1"
            rows.append((name + " row-major slots", M, N, K, res["nccl"], t_row, floor_ms, coll, mm))
        if kind == "ag" and K % 128 == 0:
            # MXFP8 form: e4m3 payloads + scale atoms on the wire, block-scaled product. Library arm: NCCL all-gather of the
            # quantised payload and of the scale atoms, then the block-scaled GEMM.
            from elfa_b200.ops.gemm_mxfp8 import Mxfp8Operand, gemm_mxfp8, quantize_mxfp8, sf_numel
            from elfa_b200.parallel import fused
            w_op, _ = quantize_mxfp8(w.t().contiguous(), right=True)
            Ml = M // world
            pay = torch.empty(M, K, device=dev, dtype=torch.uint8)
            sf = torch.empty(sf_numel(M, K), device=dev, dtype=torch.uint8)

            def lib_arm():
                op, _ = quantize_mxfp8(x)
                dist.all_gather_into_tensor(pay, op.payload, group=pc.tp_group)
                dist.all_gather_into_tensor(sf, op.scales, group=pc.tp_group)
                return gemm_mxfp8(Mxfp8Operand(pay, sf, M, K, False), w_op)
            pc.comm_backend = "fused"
            t_lib = timed(lib_arm)
            xa, _ = quantize_mxfp8(torch.randn(M, K, device=dev).to(torch.bfloat16))
            mm8 = timed(lambda: gemm_mxfp8(xa, w_op))
            coll8 = timed(lambda: dist.all_gather_into_tensor(pay, xa.payload[:Ml], group=pc.tp_group))
            for one in (True, False):
                fused._ONE_KERNEL = one

                def fused_arm():
                    y, _, _ = fused.ag_gemm_mxfp8(x, w_op, pc)
                    fused.wait_pending_copies(pc)
                    return y
                t = timed(fused_arm)
                wire8 = (world - 1) / world * M * K * (1 + 1 / 32)
                fl8 = max(flops / (2 * peak), wire8 / link) * 1e3        # nominal fp8 rate = 2 x bf16
                rows.append((name.replace("(AG->GEMM)", "mxfp8 " + ("one kernel" if one else "4 launches")), M, N, K, t_lib, t, fl8, coll8, mm8))
            fused._ONE_KERNEL = True
    if pc.rank == 0:
        print(f"world={world} tokens={M}")
        print(f"{'op':24s} {'M':>6s} {'N':>6s} {'K':>6s} {'nccl ms':>9s} {'fused ms':>9s} {'speedup':>8s} {'floor ms':>9s} {'floor/fused':>11s} "
              f"{'coll only':>9s} {'gemm only':>9s}")
        for name, m, n, k, t0, t1, fl, coll, mm in rows:
            print(f"{name:24s} {m:6d} {n:6d} {k:6d} {t0:9.3f} {t1:9.3f} {t0 / t1:8.2f} {fl:9.3f} {fl / t1:11.2f} {coll:9.3f} {mm:9.3f}")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
