"""Peer-memory copy rates of the mechanisms the fused kernels can use, apart from any GEMM:
per-thread 16-byte stores against a bulk-copy pipeline through shared memory, for several grid sizes, piece sizes and
pipeline depths; plus NCCL's all-gather (on local tensors) for reference.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29570 \
        baseline/link_probe.py [--mb 256]

Every rank sends to rank + 1 at the same time (the pattern of one phase of the fused all-gather). Device timing (CUDA events),
max over ranks."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from elfa_b200.native import lib, stream_ptr  # noqa: E402
from elfa_b200.parallel.mesh import build_context, init_distributed  # noqa: E402
from elfa_b200.runtime.symm import SymmetricArena  # noqa: E402


def timed(fn, iters=10, warm=3):
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
    ap.add_argument("--mb", type=int, default=256)
    a = ap.parse_args()
    world = init_distributed("nccl")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    pc = build_context(world, True, "nccl")
    nbytes = a.mb << 20
    arena = SymmetricArena.for_group(pc.tp_group, dev, nbytes + (64 << 20))
    recv = arena.alloc(nbytes, "probe_recv")
    src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device=dev)
    peer = (pc.rank + 1) % world
    dst = arena.peer_address(peer, recv)
    arena.barrier()
    rows = []

    def run(mode, ctas, warps=2, piece=8192, depth=2):
        lib.call("elfa_p2p_probe", src, dst, nbytes, mode, ctas, warps, piece, depth, stream_ptr(src))

    for ctas in (32, 74, 148, 296):
        rows.append((f"16-byte stores, {ctas} CTAs x 256 threads", timed(lambda: run(0, ctas))))
    for ctas, warps, piece, depth in [(148, 2, 8192, 2), (148, 2, 16384, 2), (148, 2, 8192, 4), (148, 4, 8192, 4), (148, 4, 16384, 3),
                                      (148, 8, 8192, 2), (64, 4, 16384, 3), (32, 4, 16384, 3), (16, 4, 16384, 3), (296, 2, 8192, 2)]:
        rows.append((f"bulk pipeline, {ctas} CTAs x {warps} lanes, {piece} B x {depth}", timed(lambda: run(1, ctas, warps, piece, depth))))
    # correctness of the last transfer: the receiver holds the sender's bytes
    arena.barrier()
    got = recv.view(torch.uint8, (nbytes,))
    ref = [torch.empty_like(src) for _ in range(world)]
    dist.all_gather(ref, src, group=pc.tp_group)
    assert torch.equal(got, ref[(pc.rank - 1) % world]), "probe: received bytes differ"
    full = torch.empty(world * (nbytes // 8), dtype=torch.uint8, device=dev)
    t_ag = timed(lambda: dist.all_gather_into_tensor(full, src[: nbytes // 8], group=pc.tp_group))
    if pc.rank == 0:
        print(f"world={world} bytes={nbytes}")
        for name, ms in rows:
            print(f"{name:56s} {ms:8.3f} ms {nbytes / ms / 1e6:8.1f} GB/s")
        print(f"{'NCCL all-gather of bytes/8 per rank':56s} {t_ag:8.3f} ms {(world - 1) * (nbytes // 8) / t_ag / 1e6:8.1f} GB/s received per rank")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
