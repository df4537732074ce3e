"""ZeRO stages 2 and 3: gradients and optimizer state (stage 3: parameters too) sharded over the data-parallel group.

At rest every rank holds ``1/dp`` of each bucket of parameters (model dtype), of its fp32 gradient
and of the optimizer state. A bucket is one transformer block; everything outside the blocks
(embeddings, final norm, head) forms the bucket ``rest``.

* ``rest`` is gathered once per optimizer step (it is needed at both ends of forward and backward)
  and its gradient is reduce-scattered once, after the last micro-batch.
* A block is gathered right before its forward and again right before its backward, into one of two
  full-size slots (block ``i`` always uses slot ``i % 2``, so the tensors autograd saved stay valid
  once the slot is refilled). The gather of the next block is issued on a side stream while the
  current block computes. The block's fp32 gradient is accumulated by the backward kernels in a
  slot of the same shape and reduce-scattered (averaged) into the rank's gradient shard when the
  next block's backward starts.
* ``gather_in_gemm`` (``ELFA_ZERO3_GATHER_IN_GEMM=1``; needs the symmetric arena): in forward no kernel gathers a block's
  matrices. The product that consumes a matrix fetches it itself - ``elfa_gemm_gb``: two warps of every CTA copy the owners'
  pieces into the local slot while the tensor cores work through the K blocks that have arrived - and only the rest of the
  bucket (norm weights) is gathered by a small windowed copy. Backward keeps the whole-block gather one block ahead.
* Stage 2 (``shard_params=False``) keeps every block's parameters whole and resident; it shares the gradient path: per-block
  fp32 gradient slots that are reused once their reduce-scatter has run (the full-size gradient buffer of stages 0 / 1 does
  not exist), the reduce-scatter of a block issued on a side stream while the next block's backward runs, bf16 on the wire
  with fp32 sums, and after the update an all-gather of the parameter shards into the resident copies.
* The optimizer sees only the local shards: :class:`Zero3Shards` has the interface of
  ``optim.flat.FlatParams`` with ``presharded = True`` (no gradient reduction or parameter gather
  in the optimizer; the gradient norm is summed over the group).

reference: ``src/distributed/zero_sharding.zig:73-113`` (``shardParameter`` / ``gatherParameter``:
``len / num_gpus`` per GPU), ``:115-157`` (``allGatherParameters`` before use), ``:159-181``
(``reduceScatterGradients`` then x 1/N), stage predicates ``src/tensor/sharding.zig:344-354``. The
reference gathers into a fresh full-size tensor per call and has no consumer; here the gather
overlaps the previous block's compute and, on GPUs with a symmetric arena, is a peer-load kernel.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..optim.flat import ALIGN
from .mesh import ParallelContext


@dataclass
class _Bucket:
    name: str
    names: List[str]
    params: List[torch.nn.Parameter]
    offsets: List[int] = field(default_factory=list)      # element offsets inside the bucket
    numel: int = 0                                          # padded to dp * ALIGN
    shard: int = 0                                          # numel / dp
    base: int = 0                                           # offset of this bucket's shard in the local flat buffers
    full: Optional[torch.Tensor] = None                     # full-size parameter slot (shared between blocks of equal parity)
    full_grad: Optional[torch.Tensor] = None                # full-size fp32 gradient slot
    slot: int = 0                                           # gradient slot index (-1: the rest bucket's own buffer)
    module: Optional[torch.nn.Module] = None
    state: str = "sharded"                                  # sharded | fwd | bwd
    ready: Optional[object] = None                          # CUDA event: gather finished
    fetch_end: int = 0                                      # elements [0, fetch_end) are matrices their forward products fetch themselves
    fused_fwd: bool = False                                 # forward of this block is running with such products
    fetched: set = field(default_factory=set)               # matrices already fetched in this forward
    src_addrs: Optional[object] = None                      # ctypes array: address of every rank's shard of this bucket


class _GemmGather:
    """Attached to a matrix (``w._gemm_gather``) whose forward product may fetch it from the owners' shards itself."""

    def __init__(self, shards: "Zero3Shards", bucket: _Bucket, offset: int):
        self.shards, self.bucket, self.offset = shards, bucket, offset

    def pending(self, w: torch.Tensor) -> bool:
        return self.bucket.fused_fwd and id(w) not in self.bucket.fetched

    def gemm(self, x2: torch.Tensor, w: torch.Tensor, gelu: bool, pre: Optional[torch.Tensor]) -> torch.Tensor:
        z, b = self.shards, self.bucket
        if not x2.is_cuda:
            # CPU ranks (gloo): the same bookkeeping with a library all-gather in place of the kernel's copy warps
            from ..ops.gemm import gemm
            full = z._all_gather_shards(b)
            n = w.numel()
            b.full[self.offset:self.offset + n].copy_(full[self.offset:self.offset + n])
            b.fetched.add(id(w))
            z.gemm_gathers += 1
            return gemm(x2, w, b_mn=True, gelu=gelu, preact=pre, out_dtype=x2.dtype)
        import ctypes
        from ..native import EPI_GELU, EPI_STORE_PREACT, lib, stream_ptr
        M, K = x2.shape
        N = w.shape[1]
        y = torch.empty((M, N), dtype=x2.dtype, device=x2.device)
        counters = torch.zeros(z.dp, dtype=torch.int32, device=x2.device)       # one per owner, raised by the kernel's copy warps
        esz = z.flat.element_size()
        flags = (EPI_GELU | (EPI_STORE_PREACT if pre is not None else 0)) if gelu else 0
        lib.call("elfa_gemm_gb", x2, x2.stride(0), y, y.stride(0), M, N, K, pre, pre.stride(0) if pre is not None else 0, flags,
                 ctypes.addressof(b.src_addrs), b.full, self.offset * esz, b.shard * esz, counters, z.rank, z.dp, 0, stream_ptr(x2))
        b.fetched.add(id(w))
        z.gemm_gathers += 1
        return y


def _is_no_decay(p: torch.nn.Parameter) -> bool:
    return bool(getattr(p, "no_decay", False)) or p.dim() < 2


class Zero3Shards:
    presharded = True
    symm = None

    def __init__(self, model: torch.nn.Module, pc: ParallelContext, blocks: Optional[Iterable[torch.nn.Module]] = None,
                 grad_dtype: torch.dtype = torch.float32, prefetch: bool = True, arena=None, shard_params: bool = True,
                 wire_bf16: bool = True, gather_in_gemm: Optional[bool] = None):
        """``arena``: a symmetric arena of the data-parallel group. With it the shards and the gradient
        slots live in peer-addressable memory and both collectives are this library's peer-load kernels
        (gather: every rank reads the peers' shards; reduce-scatter: every rank sums its slice of the
        peers' gradient slots in fixed rank order), ordered by signal-word barriers."""
        if pc.tp_size != 1:
            raise ValueError("per-block gradient / parameter sharding is implemented for pure data parallelism (tensor_parallel_size 1)")
        self.pc, self.model = pc, model
        self.shard_params = shard_params
        self.wire_bf16 = wire_bf16
        self.dp, self.rank = pc.dp_size, pc.dp_rank
        self.group = pc.dp_group
        named = list(model.named_checkpoint_parameters()) if hasattr(model, "named_checkpoint_parameters") else list(model.named_parameters())
        named = [(n, p) for n, p in named if p.requires_grad]
        self.dtype = max((p for _, p in named), key=lambda p: p.numel()).dtype      # the weights' dtype, not a leading scalar's
        self.device = named[0][1].device
        self.cuda = self.device.type == "cuda"
        blocks = list(blocks if blocks is not None else getattr(model, "blocks", []))
        by_id = {id(p): n for n, p in named}
        taken = set()
        self.buckets: List[_Bucket] = []
        for i, m in enumerate(blocks):
            ps = [p for p in m.parameters() if id(p) in by_id and id(p) not in taken]
            for p in ps:
                taken.add(id(p))
            self.buckets.append(_Bucket(f"block{i}", [by_id[id(p)] for p in ps], ps, module=m))
        rest = [(n, p) for n, p in named if id(p) not in taken]
        self.rest = _Bucket("rest", [n for n, _ in rest], [p for _, p in rest])
        self.block_buckets = list(self.buckets)
        self.buckets.append(self.rest)
        q = self.dp * ALIGN
        base = 0
        for b in self.buckets:
            order = sorted(range(len(b.params)), key=lambda j: 1 if _is_no_decay(b.params[j]) else 0)   # decay first (stable)
            b.params = [b.params[j] for j in order]
            b.names = [b.names[j] for j in order]
            off = 0
            for p in b.params:
                b.offsets.append(off)
                off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
            b.numel = (off + q - 1) // q * q
            b.shard = b.numel // self.dp
            b.base = base
            base += b.shard
        self.numel = base                       # local elements: what the optimizer updates
        self.arena = arena if (arena is not None and self.device.type == "cuda" and grad_dtype == torch.float32) else None
        esz = torch.empty(0, dtype=self.dtype).element_size()
        if self.arena is not None:
            self._r_flat = self.arena.alloc(self.numel * esz, "zero3.shards")
            self.flat = self._r_flat.view(self.dtype, (self.numel,))
            self.flat.zero_()
        else:
            self.flat = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
        self.grads = torch.zeros(self.numel, dtype=grad_dtype, device=self.device)
        self.replicated_end = 0
        self.shard_lo, self.shard_hi, self.shard_size = 0, self.numel, self.numel
        self.params = [p for b in self.buckets for p in b.params]
        self.names = [n for b in self.buckets for n in b.names]
        # full-size slots: two for the blocks, one for the rest
        nslot = max((b.numel for b in self.block_buckets), default=0)
        if shard_params:
            self._pslots = [torch.zeros(nslot, dtype=self.dtype, device=self.device) for _ in range(2)] if nslot else []
        else:       # stage 2: every block keeps its own whole parameters
            self._pslots = [torch.zeros(b.numel, dtype=self.dtype, device=self.device) for b in self.block_buckets]
        self._g_regions = []
        if self.arena is not None:
            import ctypes
            self._g_regions = [self.arena.alloc(max(nslot, 4) * 4, f"zero3.gslot{j}") for j in range(2)]
            self._gslots = [r.view(grad_dtype, (nslot,)) for r in self._g_regions] if nslot else []
            self._r_rest_grad = self.arena.alloc(self.rest.numel * 4, "zero3.rest_grad")
            rest_grad = self._r_rest_grad.view(grad_dtype, (self.rest.numel,))
            flags = self.arena.alloc(1024, "zero3.barrier")
            w = self.arena.world
            mk = lambda region: (ctypes.c_uint64 * w)(*[self.arena.peer_address(r, region) for r in range(w)])
            self._peer = {"flat": mk(self._r_flat), "gslot": [mk(r) for r in self._g_regions], "rest_grad": mk(self._r_rest_grad),
                          "flags": mk(flags), "my_flags": flags, "epoch": 0}
            if wire_bf16:
                # bf16 staging regions the peers read instead of the fp32 slots (half the NVLink bytes)
                self._stage = [self.arena.alloc(max(nslot, 8) * 2, f"zero3.stage{j}") for j in range(2)]
                self._stage_rest = self.arena.alloc(self.rest.numel * 2, "zero3.stage_rest")
                self._peer["stage"] = [mk(r) for r in self._stage]
                self._peer["stage_rest"] = mk(self._stage_rest)
            for g in self._gslots:
                g.zero_()
            rest_grad.zero_()
        else:
            self._gslots = [torch.zeros(nslot, dtype=grad_dtype, device=self.device) for _ in range(2)] if nslot else []
            rest_grad = torch.zeros(self.rest.numel, dtype=grad_dtype, device=self.device)
        for i, b in enumerate(self.block_buckets):
            b.full = self._pslots[i % 2][:b.numel] if shard_params else self._pslots[i]
            b.full_grad = self._gslots[i % 2][:b.numel]
            b.slot = i % 2
        self.rest.full = torch.zeros(self.rest.numel, dtype=self.dtype, device=self.device)
        self.rest.full_grad = rest_grad
        self.rest.slot = -1
        # move every parameter into its slot view; keep this rank's slice as the persistent shard
        with torch.no_grad():
            for b in self.buckets:
                tmp = torch.zeros(b.numel, dtype=self.dtype, device=self.device)
                for p, o in zip(b.params, b.offsets):
                    tmp[o:o + p.numel()].copy_(p.data.reshape(-1))
                self.flat[b.base:b.base + b.shard].copy_(tmp[self.rank * b.shard:(self.rank + 1) * b.shard])
                if not shard_params:
                    b.full.copy_(tmp)
                for p, o in zip(b.params, b.offsets):
                    p.data = b.full[o:o + p.numel()].view(p.shape)
                    p.main_grad = b.full_grad[o:o + p.numel()].view(p.shape)
                    p._grad_fresh = False
        self.side = torch.cuda.Stream(self.device) if (self.cuda and prefetch) else None
        self._pending_rs: List[_Bucket] = []
        self._slot_free = {}          # gradient slot -> event of the reduce-scatter that last read it (side stream)
        self._rest_valid = not shard_params
        self.gathers = 0          # statistics (tests)
        self.reduce_scatters = 0
        self.gemm_gathers = 0
        # parameter gather inside the consuming GEMM (forward): matrices the block declares, laid out first in the bucket
        import os
        if gather_in_gemm is None:
            gather_in_gemm = os.environ.get("ELFA_ZERO3_GATHER_IN_GEMM", "0") == "1"
        kernel_form = self.arena is not None and self.dtype == torch.bfloat16        # GPUs with a symmetric arena
        self.gather_in_gemm = bool(gather_in_gemm and shard_params and self.dp > 1 and (kernel_form or not self.cuda))
        if self.gather_in_gemm:
            import ctypes
            esz = self.flat.element_size()
            for b in self.block_buckets:
                own = {id(p) for p in (b.module.gemm_weights() if hasattr(b.module, "gemm_weights") else [])}
                end = 0
                for p, o in zip(b.params, b.offsets):        # the leading run of declared matrices
                    if id(p) in own and p.dim() == 2 and o == end and p.shape[0] % 8 == 0 and p.shape[1] % 8 == 0:
                        p._gemm_gather = _GemmGather(self, b, o)
                        end = o + (p.numel() + ALIGN - 1) // ALIGN * ALIGN
                    else:
                        break
                b.fetch_end = end
                if kernel_form:
                    b.src_addrs = (ctypes.c_uint64 * self.dp)(*[self.arena.peer_address(r, self._r_flat) + b.base * esz for r in range(self.dp)])
        for i, b in enumerate(self.block_buckets):
            self._hook(i, b)
        if self.arena is not None:
            self.arena.barrier()          # every rank's shards are in place before the first peer load

    def _barrier(self) -> None:
        """Device-side barrier over the group on the current stream (bounded wait)."""
        import ctypes
        from ..native import lib, stream_ptr
        z = self._peer
        z["epoch"] += 1
        lib.call("elfa_symm_barrier", ctypes.addressof(z["flags"]), z["my_flags"].tensor, self.rank, self.dp, z["epoch"], 0,
                 stream_ptr(self.flat))

    # ------------------------------------------------------------------ collectives on one bucket
    def _gather_into(self, b: _Bucket) -> None:
        shard = self.flat[b.base:b.base + b.shard]
        self.gathers += 1
        if self.dp == 1:
            b.full.copy_(shard)
        elif self.arena is not None:
            import ctypes
            from ..native import lib, stream_ptr
            esz = self.flat.element_size()
            lib.call("elfa_zero3_gather", ctypes.addressof(self._peer["flat"]), self.dp, b.base * esz, b.shard * esz, b.full,
                     stream_ptr(b.full))
        elif self.cuda:
            dist.all_gather_into_tensor(b.full, shard, group=self.group)
        else:
            parts = [torch.empty_like(shard) for _ in range(self.dp)]
            dist.all_gather(parts, shard.contiguous(), group=self.group)
            b.full.copy_(torch.cat(parts))

    def _all_gather_shards(self, b: _Bucket) -> torch.Tensor:
        """The bucket's concatenated shards through the library (CPU ranks)."""
        shard = self.flat[b.base:b.base + b.shard]
        parts = [torch.empty_like(shard) for _ in range(self.dp)]
        dist.all_gather(parts, shard.contiguous(), group=self.group)
        return torch.cat(parts)

    def _gather_rest_of(self, b: _Bucket) -> None:
        """What no product fetches itself (``[fetch_end, numel)``: norm weights, biases) by a windowed peer-load copy."""
        if self.arena is None:
            b.full[b.fetch_end:b.numel].copy_(self._all_gather_shards(b)[b.fetch_end:b.numel])
            return
        import ctypes
        from ..native import lib, stream_ptr
        esz = self.flat.element_size()
        lib.call("elfa_zero3_gather_window", ctypes.addressof(self._peer["flat"]), self.dp, b.base * esz, b.shard * esz,
                 b.fetch_end * esz, b.numel * esz, b.full, stream_ptr(b.full))

    def _gather(self, b: _Bucket, state: str, asynchronous: bool = False) -> None:
        if b.state != "sharded":
            b.state = state if b.state != "bwd" else b.state
            return
        if asynchronous and self.side is not None:
            self.side.wait_stream(torch.cuda.current_stream(self.device))   # the slot's previous user is done
            with torch.cuda.stream(self.side):
                self._gather_into(b)
                ev = torch.cuda.Event()
                ev.record(self.side)
            b.ready = ev
        else:
            self._gather_into(b)
            b.ready = None
        b.state = state

    def _wait(self, b: _Bucket) -> None:
        if b.ready is not None:
            torch.cuda.current_stream(self.device).wait_event(b.ready)
            b.ready = None

    def _reduce_scatter(self, b: _Bucket) -> None:
        """full fp32 gradient of ``b`` (plus what autograd left in ``.grad``) → averaged, added to the shard."""
        for p in b.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None
        dst = self.grads[b.base:b.base + b.shard]
        self.reduce_scatters += 1
        if self.dp == 1:
            dst.add_(b.full_grad)
        elif self.arena is not None:
            import ctypes
            from ..native import lib, stream_ptr
            if self.wire_bf16:
                stage = self._stage_rest if b.slot < 0 else self._stage[b.slot]
                lib.call("elfa_zero_pack_bf16", b.full_grad, stage.tensor, b.numel, stream_ptr(dst))
                self._barrier()           # every rank's staged gradient of this bucket is complete and visible
                peers = self._peer["stage_rest"] if b.slot < 0 else self._peer["stage"][b.slot]
                lib.call("elfa_zero3_reduce_acc_bf16", ctypes.addressof(peers), self.dp, self.rank * b.shard, b.shard, dst,
                         1.0 / self.dp, stream_ptr(dst))
            else:
                self._barrier()           # every rank's gradient of this bucket is complete and visible
                peers = self._peer["rest_grad"] if b.slot < 0 else self._peer["gslot"][b.slot]
                lib.call("elfa_zero3_reduce_acc", ctypes.addressof(peers), self.dp, self.rank * b.shard, b.shard, dst, 1.0 / self.dp,
                         stream_ptr(dst))
        elif self.cuda:
            out = torch.empty_like(dst)
            dist.reduce_scatter_tensor(out, b.full_grad, op=dist.ReduceOp.AVG, group=self.group)
            dst.add_(out)
        else:
            g = b.full_grad.clone()
            dist.all_reduce(g, group=self.group)
            dst.add_(g[self.rank * b.shard:(self.rank + 1) * b.shard] / self.dp)

    def _flush_pending(self) -> None:
        """Reduce-scatters the blocks whose backward has finished. On a GPU the collective runs on the side stream, next to
        the following block's backward; the slot's next user waits for the event recorded here."""
        for b in self._pending_rs:
            if self.side is not None and self.dp > 1:
                self.side.wait_stream(torch.cuda.current_stream(self.device))      # the block's gradient is complete
                with torch.cuda.stream(self.side):
                    self._reduce_scatter(b)
                    ev = torch.cuda.Event()
                    ev.record(self.side)
                self._slot_free[b.slot] = ev
            else:
                self._reduce_scatter(b)
            b.state = "sharded"
        self._pending_rs = []

    def _wait_slot(self, slot: int) -> None:
        ev = self._slot_free.pop(slot, None)
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)

    # ------------------------------------------------------------------ hooks on the blocks
    def _hook(self, i: int, b: _Bucket) -> None:
        blocks = self.block_buckets

        def pre_forward(module, args):
            if not self.shard_params:
                return                      # stage 2: the parameters are resident
            if self.gather_in_gemm and b.fetch_end > 0 and b.state == "sharded":
                # the block's products fetch their matrices themselves; only the rest of the bucket is copied here
                self._gather_rest_of(b)
                b.state, b.fused_fwd, b.fetched = "fwd", True, set()
                return
            if b.state == "sharded":
                self._gather(b, "fwd")
            self._wait(b)
            if i + 1 < len(blocks) and blocks[i + 1].state == "sharded" and torch.is_grad_enabled() and b.state == "fwd":
                # the other slot was last used by block i-1, whose forward has been issued already
                self._gather(blocks[i + 1], "fwd", asynchronous=True)

        def post_forward(module, args, out):
            if not self.shard_params:
                return
            b.fused_fwd = False
            if b.state == "fwd":
                b.state = "sharded"         # the slot may be overwritten; backward gathers again

        def pre_backward(module, grad_out):
            self._flush_pending()
            if b.state != "bwd":
                if b.state == "sharded" and self.shard_params:
                    self._gather(b, "bwd")
                b.state = "bwd"
                self._wait_slot(b.slot)     # the reduce-scatter that last read this gradient slot has finished
                b.full_grad.zero_()
            if not self.shard_params:
                return
            self._wait(b)
            if i - 1 >= 0 and blocks[i - 1].state == "sharded":
                self._gather(blocks[i - 1], "bwd_prefetched", asynchronous=True)

        def post_backward(module, grad_in, grad_out):
            if b not in self._pending_rs:
                self._pending_rs.append(b)

        b.module.register_forward_pre_hook(pre_forward)
        b.module.register_forward_hook(post_forward)
        b.module.register_full_backward_pre_hook(pre_backward)
        b.module.register_full_backward_hook(post_backward)

    # ------------------------------------------------------------------ step protocol (called by the trainer / optimizer)
    def before_forward(self) -> None:
        """Makes the ``rest`` bucket valid (once per optimizer step) and resets block states."""
        if not self._rest_valid and self.shard_params:
            self._gather_into(self.rest)
            self._rest_valid = True
        for b in self.block_buckets:
            if b.state == "bwd_prefetched":
                b.state = "sharded"

    def after_backward(self) -> None:
        """End of one micro-batch's backward: reduce-scatter what is still pending."""
        self._flush_pending()
        for b in self.block_buckets:
            b.state = "sharded"
            b.ready = None
        if self.side is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.side)
            self._slot_free.clear()
        if self.arena is not None and self.dp > 1:
            # the last reduce-scatter of this micro-batch read the peers' gradient slots: nobody may zero or refill a slot
            # for the next micro-batch before every rank has finished that read
            self._barrier()

    def fold_autograd_grads(self) -> None:
        """Called by the optimizer before the update: the ``rest`` gradient (accumulated over all
        micro-batches in its full-size buffer) is reduce-scattered now."""
        self._flush_pending()
        if self.side is not None:
            # barriers are counted: the ones issued on the side stream must run before the next one on this stream
            torch.cuda.current_stream(self.device).wait_stream(self.side)
            self._slot_free.clear()
        self._reduce_scatter(self.rest)
        self.rest.full_grad.zero_()

    def after_step(self) -> None:
        self._rest_valid = False
        if self.arena is not None and self.dp > 1:
            self._barrier()               # all shards updated before anyone gathers them again
        if not self.shard_params:
            # stage 2: the updated shards go back into every rank's resident parameters
            for b in self.buckets:
                self._gather_into(b)
            self._rest_valid = True
            if self.arena is not None and self.dp > 1:
                self._barrier()           # nobody updates its shards again while a peer still reads them

    def zero_grad(self) -> None:
        self.grads.zero_()
        self.rest.full_grad.zero_()
        for p in self.params:
            p.grad = None

    # ------------------------------------------------------------------ FlatParams interface used by the optimizers
    def wd_ranges(self, lo: Optional[int] = None, hi: Optional[int] = None) -> List[Tuple[int, int, bool]]:
        lo = 0 if lo is None else lo
        hi = self.numel if hi is None else hi
        out: List[Tuple[int, int, bool]] = []
        for b in self.buckets:
            s0 = self.rank * b.shard                 # bucket coordinates of this rank's slice
            decay_end = b.numel
            for p, o in zip(b.params, b.offsets):
                if _is_no_decay(p):
                    decay_end = o
                    break
            for a, e, wd in ((0, decay_end, True), (decay_end, b.numel, False)):
                a2, e2 = max(a, s0), min(e, s0 + b.shard)
                if a2 >= e2:
                    continue
                ga, ge = b.base + a2 - s0, b.base + e2 - s0
                ga, ge = max(ga, lo), min(ge, hi)
                if ga >= ge:
                    continue
                if out and out[-1][2] == wd and out[-1][1] == ga:
                    out[-1] = (out[-1][0], ge, wd)
                else:
                    out.append((ga, ge, wd))
        return out

    def param_slices(self) -> Dict[str, Tuple[int, int]]:
        raise NotImplementedError("stage 3 shards do not hold whole parameters; use full_tensors()")

    # ------------------------------------------------------------------ checkpoints
    def full_tensors(self) -> List[Tuple[str, torch.Tensor]]:
        """(name, full tensor) for every parameter, gathered bucket by bucket (every rank must call)."""
        out = []
        for b in self.buckets:
            self._gather_into(b)
            if self.cuda:
                torch.cuda.current_stream(self.device).synchronize()
            for n, p, o in zip(b.names, b.params, b.offsets):
                out.append((n, b.full[o:o + p.numel()].view(p.shape).detach().clone()))
            if b is not self.rest:
                b.state = "sharded"
        self._rest_valid = True
        return out if self.shard_params else [(n, t) for n, t in out]

    @torch.no_grad()
    def load_full(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Writes full tensors (same on every rank) into the local shards."""
        for b in self.buckets:
            tmp = torch.zeros(b.numel, dtype=self.dtype, device=self.device)
            for n, p, o in zip(b.names, b.params, b.offsets):
                if n not in tensors:
                    raise KeyError(f"checkpoint is missing tensor '{n}'")
                t = tensors[n]
                if tuple(t.shape) != tuple(p.shape):
                    raise ValueError(f"tensor '{n}': checkpoint shape {tuple(t.shape)} != model shape {tuple(p.shape)}")
                tmp[o:o + p.numel()].copy_(t.reshape(-1).to(self.device, self.dtype))
            self.flat[b.base:b.base + b.shard].copy_(tmp[self.rank * b.shard:(self.rank + 1) * b.shard])
            if not self.shard_params:
                b.full.copy_(tmp)
        self._rest_valid = not self.shard_params

    def logical_state(self, v: torch.Tensor, lo: int, hi: int, pc) -> Dict[str, torch.Tensor]:
        """One optimizer-state buffer (laid out like the local shards) as full per-parameter host tensors (collective)."""
        out: Dict[str, torch.Tensor] = {}
        v = v.detach()
        for b in self.buckets:
            local = v[b.base:b.base + b.shard].contiguous()
            if self.dp == 1:
                full = local
            elif self.cuda:
                full = torch.empty(b.numel, dtype=v.dtype, device=v.device)
                dist.all_gather_into_tensor(full, local, group=self.group)
            else:
                parts = [torch.empty_like(local) for _ in range(self.dp)]
                dist.all_gather(parts, local, group=self.group)
                full = torch.cat(parts)
            for n, p, o in zip(b.names, b.params, b.offsets):
                out[n] = full[o:o + p.numel()].view(p.shape).cpu().clone()
        return out

    @torch.no_grad()
    def load_logical_state(self, tensors: Dict[str, torch.Tensor], v: torch.Tensor, lo: int, hi: int, pc) -> None:
        for b in self.buckets:
            tmp = torch.zeros(b.numel, dtype=v.dtype, device=v.device)
            for n, p, o in zip(b.names, b.params, b.offsets):
                if n not in tensors:
                    raise KeyError(f"optimizer state is missing tensor '{n}'")
                tmp[o:o + p.numel()].copy_(tensors[n].reshape(-1).to(v.device, v.dtype))
            v[b.base:b.base + b.shard].copy_(tmp[self.rank * b.shard:(self.rank + 1) * b.shard])

    def memory_report(self) -> Dict[str, int]:
        esz = self.flat.element_size()
        full = sum(b.numel for b in self.buckets)
        gslots = sum(g.numel() for g in self._gslots) + self.rest.numel
        return {"param_bytes_at_rest": (self.numel if self.shard_params else full + self.numel) * esz, "param_bytes_unsharded": full * esz,
                "transient_bytes": ((sum(s.numel() for s in self._pslots) if self.shard_params else 0) + self.rest.numel) * esz,
                # fp32 gradient memory: this rank's shard plus the reusable block slots, against one full-size buffer
                "grad_bytes": (self.numel + gslots) * 4, "grad_bytes_unsharded": full * 4}
