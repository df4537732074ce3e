"""A host model of the device-side flag protocols, with threads as ranks and random delays.

``compute-sanitizer --tool racecheck`` sees one GPU; the protocols here synchronise several. Their rules are
therefore also written down as plain Python over shared lists, run with one thread per rank and random sleeps
between every step, and checked for the two properties that matter: nothing is read before it was written
for this operation, and nothing is overwritten while a peer may still read it.

Modelled (same rules as the kernels and their host bookkeeping):

* :class:`PushGatherModel` - the all-gather of the fused all-gather->GEMM kernel (``parallel/fused.py``,
  ``csrc/gemm_bf16.cu``): a ring of ``ring`` slots per rank, every rank pushes its shard into the slot of
  every peer and then raises that peer's arrival counter; counters only grow, the wait target of the
  ``n``-th use of a slot is ``(n + 1) * world``. With ``ring=2`` the protocol is safe; ``ring=1`` is the
  negative control (a fast rank overwrites data a slow one has not read yet).
* :class:`DeferredSignalPushModel` - the push role of the fused all-gather kernels as it runs now (``csrc/comm.cuh``
  ``push_ranges``): stores are asynchronous (bulk copies that complete some time after they were issued, in any order), the
  peers are served one after the other without draining the pipeline, and a peer's counter is raised only after the NEXT
  peer's stores have been issued and every store older than those is known to be complete (``cp.async.bulk.wait_group n``
  with ``n`` = the stores issued since). Raising the counter without that wait is the negative control.
* :class:`MailboxModel` - the two-slot neighbour mailbox of ``parallel/sp.py`` (``csrc/p2p.cu``):
  arrival counter on the receiver, acknowledgement counter on the sender, a send waits for the
  acknowledgement of the message that used the same slot two sends ago.
* :class:`BarrierModel` - the epoch barrier on per-sender signal words (``csrc/zero.cu`` ``elfa_symm_barrier``).

Every wait is bounded, as on the device: when the limit passes the rank records a timeout status and stops
(`status` is non-zero), it never spins for ever.

reference: ``scripts/profile.sh:43-57`` (``compute-sanitizer`` memcheck / racecheck on the single-GPU smoke test
is all the reference has).
"""
from __future__ import annotations

import random
import threading
import time
from typing import List, Optional

TIMEOUT = 1


class _Rank:
    def __init__(self):
        self.status = 0
        self.errors: List[str] = []


def _wait(pred, limit_s: float) -> bool:
    t0 = time.perf_counter()
    while not pred():
        if time.perf_counter() - t0 > limit_s:
            return False
        time.sleep(0)
    return True


class PushGatherModel:
    def __init__(self, world: int, ring: int = 2, seed: int = 0, max_delay_s: float = 2e-4, wait_limit_s: float = 5.0,
                 skip_signal: Optional[tuple] = None):
        self.world, self.ring = world, ring
        self.rng = random.Random(seed)
        self.max_delay, self.limit = max_delay_s, wait_limit_s
        self.skip_signal = skip_signal                    # (rank, op): that rank does not raise the counters of that op
        # slots[rank][slot][source] = stamp (op, source) of the shard last written there
        self.slots = [[[None] * world for _ in range(ring)] for _ in range(world)]
        self.arrivals = [[0] * ring for _ in range(world)]
        self.lock = threading.Lock()                      # stands for the atomicity of one counter increment
        self.ranks = [_Rank() for _ in range(world)]

    def _delay(self, rng):
        time.sleep(rng.random() * self.max_delay)

    def _run_rank(self, r: int, ops: int):
        rng = random.Random(self.rng.random() + r)
        me = self.ranks[r]
        for n in range(ops):
            slot = n % self.ring
            target = (n // self.ring + 1) * self.world   # arrivals promised to this slot so far (host bookkeeping)
            for peer in range(self.world):               # push: data first, then the counter (release order)
                self._delay(rng)
                self.slots[peer][slot][r] = (n, r)
                if self.skip_signal == (r, n):
                    continue
                with self.lock:
                    self.arrivals[peer][slot] += 1
            if not _wait(lambda: self.arrivals[r][slot] >= target, self.limit):
                me.status = TIMEOUT                      # the kernel sets the status word and returns
                return
            for src in range(self.world):                # consume (the GEMM's tile loads)
                self._delay(rng)
                got = self.slots[r][slot][src]
                if got != (n, src):
                    me.errors.append(f"rank {r} op {n}: slot {slot} source {src} holds {got}")

    def run(self, ops: int) -> List[_Rank]:
        ts = [threading.Thread(target=self._run_rank, args=(r, ops)) for r in range(self.world)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return self.ranks


class DeferredSignalPushModel:
    """``world`` ranks, each pushes ``pieces`` pieces of its shard to every peer per operation. A store is issued into the
    rank's queue and lands when the rank's link thread gets to it (random order among the queued ones, random delays);
    ``wait_all_but(n)`` returns once every store except the ``n`` most recently issued has landed."""

    def __init__(self, world: int, pieces: int = 3, ring: int = 2, seed: int = 0, max_delay_s: float = 2e-4, wait_limit_s: float = 5.0,
                 wait_for_completion: bool = True):
        self.world, self.pieces, self.ring = world, pieces, ring
        self.rng = random.Random(seed)
        self.max_delay, self.limit = max_delay_s, wait_limit_s
        self.wait_for_completion = wait_for_completion
        # data[rank][slot][source][piece] = stamp (op, source, piece); arrivals[rank][slot][source] = uses signalled so far
        self.data = [[[[None] * pieces for _ in range(world)] for _ in range(ring)] for _ in range(world)]
        self.arrivals = [[[0] * world for _ in range(ring)] for _ in range(world)]
        self.queue = [[] for _ in range(world)]           # per sender: [issue index, landed?, (peer, slot, piece, stamp)]
        self.issued = [0] * world
        self.lock = threading.Lock()
        self.stop = False
        self.ranks = [_Rank() for _ in range(world)]

    def _link(self, r: int):
        """The sender's link: lands queued stores one at a time, any of the queued ones next."""
        rng = random.Random(self.rng.random() + 100 + r)
        while not self.stop:
            with self.lock:
                waiting = [e for e in self.queue[r] if not e[1]]
                e = rng.choice(waiting) if waiting else None
            if e is None:
                time.sleep(0)
                continue
            time.sleep(rng.random() * self.max_delay)
            peer, slot, piece, stamp = e[2]
            self.data[peer][slot][r][piece] = stamp
            with self.lock:
                e[1] = True

    def _wait_all_but(self, r: int, n: int) -> bool:
        def done():
            with self.lock:
                limit = self.issued[r] - n
                ok = all(e[1] for e in self.queue[r] if e[0] < limit)
                if ok:
                    self.queue[r] = [e for e in self.queue[r] if not (e[1] and e[0] < limit)]
                return ok
        return _wait(done, self.limit)

    def _run_rank(self, r: int, ops: int):
        rng = random.Random(self.rng.random() + r)
        me = self.ranks[r]
        for n in range(ops):
            slot, use = n % self.ring, n // self.ring + 1
            for p in range(self.pieces):                 # the own shard is a local copy
                self.data[r][slot][r][p] = (n, r, p)
            self.arrivals[r][slot][r] = use
            prev = None
            for i in range(1, self.world):
                peer = (r + i) % self.world
                for p in range(self.pieces):
                    time.sleep(rng.random() * self.max_delay)
                    with self.lock:
                        self.queue[r].append([self.issued[r], False, (peer, slot, p, (n, r, p))])
                        self.issued[r] += 1
                if prev is not None:
                    if self.wait_for_completion and not self._wait_all_but(r, self.pieces):
                        me.status = TIMEOUT
                        return
                    self.arrivals[prev][slot][r] = use   # release: everything older has landed
                prev = peer
            if prev is not None:
                if self.wait_for_completion and not self._wait_all_but(r, 0):
                    me.status = TIMEOUT
                    return
                self.arrivals[prev][slot][r] = use
            for i in range(self.world):                  # consume in arrival order: own shard, then rank - 1, rank - 2, ...
                src = (r - i) % self.world
                if not _wait(lambda: self.arrivals[r][slot][src] >= use, self.limit):
                    me.status = TIMEOUT
                    return
                for p in range(self.pieces):
                    got = self.data[r][slot][src][p]
                    if got != (n, src, p):
                        me.errors.append(f"rank {r} op {n}: slot {slot} source {src} piece {p} holds {got}")

    def run(self, ops: int) -> List[_Rank]:
        links = [threading.Thread(target=self._link, args=(r,)) for r in range(self.world)]
        ts = [threading.Thread(target=self._run_rank, args=(r, ops)) for r in range(self.world)]
        for t in links + ts:
            t.start()
        for t in ts:
            t.join()
        self.stop = True
        for t in links:
            t.join()
        return self.ranks


class MailboxModel:
    """Ring of ``world`` ranks, each sends ``msgs`` messages to its right neighbour and receives as many from the left."""

    def __init__(self, world: int, seed: int = 0, max_delay_s: float = 2e-4, wait_limit_s: float = 5.0, wait_for_ack: bool = True):
        self.world = world
        self.rng = random.Random(seed)
        self.max_delay, self.limit, self.wait_for_ack = max_delay_s, wait_limit_s, wait_for_ack
        self.box = [[None, None] for _ in range(world)]   # two slots per receiver
        self.arrivals = [0] * world
        self.acks = [0] * world                           # on the sender: messages its right neighbour has consumed
        self.ranks = [_Rank() for _ in range(world)]

    def _sender(self, r: int, msgs: int):
        rng = random.Random(self.rng.random() + r)
        right = (r + 1) % self.world
        for m in range(msgs):
            if m >= 2 and self.wait_for_ack and not _wait(lambda: self.acks[r] >= m - 1, self.limit):
                self.ranks[r].status = TIMEOUT
                return
            time.sleep(rng.random() * self.max_delay)
            self.box[right][m % 2] = (m, r)
            self.arrivals[right] = m + 1                  # single writer: the left neighbour

    def _receiver(self, r: int, msgs: int):
        rng = random.Random(self.rng.random() + 100 + r)
        left = (r - 1) % self.world
        for m in range(msgs):
            if not _wait(lambda: self.arrivals[r] >= m + 1, self.limit):
                self.ranks[r].status = TIMEOUT
                return
            time.sleep(rng.random() * self.max_delay)
            got = self.box[r][m % 2]
            if got != (m, left):
                self.ranks[r].errors.append(f"rank {r} message {m}: slot holds {got}")
            self.acks[left] = m + 1                       # acknowledge after the copy out of the slot

    def run(self, msgs: int) -> List[_Rank]:
        ts = []
        for r in range(self.world):
            ts.append(threading.Thread(target=self._sender, args=(r, msgs)))
            ts.append(threading.Thread(target=self._receiver, args=(r, msgs)))
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return self.ranks


class BarrierModel:
    """The stream-ordered barrier of ``csrc/zero.cu`` (``elfa_symm_barrier``): rank r adds one to word ``[r]`` of every
    peer's signal array, then waits until each word ``[p]`` of its own array has reached the barrier's epoch. The words
    only grow (one increment per barrier and sender), so a fast rank that already signals barrier ``e + 1`` cannot be
    mistaken for, or hide, barrier ``e``. Between barriers every rank does one epoch of "work"; the model records a violation
    when some rank starts epoch ``e + 1``'s work before every rank has finished epoch ``e``'s."""

    def __init__(self, world: int, seed: int = 0, max_delay_s: float = 2e-4, wait_limit_s: float = 5.0, absent: Optional[tuple] = None):
        self.world = world
        self.rng = random.Random(seed)
        self.max_delay, self.limit = max_delay_s, wait_limit_s
        self.absent = absent                               # (rank, epoch): that rank never signals that barrier (it left)
        self.words = [[0] * world for _ in range(world)]   # words[receiver][sender]
        self.lock = threading.Lock()
        self.done = [[False] * world for _ in range(64)]   # done[epoch][rank]: work of that epoch finished
        self.ranks = [_Rank() for _ in range(world)]

    def _run_rank(self, r: int, epochs: int):
        rng = random.Random(self.rng.random() + r)
        me = self.ranks[r]
        for e in range(1, epochs + 1):
            # work of epoch e: everybody must be through barrier e - 1, i.e. have finished the work of epoch e - 1
            if e > 1 and not all(self.done[e - 1]):
                me.errors.append(f"rank {r} began epoch {e} while {[p for p in range(self.world) if not self.done[e - 1][p]]} were in {e - 1}")
            time.sleep(rng.random() * self.max_delay)
            self.done[e][r] = True
            if self.absent == (r, e):
                return
            for p in range(self.world):                   # signal: one increment per peer
                if p != r:
                    with self.lock:
                        self.words[p][r] += 1
            for p in range(self.world):                   # wait: signed comparison against the epoch, bounded
                if p != r and not _wait(lambda: self.words[r][p] - e >= 0, self.limit):
                    me.status = TIMEOUT
                    return

    def run(self, epochs: int) -> List[_Rank]:
        ts = [threading.Thread(target=self._run_rank, args=(r, epochs)) for r in range(self.world)]
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return self.ranks
