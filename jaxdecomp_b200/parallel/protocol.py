"""Host-side model of the cross-GPU signalling protocol, and rank liveness.

``FlagBoard`` restates the device protocol of ``csrc/signal.cu`` in Python:
every rank owns one 32-bit epoch slot per peer; a barrier with epoch ``e``
stores ``e`` into slot ``me`` of every peer and waits until all of its own
slots hold a value ``>= e`` in wrap-around arithmetic.  A wait that runs out of
budget returns ``TIMEOUT_PEER_SIGNAL`` with the peer, the expected and the
observed epoch; a slot that is *ahead* of the expected epoch by more than one
barrier is reported as ``STALE_EPOCH`` (a rank replayed or skipped barriers).
A rank whose wait failed sets the abort word of every rank; an aborted rank
signals nothing more and its barriers return ``PEER_ABORTED``, as do the
kernels' (``csrc/signal.cu``).  ``PipelineModel`` runs the per-chunk barriers
of the pipelined transports on top of it.  The model lets fault scenarios -- a withheld signal, a corrupted epoch -- be
tested on CPU ranks without ever making a GPU wait on something that cannot
arrive.  The reference has no failure detection: a dead peer blocks its NCCL or
MPI collective forever (``src/csrc/include/checks.h:29-72``).

``HealthMonitor`` is the host watchdog: ranks publish heartbeats in the
``torch.distributed`` store and learn about a missing peer *before* their next
launch instead of inside a kernel.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch.distributed as dist

from ..utils.errors import DecompError

OK = 0
TIMEOUT_PEER_SIGNAL = -3
STALE_EPOCH = -4
PEER_ABORTED = -8
_MASK = 0xFFFFFFFF


def _ahead(a: int, b: int) -> int:
    """Signed 32-bit difference a - b (wrap-around safe), as the kernels compute it."""
    d = (a - b) & _MASK
    return d - (1 << 32) if d & 0x80000000 else d


@dataclass
class WaitResult:
    code: int
    peer: int = -1
    expected: int = -1
    seen: int = -1


class FlagBoard:
    """Epoch slots of ``n`` ranks: ``slots[r][p]`` is what rank ``p`` last signalled to rank ``r``."""

    def __init__(self, n: int, drop: Optional[Callable[[int, int, int], bool]] = None):
        self.n = n
        self.slots: List[List[int]] = [[0] * n for _ in range(n)]
        self.counter = [0] * n
        self.aborted = [0] * n  # abort word of every rank: 0, or 1 + the rank whose wait failed
        self.drop = drop  # drop(src, dst, epoch) -> True withholds that signal

    def signal(self, src: int, epoch: int) -> None:
        for dst in range(self.n):
            if self.drop is not None and self.drop(src, dst, epoch):
                continue
            self.slots[dst][src] = epoch & _MASK

    def wait(self, me: int, epoch: int, polls: int = 8) -> WaitResult:
        """Bounded wait: ``polls`` looks at every slot, then give up (the device uses a time budget)."""
        for _ in range(max(1, polls)):
            pending = None
            for p in range(self.n):
                seen = self.slots[me][p]
                d = _ahead(seen, epoch & _MASK)
                if d > 1:
                    return WaitResult(STALE_EPOCH, p, epoch & _MASK, seen)
                if d < 0 and pending is None:
                    pending = (p, seen)
            if pending is None:
                return WaitResult(OK)
        return WaitResult(TIMEOUT_PEER_SIGNAL, pending[0], epoch & _MASK, pending[1])

    def barrier_all(self, polls: int = 8) -> List[WaitResult]:
        """One barrier round executed by every rank: all signal, then all wait.  An aborted rank
        counts the barrier but neither signals nor waits; a rank whose wait fails aborts everyone."""
        epochs = []
        for r in range(self.n):
            self.counter[r] = (self.counter[r] + 1) & _MASK
            epochs.append(self.counter[r])
            if not self.aborted[r]:
                self.signal(r, self.counter[r])
        out, failed = [], []
        for r in range(self.n):
            if self.aborted[r]:
                out.append(WaitResult(PEER_ABORTED, self.aborted[r] - 1, epochs[r]))
                continue
            w = self.wait(r, epochs[r], polls)
            if w.code != OK:
                failed.append(r)
            out.append(w)
        # a wait fails only after its whole budget, by which time the healthy ranks have left this
        # barrier: they see the abort word in their next one
        for r in failed:
            for q in range(self.n):
                if not self.aborted[q]:
                    self.aborted[q] = r + 1
        return out


class PipelineModel:
    """Per-chunk barriers of a pipelined exchange (``csrc/runtime.cpp``, ``run_pipelined``).

    Every rank issues its exchange chunks in order; before the local pass may work on chunk ``k`` the
    rank runs one barrier, which it can only signal once its own chunk ``k`` has been issued and which
    completes once every rank has signalled.  ``run`` plays the chunks of all ranks in lock step and
    returns ``(rank, chunk, code)`` for every barrier; ``consumed_before_produced`` counts local
    passes that started on a chunk some rank had not produced yet (must stay 0)."""

    def __init__(self, board: FlagBoard, chunks: int):
        self.board, self.chunks = board, chunks
        self.consumed_before_produced = 0

    def run(self, polls: int = 8):
        n = self.board.n
        produced = [[False] * self.chunks for _ in range(n)]
        log = []
        for k in range(self.chunks):
            for r in range(n):
                if not self.board.aborted[r]:
                    produced[r][k] = True  # exchange chunk k of rank r: stores into every peer
            res = self.board.barrier_all(polls)
            for r in range(n):
                log.append((r, k, res[r].code))
                if res[r].code == OK and not all(produced[q][k] for q in range(n)):
                    self.consumed_before_produced += 1
        return log


class PeerDeadError(DecompError):
    """One or more ranks stopped publishing heartbeats."""

    def __init__(self, ranks, max_age):
        super().__init__(f"ranks {sorted(ranks)} published no heartbeat for more than {max_age:.1f} s")
        self.ranks = sorted(ranks)


class HealthMonitor:
    """Heartbeats through the process-group store.

    Every rank runs a daemon thread that writes ``hb/<rank>`` = wall-clock time
    every ``period`` seconds.  ``check()`` reads all keys and raises
    :class:`PeerDeadError` for ranks whose last beat is older than ``max_age``;
    call it between steps, before launching kernels that would wait on peers.
    """

    def __init__(self, period: float = 0.2, max_age: float = 2.0, store=None, rank: Optional[int] = None,
                 world_size: Optional[int] = None):
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        self.period, self.max_age = period, max_age
        self._stop = threading.Event()
        self._beat()
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _beat(self):
        self.store.set(f"hb/{self.rank}", repr(time.time()))

    def _run(self):
        while not self._stop.wait(self.period):
            try:
                self._beat()
            except Exception:  # noqa: BLE001 - the store is gone at shutdown
                return

    def ages(self) -> List[float]:
        now = time.time()
        out = []
        for r in range(self.world):
            key = f"hb/{r}"
            try:
                # get() on a key that was never written blocks for the store's own time-out (minutes):
                # ask first whether the key exists, and treat a missing key as "never seen"
                if not self.store.check([key]):
                    out.append(float("inf"))
                    continue
                out.append(now - float(self.store.get(key).decode()))
            except Exception:  # noqa: BLE001 - the store is gone
                out.append(float("inf"))
        return out

    def check(self) -> None:
        dead = [r for r, a in enumerate(self.ages()) if a > self.max_age and r != self.rank]
        if dead:
            raise PeerDeadError(dead, self.max_age)

    def stop(self) -> None:
        """Stop publishing (used by tests to model a rank that went away)."""
        self._stop.set()
        self._thread.join(timeout=2 * self.period + 1.0)
