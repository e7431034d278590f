"""Host-side model of the cross-GPU signalling protocol, and rank liveness.

``FlagBoard`` restates the device protocol of ``csrc/signal.cu`` in Python:
every rank owns one 32-bit epoch slot per peer; a barrier with epoch ``e``
stores ``e`` into slot ``me`` of every peer and waits until all of its own
slots hold a value ``>= e`` in wrap-around arithmetic.  A wait that runs out of
budget returns ``TIMEOUT_PEER_SIGNAL`` with the peer, the expected and the
observed epoch; a slot that is *ahead* of the expected epoch by more than one
barrier is reported as ``STALE_EPOCH`` (a rank replayed or skipped barriers).
The model lets fault scenarios -- a withheld signal, a corrupted epoch -- be
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
        """One barrier round executed by every rank: all signal, then all wait."""
        epochs = []
        for r in range(self.n):
            self.counter[r] = (self.counter[r] + 1) & _MASK
            epochs.append(self.counter[r])
            self.signal(r, self.counter[r])
        return [self.wait(r, epochs[r], polls) for r in range(self.n)]


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
            try:
                out.append(now - float(self.store.get(f"hb/{r}").decode()))
            except Exception:  # noqa: BLE001 - key not written yet
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
