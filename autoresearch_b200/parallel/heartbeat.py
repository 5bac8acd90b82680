"""Rank liveness: every rank publishes a heartbeat counter in a key-value store (the process
group's TCP store or any object with ``set``/``get``), a watchdog thread compares the peers'
counters with the clock and the training loop asks ``check()`` between steps, before it launches
anything that would wait for a dead peer.

The reference has no liveness protocol: a hung peer hangs the job (brain/src/nccl.rs:50-59 spins
on the rendez-vous file without bound, send/recv have no timeout).  Device-side waits in this
package are bounded as well (``ops/csrc/ptx.cuh``) and report through an error word
(``ops.kernels.check_err_flag``); this module is the host-side half.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional


class RankFailure(RuntimeError):
    def __init__(self, ranks: List[int], age_s: float):
        super().__init__(f"rank(s) {ranks} sent no heartbeat for {age_s:.1f}s")
        self.ranks = ranks


class DictStore:
    """In-process stand-in for the TCP store (tests, single-process runs)."""

    def __init__(self):
        self.d: Dict[str, bytes] = {}
        self.lock = threading.Lock()

    def set(self, k: str, v):
        with self.lock:
            self.d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        with self.lock:
            if k not in self.d:
                raise KeyError(k)
            return self.d[k]


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval_s: float = 1.0, timeout_s: float = 10.0,
                 prefix: str = "hb", clock: Callable[[], float] = time.monotonic):
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix, self.clock = interval_s, timeout_s, prefix, clock
        self._stop = threading.Event()
        self._paused = threading.Event()
        self._beat = 0
        self._seen: Dict[int, tuple] = {}      # rank -> (counter, local time it last changed)
        self._dead: List[int] = []
        self._lock = threading.Lock()
        self._th: Optional[threading.Thread] = None

    # -- publishing / observing (also callable directly, without the thread) -----------------
    def beat(self) -> None:
        if self._paused.is_set():
            return                                   # fault injection: this rank "drops" its messages
        self._beat += 1
        self.store.set(f"{self.prefix}/{self.rank}", str(self._beat))

    def observe(self) -> None:
        now = self.clock()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                c = int(self.store.get(f"{self.prefix}/{r}"))
            except Exception:
                c = -1
            last = self._seen.get(r)
            if last is None or last[0] != c:
                self._seen[r] = (c, now)
            elif now - last[1] > self.timeout:
                dead.append(r)
        with self._lock:
            self._dead = dead

    def _run(self):
        while not self._stop.wait(self.interval):
            try:
                self.beat()
                self.observe()
            except Exception:
                pass

    def start(self):
        self.beat()
        self.observe()
        self._th = threading.Thread(target=self._run, daemon=True, name=f"heartbeat-{self.rank}")
        self._th.start()
        return self

    def stop(self):
        self._stop.set()
        if self._th is not None:
            self._th.join(timeout=2 * self.interval + 1)

    def pause(self):
        self._paused.set()

    def resume(self):
        self._paused.clear()

    # -- the training loop's side ------------------------------------------------------------------
    def dead_ranks(self) -> List[int]:
        with self._lock:
            return list(self._dead)

    def check(self) -> None:
        """Raise RankFailure if a peer has been silent for longer than the timeout."""
        d = self.dead_ranks()
        if d:
            raise RankFailure(d, self.timeout)
