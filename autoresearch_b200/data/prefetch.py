"""Background batch producer with a ring of (pinned) host slots.

The reference reads stdin rows on a background thread into a bounded channel of 16 batches and
copies each batch through ONE pinned buffer (brain/src/train.rs:348-409,31-97).  Here every
loader (synthetic streams, TKNS shards, the stdin stream) is driven by the same thread:

* the thread fills free slots ahead of the training loop, so token generation / shard reads /
  pipe reads never sit between two kernel launches of a step;
* a slot is handed back with the CUDA event recorded after its host->device copy, and the
  thread waits for that event before it writes into the slot again, so a queued copy can
  never read a half-overwritten buffer however far the host runs ahead of the GPU;
* the loader's position after each batch travels with the batch, so ``state_dict()`` is the
  position after the last batch the CONSUMER took (exact resume with batches in flight).
"""
from __future__ import annotations

import queue
import threading
from typing import Optional

import torch

_END = object()


class PinnedPrefetcher:
    def __init__(self, loader, batch_size: int, seq_len: int, depth: int = 3, pin: bool = False):
        self.loader = loader
        self.B, self.T = batch_size, seq_len
        self.depth = max(2, int(depth))
        pin = bool(pin and torch.cuda.is_available())
        self.slots = [(torch.empty(batch_size, seq_len, dtype=torch.int32, pin_memory=pin),
                       torch.empty(batch_size, seq_len, dtype=torch.int32, pin_memory=pin))
                      for _ in range(self.depth)]
        self._events = [None] * self.depth
        self._has_state = hasattr(loader, "state_dict")
        self._consumed_state = loader.state_dict() if self._has_state else None
        self._start()

    # ---- producer ---------------------------------------------------------------------------
    def _start(self):
        self._free: "queue.Queue" = queue.Queue()
        self._ready: "queue.Queue" = queue.Queue()
        self._peeked = []
        self._stop = threading.Event()
        self._ended = False
        for i in range(self.depth):
            self._free.put(i)
        self._thread = threading.Thread(target=self._run, name="batch-prefetch", daemon=True)
        self._thread.start()

    def _run(self):
        while not self._stop.is_set():
            try:
                i = self._free.get(timeout=0.05)
            except queue.Empty:
                continue
            ev = self._events[i]
            if ev is not None:
                ev.synchronize()             # the copy that read this slot has finished
                self._events[i] = None
            try:
                got = self.loader.next_batch(*self.slots[i])
            except BaseException as e:        # surfaces in the consumer
                self._ready.put(e)
                return
            if got is None:
                self._ready.put(_END)
                return
            self._ready.put((i, self.loader.state_dict() if self._has_state else None))

    # ---- consumer ---------------------------------------------------------------------------
    def _take(self, timeout: Optional[float] = None):
        if self._peeked:
            return self._peeked.pop(0)
        if self._ended:
            return _END
        item = self._ready.get(timeout=timeout)
        if item is _END:
            self._ended = True
        return item

    def wait_for(self, n: int) -> bool:
        """Blocks until `n` batches are ready (n <= depth) or the source has ended; True when they are."""
        n = min(n, self.depth)
        while len(self._peeked) < n:
            if self._ended:
                return False
            item = self._ready.get()
            if item is _END:
                self._ended = True
                return False
            self._peeked.append(item)
            if isinstance(item, BaseException):
                raise item
        return True

    def next(self):
        """-> (slot, ids, targets) host tensors, or None at the end of the data."""
        item = self._take()
        if item is _END:
            return None
        if isinstance(item, BaseException):
            raise item
        i, state = item
        if state is not None:
            self._consumed_state = state
        return (i,) + self.slots[i]

    def release(self, slot: int, event=None) -> None:
        """The consumer is done with the slot's host memory once `event` (or nothing) has completed."""
        self._events[slot] = event
        self._free.put(slot)

    # ---- position ---------------------------------------------------------------------------
    def state_dict(self):
        return self._consumed_state

    def load_state_dict(self, d) -> None:
        self.close()
        self.loader.load_state_dict(d)
        self._consumed_state = self.loader.state_dict()
        self._events = [None] * self.depth
        self._start()

    def close(self) -> None:
        self._stop.set()
        t = getattr(self, "_thread", None)
        if t is not None and t.is_alive() and t is not threading.current_thread():
            t.join(timeout=5.0)

    def __del__(self):
        try:
            self._stop.set()
        except Exception:
            pass
