"""Synthetic token streams (no I/O).

* ``lcg``  – the reference's MFU stream: a 64-bit LCG, tokens in [1, vocab-1], eight
  batches generated once and cycled (brain/src/train.rs:411-444).
* ``zipf`` – Zipf(1.1)-distributed ids from a seed, packed into full sequences; every
  (rank, step, micro-step) draws from a counter-based stream so that any data-parallel
  decomposition of a step sees the same global batch.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from .. import native


class LcgStream:
    def __init__(self, batch_size: int, seq_len: int, vocab: int = 8192, cycle: int = 8):
        self.B, self.T = batch_size, seq_len
        lib = native.lib()
        rows = batch_size * cycle
        buf = np.empty(rows * (seq_len + 1), dtype=np.int32)
        st = C.c_uint64(0xdeadbeef12345678)
        lib.ar_lcg_tokens(C.byref(st), buf.size, vocab, buf.ctypes.data)
        self.buf = torch.from_numpy(buf).view(rows, seq_len + 1)
        self.pos = 0

    def next_batch(self, ids_out: torch.Tensor = None, tgt_out: torch.Tensor = None):
        rows = self.buf.shape[0]
        idx = (torch.arange(self.B) + self.pos) % rows
        chunk = self.buf[idx]
        self.pos = (self.pos + self.B) % rows
        ids, tgt = chunk[:, :-1], chunk[:, 1:]
        if ids_out is not None:
            ids_out.copy_(ids)
            tgt_out.copy_(tgt)
            return ids_out, tgt_out
        return ids.contiguous(), tgt.contiguous()

    def state_dict(self):
        return {"pos": self.pos}

    def load_state_dict(self, d):
        self.pos = int(d["pos"])


class ZipfStream:
    """Global sequence index -> tokens is a pure function of (seed, index)."""

    def __init__(self, batch_size: int, seq_len: int, vocab: int = 8192, s: float = 1.1,
                 seed: int = 1234, rank: int = 0, world: int = 1):
        self.B, self.T, self.vocab = batch_size, seq_len, vocab
        self.seed, self.rank, self.world = seed, rank, world
        self.lib = native.lib()
        self.h = self.lib.ar_zipf_create(vocab, float(s), seed)
        self.cursor = 0  # global micro-batch counter

    def _row(self, global_row: int, out: np.ndarray):
        self.lib.ar_zipf_seek(self.h, self.seed, global_row * (self.T + 1))
        self.lib.ar_zipf_fill(self.h, self.T + 1, out.ctypes.data)

    def next_batch(self, ids_out: torch.Tensor = None, tgt_out: torch.Tensor = None):
        buf = np.empty((self.B, self.T + 1), dtype=np.int32)
        base = (self.cursor * self.world + self.rank) * self.B
        for b in range(self.B):
            self._row(base + b, buf[b])
        self.cursor += 1
        t = torch.from_numpy(buf)
        ids, tgt = t[:, :-1], t[:, 1:]
        if ids_out is not None:
            ids_out.copy_(ids)
            tgt_out.copy_(tgt)
            return ids_out, tgt_out
        return ids.contiguous(), tgt.contiguous()

    def state_dict(self):
        return {"cursor": self.cursor}

    def load_state_dict(self, d):
        self.cursor = int(d["cursor"])

    def __del__(self):
        try:
            self.lib.ar_zipf_destroy(self.h)
        except Exception:
            pass
