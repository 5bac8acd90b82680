"""TKNS shard files and the stdin row stream.

Shard format and the train/val split follow brain/src/train.rs:247-318,447-622: files
``shard_*.bin`` sorted by name; ``NUM_TRAIN_SHARDS`` train shards (rest = validation) or
"all but the last"; shard order reshuffled every epoch with a xorshift64 Fisher-Yates
(seed + epoch); rows shorter than SEQ+1 are concatenated ceil((SEQ+1)/row_len) at a time.
The stdin stream is rows of SEQ+1 little-endian u16 without framing
(brain/src/train.rs:348-409), read by a native background thread into a bounded queue.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import List, Optional

import numpy as np
import torch

from .. import native

_ERR = {-1: "cannot read file", -2: "shard too small for header", -3: "bad magic bytes",
        -4: "unsupported shard version", -5: "shard truncated"}


class Shard:
    def __init__(self, path):
        self.lib = native.lib()
        self.h = None
        h, v, s, n = C.c_void_p(), C.c_uint32(), C.c_uint32(), C.c_uint32()
        rc = self.lib.ar_shard_open(str(path).encode(), C.byref(h), C.byref(v), C.byref(s), C.byref(n))
        if rc != 0:
            raise ValueError(f"{path}: {_ERR.get(rc, rc)}")
        self.h, self.vocab, self.seq_len, self.num_rows = h, v.value, s.value, n.value

    def row(self, i: int) -> np.ndarray:
        p = self.lib.ar_shard_row(self.h, i)
        if not p:
            raise IndexError(i)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint16)), shape=(self.seq_len,))

    def close(self):
        if self.h:
            self.lib.ar_shard_close(self.h)
            self.h = None

    def __del__(self):
        self.close()


def write_shard(path, rows: np.ndarray, vocab: int) -> None:
    rows = np.ascontiguousarray(rows, dtype=np.uint16)
    rc = native.lib().ar_shard_write(str(path).encode(), vocab, rows.shape[1], rows.shape[0],
                                     rows.ctypes.data)
    if rc != 0:
        raise OSError(f"cannot write {path}")


def list_shard_files(d) -> List[Path]:
    return sorted(p for p in Path(d).iterdir() if p.name.startswith("shard_") and p.suffix == ".bin")


def shuffle_order(n: int, seed: int) -> List[int]:
    arr = np.empty(n, dtype=np.int64)
    native.lib().ar_shuffle_order(arr.ctypes.data, n, seed)
    return arr.tolist()


class ShardLoader:
    def __init__(self, data_dir, batch_size: int, seq_len: int, split: str = "train",
                 num_train_shards: Optional[int] = None, seed: int = 42,
                 rank: int = 0, world: int = 1):
        files = list_shard_files(data_dir)
        if not files:
            raise FileNotFoundError(f"no shard_*.bin under {data_dir}")
        if num_train_shards is not None:
            nt = min(num_train_shards, len(files))
        else:
            nt = max(len(files) - 1, 1)
        self.files = files[:nt] if split == "train" else (files[nt:] or files[-1:])
        self.split = split
        self.B, self.T = batch_size, seq_len
        self.seed, self.epoch = seed, 0
        self.rank, self.world = rank, world
        self.order = list(range(len(self.files)))
        if split == "train":
            self.order = shuffle_order(len(self.files), seed)
        self.si, self.ri = 0, 0
        self.cur: Optional[Shard] = None
        self._skip = 0

    def _open(self):
        if self.cur is not None:
            self.cur.close()
        self.cur = Shard(self.files[self.order[self.si]])
        self.ri = 0

    def _next_raw_row(self) -> Optional[np.ndarray]:
        while True:
            if self.cur is None:
                self._open()
            if self.ri < self.cur.num_rows:
                r = self.cur.row(self.ri)
                self.ri += 1
                return r
            self.si += 1
            if self.si >= len(self.files):
                if self.split != "train":
                    return None
                self.epoch += 1
                self.order = shuffle_order(len(self.files), self.seed + self.epoch)
                self.si = 0
            self._open()

    def _next_seq(self) -> Optional[np.ndarray]:
        need = self.T + 1
        parts, have = [], 0
        while have < need:
            r = self._next_raw_row()
            if r is None:
                return None
            parts.append(r)
            have += len(r)
        return np.concatenate(parts)[:need] if len(parts) > 1 else parts[0][:need]

    def state_dict(self):
        """Position of the stream: epoch, index into the epoch's shard order, next row of that shard (the order
        itself follows from seed + epoch)."""
        return {"epoch": self.epoch, "si": self.si, "ri": self.ri if self.cur is not None else 0}

    def load_state_dict(self, d) -> None:
        self.epoch, self.si = int(d["epoch"]), int(d["si"])
        if self.split == "train":
            self.order = shuffle_order(len(self.files), self.seed + self.epoch)
        if self.si >= len(self.files):
            raise ValueError(f"data position names shard {self.si} of {len(self.files)}")
        self._open()
        self.ri = int(d["ri"])

    def next_batch(self, ids_out=None, tgt_out=None):
        """Round-robin over data-parallel ranks: rank r takes sequences r, r+world, ..."""
        rows = []
        while len(rows) < self.B:
            for r in range(self.world):
                s = self._next_seq()
                if s is None:
                    return None
                if r == self.rank:
                    rows.append(s.astype(np.int32))
        t = torch.from_numpy(np.stack(rows))
        ids, tgt = t[:, :-1], t[:, 1:]
        if ids_out is not None:
            ids_out.copy_(ids)
            tgt_out.copy_(tgt)
            return ids_out, tgt_out
        return ids.contiguous(), tgt.contiguous()


class StdinRowStream:
    """Rows of SEQ+1 little-endian u16 from a file descriptor (default: stdin)."""

    def __init__(self, batch_size: int, seq_len: int, fd: int = 0, depth: int = 16):
        self.lib = native.lib()
        self.B, self.T = batch_size, seq_len
        self.h = self.lib.ar_rowstream_open(fd, seq_len + 1, batch_size, depth)
        if not self.h:
            raise ValueError("bad row stream parameters")
        self._batches = 0

    def next_batch(self, ids_out=None, tgt_out=None, timeout_ms: int = -1):
        if ids_out is None:
            ids_out = torch.empty(self.B, self.T, dtype=torch.int32)
            tgt_out = torch.empty(self.B, self.T, dtype=torch.int32)
        rc = self.lib.ar_rowstream_next(self.h, ids_out.data_ptr(), tgt_out.data_ptr(), timeout_ms)
        if rc == 1:
            self._batches += 1
            return ids_out, tgt_out
        if rc == 0:
            return None
        if rc == -2:
            raise TimeoutError("no batch from the feeder within the time limit")
        raise RuntimeError("feeder stream ended unexpectedly (truncated row or read error)")

    def rows_read(self) -> int:
        return int(self.lib.ar_rowstream_rows_read(self.h))

    def state_dict(self):
        return {"batches": self._batches}

    def load_state_dict(self, d) -> None:
        """A pipe cannot seek: the batches already consumed are read and dropped, which restores the position
        when the feeder replays the same stream (a seeded feeder does)."""
        ids = torch.empty(self.B, self.T, dtype=torch.int32)
        tgt = torch.empty(self.B, self.T, dtype=torch.int32)
        for _ in range(int(d.get("batches", 0)) - self._batches):
            if self.next_batch(ids, tgt) is None:
                break

    def close(self):
        if self.h:
            self.lib.ar_rowstream_close(self.h)
            self.h = None
