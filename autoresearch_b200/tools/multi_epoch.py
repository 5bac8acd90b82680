"""Replay a fixed set of documents for several epochs with a per-epoch shuffle, feeding the packed row stream
(brain/tools/multi_epoch.py:28-164: documents collected once, order reshuffled with seed 42 + epoch, the collection
spilled to disk when it outgrows memory).

    python -m autoresearch_b200.tools.multi_epoch --input DIR --epochs 4 --tokenizer-dir DIR | trainer --stream-input ...
    python -m autoresearch_b200.tools.multi_epoch --jsonl docs.jsonl --epochs 3 --target-rows 20000 ...

The documents are tokenised ONCE (the reference keeps the text and re-tokenises every epoch) and held as one flat
u16 array plus offsets.  Above ``--mem-limit-mb`` of tokens the array is written to a temporary file and memory-mapped,
so a collection larger than RAM replays at page-cache speed; the file is removed when the stream ends.
``--target-rows`` stops collecting documents once epochs x collected tokens covers that many packed rows
(the reference's ``estimate_parquets_needed``, done on actual token counts instead of an average).
"""
from __future__ import annotations

import argparse
import os
import random
import sys
import tempfile
import time
import types
from typing import Iterable, Iterator, List, Optional

import numpy as np

from ..data import feeder as F
from ..data.tokenizer import Tokenizer


class DocStore:
    """Token ids of many documents as one flat little-endian u16 array with offsets; in RAM up to `mem_limit` bytes,
    then appended to a temporary file that is memory-mapped for reading."""

    def __init__(self, mem_limit: int = 4 << 30, tmp_dir: Optional[str] = None):
        self.mem_limit = int(mem_limit)
        self.tmp_dir = tmp_dir
        self.offsets: List[int] = [0]
        self._chunks: List[np.ndarray] = []
        self._bytes = 0
        self._file = None
        self.path: Optional[str] = None
        self._flat: Optional[np.ndarray] = None

    @property
    def on_disk(self) -> bool:
        return self.path is not None

    def __len__(self) -> int:
        return len(self.offsets) - 1

    @property
    def n_tokens(self) -> int:
        return self.offsets[-1]

    def add(self, ids) -> None:
        a = np.asarray(ids, dtype="<u2")
        self.offsets.append(self.offsets[-1] + a.size)
        if self._file is not None:
            self._file.write(a.tobytes())
            return
        self._chunks.append(a)
        self._bytes += a.nbytes
        if self._bytes > self.mem_limit:
            fd, self.path = tempfile.mkstemp(prefix="multi_epoch_", suffix=".u16", dir=self.tmp_dir)
            self._file = os.fdopen(fd, "wb")
            print(f"[multi_epoch] {self._bytes / 2**20:.0f} MB of tokens exceed the memory limit, spilling to {self.path}",
                  file=sys.stderr)
            for c in self._chunks:
                self._file.write(c.tobytes())
            self._chunks = []

    def seal(self) -> None:
        if self._file is not None:
            self._file.close()
            self._file = None
            self._flat = np.memmap(self.path, dtype="<u2", mode="r") if self.n_tokens else np.empty(0, "<u2")
        else:
            self._flat = np.concatenate(self._chunks) if self._chunks else np.empty(0, "<u2")
            self._chunks = []

    def doc(self, i: int) -> np.ndarray:
        return np.asarray(self._flat[self.offsets[i]:self.offsets[i + 1]])

    def close(self) -> None:
        self._flat = None
        if self.path and os.path.exists(self.path):
            os.remove(self.path)
        self.path = None


def epoch_stream(docs, epochs: int, seed: int = 42) -> Iterator:
    """docs: a DocStore or a list; yields every document once per epoch in that epoch's shuffled order."""
    n = len(docs)
    get = docs.doc if isinstance(docs, DocStore) else docs.__getitem__
    for ep in range(epochs):
        order = list(range(n))
        random.Random(seed + ep).shuffle(order)
        for i in order:
            yield get(i)


def collect(texts: Iterable[str], tok, epochs: int, row_len: int, target_rows: Optional[int], mem_limit: int,
            tmp_dir: Optional[str] = None) -> DocStore:
    store = DocStore(mem_limit, tmp_dir)
    need = None if not target_rows else target_rows * row_len
    for t in texts:
        store.add(tok.encode(t, bos=True))
        if need is not None and store.n_tokens * epochs >= need:
            break
    store.seal()
    return store


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", default=None, help="directory of shard_*.parquet files")
    ap.add_argument("--jsonl", default=None, help="JSONL file ('-' = stdin) instead of parquet shards")
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--tokenizer-dir", required=True)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--target-rows", type=int, default=None)
    ap.add_argument("--mem-limit-mb", type=float, default=4096.0)
    ap.add_argument("--tmp-dir", default=None)
    a = ap.parse_args(argv)
    if not a.input and not a.jsonl:
        ap.error("one of --input / --jsonl is required")
    src = types.SimpleNamespace(jsonl=a.jsonl, stream=False, input=a.input, seed=None, prefetch=1, cache_dir="", keep=True)
    tok = Tokenizer(a.tokenizer_dir)
    t0 = time.time()
    store = collect(F.iter_documents(src), tok, a.epochs, a.seq_len + 1, a.target_rows, int(a.mem_limit_mb * 2**20), a.tmp_dir)
    print(f"[multi_epoch] {len(store)} documents, {store.n_tokens} tokens ({'disk' if store.on_disk else 'memory'}) "
          f"collected in {time.time() - t0:.1f}s; {a.epochs} epochs", file=sys.stderr)
    out = sys.stdout.buffer
    rows = 0
    try:
        for row in F.pack_rows(epoch_stream(store, a.epochs, a.seed), a.seq_len + 1):
            out.write(row.astype("<u2").tobytes())
            rows += 1
        out.flush()
    except BrokenPipeError:
        pass
    finally:
        store.close()
    print(f"[multi_epoch] wrote {rows} rows", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
