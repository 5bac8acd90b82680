"""Replay a fixed set of documents for several epochs with a per-epoch shuffle, feeding the packed
row stream (brain/tools/multi_epoch.py:28-164: seed 42 + epoch, documents collected once).

    python -m autoresearch_b200.tools.multi_epoch --input DIR --epochs 4 --tokenizer-dir DIR | trainer ...
"""
from __future__ import annotations

import argparse
import random
import sys
import types

from ..data import feeder as F
from ..data.tokenizer import Tokenizer


def epoch_stream(docs, epochs: int, seed: int = 42):
    for ep in range(epochs):
        order = list(range(len(docs)))
        random.Random(seed + ep).shuffle(order)
        for i in order:
            yield docs[i]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--input", required=True)
    ap.add_argument("--epochs", type=int, default=2)
    ap.add_argument("--tokenizer-dir", required=True)
    ap.add_argument("--seq-len", type=int, default=2048)
    a = ap.parse_args(argv)
    src = types.SimpleNamespace(jsonl=None, stream=False, input=a.input, seed=None, prefetch=1, cache_dir="", keep=True)
    tok = Tokenizer(a.tokenizer_dir)
    docs = [tok.encode(t, bos=True) for t in F.iter_documents(src)]
    print(f"[multi_epoch] {len(docs)} documents x {a.epochs} epochs", file=sys.stderr)
    out = sys.stdout.buffer
    try:
        for row in F.pack_rows(epoch_stream(docs, a.epochs), a.seq_len + 1):
            out.write(row.astype("<u2").tobytes())
        out.flush()
    except BrokenPipeError:
        pass
    return 0


if __name__ == "__main__":
    sys.exit(main())
