"""One-time preparation: train a byte-level BPE vocabulary on local text and write the tokenizer files
the engine reads.

    python -m autoresearch_b200.tools.prepare --input corpus_dir_or_file --out tok_dir --vocab-size 8192

Role of original/prepare.py:57-203 (which downloads parquet shards and trains with the rustbpe crate):
no downloads here, the corpus is whatever ``--input`` holds (``.txt`` files, ``.jsonl`` files with a
``text`` field, or ``.parquet`` files with a ``text`` column).  Output, in ``--out``:

* ``tokenizer.json``   {"pattern", "mergeable_ranks": [[base64, rank]...], "special_tokens": [[name, rank]...]}
  with vocab_size - 4 mergeable entries and the four specials ``<|reserved_0..3|>`` at the top ranks
  (``<|reserved_0|>`` is BOS), the layout of results/tokenizer/tokenizer.json;
* ``token_bytes.json`` the UTF-8 byte length of every token (0 for specials) used by the bits-per-byte eval.

Ranks follow tiktoken's convention: ranks 0..255 are the single bytes in byte order, rank 256+i is the
i-th merge.  The pre-tokenisation pattern is the GPT-4 style split of original/prepare.py:48.
"""
from __future__ import annotations

import argparse
import base64
import ctypes as C
import json
from collections import Counter
from pathlib import Path
from typing import Iterable, Iterator

import numpy as np

SPLIT_PATTERN = (r"""'(?i:[sdmt]|ll|ve|re)|[^\r\n\p{L}\p{N}]?+\p{L}+|\p{N}{1,2}| ?[^\s\p{L}\p{N}]++[\r\n]*|\s*[\r\n]|\s+(?!\S)|\s+""")
SPECIALS = [f"<|reserved_{i}|>" for i in range(4)]


def iter_texts(path) -> Iterator[str]:
    p = Path(path)
    files = sorted(p.rglob("*")) if p.is_dir() else [p]
    for f in files:
        if f.suffix == ".txt":
            yield f.read_text(encoding="utf-8", errors="replace")
        elif f.suffix == ".jsonl":
            with open(f, encoding="utf-8", errors="replace") as fh:
                for line in fh:
                    line = line.strip()
                    if line:
                        d = json.loads(line)
                        if isinstance(d.get("text"), str):
                            yield d["text"]
        elif f.suffix == ".parquet":
            import pyarrow.parquet as pq
            for batch in pq.ParquetFile(f).iter_batches(columns=["text"], batch_size=1024):
                for t in batch.column(0).to_pylist():
                    if t:
                        yield t


def train_bpe(texts: Iterable[str], vocab_size: int, splitter) -> list:
    """Returns the merges as (left bytes, right bytes) in rank order.  `splitter(text)` yields the
    pre-tokenised pieces (str)."""
    from .. import native
    words = Counter()
    for t in texts:
        words.update(splitter(t))
    items = [(w.encode("utf-8"), c) for w, c in words.items() if len(w.encode("utf-8")) > 1]
    blob = b"".join(b for b, _ in items)
    offsets = np.zeros(len(items) + 1, dtype=np.int64)
    np.cumsum([len(b) for b, _ in items], out=offsets[1:])
    counts = np.asarray([c for _, c in items], dtype=np.int64)
    n_merge_max = vocab_size - 256
    merges = np.zeros(max(1, 2 * n_merge_max), dtype=np.int32)
    L = native.lib()
    f = L.ar_bpe_train
    f.restype = C.c_int32
    f.argtypes = [C.c_char_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]
    n = f(blob, offsets.ctypes.data, counts.ctypes.data, len(items), vocab_size, merges.ctypes.data)
    if n < 0:
        raise RuntimeError("ar_bpe_train failed")
    table = [bytes([i]) for i in range(256)]
    out = []
    for i in range(n):
        a, b = table[merges[2 * i]], table[merges[2 * i + 1]]
        out.append((a, b))
        table.append(a + b)
    return out


def write_tokenizer(out_dir, merges, vocab_size: int) -> Path:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    tokens = [bytes([i]) for i in range(256)] + [a + b for a, b in merges]
    n_merge_tokens = vocab_size - len(SPECIALS)
    tokens = tokens[:n_merge_tokens]
    ranks = [[base64.b64encode(t).decode("ascii"), i] for i, t in enumerate(tokens)]
    specials = [[name, len(tokens) + i] for i, name in enumerate(SPECIALS)]
    (out / "tokenizer.json").write_text(json.dumps({"pattern": SPLIT_PATTERN, "mergeable_ranks": ranks,
                                                     "special_tokens": specials}))
    (out / "token_bytes.json").write_text(json.dumps([len(t) for t in tokens] + [0] * len(SPECIALS)))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--vocab-size", type=int, default=8192)
    ap.add_argument("--max-chars", type=int, default=2_000_000_000, help="stop reading the corpus after this many characters")
    a = ap.parse_args(argv)
    if a.vocab_size < 256 + len(SPECIALS):
        raise SystemExit("vocab size must be at least 260")
    import tempfile
    from ..data.tokenizer import Tokenizer
    # a bootstrap tokenizer (the 256 bytes + specials) gives access to the native pre-tokenisation split
    with tempfile.TemporaryDirectory(prefix="arb_tok_") as td:
        write_tokenizer(td, [], 256 + len(SPECIALS))
        boot = Tokenizer(Path(td) / "tokenizer.json")

    def texts():
        seen = 0
        for t in iter_texts(a.input):
            yield t
            seen += len(t)
            if seen >= a.max_chars:
                return

    merges = train_bpe(texts(), a.vocab_size - len(SPECIALS), boot.split)
    out = write_tokenizer(a.out, merges, a.vocab_size)
    tok = Tokenizer(out / "tokenizer.json")
    probe = "Hello world! Numbers: 123.\n"
    assert tok.decode(tok.encode(probe)) == probe, "round-trip check failed"
    (out / "token_bytes.json").write_text(json.dumps(tok.token_bytes()))   # decode semantics of the bpb eval
    print(f"wrote {out}/tokenizer.json ({tok.vocab_size} ids, {len(merges)} merges) and token_bytes.json")


if __name__ == "__main__":
    main()
