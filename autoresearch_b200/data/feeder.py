"""Data feeder front end: parquet / JSONL documents -> packed token rows on stdout.

    python -m autoresearch_b200.data.feeder --input DIR --tokenizer-dir DIR [--seq-len 2048]
    python -m autoresearch_b200.data.feeder --stream --tokenizer-dir DIR      (download shards)
    python -m autoresearch_b200.data.feeder --jsonl FILE --tokenizer-dir DIR

Same behaviour as the reference feeders (brain/feeder.py:57-425, brain/src/bin/feeder.rs:18-129):
documents are read from ``shard_{i:05}.parquet`` files (column ``text``) or JSONL records
(``text``, or ``messages`` / ``turns`` lists with ``content``), tokenised with BOS, best-fit
packed into rows of SEQ+1 tokens and written as little-endian u16 without framing.  ``--stream``
downloads shards in the background (5 retries with exponential back-off, ``.tmp`` + rename,
deleted after use), ``--seed`` shuffles the shard order, the validation shard is excluded.

Tokenisation and packing run in the native C++ ``feeder`` binary; this module only extracts the
text (parquet needs pyarrow, which has no C++ headers on the target image) and pipes JSONL into
it.  ``--python`` keeps everything in this process through the native library's ctypes binding.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import threading
import time
import urllib.request
from pathlib import Path
from typing import Iterable, Iterator, List, Optional

import numpy as np

from .. import native

BASE_URL = "https://huggingface.co/datasets/karpathy/climbmix-400b-shuffle/resolve/main"
MAX_SHARD = 6542          # last shard = validation (excluded from training streams)
BUFFER_DOCS = 1000


def shard_name(i: int) -> str:
    return f"shard_{i:05d}.parquet"


def download_shard(i: int, cache: Path, retries: int = 5, opener=urllib.request.urlopen) -> Optional[Path]:
    """Fetch one parquet shard with exponential back-off; None when every attempt failed."""
    dst = cache / shard_name(i)
    if dst.exists():
        return dst
    cache.mkdir(parents=True, exist_ok=True)
    tmp = dst.with_suffix(".tmp")
    for attempt in range(retries):
        try:
            with opener(f"{BASE_URL}/{shard_name(i)}", timeout=60) as r, open(tmp, "wb") as f:
                while True:
                    chunk = r.read(1 << 20)
                    if not chunk:
                        break
                    f.write(chunk)
            os.replace(tmp, dst)
            return dst
        except Exception as e:  # network errors are retried, then reported
            print(f"[feeder] download {shard_name(i)} attempt {attempt + 1}/{retries} failed: {e}", file=sys.stderr)
            time.sleep(min(2 ** attempt, 30) if opener is urllib.request.urlopen else 0)
    return None


def parquet_texts(path: Path) -> Iterator[str]:
    import pyarrow.parquet as pq
    try:
        pf = pq.ParquetFile(path)
    except Exception as e:
        print(f"[feeder] skipping corrupt parquet {path}: {e}", file=sys.stderr)
        return
    for rg in range(pf.num_row_groups):
        for t in pf.read_row_group(rg, columns=["text"]).column("text").to_pylist():
            if t:
                yield t


def jsonl_text(rec: dict) -> Optional[str]:
    """text | messages[].content | turns[].content (brain/feeder.py:167-238)."""
    t = rec.get("text")
    if isinstance(t, str) and t:
        return t
    for key in ("messages", "turns"):
        seq = rec.get(key)
        if isinstance(seq, list):
            parts = [m["content"] for m in seq if isinstance(m, dict) and isinstance(m.get("content"), str)]
            if parts:
                return "\n".join(parts)
    return None


def jsonl_texts(path) -> Iterator[str]:
    f = sys.stdin if str(path) == "-" else open(path, "r", encoding="utf-8")
    with f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            try:
                t = jsonl_text(json.loads(line))
            except json.JSONDecodeError:
                continue
            if t:
                yield t


def iter_documents(args) -> Iterator[str]:
    if args.jsonl:
        yield from jsonl_texts(args.jsonl)
        return
    if args.stream:
        order = list(range(MAX_SHARD))
        if args.seed is not None:
            random.Random(args.seed).shuffle(order)
        cache = Path(args.cache_dir)
        ahead: List = []
        lock = threading.Condition()
        done = [False]

        def fetch():
            for i in order:
                with lock:
                    while len(ahead) >= max(args.prefetch, 1):
                        lock.wait()
                p = download_shard(i, cache)
                with lock:
                    ahead.append(p)
                    lock.notify_all()
            with lock:
                done[0] = True
                lock.notify_all()

        threading.Thread(target=fetch, daemon=True).start()
        while True:
            with lock:
                while not ahead and not done[0]:
                    lock.wait()
                if not ahead and done[0]:
                    return
                p = ahead.pop(0)
                lock.notify_all()
            if p is None:
                continue
            yield from parquet_texts(p)
            if not args.keep:
                p.unlink(missing_ok=True)
        return
    d = Path(args.input)
    files = sorted(p for p in d.iterdir() if p.suffix in (".parquet", ".jsonl", ".txt"))
    files = [p for p in files if p.name != shard_name(MAX_SHARD)]
    if args.seed is not None:
        random.Random(args.seed).shuffle(files)
    for p in files:
        if p.suffix == ".parquet":
            yield from parquet_texts(p)
        elif p.suffix == ".jsonl":
            yield from jsonl_texts(p)
        else:
            yield p.read_text(encoding="utf-8", errors="replace")


def pack_rows(docs: Iterable[List[int]], row_capacity: int, buffer_docs: int = BUFFER_DOCS) -> Iterator[np.ndarray]:
    """Best-fit packing through the native packer (same rule as brain/feeder.py pack_rows)."""
    lib = native.lib()
    p = lib.ar_packer_create(row_capacity, buffer_docs)
    out = np.zeros(row_capacity, dtype=np.uint16)
    try:
        for d in docs:
            a = np.asarray(d, dtype=np.int32)
            lib.ar_packer_add_doc(p, a.ctypes.data, len(a))
            while lib.ar_packer_next_row(p, 0, out.ctypes.data):
                yield out.copy()
        while lib.ar_packer_next_row(p, 1, out.ctypes.data):
            yield out.copy()
    finally:
        lib.ar_packer_destroy(p)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="autoresearch data feeder")
    ap.add_argument("--stream", action="store_true")
    ap.add_argument("--input", default=None)
    ap.add_argument("--jsonl", default=None)
    ap.add_argument("--prefetch", type=int, default=4)
    ap.add_argument("--no-prefetch", action="store_true")
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--tokenizer-dir", default=os.path.expanduser("~/.cache/autoresearch/tokenizer"))
    ap.add_argument("--cache-dir", default=os.path.expanduser("~/.cache/autoresearch/data"))
    ap.add_argument("--seq-len", type=int, default=int(os.environ.get("SEQ_LEN", "2048")))
    ap.add_argument("--max-rows", type=int, default=-1)
    ap.add_argument("--keep", action="store_true", help="keep downloaded shards")
    ap.add_argument("--python", action="store_true", help="tokenise and pack in this process")
    args = ap.parse_args(argv)
    if args.no_prefetch:
        args.prefetch = 1
    if not (args.stream or args.input or args.jsonl):
        ap.error("one of --stream, --input or --jsonl is required")
    t0 = time.time()
    if args.python:
        from .tokenizer import Tokenizer
        tok = Tokenizer(args.tokenizer_dir)
        out = sys.stdout.buffer
        rows = 0
        try:
            for row in pack_rows((tok.encode(t, bos=True) for t in iter_documents(args)), args.seq_len + 1):
                out.write(row.astype("<u2").tobytes())
                rows += 1
                if 0 <= args.max_rows <= rows:
                    break
            out.flush()
        except BrokenPipeError:
            pass
        print(f"[feeder] done: rows={rows} total={time.time() - t0:.1f}s", file=sys.stderr)
        return 0
    cmd = [str(native.feeder_binary()), "--tokenizer-dir", args.tokenizer_dir, "--jsonl", "-",
           "--seq-len", str(args.seq_len), "--max-rows", str(args.max_rows)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE)
    try:
        for t in iter_documents(args):
            proc.stdin.write(json.dumps({"text": t}).encode("utf-8") + b"\n")
            if proc.poll() is not None:
                break
        proc.stdin.close()
    except BrokenPipeError:
        pass
    return proc.wait()


if __name__ == "__main__":
    sys.exit(main())
