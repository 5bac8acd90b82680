"""Throughput of the native feeder (tokenise + best-fit pack + write rows) on a generated JSONL corpus.

    python -m autoresearch_b200.bench.feeder_bench --docs 20000 --seq-len 32768 --workers 1,4,16

The training step consumes tokens_per_step / step_time tokens per second (1.8 M tok/s for the 428 M model on eight
B200s); the feeder has to stay above that.  CPU only.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import tempfile
import time
from pathlib import Path

from .. import native

WORDS = ["the", "quick", "brown", "fox", "jumps", "over", "lazy", "dog", "transformer", "attention", "gradient", "Blackwell",
         "tensor", "memory", "kernel", "pipeline", "2026", "data-parallel", "NVLink", "optimizer", "é", "naïve", "数据",
         "— and so on."]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--docs", type=int, default=20000)
    ap.add_argument("--seq-len", type=int, default=32768)
    ap.add_argument("--workers", default="1,4,16")
    ap.add_argument("--tokenizer-dir", default=str(Path(__file__).resolve().parents[2] / "tests" / "data" / "tokenizer"))
    a = ap.parse_args()
    native.build()
    feeder = Path(native.__file__).parent / "feeder"
    rng = random.Random(0)
    with tempfile.TemporaryDirectory(prefix="feeder_bench_") as td:
        path = os.path.join(td, "docs.jsonl")
        with open(path, "w") as f:
            for _ in range(a.docs):
                f.write(json.dumps({"text": " ".join(rng.choice(WORDS) for _ in range(rng.randint(200, 3000)))}) + "\n")
        nbytes = os.path.getsize(path)
        row = a.seq_len + 1
        for w in [int(x) for x in a.workers.split(",")]:
            t0 = time.time()
            p = subprocess.run([str(feeder), "--tokenizer-dir", a.tokenizer_dir, "--jsonl", path, "--seq-len", str(a.seq_len),
                                "--workers", str(w)], capture_output=True, check=True)
            dt = time.time() - t0
            rows = len(p.stdout) // (2 * row)
            print(json.dumps({"workers": w, "rows": rows, "seconds": round(dt, 2), "mtok_per_s": round(rows * row / dt / 1e6, 2),
                              "jsonl_mb_per_s": round(nbytes / dt / 1e6, 1), "cpus": os.cpu_count()}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
