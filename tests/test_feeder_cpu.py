"""Feeder: native binary and Python front end produce the same packed rows; rows feed the trainer's
row stream; JSONL extraction rules; download retry logic against a fake opener."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from autoresearch_b200 import native
from autoresearch_b200.data import feeder as F
from autoresearch_b200.data.tokenizer import Tokenizer

TOK = Path(__file__).parent / "data" / "tokenizer"


def _docs(n=40):
    words = ["alpha", "beta", "gamma", "delta", "epsilon", "The", "quick", "brown", "fox", "123", "你好", "\n"]
    return [" ".join(words[(i * 7 + j) % len(words)] for j in range(5 + (i * 13) % 60)) for i in range(n)]


def test_native_feeder_matches_python_pipeline(tmp_path):
    docs = _docs()
    jl = tmp_path / "d.jsonl"
    with open(jl, "w") as f:
        for i, d in enumerate(docs):
            rec = {"text": d} if i % 3 else {"messages": [{"role": "u", "content": d[:10]}, {"role": "a", "content": d[10:]}]}
            f.write(json.dumps(rec) + "\n")
        f.write("{not json\n")
    T = 64
    r = subprocess.run([str(native.feeder_binary()), "--tokenizer-dir", str(TOK), "--jsonl", str(jl), "--seq-len", str(T)],
                       capture_output=True, timeout=120)
    assert r.returncode == 0, r.stderr.decode()[-1000:]
    rows = np.frombuffer(r.stdout, dtype="<u2").reshape(-1, T + 1)
    tok = Tokenizer(TOK)
    texts = [d if i % 3 else d[:10] + "\n" + d[10:] for i, d in enumerate(docs)]
    want = np.stack(list(F.pack_rows((tok.encode(t, bos=True) for t in texts), T + 1)))
    assert rows.shape == want.shape and (rows == want).all()
    assert (rows[:, 0] == 8188).sum() >= 1 and rows.max() < 8192
    total = sum(len(tok.encode(t, bos=True)) for t in texts)
    assert rows.shape[0] <= total // (T + 1) + 1     # cropping discards document tails, never invents tokens


def test_python_front_end_pipes_into_native_binary(tmp_path):
    d = tmp_path / "in"
    d.mkdir()
    (d / "a.jsonl").write_text("\n".join(json.dumps({"text": t}) for t in _docs(10)) + "\n")
    (d / "b.txt").write_text("plain text document " * 30)
    env = dict(os.environ, PYTHONPATH=str(Path(__file__).parent.parent))
    outs = []
    for extra in ([], ["--python"]):
        r = subprocess.run([sys.executable, "-m", "autoresearch_b200.data.feeder", "--input", str(d), "--tokenizer-dir", str(TOK),
                            "--seq-len", "32"] + extra, capture_output=True, timeout=180, env=env)
        assert r.returncode == 0, r.stderr.decode()[-1500:]
        outs.append(r.stdout)
    assert outs[0] == outs[1] and len(outs[0]) % (33 * 2) == 0 and len(outs[0]) > 0


def test_feeder_rows_drive_the_row_stream(tmp_path):
    from autoresearch_b200.data.shards import StdinRowStream
    jl = tmp_path / "d.jsonl"
    jl.write_text("\n".join(json.dumps({"text": t}) for t in _docs(60)) + "\n")
    T = 32
    p = subprocess.Popen([str(native.feeder_binary()), "--tokenizer-dir", str(TOK), "--jsonl", str(jl), "--seq-len", str(T)],
                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL)
    s = StdinRowStream(batch_size=4, seq_len=T, fd=p.stdout.fileno(), depth=4)
    n = 0
    while True:
        b = s.next_batch(timeout_ms=20000)
        if b is None:
            break
        ids, tgt = b
        assert ids.shape == (4, T) and (ids[:, 1:] == tgt[:, :-1]).all()
        n += 1
    assert n >= 2
    p.wait()
    s.close()


def test_jsonl_text_rules():
    assert F.jsonl_text({"text": "a"}) == "a"
    assert F.jsonl_text({"messages": [{"content": "x"}, {"content": "y"}]}) == "x\ny"
    assert F.jsonl_text({"turns": [{"content": "q"}, {"nope": 1}]}) == "q"
    assert F.jsonl_text({"other": 1}) is None


def test_download_retries_then_gives_up(tmp_path):
    calls = []

    def failing(url, timeout=0):
        calls.append(url)
        raise OSError("network down")

    assert F.download_shard(3, tmp_path, retries=5, opener=failing) is None
    assert len(calls) == 5 and calls[0].endswith("shard_00003.parquet")
    assert not (tmp_path / "shard_00003.parquet").exists()

    class Resp:
        def __init__(self): self.data = [b"abc", b""]
        def read(self, n): return self.data.pop(0)
        def __enter__(self): return self
        def __exit__(self, *a): return False

    flaky = {"n": 0}

    def second_try(url, timeout=0):
        flaky["n"] += 1
        if flaky["n"] == 1:
            raise OSError("reset")
        return Resp()

    p = F.download_shard(4, tmp_path, retries=5, opener=second_try)
    assert p is not None and p.read_bytes() == b"abc" and not p.with_suffix(".tmp").exists()


def test_parquet_source(tmp_path):
    pa = pytest.importorskip("pyarrow")
    import pyarrow.parquet as pq
    pq.write_table(pa.table({"text": ["one doc", "", "two doc"]}), tmp_path / "shard_00000.parquet")
    (tmp_path / "shard_00001.parquet").write_bytes(b"garbage")
    assert list(F.parquet_texts(tmp_path / "shard_00000.parquet")) == ["one doc", "two doc"]
    assert list(F.parquet_texts(tmp_path / "shard_00001.parquet")) == []


def test_multi_epoch_replays_with_distinct_orders():
    from autoresearch_b200.tools.multi_epoch import epoch_stream
    docs = [[i] for i in range(20)]
    out = [d[0] for d in epoch_stream(docs, 3)]
    assert len(out) == 60 and sorted(out[:20]) == list(range(20)) and out[:20] != out[20:40]
