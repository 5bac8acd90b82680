"""C++ BPE tokenizer: golden token ids for the strings the reference tests
(brain/src/feeder/tokenizer.rs:393-431; the ids there belong to a differently trained vocabulary,
the ones below are tiktoken's output for the vocabulary checked in under tests/data/tokenizer),
agreement with tiktoken and with the `regex` module's split on random text, the .tiktoken round
trip and the byte table."""
import base64
import json
import random
from pathlib import Path

import pytest

from autoresearch_b200.data.tokenizer import Tokenizer

DATA = Path(__file__).parent / "data" / "tokenizer"

GOLDEN = [
    ('Hello', [72, 461, 111]),
    ('a', [97]),
    ('', []),
    ('Hello world!', [72, 461, 111, 996, 33]),
    ('Numbers: 123.', [78, 374, 1564, 58, 32, 1120, 51, 46]),
    ('The quick brown fox jumps over the lazy dog.', [488, 1818, 3758, 278, 1551, 523, 5043, 642, 262, 300, 1630, 121, 980, 46]),
    ('  spaces  ', [32, 5054, 1736]),
    ('line1\nline2\nline3', [1310, 49, 10, 1310, 50, 10, 1310, 51]),
    ("It's a test. I've been here. They're going.", [1311, 387, 257, 1121, 46, 332, 1412, 741, 1454, 46, 886, 896, 1456, 46]),
    ('def foo(x):\n    return x * 2', [100, 856, 278, 507, 40, 120, 41, 1118, 6354, 3259, 2904, 4105, 32, 50]),
    ('Hello world! Numbers: 123. Unicode: 你好', [72, 461, 111, 996, 33, 487, 374, 1564, 58, 32, 1120, 51, 46, 1009, 291, 1573, 58, 32, 228, 189, 160, 229, 165, 189]),
]


@pytest.fixture(scope="module")
def tok():
    return Tokenizer(DATA)


def test_load(tok):
    assert tok.bos_token_id == 8188 and tok.vocab_size == 8192


@pytest.mark.parametrize("text,ids", GOLDEN)
def test_golden_ids(tok, text, ids):
    assert tok.encode(text) == ids
    assert tok.decode(ids) == text


def test_batch_with_bos(tok):
    b = tok.encode_batch_with_bos(["Hello world", "test"])
    assert b[0][0] == 8188 and b[1][0] == 8188
    assert b[0][1:] == tok.encode("Hello world") and b[1][1:] == tok.encode("test")


def _corpus(n, seed):
    rng = random.Random(seed)
    alphabet = ["a", "b", "Z", "é", "ß", "你", "好", "д", "ا", "1", "2", "٣", " ", "  ", "\n", "\r\n", "\t", "'s", "'LL", "'x",
                ".", ",", "!", "?", "(", ")", "_", "-", " ", " ", "😀", "x", "The", "quick", "3.14", "''", "re"]
    out = []
    for _ in range(n):
        out.append("".join(rng.choice(alphabet) for _ in range(rng.randint(1, 60))))
    return out


def test_split_matches_regex_module(tok):
    regex = pytest.importorskip("regex")
    pat = regex.compile(json.loads((DATA / "tokenizer.json").read_text())["pattern"])
    for text in _corpus(400, 1) + [g[0] for g in GOLDEN]:
        assert tok.split(text) == pat.findall(text), repr(text)


def test_matches_tiktoken_on_random_text(tok):
    tiktoken = pytest.importorskip("tiktoken")
    d = json.loads((DATA / "tokenizer.json").read_text())
    enc = tiktoken.Encoding(name="ref", pat_str=d["pattern"],
                            mergeable_ranks={base64.b64decode(k): v for k, v in d["mergeable_ranks"]},
                            special_tokens={k: v for k, v in d["special_tokens"]})
    for text in _corpus(300, 2):
        assert tok.encode(text) == enc.encode_ordinary(text), repr(text)


def test_tiktoken_format_roundtrip(tok, tmp_path):
    from autoresearch_b200.tools.convert_tokenizer import convert
    convert(DATA, tmp_path)
    t2 = Tokenizer(tmp_path)
    assert t2.bos_token_id == 8188
    for text, ids in GOLDEN:
        assert t2.encode(text) == ids


def test_token_bytes_table_matches_reference_artifact(tok):
    ref = json.loads((DATA / "token_bytes.json").read_text())
    assert tok.token_bytes() == ref


def test_bpe_training_matches_a_plain_python_trainer(tmp_path):
    """The native trainer against a direct restatement of byte-pair merging (most frequent pair,
    ties to the smaller pair of ids), and the written tokenizer round-trips text."""
    import json
    from collections import Counter
    from autoresearch_b200.tools import prepare

    corpus = ("the quick brown fox jumps over the lazy dog. " * 20 + "pack my box with five dozen liquor jugs! " * 13 +
              "sphinx of black quartz, judge my vow? 12345 67890 " * 7 + "naïve café déjà vu — ünïcödé tëxt. " * 5)
    (tmp_path / "c.txt").write_text(corpus)
    prepare.main(["--input", str(tmp_path / "c.txt"), "--out", str(tmp_path / "tok"), "--vocab-size", "300"])
    d = json.loads((tmp_path / "tok" / "tokenizer.json").read_text())
    assert len(d["mergeable_ranks"]) == 296 and len(d["special_tokens"]) == 4
    from autoresearch_b200.data.tokenizer import Tokenizer
    tok = Tokenizer(tmp_path / "tok")
    assert tok.vocab_size == 300 and tok.bos_token_id == 296
    assert tok.decode(tok.encode(corpus)) == corpus
    assert len(tok.encode(corpus)) < len(corpus.encode()) // 2
    tb = json.loads((tmp_path / "tok" / "token_bytes.json").read_text())
    assert len(tb) == 300 and tb[-4:] == [0, 0, 0, 0]

    # plain trainer on the same pre-tokenised words
    words = Counter(tok.split(corpus))
    seqs = {w: list(w.encode()) for w in words}
    merges = []
    for new_id in range(256, 296):
        stat = Counter()
        for w, ids in seqs.items():
            for a, b in zip(ids, ids[1:]):
                stat[(a, b)] += words[w]
        if not stat:
            break
        best = min(stat, key=lambda p: (-stat[p], p))
        merges.append(best)
        for w, ids in seqs.items():
            out, i = [], 0
            while i < len(ids):
                if i + 1 < len(ids) and (ids[i], ids[i + 1]) == best:
                    out.append(new_id); i += 2
                else:
                    out.append(ids[i]); i += 1
            seqs[w] = out
    import base64
    table = [bytes([i]) for i in range(256)]
    for a, b in merges:
        table.append(table[a] + table[b])
    got = [base64.b64decode(k) for k, _ in d["mergeable_ranks"]]
    assert got == table[:296]
