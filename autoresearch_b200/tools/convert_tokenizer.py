"""tokenizer.json -> tokenizer.tiktoken + tokenizer_config.txt (and a round-trip check).

Same file formats as the reference's converter (brain/tools/convert_tokenizer.py:21-93):
``tokenizer.tiktoken`` holds one ``<base64 bytes> <rank>`` line per merge, sorted by rank;
``tokenizer_config.txt`` holds ``pat_str:``, one ``special:<name> <rank>`` line per special token
and ``bos_id:``.
"""
from __future__ import annotations

import argparse
import base64
import json
from pathlib import Path


def convert(src_dir, dst_dir=None) -> Path:
    src, dst = Path(src_dir), Path(dst_dir or src_dir)
    d = json.loads((src / "tokenizer.json").read_text())
    specials = {k: v for k, v in d["special_tokens"]}
    bos = specials.get("<|reserved_0|>")
    if bos is None:
        raise ValueError("<|reserved_0|> is not among the special tokens")
    dst.mkdir(parents=True, exist_ok=True)
    ranks = sorted(((base64.b64decode(k), v) for k, v in d["mergeable_ranks"]), key=lambda x: x[1])
    with open(dst / "tokenizer.tiktoken", "w") as f:
        for b, r in ranks:
            f.write(f"{base64.b64encode(b).decode('ascii')} {r}\n")
    with open(dst / "tokenizer_config.txt", "w") as f:
        f.write(f"pat_str:{d['pattern']}\n")
        for name, r in sorted(specials.items(), key=lambda x: x[1]):
            f.write(f"special:{name} {r}\n")
        f.write(f"bos_id:{bos}\n")
    # round trip through the native loader
    from ..data.tokenizer import Tokenizer
    a = Tokenizer(src / "tokenizer.json")
    tmp_only = dst / "tokenizer.json"
    b = Tokenizer(dst) if not tmp_only.exists() else None
    if b is not None:
        probe = "Hello world! Numbers: 123."
        if a.encode(probe) != b.encode(probe):
            raise RuntimeError("round-trip check failed")
    return dst


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("tokenizer_dir")
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    print(f"wrote {convert(a.tokenizer_dir, a.out)}/tokenizer.tiktoken and tokenizer_config.txt")


if __name__ == "__main__":
    main()
