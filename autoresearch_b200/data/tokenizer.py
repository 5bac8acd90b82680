"""BPE tokenizer (native C++ implementation, tiktoken-compatible for the reference vocabulary)."""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import List

import numpy as np

from .. import native


class Tokenizer:
    def __init__(self, path):
        """`path`: a directory holding tokenizer.json (or tokenizer.tiktoken + tokenizer_config.txt),
        or the tokenizer.json file itself."""
        self.lib = native.lib()
        p = Path(path)
        err = C.create_string_buffer(256)
        self.h = None
        if p.is_file():
            self.h = self.lib.ar_tok_load_json(str(p).encode(), err, 256)
        elif (p / "tokenizer.json").exists():
            self.h = self.lib.ar_tok_load_json(str(p / "tokenizer.json").encode(), err, 256)
        elif (p / "tokenizer.tiktoken").exists():
            self.h = self.lib.ar_tok_load_tiktoken(str(p / "tokenizer.tiktoken").encode(),
                                                   str(p / "tokenizer_config.txt").encode(), err, 256)
        else:
            raise FileNotFoundError(f"no tokenizer.json or tokenizer.tiktoken under {p}")
        if not self.h:
            raise ValueError(f"{p}: {err.value.decode()}")

    @property
    def vocab_size(self) -> int:
        return int(self.lib.ar_tok_vocab(self.h))

    @property
    def bos_token_id(self) -> int:
        return int(self.lib.ar_tok_bos(self.h))

    def encode(self, text: str, bos: bool = False) -> List[int]:
        b = text.encode("utf-8")
        n = self.lib.ar_tok_encode(self.h, b, len(b), int(bos), None, 0)
        out = np.empty(max(n, 1), dtype=np.int32)
        self.lib.ar_tok_encode(self.h, b, len(b), int(bos), out.ctypes.data, n)
        return out[:n].tolist()

    def encode_batch_with_bos(self, texts) -> List[List[int]]:
        return [self.encode(t, bos=True) for t in texts]

    def split(self, text: str) -> List[str]:
        b = text.encode("utf-8")
        n = self.lib.ar_tok_split(self.h, b, len(b), None, 0)
        ends = np.empty(max(n, 1), dtype=np.int64)
        self.lib.ar_tok_split(self.h, b, len(b), ends.ctypes.data, n)
        out, a = [], 0
        for e in ends[:n].tolist():
            out.append(b[a:e].decode("utf-8", errors="replace"))
            a = e
        return out

    def decode(self, ids) -> str:
        arr = np.asarray(ids, dtype=np.int32)
        n = self.lib.ar_tok_decode(self.h, arr.ctypes.data, len(arr), None, 0)
        buf = C.create_string_buffer(max(n, 1))
        self.lib.ar_tok_decode(self.h, arr.ctypes.data, len(arr), buf, n)
        return buf.raw[:n].decode("utf-8", errors="replace")

    def token_bytes(self) -> List[int]:
        """UTF-8 byte length of every token's decoded text (0 for special tokens): the table that
        bits-per-byte evaluation needs.  A token that is not valid UTF-8 on its own decodes to
        U+FFFD per invalid byte sequence, as in the reference's table (original/prepare.py:176-190)."""
        out = []
        for i in range(self.vocab_size):
            arr = np.asarray([i], dtype=np.int32)
            n = self.lib.ar_tok_decode(self.h, arr.ctypes.data, 1, None, 0)
            buf = C.create_string_buffer(max(n, 1))
            self.lib.ar_tok_decode(self.h, arr.ctypes.data, 1, buf, n)
            out.append(len(buf.raw[:n].decode("utf-8", errors="replace").encode("utf-8")))
        return out

    def __del__(self):
        try:
            if self.h:
                self.lib.ar_tok_destroy(self.h)
        except Exception:
            pass
