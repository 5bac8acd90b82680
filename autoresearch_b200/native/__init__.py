"""ctypes binding of the host-side native library (C++17, no CUDA, no torch headers).

The shared object is built in-tree next to this file by ``build()`` (g++), and rebuilt
only when the content hash of the sources changes.
"""
from __future__ import annotations

import ctypes as C
import hashlib
import os
import subprocess
import threading
from pathlib import Path

_DIR = Path(__file__).resolve().parent
_SRC = _DIR / "src"
_SO = _DIR / "_ar_native.so"
_STAMP = _DIR / "_ar_native.stamp"
_FEEDER = _DIR / "feeder"
_lock = threading.Lock()
_lib = None

LIB_SOURCES = ["rng.cpp", "data.cpp", "packer.cpp", "safetensors.cpp", "tokenizer.cpp",
               "unicode_tables.cpp", "bpe_train.cpp"]


def _hash() -> str:
    h = hashlib.sha256()
    for f in sorted(_SRC.iterdir()):
        if f.suffix in (".cpp", ".h"):
            h.update(f.name.encode())
            h.update(f.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the shared library and the stand-alone ``feeder`` binary."""
    with _lock:
        want = _hash()
        if (not force and _SO.exists() and _FEEDER.exists() and _STAMP.exists()
                and _STAMP.read_text().strip() == want):
            return _SO
        srcs = [str(_SRC / s) for s in LIB_SOURCES if (_SRC / s).exists()]
        tmp = _SO.with_suffix(f".tmp{os.getpid()}.so")
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-pthread", "-o", str(tmp)] + srcs
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
        os.replace(tmp, _SO)
        main = _SRC / "feeder_main.cpp"
        if main.exists():
            tmpb = _FEEDER.with_suffix(f".tmp{os.getpid()}")
            cmd = ["g++", "-std=c++17", "-O2", "-pthread", "-o", str(tmpb), str(main)] + srcs
            if verbose:
                print(" ".join(cmd))
            subprocess.run(cmd, check=True)
            os.replace(tmpb, _FEEDER)
        _STAMP.write_text(want)
        return _SO


def feeder_binary() -> Path:
    build()
    return _FEEDER


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    build()
    L = C.CDLL(str(_SO))
    vp, i32, i64, u32, u64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_uint64
    P = C.POINTER

    def sig(name, res, args):
        if hasattr(L, name):
            f = getattr(L, name)
            f.restype, f.argtypes = res, args

    sig("ar_uniform_bf16", None, [P(u64), i64, C.c_double, vp])
    sig("ar_uniform_f32", None, [P(u64), i64, C.c_double, vp])
    sig("ar_randn_f32", None, [P(u64), i64, C.c_float, vp])
    sig("ar_randn_bf16", None, [P(u64), i64, C.c_float, vp])
    sig("ar_shuffle_order", None, [vp, i64, u64])
    sig("ar_lcg_tokens", None, [P(u64), i64, u32, vp])
    sig("ar_zipf_create", vp, [u32, C.c_double, u64])
    sig("ar_zipf_fill", None, [vp, i64, vp])
    sig("ar_zipf_seek", None, [vp, u64, u64])
    sig("ar_zipf_destroy", None, [vp])
    sig("ar_shard_open", C.c_int, [C.c_char_p, P(vp), P(u32), P(u32), P(u32)])
    sig("ar_shard_row", vp, [vp, u32])
    sig("ar_shard_close", None, [vp])
    sig("ar_shard_write", C.c_int, [C.c_char_p, u32, u32, u32, vp])
    sig("ar_rowstream_open", vp, [C.c_int, i32, i32, i32])
    sig("ar_rowstream_next", C.c_int, [vp, vp, vp, i32])
    sig("ar_rowstream_rows_read", i64, [vp])
    sig("ar_rowstream_close", None, [vp])
    sig("ar_packer_create", vp, [i32, i32])
    sig("ar_packer_add_doc", None, [vp, vp, i32])
    sig("ar_packer_buffered", i32, [vp])
    sig("ar_packer_next_row", C.c_int, [vp, C.c_int, vp])
    sig("ar_packer_destroy", None, [vp])
    sig("ar_st_writer_create", vp, [])
    sig("ar_st_writer_add", None, [vp, C.c_char_p, C.c_char_p, P(i64), i32, vp, i64])
    sig("ar_st_writer_finish", C.c_int, [vp, C.c_char_p])
    sig("ar_st_open", vp, [C.c_char_p, C.c_char_p, i32])
    sig("ar_st_count", i32, [vp])
    sig("ar_st_name", C.c_char_p, [vp, i32])
    sig("ar_st_dtype", C.c_char_p, [vp, i32])
    sig("ar_st_ndim", i32, [vp, i32])
    sig("ar_st_dim", i64, [vp, i32, i32])
    sig("ar_st_data", vp, [vp, i32, P(i64)])
    sig("ar_st_close", None, [vp])
    sig("ar_tok_load_json", vp, [C.c_char_p, C.c_char_p, i32])
    sig("ar_tok_load_tiktoken", vp, [C.c_char_p, C.c_char_p, C.c_char_p, i32])
    sig("ar_tok_vocab", i32, [vp])
    sig("ar_tok_bos", i32, [vp])
    sig("ar_tok_encode", i64, [vp, C.c_char_p, i64, C.c_int, vp, i64])
    sig("ar_tok_split", i64, [vp, C.c_char_p, i64, vp, i64])
    sig("ar_tok_decode", i64, [vp, vp, i64, vp, i64])
    sig("ar_tok_destroy", None, [vp])
    _lib = L
    return L
