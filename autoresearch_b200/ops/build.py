"""In-tree build of the sm_100a kernel library.

Each ``csrc/*.cu`` is compiled by nvcc with ``-gencode arch=compute_100a,code=sm_100a``
(cross-compiles without a GPU) and linked into ``_arb_kernels.so`` next to this file.  The
library exposes a flat C interface (``csrc/api.h``) that Python binds with ctypes, so no
torch headers are involved and a rebuild takes seconds.  A content hash of the sources
decides whether a rebuild is needed (file times do not survive a copy of the tree).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import tempfile
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

_DIR = Path(__file__).resolve().parent
CSRC = _DIR / "csrc"
SO = _DIR / "_arb_kernels.so"
STAMP = _DIR / "_arb_kernels.stamp"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
# extra flags for experiments (e.g. ARB_NVCC_EXTRA="-DARB_ATTN_POLY_OF_8=0"); part of the rebuild hash
NVCC_FLAGS += os.environ.get("ARB_NVCC_EXTRA", "").split()


def sources():
    return sorted(CSRC.glob("*.cu"))


def _hash() -> str:
    h = hashlib.sha256()
    for f in sorted(CSRC.iterdir()):
        if f.suffix in (".cu", ".cuh", ".h"):
            h.update(f.name.encode())
            h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def nvcc_path() -> str:
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found; the sm_100a kernel library cannot be built")
    return p


def is_current() -> bool:
    return SO.exists() and STAMP.exists() and STAMP.read_text().strip() == _hash()


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and is_current():
        return SO
    nvcc = nvcc_path()
    want = _hash()
    with tempfile.TemporaryDirectory(prefix="arb_build_") as td:
        logs = {}

        def one(src: Path):
            obj = Path(td) / (src.stem + ".o")
            cmd = [nvcc] + NVCC_FLAGS + ["-c", str(src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            logs[src.name] = r.stderr
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stderr[-4000:]}")
            return obj

        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            objs = list(ex.map(one, sources()))
        tmp = SO.with_suffix(f".tmp{os.getpid()}.so")
        cmd = [nvcc, "-shared", "-o", str(tmp)] + [str(o) for o in objs] + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
        os.replace(tmp, SO)
        if verbose:
            for name, log in logs.items():
                spills = [l for l in log.splitlines() if "spill" in l and "0 bytes spill stores" not in l]
                print(f"{name}: {len(spills)} kernels with spills")
    STAMP.write_text(want)
    return SO


if __name__ == "__main__":
    print(build(force=True, verbose=True))
