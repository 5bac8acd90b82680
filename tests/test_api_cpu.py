"""The ctypes table of ops/kernels.py against the declarations of ops/csrc/api.h: same names, same argument counts,
pointer / integer / float in the same places.  Needs neither a GPU nor the built library."""
import ctypes as C
import re
from pathlib import Path

from autoresearch_b200.ops import kernels as K

API_H = Path(K.__file__).parent / "csrc" / "api.h"


def _declarations():
    text = re.sub(r"//[^\n]*", "", API_H.read_text())
    out = {}
    for m in re.finditer(r"\bint\s+(arb_\w+)\s*\(([^;{]*)\)\s*;", text):
        params = [p.strip() for p in m.group(2).replace("\n", " ").split(",") if p.strip()]
        out[m.group(1)] = params
    return out


def _kind(param: str) -> str:
    if "*" in param or "cudaStream_t" in param:
        return "ptr"
    if re.search(r"\b(float|double)\b", param):
        return "float"
    return "long" if "long long" in param else "int"


def test_every_bound_entry_point_is_declared_with_the_same_arguments():
    decl = _declarations()
    kinds = {C.c_void_p: "ptr", C.c_int: "int", C.c_longlong: "long", C.c_float: "float"}
    for name, args in K._signatures().items():
        assert name in decl, f"{name} is bound in kernels.py but not declared in api.h"
        want = [_kind(p) for p in decl[name]]
        got = [kinds[a] for a in args]
        assert got == want, f"{name}: kernels.py binds {got}, api.h declares {want}"
