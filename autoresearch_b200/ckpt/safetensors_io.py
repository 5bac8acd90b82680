"""safetensors read / write through the native C++ reader and writer."""
from __future__ import annotations

import ctypes as C
from typing import Dict

import numpy as np
import torch

from .. import native

_DT = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16,
       "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8, "F64": torch.float64}
_DT_INV = {v: k for k, v in _DT.items()}


def save_file(tensors: Dict[str, torch.Tensor], path: str) -> None:
    lib = native.lib()
    w = lib.ar_st_writer_create()
    keep = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        keep.append(t)
        shape = (C.c_int64 * t.dim())(*t.shape)
        lib.ar_st_writer_add(w, name.encode(), _DT_INV[t.dtype].encode(), shape, t.dim(),
                             t.data_ptr(), t.numel() * t.element_size())
    if lib.ar_st_writer_finish(w, str(path).encode()) != 0:
        raise OSError(f"cannot write {path}")


def load_file(path: str) -> Dict[str, torch.Tensor]:
    lib = native.lib()
    err = C.create_string_buffer(256)
    r = lib.ar_st_open(str(path).encode(), err, 256)
    if not r:
        raise ValueError(f"{path}: {err.value.decode()}")
    out: Dict[str, torch.Tensor] = {}
    try:
        for i in range(lib.ar_st_count(r)):
            name = lib.ar_st_name(r, i).decode()
            dt = _DT[lib.ar_st_dtype(r, i).decode()]
            shape = [lib.ar_st_dim(r, i, d) for d in range(lib.ar_st_ndim(r, i))]
            nb = C.c_int64()
            p = lib.ar_st_data(r, i, C.byref(nb))
            want = int(np.prod(shape)) * torch.empty((), dtype=dt).element_size() if shape else torch.empty((), dtype=dt).element_size()
            if nb.value != want:
                raise ValueError(f"{path}: tensor {name} has {nb.value} bytes, shape needs {want}")
            if nb.value == 0:
                out[name] = torch.empty(shape, dtype=dt)
                continue
            raw = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(nb.value,)).copy()
            out[name] = torch.from_numpy(raw).view(dt).view(*shape)
    finally:
        lib.ar_st_close(r)
    return out
