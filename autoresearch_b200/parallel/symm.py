"""Symmetric peer-mapped device memory.

Every rank allocates a buffer of the same size; after the rendez-vous each rank holds a device
pointer to every peer's buffer (NVLink peer mapping) and, where the fabric supports it, one
multicast pointer whose loads are reduced and whose stores are replicated inside the NVSwitch.
Kernels of this package read and write those pointers directly.

The reference's closest relative is its unused CUDA-IPC transport (brain/src/cuda_ipc.rs:127-215:
IPC memory handles exchanged through files, D2D copies from the mapped pointer); here the
mapping is set up by ``torch.distributed._symmetric_memory`` (CUDA VMM allocations whose
handles travel through the process group's store) and the data movement happens inside the
compute kernels.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist


class SymmBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, device, group=None):
        import torch.distributed._symmetric_memory as sm
        self.group = group if group is not None else dist.group.WORLD
        self.tensor = sm.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self._sm = sm
        self.handle = None

    def rendezvous(self):
        gname = self.group.group_name
        try:
            if not self._sm.is_symm_mem_enabled_for_group(gname):
                self._sm.enable_symm_mem_for_group(gname)
        except Exception:
            pass
        self.handle = self._sm.rendezvous(self.tensor, self.group)
        return self

    @property
    def peer_ptrs(self) -> List[int]:
        return [int(p) for p in self.handle.buffer_ptrs]

    def peer_tensor(self, rank: int, shape, dtype: Optional[torch.dtype] = None, offset: int = 0) -> torch.Tensor:
        """A tensor that aliases `rank`'s buffer (its own memory, mapped here over NVLink), starting
        `offset` elements into it.  Kernels of this package may write it (peer stores) or read it."""
        return self.handle.get_buffer(int(rank), tuple(int(x) for x in shape), dtype or self.tensor.dtype, int(offset))

    @property
    def multicast_ptr(self) -> int:
        if os.environ.get("ARB_DISABLE_MULTIMEM", "0") == "1":
            return 0
        try:
            if not self.handle.has_multicast_support(self.tensor.device.type, self.tensor.device.index):
                return 0
        except Exception:
            pass
        try:
            return int(self.handle.multicast_ptr or 0)
        except Exception:
            return 0

    @property
    def rank(self) -> int:
        return int(self.handle.rank)

    @property
    def world(self) -> int:
        return int(self.handle.world_size)
