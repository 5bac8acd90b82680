"""Expert parallelism: the experts of a MoE layer are spread over the ranks of a group and the
token exchange (dispatch / combine all-to-all) is done by the MoE kernels themselves through
NVLink peer pointers into symmetric staging buffers.

The reference has no expert parallelism (its MoE runs on one GPU and loops over the experts,
brain/src/forward.rs:642-679).  Layout of every staging buffer on the rank that owns the
experts: ``[E_local, world, cap_src, D]`` - one slab of ``cap_src`` rows per (local expert,
source rank).  A source rank writes its routed tokens into its own slab of the owner's buffer
(peer stores) and later reads the expert outputs back from the same rows (peer loads).  Three
bounded flag barriers order zero-fill, dispatch, expert GEMMs and combine.
"""
from __future__ import annotations

import ctypes as C
import math

import torch
import torch.distributed as dist

from ..ops import kernels as K
from .symm import SymmBuffer


class EPContext:
    def __init__(self, group, device, n_experts: int, d_model: int, max_tokens: int, top_k: int,
                 capacity_factor: float):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if n_experts % self.world:
            raise ValueError(f"{n_experts} experts do not divide over {self.world} ranks")
        self.E, self.E_local, self.D, self.K = n_experts, n_experts // self.world, d_model, top_k
        if capacity_factor <= 0:
            raise ValueError("expert parallelism needs a capacity factor (fixed-size exchange buffers)")
        self.cap_src = int(math.ceil(capacity_factor * max_tokens * top_k / n_experts))
        self.cap_src = (self.cap_src + 7) // 8 * 8
        self.rows_local = self.E_local * self.world * self.cap_src
        n = self.rows_local * d_model
        self.device = torch.device(device)
        self.bufs = {name: SymmBuffer(n, torch.bfloat16, self.device, group) for name in ("x", "y", "dy", "dx")}
        self.flags = SymmBuffer(64, torch.int32, self.device, group)
        for b in list(self.bufs.values()) + [self.flags]:
            b.rendezvous()
        dist.barrier(group=group)
        self._flag_ptrs = (C.c_void_p * self.world)(*self.flags.peer_ptrs)
        self.epoch = 0
        self._tables = {name: self._expert_table(b) for name, b in self.bufs.items()}

    def _expert_table(self, buf: SymmBuffer):
        """Pointer of this rank's slab inside every expert's buffer (host array of E pointers)."""
        ptrs = []
        slab = self.cap_src * self.D * 2
        for e in range(self.E):
            owner, el = divmod(e, self.E_local)
            ptrs.append(buf.peer_ptrs[owner] + (el * self.world + self.rank) * slab)
        return (C.c_void_p * self.E)(*ptrs)

    def table(self, name: str):
        return self._tables[name]

    def local(self, name: str) -> torch.Tensor:
        """This rank's staging buffer viewed as [E_local, world * cap_src, D]."""
        return self.bufs[name].tensor.view(self.E_local, self.world * self.cap_src, self.D)

    # ---- receive side of the expert-output exchange -------------------------------------------------
    # The "y" and "dx" buffers are laid out by the rank that RECEIVES them: [E, cap_src, D], expert e's rows for
    # this rank's tokens.  The owner of expert e writes them with the epilogue of its output GEMM (TMA stores
    # over NVLink), so the combine kernels read local memory only.
    def recv_view(self, name: str, dst_rank: int) -> torch.Tensor:
        """Rank `dst_rank`'s receive area for this rank's experts: [E_local, cap_src, D]."""
        shape = (self.E_local, self.cap_src, self.D)
        off = self.rank * self.E_local * self.cap_src * self.D
        if dst_rank == self.rank:
            return self.bufs[name].tensor[off: off + self.E_local * self.cap_src * self.D].view(shape)
        return self.bufs[name].peer_tensor(dst_rank, shape, torch.bfloat16, off)

    def recv_table(self, name: str):
        """Local pointer of every expert's rows in this rank's receive area (host array of E pointers)."""
        key = ("recv", name)
        if key not in self._tables:
            base = self.bufs[name].tensor.data_ptr()
            slab = self.cap_src * self.D * 2
            self._tables[key] = (C.c_void_p * self.E)(*[base + e * slab for e in range(self.E)])
        return self._tables[key]

    def barrier(self):
        self.epoch += 1
        rc = K.lib().arb_peer_barrier(self._flag_ptrs, self.world, self.rank, self.epoch,
                                      K.err_flag(self.device).data_ptr(), K._stream())
        K._check(rc, "peer_barrier")
