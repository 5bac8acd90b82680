"""Expert parallelism: the experts of a MoE layer are spread over the ranks of a group and the
token exchange (dispatch / combine all-to-all) is done by the MoE kernels themselves through
NVLink peer pointers into symmetric staging buffers.

The reference has no expert parallelism (its MoE runs on one GPU and loops over the experts,
brain/src/forward.rs:642-679).  Layout of every staging buffer on the rank that owns the
experts: ``[E_local, world, cap_src, D]`` - one slab of ``cap_src`` rows per (local expert,
source rank) - beside a row-count table ``[E_local, world]``.

Forward of a layer: a source rank writes its routed tokens into its slab of the owner's ``x``
buffer (peer stores), writes how many it sent into the owner's count table and zeroes the rows
up to the next tile boundary; ONE bounded flag barrier; the owner runs its experts as ragged
grouped GEMMs over the slabs in place (row counts from the table: empty tiles are skipped,
nothing is copied or cleared); a second barrier; every source reads the expert outputs of its
tokens straight from the owners' ``y`` buffers while it applies gates and residual (peer loads
in the combine kernel).  The backward mirrors it with ``dy`` / ``dx``.  ``x`` and ``y`` exist
once per layer (the backward needs them: nothing is cloned), ``dy`` / ``dx`` once.
"""
from __future__ import annotations

import ctypes as C
import math

import torch
import torch.distributed as dist

from ..ops import kernels as K
from .symm import SymmBuffer


class EPContext:
    TILE = 256            # rows per GEMM tile: the dispatch zero-pads every slab to this boundary
    mode = "fused"

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
        # slots one source may send to one expert, and the rows of a slab: a multiple of 64 (K blocks of the
        # weight-gradient GEMMs)
        self.keep = (int(math.ceil(capacity_factor * max_tokens * top_k / n_experts)) + 7) // 8 * 8
        self.cap_src = (self.keep + 63) // 64 * 64
        self.rows_local = self.E_local * self.world * self.cap_src
        self.G = self.E_local * self.world                    # slabs = batch items of the grouped GEMMs
        self.device = torch.device(device)
        self.flags = SymmBuffer(64, torch.int32, self.device, group)
        self.flags.rendezvous()
        self._flag_ptrs = (C.c_void_p * self.world)(*self.flags.peer_ptrs)
        self.epoch = 0
        self._bufs = {}
        self._tables = {}
        dist.barrier(group=group)

    # ---- buffers (created on first use: a collective, reached by all ranks in the same order) ------------
    def buf(self, name: str, layer: int = -1) -> SymmBuffer:
        key = (name, layer)
        b = self._bufs.get(key)
        if b is None:
            if name == "cnt":
                b = SymmBuffer(max(self.G, 16), torch.int32, self.device, self.group)
            else:
                b = SymmBuffer(self.rows_local * self.D, torch.bfloat16, self.device, self.group)
            b.rendezvous()
            self._bufs[key] = b
        return b

    def table(self, name: str, layer: int = -1):
        """For every expert e: pointer to THIS rank's slab inside the owner's buffer (host array of E pointers; peer
        mappings for experts that live elsewhere).  For "cnt": pointer to this rank's entry in the owner's count table."""
        key = (name, layer)
        t = self._tables.get(key)
        if t is None:
            b = self.buf(name, layer)
            unit = 4 if name == "cnt" else self.cap_src * self.D * 2
            ptrs = []
            for e in range(self.E):
                owner, el = divmod(e, self.E_local)
                ptrs.append(b.peer_ptrs[owner] + (el * self.world + self.rank) * unit)
            t = (C.c_void_p * self.E)(*ptrs)
            self._tables[key] = t
        return t

    def local(self, name: str, layer: int = -1) -> torch.Tensor:
        """This rank's own buffer as the batch of slabs the grouped GEMMs see: [E_local * world, cap_src, D]
        (the count table: int32 [E_local * world])."""
        t = self.buf(name, layer).tensor
        if name == "cnt":
            return t[:self.G]
        return t.view(self.G, self.cap_src, self.D)

    def barrier(self):
        self.epoch += 1
        rc = K.lib().arb_peer_barrier(self._flag_ptrs, self.world, self.rank, self.epoch,
                                      K.err_flag(self.device).data_ptr(), K._stream())
        K._check(rc, "peer_barrier")

    def symmetric_bytes(self) -> int:
        return sum(b.tensor.numel() * b.tensor.element_size() for b in self._bufs.values())


class LibraryEPContext:
    """The comparison arm: the same capacity rule and slab layout, but the token exchange is the library's
    all-to-all (``ncclSend/Recv`` grouped by ``all_to_all_single``) on padded fixed-size slabs, between local
    dispatch / combine kernels.  Used to measure what the peer-memory path buys."""

    mode = "library"

    def __init__(self, group, device, n_experts: int, d_model: int, max_tokens: int, top_k: int, capacity_factor: float):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if n_experts % self.world:
            raise ValueError(f"{n_experts} experts do not divide over {self.world} ranks")
        if capacity_factor <= 0:
            raise ValueError("expert parallelism needs a capacity factor (fixed-size exchange buffers)")
        self.E, self.E_local, self.D, self.K = n_experts, n_experts // self.world, d_model, top_k
        self.keep = (int(math.ceil(capacity_factor * max_tokens * top_k / n_experts)) + 7) // 8 * 8
        self.cap_src = (self.keep + 63) // 64 * 64
        self.G = self.E_local * self.world
        self.device = torch.device(device)
        self.bytes = 0

    def to_owners(self, t: torch.Tensor) -> torch.Tensor:
        """[E, ...] by expert (owner-major) on every source -> [E_local * world, ...] by (local expert, source) on the
        owner: the all-to-all plus, with several experts per rank, the re-ordering of the received blocks."""
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t.contiguous(), group=self.group)
        self.bytes += t.numel() * t.element_size() * (self.world - 1) // self.world
        if self.E_local > 1:
            out = out.view(self.world, self.E_local, *t.shape[1:]).transpose(0, 1).contiguous().view_as(t)
        return out

    def to_sources(self, t: torch.Tensor) -> torch.Tensor:
        """The inverse of to_owners."""
        if self.E_local > 1:
            t = t.view(self.E_local, self.world, *t.shape[1:]).transpose(0, 1).contiguous().view_as(t)
        out = torch.empty_like(t)
        dist.all_to_all_single(out, t.contiguous(), group=self.group)
        self.bytes += t.numel() * t.element_size() * (self.world - 1) // self.world
        return out
