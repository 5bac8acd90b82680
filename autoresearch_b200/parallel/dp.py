"""Data-parallel gradient reduce-scatter and parameter all-gather over a ParamLayout.

The reference has no data parallelism at all (its only collective-free transports are
pipeline send/recv, brain/src/nccl.rs:18-24).  Three interchangeable communicators:

* ``LocalComm``  – one rank, nothing to do.
* ``LibraryComm`` – library collectives (NCCL on GPUs, gloo on CPU ranks): the measured
  baseline arm.
* ``FusedComm`` (``parallel.fused_dp``) – the peer-memory kernels: one launch pulls every
  peer's gradient shard over NVLink, sums in fp32, applies the scale and leaves the result
  in the owner's fp32 gradient; one launch pushes the owner's updated bf16 shard to every
  peer.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .layout import ParamLayout


class LocalComm:
    world = 1
    rank = 0
    name = "local"

    def reduce_scatter_grads(self, layout: ParamLayout) -> None:
        pass

    def all_gather_params(self, layout: ParamLayout) -> None:
        pass

    def barrier(self) -> None:
        pass


class LibraryComm:
    name = "library"

    def __init__(self, group=None, bucket_dtype: Optional[torch.dtype] = None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.backend = dist.get_backend(group)
        self.bucket_dtype = bucket_dtype
        self._bucket = None

    def reduce_scatter_grads(self, layout: ParamLayout) -> None:
        lo, hi = layout.shard_range()
        g = layout.flat_grad
        if self.backend == "gloo":
            dist.all_reduce(g, group=self.group)
            return
        if self.bucket_dtype is not None and self.bucket_dtype != g.dtype:
            if self._bucket is None:
                self._bucket = torch.empty_like(g, dtype=self.bucket_dtype)
            self._bucket.copy_(g)
            out = torch.empty(hi - lo, dtype=self.bucket_dtype, device=g.device)
            dist.reduce_scatter_tensor(out, self._bucket, group=self.group)
            g[lo:hi].copy_(out)
        else:
            out = torch.empty(hi - lo, dtype=g.dtype, device=g.device)
            dist.reduce_scatter_tensor(out, g, group=self.group)
            g[lo:hi].copy_(out)

    def all_gather_params(self, layout: ParamLayout) -> None:
        lo, hi = layout.shard_range()
        p = layout.flat_param
        if self.backend == "gloo":
            parts = [torch.empty(hi - lo, dtype=p.dtype) for _ in range(self.world)]
            dist.all_gather(parts, p[lo:hi].clone(), group=self.group)
            for r, t in enumerate(parts):
                p[r * layout.shard_size:(r + 1) * layout.shard_size].copy_(t)
            return
        dist.all_gather_into_tensor(p, p[lo:hi].clone(), group=self.group)

    def barrier(self) -> None:
        dist.barrier(group=self.group)
