"""Data-parallel gradient reduce-scatter and parameter all-gather done by this package's own
kernels over NVLink peer memory (no library collective on the path).

Per optimizer step, on the compute stream:

1. the fp32 main gradients are cast into this rank's bf16 bucket (symmetric memory);
2. a bounded flag barrier (kernel; every wait gives up after 2 s of device time and reports
   through the error word) makes all buckets visible;
3. ONE kernel reduces this rank's owner shard across all ranks - ``multimem.ld_reduce`` through
   the NVSwitch when a multicast mapping exists, plain peer loads otherwise - accumulating in
   fp32, applying the scale and writing the fp32 gradient the optimizer consumes;
4. the optimizer updates the owned matrices and writes bf16 parameters into the symmetric
   parameter buffer;
5. a second barrier; the dense weight matrices (wqkv, wo, wfc, wdn: 99 % of the bytes) are NOT
   copied here: each is registered as pending and the GEMMs of the next forward pass copy them from
   the owners' memory themselves: the first GEMM copies its own B operand in its prologue
   (``GemmArgs::pull_src``), and a spare warp of every GEMM copies the operand of the NEXT GEMM while
   the tiles are computed (``GemmArgs::ahead_src``), so the transfer hides under the math; one small
   kernel pulls everything else (embeddings, head, scalars, gates, experts).

Overlap with the backward pass (``exchange_bucket``): the parameters are laid out in gradient
buckets by depth (``ParamLayout(bucket_of=...)``).  As soon as the last micro-step's backward
has left a group of layers, steps 1-5 run for that bucket alone on a side stream - cast of its
slices, barrier, fused reduce-scatter + owner update of its groups, barrier, pull of its small
parameters - while the compute stream goes on with the earlier layers; only the last bucket
(the first layers, embeddings and scalars) is left for after the backward pass.

The library arm (``LibraryComm``) does the same with ncclReduceScatter / ncclAllGather and is
what this path is measured against.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import kernels as K
from .layout import ParamLayout
from .symm import SymmBuffer


class FusedComm:
    name = "fused"

    def __init__(self, group=None, device=None, bucket_dtype: torch.dtype = torch.bfloat16,
                 use_multimem: bool = True):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.bucket_dtype = bucket_dtype
        self.use_multimem = use_multimem
        self._bufs = []
        self._param: Optional[SymmBuffer] = None
        self._bucket: Optional[SymmBuffer] = None
        self._flags: Optional[SymmBuffer] = None
        self.epoch = 0
        self._staged = {}
        K.lib()

    # the layout asks for its flat tensors through this hook: parameters go to symmetric memory
    def allocator(self, numel, dtype, device):
        if self._param is None and dtype != torch.float32:
            self._param = SymmBuffer(numel, dtype, device, self.group)
            return self._param.tensor
        return torch.zeros(numel, dtype=dtype, device=device)

    def attach(self, layout: ParamLayout) -> None:
        if self._param is None:  # fp32 parameters (tests): place a bf16-free copy path
            raise RuntimeError("FusedComm needs bf16 parameters in symmetric memory")
        self._bucket = SymmBuffer(layout.total, self.bucket_dtype, self.device, self.group)
        self._flags = SymmBuffer(64, torch.int32, self.device, self.group)
        for b in (self._param, self._bucket, self._flags):
            b.rendezvous()
        dist.barrier(group=self.group)
        self._param_ptrs = self._ptr_array(self._param.peer_ptrs)
        self._bucket_ptrs = self._ptr_array(self._bucket.peer_ptrs + [self.rank])
        self._bucket_plain_ptrs = self._ptr_array(self._bucket.peer_ptrs)
        self._small_ranges = None
        self._flag_ptrs = self._ptr_array(self._flags.peer_ptrs)
        self._mc = self._bucket.multicast_ptr if self.use_multimem else 0

    @staticmethod
    def _ptr_array(ptrs):
        arr = (C.c_void_p * len(ptrs))(*ptrs)
        return arr

    def barrier(self) -> None:
        self.epoch += 1
        rc = K.lib().arb_peer_barrier(self._flag_ptrs, self.world, self.rank, self.epoch,
                                      K.err_flag(self.device).data_ptr(), K._stream())
        K._check(rc, "peer_barrier")

    fuse_into_optimizer = True

    def grad_source(self, layout: ParamLayout):
        """Per owned group: a descriptor of the un-reduced bf16 buckets, so that the optimizer
        kernels do the cross-rank sum themselves.  Groups that take the unfused optimizer path
        (tiny matrices) return None and read the separately reduced fp32 gradient."""
        from ..ops.sm100 import OptimKernels, PeerGrad
        if not (self.fuse_into_optimizer and self.bucket_dtype == torch.bfloat16):
            return None

        def src(g):
            if g.kind == "muon":
                m, n = g.shape
                if min(m, n) < OptimKernels.MIN_GEMM_DIM or (m % 8) or (n % 8):
                    return None
            elif g.numel % 8:
                return None
            return PeerGrad(self._bucket_plain_ptrs, self.world, self.rank, self._mc or 0, g.offset,
                            (g.count,) + tuple(g.shape), 1.0)
        return src

    def reduce_scatter_grads(self, layout: ParamLayout) -> None:
        K.flush_pending_pulls()   # normally empty: the forward pass has pulled every weight it used
        lo, hi = layout.shard_range()
        src_bf16 = self.bucket_dtype == torch.bfloat16
        if src_bf16:
            K.cast_f32_to_bf16(layout.flat_grad, self._bucket.tensor, 1.0)
        else:
            self._bucket.tensor.copy_(layout.flat_grad)
        self.barrier()
        L = K.lib()
        src = self.grad_source(layout)
        if src is not None:
            # everything the fused optimizer kernels will sum themselves is skipped here
            ranges = [(g.offset, g.numel) for g in layout.owned_groups() if src(g) is None]
        else:
            ranges = [(lo, hi - lo)]
        for off, n in ranges:
            n8 = (n + 7) // 8 * 8
            out = layout.flat_grad[off:off + n8]
            if self._mc:
                rc = L.arb_reduce_scatter_multimem(self._mc, off, n8, int(src_bf16), out.data_ptr(), 1.0, K._stream())
            else:
                rc = L.arb_reduce_scatter_peers(self._bucket_ptrs, self.world, off, n8, int(src_bf16), out.data_ptr(),
                                                1.0, K._stream())
            K._check(rc, "reduce_scatter")

    # ---- bucket by bucket, overlapped with the backward pass ------------------------------------------------
    def exchange_bucket(self, layout: ParamLayout, bucket: int, run_optimizer, side: "torch.cuda.Stream") -> None:
        """Called on the compute stream when the gradients of `bucket` are final.  The cast of the bucket's slices
        stays on the compute stream (it reads what the backward kernels just wrote); everything that waits for peers
        runs on `side`: barrier, `run_optimizer(bucket, grad_source)` (the owner update with the reduce-scatter fused
        into its first kernel), barrier, and the pull of the bucket's small parameters.  The dense matrices of the
        bucket are staged as pending pulls and handed to the GEMMs by ``activate_staged()`` once the compute stream has
        joined the side stream."""
        if bucket == 0:
            K.flush_pending_pulls()   # normally empty: the forward pass has pulled every weight it used
        for lo, hi in layout.bucket_ranges(bucket):
            K.cast_f32_to_bf16(layout.flat_grad[lo:hi], self._bucket.tensor[lo:hi], 1.0)
        ready = torch.cuda.Event()
        ready.record()
        L = K.lib()
        with torch.cuda.stream(side):
            side.wait_event(ready)
            self.barrier()
            src = self.grad_source(layout)
            for g in layout.owned_groups(bucket):          # groups the fused optimizer kernels do not sum themselves
                if src is not None and src(g) is not None:
                    continue
                n8 = (g.numel + 7) // 8 * 8
                out = layout.flat_grad[g.offset:g.offset + n8]
                if self._mc:
                    rc = L.arb_reduce_scatter_multimem(self._mc, g.offset, n8, 1, out.data_ptr(), 1.0, K._stream())
                else:
                    rc = L.arb_reduce_scatter_peers(self._bucket_ptrs, self.world, g.offset, n8, 1, out.data_ptr(), 1.0,
                                                    K._stream())
                K._check(rc, "reduce_scatter")
            run_optimizer(bucket, src)
            self.barrier()
            self._gather(layout, bucket, stage=True)

    def activate_staged(self) -> None:
        """Hands the staged dense matrices to the GEMMs of the next forward pass (call on the compute stream after
        it has waited for the side stream)."""
        order = K.pull_use_order
        for dst, v in sorted(self._staged.items(), key=lambda kv: order.get(kv[0], 1 << 30)):
            K.pending_pulls[dst] = v
        self._staged = {}
        K.pull_stream = K._stream()

    fuse_into_gemm = True
    GEMM_OPERANDS = (".wqkv", ".wo", ".wfc", ".wdn")

    def _plan_gather(self, layout: ParamLayout, bucket=None):
        """Per non-owned atom (of one gradient bucket, or of all): pulled by its first GEMM, or part of a range copied
        right away.  Ranges are the complement of the GEMM operands inside each peer's shard, merged and widened to 16
        bytes (a peer's shard holds only atoms that peer owns, and inside a shard the atoms of a bucket are
        neighbours, so what is copied along is current too)."""
        es = layout.flat_param.element_size()
        gemm_atoms, ranges = [], []
        for r in range(self.world):
            if r == self.rank:
                continue
            lo, hi = layout.shard_range(r)
            atoms = sorted((a for a in layout.atoms if a.owner == r and (bucket is None or a.bucket == bucket)),
                           key=lambda a: a.offset)
            if bucket is not None and atoms:               # never widen into a neighbouring bucket's atoms
                hi = min(hi, max(a.offset + a.numel for a in atoms) + 8)
            cur = None
            for a in atoms:
                is_gemm = (self.fuse_into_gemm and a.name.endswith(self.GEMM_OPERANDS) and a.param.dim() == 2
                           and (a.numel * es) % 16 == 0 and (a.offset * es) % 16 == 0)
                if is_gemm:
                    gemm_atoms.append((a, r))
                    continue
                b0 = (a.offset * es) // 16 * 16
                b1 = min(((a.offset + a.numel) * es + 15) // 16 * 16, hi * es)
                if cur is not None and b0 <= cur[1]:
                    cur[1] = max(cur[1], b1)
                else:
                    cur = [b0, b1, r]
                    ranges.append(cur)
        return gemm_atoms, ranges

    def all_gather_params(self, layout: ParamLayout) -> None:
        self.barrier()
        self._gather(layout, None, stage=False)

    def _gather(self, layout: ParamLayout, bucket, stage: bool) -> None:
        plans = self.__dict__.setdefault("_plans", {})
        if bucket not in plans:
            plans[bucket] = self._plan_gather(layout, bucket)
        gemm_atoms, ranges = plans[bucket]
        base = layout.flat_param.data_ptr()
        es = layout.flat_param.element_size()
        peers = self._param.peer_ptrs
        if stage:
            for a, r in gemm_atoms:
                self._staged[base + a.offset * es] = (peers[r] + a.offset * es, a.numel * es)
        else:
            # registered in the order in which the forward pass consumed them last time (unknown ones last), on this stream
            order = K.pull_use_order
            for a, r in sorted(gemm_atoms, key=lambda ar: order.get(base + ar[0].offset * es, 1 << 30)):
                K.pending_pulls[base + a.offset * es] = (peers[r] + a.offset * es, a.numel * es)
            K.pull_stream = K._stream()
        if ranges:
            n = len(ranges)
            src = (C.c_void_p * n)(*[peers[r] + b0 for b0, _, r in ranges])
            dst = (C.c_void_p * n)(*[base + b0 for b0, _, _ in ranges])
            nb = (C.c_longlong * n)(*[b1 - b0 for b0, b1, _ in ranges])
            K._check(K.lib().arb_pull_ranges(src, dst, nb, n, K._stream()), "pull_ranges")
        # peers may start overwriting their shards (next optimizer step) only after everyone has
        # pulled: the barrier that opens the next reduce-scatter provides that ordering, and every
        # pending operand is pulled by the forward pass (or by flush()) before that barrier.

    def flush(self) -> None:
        """Pull whatever no GEMM has pulled yet (before parameters are read by anything else)."""
        K.flush_pending_pulls()
