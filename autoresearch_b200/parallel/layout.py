"""Flat parameter / gradient storage with per-rank ownership of whole matrices.

The reference allocates every device buffer once in its BufferManager
(brain/src/buffer.rs:222-558) and re-packs wq/wk/wv into one wqkv matrix after each
optimizer step (brain/src/buffer.rs:592-625).  Here every parameter is a view into ONE
flat tensor (and every fp32 main-gradient a view into a second one) laid out as
``world`` equal shards.  A shard holds complete "atoms" (a parameter tensor); an atom is
made of one or more optimizer "units" (the matrices Muon orthogonalises: wqkv is three
[D, D] units, an expert stack is E units).  Atoms are assigned to owner ranks by a
longest-processing-time greedy rule, and inside a shard units of equal shape are
adjacent, so that

* the data-parallel gradient reduce-scatter and the parameter all-gather are single
  equal-sized collectives over the flat tensors;
* Newton-Schulz, which needs whole matrices, runs on an owner's units as a strided batch
  ``flat[a:b].view(G, m, n)`` without any gather copy;
* wq/wk/wv never need re-packing: they are row blocks of the packed parameter.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

ALIGN = 256  # elements; keeps every group start 512-byte aligned in bf16


@dataclass
class Unit:
    name: str
    shape: Tuple[int, ...]
    offset: int = 0  # element offset in the flat tensors

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


@dataclass
class Atom:
    name: str
    param: torch.nn.Parameter
    kind: str
    units: List[Unit]
    owner: int = 0
    offset: int = 0
    bucket: int = 0

    @property
    def numel(self) -> int:
        return self.param.numel()

    @property
    def unit_shape(self) -> Tuple[int, ...]:
        return self.units[0].shape


@dataclass
class Group:
    """Units of one shape and one optimizer rule that are contiguous in a shard."""
    kind: str
    shape: Tuple[int, ...]
    owner: int
    offset: int
    count: int
    atoms: List[Atom] = field(default_factory=list)
    bucket: int = 0

    @property
    def numel(self) -> int:
        n = self.count
        for s in self.shape:
            n *= s
        return n


def _split_units(name: str, p: torch.Tensor, kind: str) -> List[Unit]:
    if kind == "muon_qkv":
        d = p.shape[0] // 3
        return [Unit(f"{name}.{s}", (d, p.shape[1])) for s in ("q", "k", "v")]
    if kind == "muon_expert":
        return [Unit(f"{name}.{e}", tuple(p.shape[1:])) for e in range(p.shape[0])]
    return [Unit(name, tuple(p.shape))]


def _cost(atom: Atom) -> float:
    if atom.kind.startswith("muon"):
        m, n = atom.unit_shape
        # Newton-Schulz work per unit ~ m*n*min(m,n); elementwise work ~ m*n
        return len(atom.units) * (m * n * (1.0 + min(m, n) / 64.0))
    return float(atom.numel)


class ParamLayout:
    def __init__(self, named_groups: Sequence[Tuple[str, torch.nn.Parameter, str]],
                 world: int = 1, rank: int = 0, grad_dtype=torch.float32,
                 allocator=None, bucket_of=None, n_buckets: int = 1):
        """named_groups: (name, parameter, kind) as returned by GPT.named_matrix_groups().
        allocator(numel, dtype, device) -> flat tensor (lets the caller place the flat
        tensors in a symmetric peer-mapped heap).
        bucket_of(name) -> 0 .. n_buckets-1: parameters whose gradients become final together during the backward
        pass (bucket 0 first).  Every shard holds its atoms bucket by bucket, so the slice of a bucket inside a shard
        is one contiguous range, owners are balanced inside every bucket, and the gradient exchange and the
        optimizer can run bucket by bucket while the backward pass is still at work on the later ones."""
        self.world, self.rank = world, rank
        self.n_buckets = max(1, int(n_buckets))
        atoms = [Atom(n, p, k, _split_units(n, p, k)) for n, p, k in named_groups]
        for a in atoms:
            a.bucket = min(max(int(bucket_of(a.name)), 0), self.n_buckets - 1) if bucket_of is not None else 0
        self.atoms = atoms
        if not atoms:
            raise ValueError("no parameters")
        self.device = atoms[0].param.device
        self.param_dtype = atoms[0].param.dtype
        # ---- owner assignment (LPT greedy, deterministic) -----------------------------
        total_load = [0.0] * world
        for b in range(self.n_buckets):
            load = [0.0] * world                      # balanced inside every bucket; ties go to the lighter rank overall
            for a in sorted((a for a in atoms if a.bucket == b), key=lambda a: (-_cost(a), a.name)):
                r = min(range(world), key=lambda i: (load[i], total_load[i], i))
                a.owner = r
                load[r] += _cost(a)
                total_load[r] += _cost(a)
        # ---- offsets: per shard, sort atoms so equal-shape units are adjacent -----------
        def gkey(a: Atom):
            base = "muon" if a.kind.startswith("muon") else a.kind
            return (a.bucket, 0 if base == "muon" else 1, base, a.unit_shape)

        self.groups: List[Group] = []
        sizes = []
        per_rank: List[List[Atom]] = [[] for _ in range(world)]
        for a in atoms:
            per_rank[a.owner].append(a)
        rel_groups: List[List[Group]] = []
        for r in range(world):
            off = 0
            cur: Optional[Group] = None
            gl: List[Group] = []
            for a in sorted(per_rank[r], key=lambda a: (gkey(a), a.name)):
                k = gkey(a)
                if cur is None or (cur.bucket, cur.kind, cur.shape) != (k[0], k[2], k[3]):
                    off = (off + ALIGN - 1) // ALIGN * ALIGN
                    cur = Group(k[2], k[3], r, off, 0, bucket=k[0])
                    gl.append(cur)
                a.offset = off
                uo = off
                for u in a.units:
                    u.offset = uo
                    uo += u.numel
                cur.count += len(a.units)
                cur.atoms.append(a)
                off += a.numel
            sizes.append(off)
            rel_groups.append(gl)
        self.shard_size = max((max(sizes) + ALIGN - 1) // ALIGN * ALIGN, ALIGN)
        for r in range(world):
            base = r * self.shard_size
            for g in rel_groups[r]:
                g.offset += base
                self.groups.append(g)
            for a in per_rank[r]:
                a.offset += base
                for u in a.units:
                    u.offset += base
        self.total = self.shard_size * world
        # ---- flat storage -----------------------------------------------------------------
        alloc = allocator or (lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev))
        self.flat_param = alloc(self.total, self.param_dtype, self.device)
        self.flat_grad = alloc(self.total, grad_dtype, self.device)
        with torch.no_grad():
            for a in atoms:
                view = self.flat_param[a.offset:a.offset + a.numel].view(a.param.shape)
                view.copy_(a.param.data)
                a.param.data = view
                a.param.main_grad = self.flat_grad[a.offset:a.offset + a.numel].view(a.param.shape)
                a.param.layout_atom = a

    # ----------------------------------------------------------------------------------
    def shard_range(self, rank: Optional[int] = None) -> Tuple[int, int]:
        r = self.rank if rank is None else rank
        return r * self.shard_size, (r + 1) * self.shard_size

    def owned_groups(self, bucket: Optional[int] = None) -> List[Group]:
        return [g for g in self.groups if g.owner == self.rank and (bucket is None or g.bucket == bucket)]

    def bucket_ranges(self, bucket: int) -> List[Tuple[int, int]]:
        """Per rank shard, the element range [lo, hi) (multiples of ALIGN) that holds the atoms of `bucket`."""
        out = []
        for r in range(self.world):
            gs = [g for g in self.groups if g.owner == r and g.bucket == bucket]
            if not gs:
                continue
            lo = min(g.offset for g in gs)
            hi = max(g.offset + g.numel for g in gs)
            out.append((lo, min((hi + ALIGN - 1) // ALIGN * ALIGN, (r + 1) * self.shard_size)))
        return out

    def owned_atoms(self) -> List[Atom]:
        return [a for a in self.atoms if a.owner == self.rank]

    def group_view(self, flat: torch.Tensor, g: Group) -> torch.Tensor:
        return flat[g.offset:g.offset + g.numel].view(g.count, *g.shape)

    def zero_grad(self) -> None:
        self.flat_grad.zero_()

    def accumulate_autograd_grads(self) -> None:
        """Fold ``param.grad`` (produced by autograd on the oracle / baseline paths) into
        the fp32 main gradient and drop it."""
        for a in self.atoms:
            p = a.param
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None

    def describe(self) -> str:
        per = [0] * self.world
        for a in self.atoms:
            per[a.owner] += a.numel
        return (f"layout: {len(self.atoms)} atoms, {len(self.groups)} groups, shard "
                f"{self.shard_size} elems x {self.world}; fill " +
                ",".join(f"{x / self.shard_size:.2f}" for x in per))
