"""Device memory plan: what a training run will hold on one GPU, computed from the configuration before
anything is allocated, reserved in one piece, reported, and refused at start-up when it cannot fit.

The reference allocates every device buffer once in its buffer manager, prints the total
("48637.5 MB allocated", brain/src/buffer.rs:222-558,988-1137, brain/src/train.rs:721) and therefore
fails at start-up, never at step k.  Here tensors are produced by autograd Functions, so the same
guarantee is built in two steps:

* ``plan(...)`` lists every persistent buffer (parameters, fp32 main gradients, optimizer state, the
  bf16 gradient bucket of the peer-memory data-parallel path, Newton-Schulz work buffers) and every
  per-micro-step buffer (the tensors the backward pass needs from each layer, the chunk of logits, the
  widest backward temporaries) with its size;
* ``reserve(...)`` takes the planned bytes of the step-time part from the driver in ONE allocation and
  hands the block to the caching allocator, which then carves every later tensor out of it: a run
  whose plan holds performs no further device allocation after start-up (``device_allocs()`` lets the
  trainer and the tests check that), and a configuration that does not fit is refused before step 0.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import torch

from ..config import ModelConfig

MB = 1024.0 * 1024.0


@dataclass
class MemoryPlan:
    persistent: List[Tuple[str, int]] = field(default_factory=list)
    step: List[Tuple[str, int]] = field(default_factory=list)
    margin: float = 0.06          # allocator rounding (512-byte blocks, 2 MB segments) and small index tensors

    @property
    def persistent_bytes(self) -> int:
        return sum(b for _, b in self.persistent)

    @property
    def step_bytes(self) -> int:
        return int(sum(b for _, b in self.step) * (1.0 + self.margin))

    @property
    def total_bytes(self) -> int:
        return self.persistent_bytes + self.step_bytes

    def report(self) -> str:
        lines = [f"memory plan: {self.total_bytes / MB:.1f} MB = persistent {self.persistent_bytes / MB:.1f} MB + "
                 f"per-step {self.step_bytes / MB:.1f} MB (incl. {self.margin * 100:.0f} % margin)"]
        for title, items in (("persistent", self.persistent), ("per step", self.step)):
            for name, b in items:
                if b >= MB:
                    lines.append(f"  {title:<10} {name:<34} {b / MB:>10.1f} MB")
        return "\n".join(lines)


def plan(mcfg: ModelConfig, micro_batch: int, *, dp: int = 1, tp: int = 1, ep: int = 1, n_layer_local: int = None,
         has_embedding: bool = True, has_head: bool = True, fused_dp: bool = False, act_bytes: int = 2,
         ce_chunk: int = 16384) -> MemoryPlan:
    """Plan for one rank.  `dp`: ranks that share the optimizer state (ZeRO-1 owner shards); `tp`: tensor-parallel
    ranks (weights and the wide activations are split, the residual stream is split along the sequence);
    `n_layer_local`: layers of this pipeline stage.  Sizes follow the tensors kept by ops/sm100.py."""
    m = mcfg
    L = m.n_layer if n_layer_local is None else n_layer_local
    D, M, V, H = m.d_model, m.mlp_dim, m.vocab, m.n_head
    N = micro_batch * m.seq_len
    Dl, Ml, Hl = D // tp, M // tp, H // tp
    Ns = N // tp                                   # tokens of the sequence-sharded residual stream
    n_ve = sum(1 for l in range(m.n_layer) if m.has_ve(l)) * L // max(m.n_layer, 1)
    moe = m.moe
    # ---- parameters of this rank --------------------------------------------------------------------
    per_layer = 3 * Dl * D + D * Dl
    if moe is None:
        per_layer += 2 * Ml * D
    else:
        per_layer += moe.n_experts * D + 2 * (moe.n_experts // ep) * moe.mlp_dim_e * D
    n_param = L * per_layer + n_ve * (V * Dl + Hl * m.ve_gate_ch) + 2 * L
    if has_embedding:
        n_param += V * D
    if has_head:
        n_param += V * D
    p = MemoryPlan()
    p.persistent.append(("parameters (bf16)", n_param * act_bytes))
    p.persistent.append(("main gradients (fp32)", n_param * 4))
    p.persistent.append(("optimizer state (3 x fp32, owner shard)", 3 * 4 * (n_param + dp - 1) // dp))
    if fused_dp and dp > 1:
        p.persistent.append(("gradient bucket (bf16, peer-mapped)", n_param * 2))
    # Newton-Schulz work buffers: two copies of the largest stacked group + Gram + polynomial, per shape
    sq = (L * 4 + dp - 1) // dp * Dl * D if tp == 1 else (L * 4 + dp - 1) // dp * Dl * D
    tall = (L + dp - 1) // dp * Ml * D if moe is None else 0
    ns = 2 * (2 * sq + 2 * (L * 4 + dp - 1) // dp * min(Dl, D) ** 2) + 2 * 2 * (2 * tall + 2 * (L + dp - 1) // dp * D * D)
    p.step.append(("Newton-Schulz work buffers (first optimizer step)", ns))
    p.persistent.append(("RoPE tables, staging, flags", 2 * m.seq_len * (m.head_dim // 2) * act_bytes + 4 * N * 4 + (1 << 20)))
    # ---- tensors kept from the forward pass of one micro-batch ------------------------------------------
    a = act_bytes
    layer = [
        ("layer: x in (residual stream)", Ns * D * a),
        ("layer: xn", Ns * D * a),
        ("layer: packed qkv", N * 3 * Dl * a),
        ("layer: attention out", N * Dl * a),
        ("layer: lse + rstd", N * Hl * 4 + N * 2 * Hl * 4),
        ("layer: x mid", Ns * D * a),
        ("layer: xn2", Ns * D * a),
    ]
    if tp > 1:
        layer += [("layer: gathered xn (TP)", 2 * N * D * a)]
    if moe is None:
        layer.append(("layer: relu(h)^2", N * Ml * a))
    else:
        slots = int(N * moe.top_k * max(moe.capacity_factor, 1.0)) // ep if ep > 1 else N * moe.top_k
        layer += [("layer: expert rows + hidden", slots * (2 * D + moe.mlp_dim_e) * a),
                  ("layer: router tables", N * (moe.n_experts * 4 + moe.top_k * 12))]
    for name, b in layer:
        p.step.append((f"{name} x {L}", b * L))
    p.step.append(("value-embedding gates", n_ve * N * Hl * 4))
    if has_embedding:
        p.step.append(("embedding out + x0", 2 * Ns * D * a))
    if has_head:
        p.step.append(("final norm in/out, d_xf, losses", 3 * Ns * D * a + Ns * 4))
        p.step.append(("logits chunk", min(ce_chunk, Ns) * V * a))
    # widest moment of the backward pass: d(out), d(hidden) or d(qkv) with the attention statistics, and two
    # residual-stream gradients
    bwd = max(N * Ml * a + 2 * N * Dl * a, 2 * N * 3 * Dl * a + N * Dl * a + N * Hl * 4) + 4 * Ns * D * a
    if tp > 1:
        bwd += 2 * N * D * a
    p.step.append(("backward temporaries", bwd))
    p.step.append(("embedding-gradient plan + scratch", N * 24 + (N // 64 + V + 1) * D * 4))
    return p


def device_allocs(device=None) -> int:
    """Number of allocations the caching allocator has requested from the driver so far."""
    if not torch.cuda.is_available():
        return 0
    return int(torch.cuda.memory_stats(device).get("num_device_alloc", 0))


def reserve(nbytes: int, device) -> Dict[str, float]:
    """One driver allocation of `nbytes`, handed to the caching allocator.  Raises MemoryError (with the numbers)
    when the device cannot hold it."""
    device = torch.device(device)
    if device.type != "cuda":
        return {"reserved_mb": 0.0, "free_mb": 0.0}
    free, total = torch.cuda.mem_get_info(device)
    cached = torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
    if nbytes > free + cached:
        raise MemoryError(f"the run needs {nbytes / MB:.0f} MB more on {device} but only {(free + cached) / MB:.0f} MB "
                          f"of {total / MB:.0f} MB are free: lower BATCH_SIZE or spread the model over more GPUs")
    try:
        block = torch.empty(nbytes, dtype=torch.uint8, device=device)
    except torch.cuda.OutOfMemoryError as e:   # fragmentation of what other processes left free
        raise MemoryError(f"cannot reserve {nbytes / MB:.0f} MB in one piece on {device}") from e
    del block                                   # the segment stays with the caching allocator
    return {"reserved_mb": nbytes / MB, "free_mb": free / MB}
