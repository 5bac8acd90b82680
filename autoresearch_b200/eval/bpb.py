"""Bits-per-byte evaluation.

val_bpb = sum(nats over targets whose token has bytes > 0) / (ln 2 * sum(bytes))
(brain/src/train.rs:2489-2578; original/prepare.py:342-364).  ``token_bytes.json`` is a
JSON array with one UTF-8 byte length per token id, 0 for special tokens.  The reduction
runs on the device: only two scalars cross to the host per evaluation, where the
reference copies every per-token loss back (brain/src/train.rs:2555-2570).
"""
from __future__ import annotations

import json
import math
from pathlib import Path
from typing import Optional

import torch

EVAL_TOKENS = 40 * 524288
PROXY_EVAL_BATCHES = 4


def load_token_bytes(path, vocab: int, device="cpu") -> torch.Tensor:
    p = Path(path)
    if p.is_dir():
        p = p / "token_bytes.json"
    arr = json.loads(p.read_text())
    if not isinstance(arr, list) or len(arr) != vocab:
        raise ValueError(f"{p}: expected a JSON array of {vocab} integers, got "
                         f"{len(arr) if isinstance(arr, list) else type(arr).__name__}")
    return torch.tensor(arr, dtype=torch.int32, device=device)


@torch.no_grad()
def eval_bpb(model, loader, token_bytes: torch.Tensor, max_batches: Optional[int] = None,
             device="cpu", group=None, forward=None) -> float:
    """`loader.next_batch()` returns (ids, targets) int32 [B, T] or None at the end.

    `group`: the ranks whose sums are added (every rank scores different tokens).  They leave the loop together:
    a validation split can end on one rank first, so each batch is preceded by an agreement (MIN over the group)
    that every rank still has one.  `forward(ids, targets) -> (per_token_losses, targets_scored)` replaces the
    plain model call where a rank scores only part of a batch (tensor-parallel token shards, the last pipeline
    stage)."""
    B, T = loader.B, loader.T
    n = EVAL_TOKENS // (B * T)
    if max_batches is not None:
        n = min(n, max_batches)
    n = max(n, 1)
    nats = torch.zeros((), dtype=torch.float64, device=device)
    nbytes = torch.zeros((), dtype=torch.float64, device=device)
    was_training = model.training
    model.eval()
    dist = None
    if group is not None:
        import torch.distributed as dist
    for _ in range(n):
        batch = loader.next_batch()
        if dist is not None:
            have = torch.tensor([0 if batch is None else 1], dtype=torch.int32, device=device)
            dist.all_reduce(have, op=dist.ReduceOp.MIN, group=group)
            if int(have.item()) == 0:
                break
        elif batch is None:
            break
        ids, tgt = (t.to(device, non_blocking=True) for t in batch)
        if forward is not None:
            per_tok, scored = forward(ids, tgt)
        else:
            _, per_tok = model(ids, tgt)
            scored = tgt
        by = token_bytes[scored.reshape(-1).long()]
        m = by > 0
        nats += (per_tok.double() * m).sum()
        nbytes += by.double().sum()
    model.train(was_training)
    if dist is not None:
        pair = torch.stack([nats, nbytes])
        dist.all_reduce(pair, group=group)
        nats, nbytes = pair[0], pair[1]
    nb = float(nbytes.item())
    return float(nats.item()) / (math.log(2.0) * nb) if nb > 0 else float("nan")
