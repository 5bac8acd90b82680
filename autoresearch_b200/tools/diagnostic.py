"""Oracle dump: weights, batches and per-layer activation / per-matrix gradient norms of the
fp32 PyTorch oracle, for comparison with any other implementation's ``--diagnostic N`` output
(role of brain/tools/diagnostic.py:34-445).

Writes into --out: ``oracle_weights.safetensors`` (engine names), ``oracle_batches.bin`` (rows of
SEQ+1 little-endian u16, the stdin protocol) and ``oracle_diagnostics.jsonl`` (one record per
batch: loss, per-layer norms of q, k, v, attention output and residual stream, per-matrix
gradient norms).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from ..ckpt.checkpoint import load_weights, model_to_engine_tensors
from ..ckpt.safetensors_io import save_file
from ..config import model_preset
from ..data.synthetic import ZipfStream
from ..models.gpt import GPT
from ..models.init import init_weights
from ..ops import reference as R
from ..ops.backend import OracleBackend


class RecordingBackend(OracleBackend):
    """The oracle ops, recording L2 norms of the attention tensors and the residual stream."""

    def __init__(self):
        super().__init__()
        self.log = []

    def attention(self, q, k, v, window):
        o = R.attention(q, k, v, window)
        self.log.append({"q": q.float().norm().item(), "k": k.float().norm().item(),
                         "v": v.float().norm().item(), "attn": o.float().norm().item()})
        return o

    def mlp_add(self, xn, wfc, wdn, x):
        out = super().mlp_add(xn, wfc, wdn, x)
        self.log[-1]["h"] = out.float().norm().item()
        return out


def run(model_name: str, out_dir: str, n_batches: int = 2, batch_size: int = 2, seed: int = 42,
        init_path: str = None, device: str = "cpu"):
    cfg = model_preset(model_name)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    be = RecordingBackend().configure(cfg)
    m = GPT(cfg, be, dtype=torch.float32, device=device)
    if init_path:
        load_weights(m, init_path, strict=False)
    else:
        init_weights(m, seed=seed)
        for blk in m.blocks:            # make the zero-initialised projections participate
            torch.nn.init.normal_(blk.wo, std=0.02, generator=torch.Generator().manual_seed(seed + blk.layer))
    save_file(model_to_engine_tensors(m), str(out / "oracle_weights.safetensors"))
    stream = ZipfStream(batch_size, cfg.seq_len, cfg.vocab, seed=seed)
    records = []
    with open(out / "oracle_batches.bin", "wb") as fb:
        for b in range(n_batches):
            ids, tgt = stream.next_batch()
            rows = torch.cat([ids, tgt[:, -1:]], 1).numpy().astype("<u2")
            fb.write(rows.tobytes())
            be.log = []
            m.zero_grad()
            scaled, per_tok = m(ids.to(device), tgt.to(device), grad_scale=1.0 / ids.numel())
            scaled.backward()
            grads = {n: (p.grad.float().norm().item() if p.grad is not None else 0.0) for n, p in m.named_parameters()}
            records.append({"batch": b, "loss": per_tok.mean().item(), "layers": be.log, "grad_norms": grads})
    with open(out / "oracle_diagnostics.jsonl", "w") as f:
        for r in records:
            f.write(json.dumps(r) + "\n")
    return records


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--out", required=True)
    ap.add_argument("--batches", type=int, default=2)
    ap.add_argument("--batch-size", type=int, default=2)
    ap.add_argument("--init-weights", default=None)
    a = ap.parse_args()
    recs = run(a.model, a.out, a.batches, a.batch_size, init_path=a.init_weights)
    print(f"wrote {len(recs)} records; first loss {recs[0]['loss']:.4f}")


if __name__ == "__main__":
    main()
