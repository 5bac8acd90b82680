"""Write the engine's initial weights for a preset to an engine-named BF16 safetensors file, so
that two implementations (or two runs) start from identical parameters
(role of brain/tools/generate_init_weights.py:26-199; loaded back through INIT_WEIGHTS_PATH).

    python -m autoresearch_b200.tools.generate_init_weights --model phase1 --out init.safetensors
"""
from __future__ import annotations

import argparse

import torch

from ..ckpt.checkpoint import model_to_engine_tensors
from ..ckpt.safetensors_io import save_file
from ..config import model_preset
from ..models.gpt import GPT
from ..models.init import init_weights


def generate(model_name: str, out: str, seed: int = 42, scheme: str = "reference") -> int:
    cfg = model_preset(model_name)
    m = GPT(cfg, dtype=torch.bfloat16, device="cpu")
    init_weights(m, seed=seed, scheme=scheme)
    t = model_to_engine_tensors(m)
    save_file(t, out)
    return len(t)


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default="phase1")
    ap.add_argument("--out", required=True)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--scheme", default="reference", choices=["reference", "normal"])
    a = ap.parse_args()
    print(f"wrote {generate(a.model, a.out, a.seed, a.scheme)} tensors to {a.out}")


if __name__ == "__main__":
    main()
