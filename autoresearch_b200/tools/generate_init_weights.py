"""Write initial weights for a preset to an engine-named BF16 safetensors file, so that two implementations
(or this engine and the upstream Python trainer) start from identical parameters; loaded back through
INIT_WEIGHTS_PATH / --init-weights (role of brain/tools/generate_init_weights.py:26-199).

    python -m autoresearch_b200.tools.generate_init_weights --model phase1 --out init.safetensors
    python -m autoresearch_b200.tools.generate_init_weights --model phase1 --scheme torch --init-scale 1.0 --out init.safetensors

Schemes: ``reference`` = the engine's xorshift64 / Box-Muller stream (brain/src/train.rs:2268-2346, 2424-2483);
``torch`` = PyTorch's generator in the call order of the Python trainer's init_weights (torch.manual_seed(42); wte,
lm_head, per layer c_q c_k c_v c_fc, then the value embeddings), whose init scale is 1.0 where the engine uses 0.68;
``normal`` = every matrix N(0, 0.02).  ``--python-names`` writes the state-dict names of the Python trainer
(``transformer.h.{i}...``, ``value_embeds.{i}.weight``) instead of the engine's; both are accepted on load.
"""
from __future__ import annotations

import argparse
import dataclasses
import re

import torch

from ..ckpt.checkpoint import model_to_engine_tensors
from ..ckpt.safetensors_io import save_file
from ..config import model_preset
from ..models.gpt import GPT
from ..models.init import init_weights


def python_name(engine: str) -> str:
    """Engine tensor name -> the upstream Python state-dict name."""
    if engine == "wte.weight":
        return "transformer.wte.weight"
    m = re.match(r"^ve\.(\d+)\.weight$", engine)
    if m:
        return f"value_embeds.{m.group(1)}.weight"
    if engine.startswith("h."):
        return "transformer." + engine
    return engine


def generate(model_name: str, out: str, seed: int = 42, scheme: str = "reference", init_scale: float = None,
             python_names: bool = False, dtype=torch.bfloat16, **overrides) -> int:
    cfg = model_preset(model_name, **overrides)
    if init_scale is not None:
        cfg = dataclasses.replace(cfg, init_scale=init_scale)
    # the torch scheme draws fp32 tensors and rounds once, as the Python trainer's cast does
    m = GPT(cfg, dtype=torch.float32 if scheme == "torch" else dtype, device="cpu")
    init_weights(m, seed=seed, scheme=scheme)
    t = model_to_engine_tensors(m)
    if python_names:
        t = {python_name(k): v for k, v in t.items()}
    save_file(t, out)
    return len(t)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="phase1")
    ap.add_argument("--out", "-o", required=True)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--scheme", default="reference", choices=["reference", "torch", "normal"])
    ap.add_argument("--init-scale", type=float, default=None, help="override the preset's init scale (Python trainer: 1.0)")
    ap.add_argument("--depth", type=int, default=None, help="override the number of layers")
    ap.add_argument("--python-names", action="store_true")
    a = ap.parse_args()
    over = {"n_layer": a.depth} if a.depth else {}
    n = generate(a.model, a.out, a.seed, a.scheme, a.init_scale, a.python_names, **over)
    print(f"wrote {n} tensors to {a.out}")


if __name__ == "__main__":
    main()
