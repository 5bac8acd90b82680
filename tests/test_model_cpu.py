"""Tiny CPU plumbing configuration (fp32, seed 42): model math against an independent
restatement, one Muon+AdamW step, checkpoint round trip, resume, data-parallel parity (gloo)."""
import math
import os
import subprocess
import sys

import pytest
import torch

from autoresearch_b200.config import ScheduleConfig, TrainConfig, model_preset
from autoresearch_b200.models.gpt import GPT
from autoresearch_b200.models.init import init_weights
from autoresearch_b200.ops import reference as R
from autoresearch_b200.ops.backend import get_backend


def _tiny(seed=42, moe=False):
    cfg = model_preset("tiny_moe" if moe else "tiny")
    m = GPT(cfg, get_backend("oracle", cfg), dtype=torch.float32, device="cpu")
    init_weights(m, seed=seed, scheme="normal", std=0.02)
    return cfg, m


def _independent_forward(m, ids, tgt):
    """Straight-line restatement of the forward pass (original/train.py:267-290 with the engine's
    constants) that shares no code path with GPT.run_layers beyond basic torch ops."""
    cfg = m.cfg
    B, T = ids.shape
    D, H, hd = cfg.d_model, cfg.n_head, cfg.head_dim
    norm = lambda x: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.eps)
    x = norm(m.wte[ids.long()])
    x0 = x
    half = hd // 2
    inv = cfg.rope_base ** (-torch.arange(half, dtype=torch.float64) * 2 / hd)
    ang = torch.outer(torch.arange(T, dtype=torch.float64), inv)
    cos, sin = ang.cos().float()[None, :, None, :], ang.sin().float()[None, :, None, :]

    def rope_norm(t):
        lo, hi = t[..., :half], t[..., half:]
        return norm(torch.cat([lo * cos + hi * sin, -lo * sin + hi * cos], -1))

    for i, blk in enumerate(m.blocks):
        x = m.resid_lambdas[i] * x + m.x0_lambdas[i] * x0
        xn = norm(x)
        q, k, v = (xn @ blk.wqkv.t()).split(D, dim=-1)
        q, k, v = (t.view(B, T, H, hd) for t in (q, k, v))
        if blk.ve is not None:
            gate = 2 * torch.sigmoid(xn[..., :cfg.ve_gate_ch] @ blk.ve_gate.t())
            v = v + gate.unsqueeze(-1) * blk.ve[ids.long()].view(B, T, H, hd)
        q, k = rope_norm(q), rope_norm(k)
        att = torch.einsum("bihd,bjhd->bhij", q, k) / math.sqrt(hd)
        i_idx = torch.arange(T)[:, None]; j_idx = torch.arange(T)[None, :]
        vis = (j_idx <= i_idx) & (j_idx >= i_idx - cfg.window(blk.layer))
        att = att.masked_fill(~vis, float("-inf")).softmax(-1)
        a = torch.einsum("bhij,bjhd->bihd", att, v).reshape(B, T, D)
        x = x + a @ blk.wo.t()
        x = x + torch.relu(norm(x) @ blk.wfc.t()).pow(2) @ blk.wdn.t()
    logits = norm(x) @ m.lm_head.t()
    s = cfg.softcap * torch.tanh(logits / cfg.softcap)
    return torch.nn.functional.cross_entropy(s.view(-1, cfg.vocab), tgt.reshape(-1).long(), reduction="none")


def test_forward_and_gradients_match_independent_restatement():
    cfg, m = _tiny()
    g = torch.Generator().manual_seed(42)
    ids = torch.randint(0, cfg.vocab, (2, cfg.seq_len), generator=g, dtype=torch.int32)
    tgt = torch.randint(0, cfg.vocab, (2, cfg.seq_len), generator=g, dtype=torch.int32)
    scaled, per_tok = m(ids, tgt, grad_scale=1.0 / ids.numel())
    ref = _independent_forward(m, ids, tgt)
    assert torch.allclose(per_tok, ref, atol=1e-4, rtol=1e-4)
    assert abs(per_tok.mean().item() - math.log(cfg.vocab)) < 0.1     # near-uniform prediction at init
    scaled.backward()
    got = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    ref.mean().backward()
    for n, p in m.named_parameters():
        assert torch.allclose(got[n], p.grad, atol=1e-6, rtol=1e-3), n


def test_window_semantics_on_a_short_window():
    q = torch.randn(1, 12, 1, 8); k = torch.randn(1, 12, 1, 8); v = torch.eye(12).view(1, 12, 1, 12)
    o = R.attention(q, k, v, window=3)[0, :, 0]           # row i = attention weights over keys
    for i in range(12):
        seen = (o[i] > 0).nonzero().flatten().tolist()
        assert seen == list(range(max(0, i - 3), i + 1))     # i-3 <= j <= i : window+1 keys


def test_one_optimizer_step_matches_reference_functions():
    from autoresearch_b200.optim import muon_adamw as MA
    from autoresearch_b200.parallel.layout import ParamLayout
    cfg, m = _tiny()
    lay = ParamLayout(m.named_matrix_groups())
    sched = ScheduleConfig()
    opt = MA.MuonAdamW(lay, sched, cfg.d_model)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab, (2, cfg.seq_len), generator=g, dtype=torch.int32)
    tgt = torch.randint(0, cfg.vocab, (2, cfg.seq_len), generator=g, dtype=torch.int32)
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    scaled, _ = m(ids, tgt, grad_scale=1.0 / ids.numel())
    scaled.backward()
    grads = {n: p.grad.detach().clone() for n, p in m.named_parameters()}
    lay.accumulate_autograd_grads()
    opt.step(1, 0.0)
    # Muon on wo of layer 0 (a [D, D] matrix), by hand
    W, G = before["blocks.0.wfc"], grads["blocks.0.wfc"]
    mu = 0.85 + 0.10 * (1 / 200)
    buf = (1 - mu) * G
    u = (1 - mu) * G + mu * buf
    x = MA.newton_schulz(MA.frob_normalise(u[None]), 5)
    sec = torch.zeros(1, W.shape[0], 1)
    gf = MA.normuon(x, sec, 0.95)[0]
    lr = 0.04 * math.sqrt(max(1.0, W.shape[0] / W.shape[1]))
    mask = (gf * W) >= 0
    want = W - (lr * gf + lr * 0.2 * W * mask)
    assert torch.allclose(dict(m.named_parameters())["blocks.0.wfc"], want, atol=1e-6)
    # AdamW on lm_head by hand (bias-corrected first step: update = lr * sign-ish)
    W, G = before["lm_head"], grads["lm_head"]
    lr = 0.005 * (cfg.d_model / 768) ** -0.5
    p = W * (1 - lr * 0.01)
    mm, vv = 0.2 * G, 0.05 * G * G
    want = p - lr * (mm / 0.2) / ((vv / 0.05).sqrt() + 1e-10)
    assert torch.allclose(dict(m.named_parameters())["lm_head"], want, atol=1e-6)
    # qkv is split into three Muon units
    names = [u.name for a in lay.atoms for u in a.units]
    assert "h.0.wqkv.q" in names and "h.0.wqkv.v" in names


def test_newton_schulz_orthogonalises():
    from autoresearch_b200.optim import muon_adamw as MA
    torch.manual_seed(0)
    for shape in [(1, 32, 32), (2, 64, 16), (2, 16, 64)]:
        x = MA.newton_schulz(MA.frob_normalise(torch.randn(shape)), 5)
        s = torch.linalg.svdvals(x)
        assert s.max() < 1.3 and s.min() > 0.5, (shape, s.min().item(), s.max().item())


def test_checkpoint_roundtrip_names_and_python_name_import(tmp_path):
    from autoresearch_b200.ckpt import checkpoint as ck
    from autoresearch_b200.ckpt.safetensors_io import load_file, save_file
    cfg, m = _tiny()
    path = ck.save_checkpoint(m, str(tmp_path))
    assert path.endswith("model.safetensors")
    sd = load_file(path)
    assert list(sd) == sorted(sd)
    assert {"wte.weight", "lm_head.weight", "resid_lambdas", "x0_lambdas", "h.0.attn.c_q.weight",
            "h.1.attn.c_proj.weight", "h.0.mlp.c_fc.weight", "h.1.mlp.c_proj.weight", "ve.1.weight",
            "h.1.attn.ve_gate.weight"} <= set(sd)
    assert all(t.dtype == torch.bfloat16 for t in sd.values())
    assert tuple(sd["h.0.attn.c_k.weight"].shape) == (cfg.d_model, cfg.d_model)
    _, m2 = _tiny(seed=7)
    ck.load_weights(m2, path)
    for (n, a), (_, b) in zip(m.named_parameters(), m2.named_parameters()):
        assert torch.equal(a.to(torch.bfloat16), b.to(torch.bfloat16)), n
    # Python state-dict names and F32 tensors are accepted too
    py = {}
    for k, v in sd.items():
        if k == "wte.weight":
            py["transformer.wte.weight"] = v.float()
        elif k.startswith("h."):
            py["transformer." + k] = v.float()
        elif k.startswith("ve."):
            py["value_embeds." + k[3:]] = v.float()
        else:
            py[k] = v.float()
    save_file(py, str(tmp_path / "py.safetensors"))
    _, m3 = _tiny(seed=9)
    ck.load_weights(m3, str(tmp_path / "py.safetensors"))
    assert torch.equal(m3.blocks[1].ve.to(torch.bfloat16), m.blocks[1].ve.to(torch.bfloat16))
    # missing tensors are refused in strict mode
    del py["lm_head.weight"]
    save_file(py, str(tmp_path / "short.safetensors"))
    with pytest.raises(KeyError):
        ck.load_weights(m3, str(tmp_path / "short.safetensors"))


def test_dense_checkpoint_warm_starts_moe(tmp_path):
    from autoresearch_b200.ckpt import checkpoint as ck
    cfg, dense = _tiny()
    path = ck.save_checkpoint(dense, str(tmp_path))
    mcfg, moe = _tiny(moe=True)
    st = ck.load_weights(moe, path)
    assert st["warm_started"] == cfg.n_layer
    blk, dblk = moe.blocks[0], dense.blocks[0]
    ME = mcfg.moe.mlp_dim_e
    assert torch.equal(blk.expert_fc[0], dblk.wfc[:ME].to(torch.bfloat16).float())
    assert not torch.equal(blk.expert_fc[1], blk.expert_fc[0])
    assert (blk.expert_fc[1] - blk.expert_fc[0]).abs().max() < 0.05
    assert blk.router.abs().max() == 0


def test_moe_forward_backward_and_aux_loss():
    cfg, m = _tiny(moe=True)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, cfg.vocab, (2, cfg.seq_len), generator=g, dtype=torch.int32)
    tgt = torch.randint(0, cfg.vocab, (2, cfg.seq_len), generator=g, dtype=torch.int32)
    scaled, per = m(ids, tgt, grad_scale=1.0 / ids.numel())
    scaled.backward()
    assert m.aux_loss is not None and m.aux_loss.item() > 0
    assert m.blocks[0].router.grad is not None and m.blocks[0].expert_fc.grad.abs().sum() > 0
    # balanced routing gives aux = coeff per layer: E * sum_e (1/E)(1/E) = 1
    probs = torch.full((8, 4), 0.25); idx = torch.tensor([[0, 1], [2, 3]] * 4)
    assert abs(R.moe_aux_loss(probs, idx, 4, 0.01).item() - 0.01) < 1e-7
    # capacity rule keeps the first `cap` slots per expert in token order
    keep = R.moe_keep_mask(torch.tensor([[0, 1], [0, 1], [0, 2]]), 3, 2)
    assert keep.tolist() == [[True, True], [True, True], [False, True]]


def test_trainer_resume_is_exact(tmp_path):
    from autoresearch_b200.trainer import Trainer
    cfg = model_preset("tiny")

    def mk(resume):
        t = TrainConfig(device_batch_size=2, total_batch_size=2 * 128 * 2, max_steps=8, cooldown_steps=4,
                        synthetic_data=True, synthetic_kind="zipf", impl="oracle", cooldown_trigger_file="",
                        checkpoint_dir=str(tmp_path), resume=resume)
        return Trainer(cfg, t, device="cpu", quiet=True)

    a = mk(False)
    full = [float(a.train_step()) for _ in range(6)]
    b = mk(False)
    first = [float(b.train_step()) for _ in range(3)]
    b.save(step=None)
    c = mk(True)
    assert c.step == 3
    rest = [float(c.train_step()) for _ in range(3)]
    assert first == full[:3]
    # the weight file holds bf16 roundings, but the parameters are rebuilt from the saved fp32 masters
    assert rest == full[3:], (rest, full[3:])


DP_WORKER = r"""
import os, sys, json, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ARB_ROOT"])
from autoresearch_b200.config import TrainConfig, ParallelConfig, model_preset
from autoresearch_b200.trainer import Trainer
dist.init_process_group("gloo")
cfg = model_preset("tiny")
t = TrainConfig(device_batch_size=2, total_batch_size=4 * 128, max_steps=10, cooldown_steps=3, synthetic_data=True,
                synthetic_kind="zipf", impl="oracle", cooldown_trigger_file="", parallel=ParallelConfig(dp=2, comm="nccl"))
tr = Trainer(cfg, t, device="cpu", quiet=True)
ls = [tr.mean_loss_across_ranks(tr.train_step()) for _ in range(4)]
w = tr.model.blocks[0].wo.detach().clone()
ws = [torch.zeros_like(w) for _ in range(2)]
dist.all_gather(ws, w)
if dist.get_rank() == 0:
    print("RESULT " + json.dumps({"losses": ls, "same": bool(torch.equal(ws[0], ws[1])), "owners": sorted({a.owner for a in tr.layout.atoms})}))
dist.destroy_process_group()
"""


def test_data_parallel_gloo_matches_single_process(tmp_path):
    from autoresearch_b200.trainer import Trainer
    cfg = model_preset("tiny")
    t = TrainConfig(device_batch_size=2, total_batch_size=4 * 128, max_steps=10, cooldown_steps=3, synthetic_data=True,
                    synthetic_kind="zipf", impl="oracle", cooldown_trigger_file="")
    one = Trainer(cfg, t, device="cpu", quiet=True)
    ref = [float(one.train_step()) for _ in range(4)]
    script = tmp_path / "w.py"
    script.write_text(DP_WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, ARB_ROOT=root)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29655", str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    import json
    res = json.loads([l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1][7:])
    assert res["same"] and res["owners"] == [0, 1]
    for a, b in zip(ref, res["losses"]):
        assert abs(a - b) < 1e-3, (ref, res)


def test_fused_gather_plan_covers_every_remote_parameter():
    """The parameter all-gather plan of the peer-memory path: a dense weight of another rank is either pulled by
    its first GEMM or lies inside a range that is copied at once; ranges are 16-byte aligned and stay inside the
    owner's shard."""
    from types import SimpleNamespace
    from autoresearch_b200.config import model_preset
    from autoresearch_b200.models.gpt import GPT
    from autoresearch_b200.parallel.fused_dp import FusedComm
    from autoresearch_b200.parallel.layout import ParamLayout
    cfg = model_preset("tiny")
    model = GPT(cfg, dtype=torch.bfloat16)
    lay = ParamLayout(model.named_matrix_groups(), world=3, rank=1)
    me = SimpleNamespace(world=3, rank=1, fuse_into_gemm=True, GEMM_OPERANDS=FusedComm.GEMM_OPERANDS)
    gemm_atoms, ranges = FusedComm._plan_gather(me, lay)
    es = 2
    assert gemm_atoms and ranges
    pulled = {a.name for a, _ in gemm_atoms}
    assert all(n.endswith(FusedComm.GEMM_OPERANDS) for n in pulled)
    for b0, b1, r in ranges:
        lo, hi = lay.shard_range(r)
        assert r != 1 and b0 % 16 == 0 and b1 % 16 == 0 and lo * es <= b0 < b1 <= hi * es
    for a in lay.atoms:
        if a.owner == 1:
            assert a.name not in pulled
            continue
        if a.name in pulled:
            continue
        a0, a1 = a.offset * es, (a.offset + a.numel) * es
        assert any(b0 <= a0 and a1 <= b1 and r == a.owner for b0, b1, r in ranges), a.name
    # without the GEMM fusion everything travels in ranges
    me.fuse_into_gemm = False
    g2, r2 = FusedComm._plan_gather(me, lay)
    assert not g2 and sum(b1 - b0 for b0, b1, _ in r2) >= sum(a.numel * es for a in lay.atoms if a.owner != 1)
