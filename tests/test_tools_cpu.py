import json

import torch

from autoresearch_b200.tools import compare_train, diagnostic, generate_init_weights, monitor


def test_generated_init_weights_are_reproducible_and_loadable(tmp_path):
    from autoresearch_b200.ckpt.safetensors_io import load_file
    a, b = tmp_path / "a.safetensors", tmp_path / "b.safetensors"
    n = generate_init_weights.generate("tiny", str(a))
    generate_init_weights.generate("tiny", str(b))
    assert n > 10 and a.read_bytes() == b.read_bytes()
    sd = load_file(str(a))
    assert sd["h.0.attn.c_proj.weight"].abs().max() == 0            # zero-initialised projection
    s = 0.68 * 3 ** 0.5 / 64 ** 0.5
    assert sd["h.0.attn.c_q.weight"].float().abs().max() <= s * 1.01
    assert abs(sd["wte.weight"].float().std().item() - 1.0) < 0.05
    assert sd["resid_lambdas"].tolist() == [1.0, 1.0] and abs(sd["x0_lambdas"][0].item() - 0.1) < 1e-3


def test_oracle_dump_files(tmp_path):
    recs = diagnostic.run("tiny", str(tmp_path), n_batches=2, batch_size=2)
    assert len(recs) == 2 and len(recs[0]["layers"]) == 2 and recs[0]["layers"][0]["q"] > 0
    assert (tmp_path / "oracle_weights.safetensors").exists()
    assert (tmp_path / "oracle_batches.bin").stat().st_size == 2 * 2 * 129 * 2
    lines = (tmp_path / "oracle_diagnostics.jsonl").read_text().splitlines()
    assert json.loads(lines[1])["grad_norms"]["lm_head"] > 0


def test_compare_train_identical_implementations_agree(tmp_path):
    r = compare_train.run("tiny", "oracle", "oracle", steps=4, batch=2, csv_path=str(tmp_path / "c.csv"), device="cpu")
    assert r["max_rel"] == 0.0 and (tmp_path / "c.csv").read_text().startswith("step,loss_oracle,loss_oracle,rel_diff")


def test_compare_train_init_weights_streamed_rows_and_proxy_eval(tmp_path):
    """--init-weights, --stream-input (rows replayed to both implementations) and the proxy evaluation column."""
    import io
    import numpy as np
    init = tmp_path / "init.safetensors"
    generate_init_weights.generate("tiny", str(init), scheme="torch", init_scale=1.0, python_names=True)
    rng = np.random.default_rng(1)
    rows = rng.integers(1, 256, size=(2 * 6 + 2 * 2, 129), dtype=np.uint16)
    got = compare_train.read_rows(io.BytesIO(rows.astype("<u2").tobytes() + b"\x01"), 128, None)   # trailing partial row ignored
    assert np.array_equal(got, rows)
    csvp = tmp_path / "s.csv"
    r = compare_train.run("tiny", "oracle", "oracle", steps=6, batch=2, csv_path=str(csvp), device="cpu", cooldown=2,
                          init_weights=str(init), rows=got, eval_every=3, eval_batches=2)
    assert r["steps"] == 6 and r["max_rel"] == 0.0
    assert sorted(r["evals"]["oracle"]) == [2, 5] and r["evals"]["oracle"][5] < r["evals"]["oracle"][2] + 1.0
    lines = csvp.read_text().splitlines()
    assert lines[0].endswith("val_bpb_oracle,val_bpb_oracle") and lines[3].split(",")[-1] != "" and lines[2].split(",")[-1] == ""
    # the streamed rows, not the synthetic stream, were trained on: another stream gives another loss
    r2 = compare_train.run("tiny", "oracle", "none", steps=2, batch=2, device="cpu", init_weights=str(init))
    assert abs(r2["losses"]["oracle"][0] - r["losses"]["oracle"][0]) > 1e-4
    compare_train.write_report(r, str(tmp_path / "p.md"), "t", "cmd")
    assert "| step | oracle | oracle |" in (tmp_path / "p.md").read_text()


def test_torch_order_init_matches_the_python_trainers_draws(tmp_path):
    """scheme='torch' reproduces torch.manual_seed(42) followed by the upstream init_weights call order."""
    import math
    from autoresearch_b200.ckpt.safetensors_io import load_file
    out = tmp_path / "t.safetensors"
    generate_init_weights.generate("tiny", str(out), scheme="torch", init_scale=1.0)
    sd = load_file(str(out))
    D, V, M = 64, 256, 256
    s = math.sqrt(3) * D ** -0.5
    torch.manual_seed(42)
    wte = torch.nn.init.normal_(torch.empty(V, D), 0.0, 1.0)
    lm = torch.nn.init.normal_(torch.empty(V, D), 0.0, 0.001)
    layers = []
    for _ in range(2):
        layers.append([torch.nn.init.uniform_(torch.empty(r, D), -s, s) for r in (D, D, D, M)])
    ve1 = torch.nn.init.uniform_(torch.empty(V, D), -s, s)
    bf = lambda t: t.to(torch.bfloat16)
    assert torch.equal(sd["wte.weight"], bf(wte)) and torch.equal(sd["lm_head.weight"], bf(lm))
    for i, (q, k, v, fc) in enumerate(layers):
        assert torch.equal(sd[f"h.{i}.attn.c_q.weight"], bf(q)) and torch.equal(sd[f"h.{i}.attn.c_v.weight"], bf(v))
        assert torch.equal(sd[f"h.{i}.attn.c_k.weight"], bf(k)) and torch.equal(sd[f"h.{i}.mlp.c_fc.weight"], bf(fc))
    assert torch.equal(sd["ve.1.weight"], bf(ve1))


def test_multi_epoch_store_spills_to_disk_and_replays_every_epoch(tmp_path):
    from autoresearch_b200.tools import multi_epoch as ME

    class Tok:
        def encode(self, text, bos=True):
            return [8188] + [ord(c) for c in text]

    texts = [chr(65 + i) * (5 + 3 * i) for i in range(12)]
    in_mem = ME.collect(texts, Tok(), 2, 33, None, mem_limit=1 << 30)
    spilled = ME.collect(texts, Tok(), 2, 33, None, mem_limit=64, tmp_dir=str(tmp_path))
    assert not in_mem.on_disk and spilled.on_disk and spilled.path.startswith(str(tmp_path))
    assert len(in_mem) == len(spilled) == 12 and in_mem.n_tokens == spilled.n_tokens
    a = [d.tolist() for d in ME.epoch_stream(in_mem, 3, seed=42)]
    b = [d.tolist() for d in ME.epoch_stream(spilled, 3, seed=42)]
    assert a == b and len(a) == 36
    first, second = a[:12], a[12:24]
    assert sorted(map(tuple, first)) == sorted(map(tuple, second)) and first != second     # same set, reshuffled
    path = spilled.path
    spilled.close()
    import os
    assert not os.path.exists(path)
    # --target-rows: stop collecting once epochs x tokens covers the rows
    few = ME.collect(texts, Tok(), 2, 33, target_rows=2, mem_limit=1 << 30)
    assert len(few) < 12 and few.n_tokens * 2 >= 2 * 33


def test_monitor_parses_reference_log_lines():
    log = """autoresearch-brain
step     0 | loss 9.0037 | lr 1.000 | dt 9.960s | tok/s 52643 | mfu 25.5% | vram 53410MB | steps_left 999
timing | fwd+bwd 9926.0ms  opt 33.0ms  gpu 9959.0ms  wall_gap 0.0ms
[eval] step 25 | val_bpb 1.2345
step   995 | loss 2.6008 | lr 0.036 | dt 9.950s | tok/s 52700 | mfu 25.6% | vram 53410MB | steps_left 4
[eval] final | val_bpb 0.5392
thread 'main' panicked at src/train.rs
""".splitlines()
    p = monitor.parse(log)
    assert [s["step"] for s in p["steps"]] == [0, 995] and p["steps"][1]["tok_s"] == 52700
    assert p["evals"] == [{"step": 25, "val_bpb": 1.2345}, {"step": None, "val_bpb": 0.5392}]
    assert len(p["crashes"]) == 1 and "CRASH" in monitor.summary(p)


def test_launch_lifecycle_and_plot(tmp_path):
    """start runs a tiny CPU job to the end, salvages its checkpoint and writes the report; plot_live draws it."""
    import json
    import sys
    from autoresearch_b200.tools import launch, plot_live
    out = tmp_path / "run"
    (out / "live_checkpoints" / "rank_0").mkdir(parents=True)     # synthetic-data runs write no checkpoint themselves
    (out / "live_checkpoints" / "rank_0" / "model.safetensors").write_bytes(b"stand-in")
    rc = launch.main(["start", "--out", str(out), "--gpus", "1", "--poll-seconds", "0.5", "--cost-per-gpu-hour", "2.0", "--",
                      "MODEL=tiny", "SYNTHETIC=1", "MAX_STEPS=4", "COOLDOWN_STEPS=2", "BATCH_SIZE=2", "TOTAL_BATCH=256",
                      "EVAL_EVERY=0"])
    log = (out / "train.log").read_text()
    assert rc == 0, log[-2000:]
    rep = json.loads((out / "report.json").read_text())
    assert rep["status"] == "finished" and rep["last_step"] is not None and rep["cost"] is not None
    state = json.loads((out / "run_state.json").read_text())
    assert "ended" in state
    assert (out / "checkpoints" / "rank_0" / "model.safetensors").read_bytes() == b"stand-in", "checkpoints were not salvaged"
    assert launch.main(["status", "--out", str(out)]) == 0
    assert launch.main(["teardown", "--out", str(out)]) == 0          # nothing left to stop: only salvages
    plot_live.main([str(out / "train.log"), "--out", str(tmp_path / "c.svg")])
    svg = (tmp_path / "c.svg").read_text()
    assert svg.startswith("<svg") and "polyline" in svg


def test_report_page_from_bench_lines(tmp_path):
    """The static benchmark page: one bar per result line, grouped by metric; 'unavailable' lines become notes."""
    import json
    from autoresearch_b200.tools import report
    lines = [
        {"metric": "train tokens/sec", "value": 222063.0, "unit": "tokens/s", "n_gpus": 1, "steps": 3, "ms_per_step": 2361.0,
         "dtype": "bf16", "vs_baseline": 4.22, "impl": "sm100", "data": "synthetic",
         "config": {"model": "phase2 <428M>", "parallelism": "dp1"}, "clocks": {"sm_mhz": 1567, "reasons": ["sw_power_cap"]},
         "e2e": {"value": 221900.0}},
        {"metric": "train tokens/sec", "value": 1743016.0, "unit": "tokens/s", "n_gpus": 8, "steps": 3, "ms_per_step": 300.8,
         "dtype": "bf16", "vs_baseline": None, "impl": "sm100", "data": "synthetic", "config": {"model": "phase2", "parallelism": "dp8"}},
        {"impl": "reference", "unavailable": "needs a Hopper-only attention library"},
    ]
    src = tmp_path / "r.jsonl"
    src.write_text("noise before\n" + "\n".join(json.dumps(l) for l in lines) + "\nnot json {\n")
    out = tmp_path / "report.html"
    report.main([str(src), "--out", str(out)])
    page = out.read_text()
    assert page.count("<rect") == 2 and "1,743,016 tokens/s" in page and "4.22x published reference" in page
    assert "phase2 &lt;428M&gt;" in page                      # labels are escaped
    assert "needs a Hopper-only attention library" in page and "sw_power_cap" in page
    # the longest bar belongs to the largest value
    import re
    widths = [float(w) for w in re.findall(r'<rect x="390" y="\d+" width="([0-9.]+)"', page)]
    assert widths[1] == 420.0 and widths[0] < 60
