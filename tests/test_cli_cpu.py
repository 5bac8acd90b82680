import subprocess
import sys

from autoresearch_b200.cli import banner, parse_args


def test_flag_and_env_precedence():
    env = {"HOME": "/h", "MAX_STEPS": "50", "PEAK_LR": "0.02", "BATCH_SIZE": "4", "COOLDOWN_STEPS": "300",
           "TOTAL_BATCH": "524288", "SYNTHETIC": "1", "CHECKPOINT_DIR": "/ck", "MODEL": "phase2"}
    m, t = parse_args(["train", "--max-steps", "7", "--diagnostic", "2", "--bogus-flag", "--stream-input",
                       "--tokenizer-path", "/tok", "--pipeline", "2"], env)
    assert t.max_steps == 7 and t.diagnostic_steps == 2 and t.stream_input and t.synthetic_data
    assert t.tokenizer_dir == "/tok" and t.checkpoint_dir == "/ck" and t.n_pipeline_stages == 2
    assert t.device_batch_size == 4 and t.cooldown_steps == 300 and m.name == "phase2"
    assert abs(t.schedule_cfg.embedding_lr - 0.45) < 1e-12
    m2, t2 = parse_args([], {"HOME": "/h"})
    assert t2.max_steps is None and t2.data_dir == "/h/.cache/autoresearch/shards" and t2.eval_interval == 25
    b = banner(m, t)
    assert "autoresearch-brain" in b and "SYNTHETIC" in b and "(LRs scaled 0.5x" in b


def test_cli_trains_tiny_model_and_prints_reference_log_lines(tmp_path):
    import os
    env = dict(os.environ, MODEL="tiny", SYNTHETIC="1", MAX_STEPS="6", COOLDOWN_STEPS="2", BATCH_SIZE="2",
               TOTAL_BATCH="512", CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-m", "autoresearch_b200", "train", "--impl", "oracle"], env=env,
                       capture_output=True, text=True, timeout=300,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stderr[-2000:]
    out = r.stdout
    import re
    assert re.search(r"step\s+0 \| loss \d+\.\d{4} \| lr 1\.000 \| dt \d+\.\d{3}s \| tok/s \d+ \| mfu \d+\.\d% \| vram \d+MB \| steps_left 5", out)
    assert re.search(r"timing \| fwd\+bwd [\d.]+ms  opt [\d.]+ms  gpu [\d.]+ms  wall_gap [\d.]+ms", out)
    assert "num_steps:        6" in out and "depth:            2" in out
