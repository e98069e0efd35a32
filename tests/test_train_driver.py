"""The benchmark entry points end to end on one CPU rank: real-data pipeline from a token file, training epochs with
per-phase timers, the separate test pass, checkpoint save and resume."""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, args, port):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", RANK="0", LOCAL_RANK="0", WORLD_SIZE="1", MASTER_ADDR="127.0.0.1",
               MASTER_PORT=str(port), COLUMNS="400")
    r = subprocess.run([sys.executable, os.path.join(ROOT, script)] + args + ["--backend", "gloo"], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    return r.stdout + r.stderr


def test_gpt2_driver_token_file_eval_and_resume(tmp_path):
    from cubework_b200.utils import free_port
    tokens = tmp_path / "tokens.npy"
    np.save(tokens, np.random.default_rng(0).integers(0, 1024, size=64 * 80).astype(np.int32))
    save = tmp_path / "ckpt"
    out = _run("benchmark/gpt2/train.py", ["-m", "gpt2_tiny", "--seq_length", "64", "--bs", "4", "--n_step", "3",
                                           "--dataset_path", str(tokens), "--eval", "--clip", "1.0", "--save_dir",
                                           str(save)], free_port())
    assert "/ Train]" in out and "/ Test]" in out and "Perplexity" in out and "data " in out and "bwd " in out
    assert "18 training / 2 test batches" in out.replace("\n", " ")
    assert (save / "step_3" / "meta.json").exists() and (save / "step_3" / "tp0_dp0.pt").exists()
    out = _run("benchmark/gpt2/train.py", ["-m", "gpt2_tiny", "--seq_length", "64", "--bs", "4", "--n_step", "2",
                                           "--dataset_path", str(tokens), "--save_dir", str(save), "--resume_step", "3"],
               free_port())
    assert "resumed from step 3" in out and (save / "step_5" / "meta.json").exists()


def test_opt_and_vit_drivers_synthetic():
    from cubework_b200.utils import free_port
    out = _run("benchmark/opt/train.py", ["-m", "opt_tiny", "--seq_length", "64", "--bs", "4", "--n_step", "2", "--eval"],
               free_port())
    assert "/ Test]" in out
    loss = float(out.split("/ Train]: Loss = ")[1].split()[0])
    assert abs(loss - np.log(512)) < 0.5, loss          # N(0, 0.02) weights: the loss starts at ln(vocabulary)
    out = _run("benchmark/vit/train.py", ["-m", "vit_tiny", "--bs", "8", "--n_step", "2", "--eval"], free_port())
    assert "images/sec" in out and "Accuracy" in out
