"""Every example script runs end to end on CPU with a few steps and prints its JSON summary."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CASES = {
    "train_dpsgd.py": ["--steps", "3", "--n", "2000"],
    "train_dpsgd_lm.py": ["--preset", "smoke"],
    "train_dpftrl.py": ["--steps", "4", "--n", "256"],
    "train_sft.py": ["--steps", "2", "--n", "64"],
    "train_dpo.py": ["--steps", "2", "--n", "64"],
    "train_dpsgd_trainer.py": ["--max_steps", "2", "--n", "128"],
    "train_sft_trainer.py": ["--max_steps", "2", "--n", "64"],
    "train_dpo_trainer.py": ["--max_steps", "2", "--n", "64"],
}


@pytest.mark.parametrize("script", sorted(CASES))
def test_example_runs(script, tmp_path):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    env.pop("WORLD_SIZE", None)
    run = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script), *CASES[script]], capture_output=True,
                         text=True, timeout=900, cwd=tmp_path, env=env)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-3000:]
    last = [line for line in run.stdout.strip().splitlines() if line.startswith("{")]
    assert last, run.stdout[-2000:]
    summary = json.loads(last[-1])
    eps = summary.get("epsilon")
    assert eps is None or eps >= 0
