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


def _run(script, args, cwd):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    env.pop("WORLD_SIZE", None)
    run = subprocess.run([sys.executable, "-W", "ignore", os.path.join(ROOT, "examples", script), *args], capture_output=True, text=True,
                         timeout=900, cwd=cwd, env=env)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-3000:]
    return json.loads([line for line in run.stdout.strip().splitlines() if line.startswith("{")][-1])


def test_examples_read_local_jsonl_data(tmp_path):
    """The language-model, SFT and DPO scripts on local files: text rows, chat messages (fallback template, completion-only
    masks), preference rows; Llama model with LoRA, calibration to a target epsilon, held-out metrics, canary audit."""
    with open(tmp_path / "chats.jsonl", "w") as f:
        for i in range(160):
            f.write(json.dumps({"text": f"record {i}: the answer is {i + 1}. " * 2,
                                "messages": [{"role": "user", "content": f"what is {i} plus one?"}, {"role": "assistant", "content": f"it is {i + 1}."}],
                                "prompt": f"{i} plus one is", "chosen": f" {i + 1}", "rejected": f" {i + 7}"}) + "\n")
    data = str(tmp_path / "chats.jsonl")
    lm = _run("train_dpsgd_lm.py", ["--preset", "smoke", "--dataset", data, "--num-train-samples", "128", "--num-eval-samples", "16",
                                    "--audit", "--audit-canaries", "8", "--output", str(tmp_path / "log.jsonl")], tmp_path)
    assert lm["event"] == "end" and lm["eval_ppl"] > 1 and "audit_epsilon_lower_bound" in lm and lm["audit_epsilon_lower_bound"] <= lm["epsilon"] + 1e-9
    assert sum(1 for _ in open(tmp_path / "log.jsonl")) >= 3
    sft = _run("train_sft.py", ["--model", "tiny", "--lora-r", "4", "--dataset", data, "--format", "messages", "--n", "96", "--eval-n", "16",
                                "--batch", "16", "--steps", "2", "--target-epsilon", "8", "--max-seq-len", "48", "--microbatch", "8"], tmp_path)
    assert 7.9 < sft["epsilon"] <= 8.0 + 1e-6 and 0 <= sft["eval_token_accuracy"] <= 1 and sft["noise_multiplier"] > 0.3
    dpo = _run("train_dpo.py", ["--dataset", data, "--n", "96", "--eval-n", "16", "--batch", "16", "--steps", "2", "--loss_type", "sigmoid,sft",
                                "--loss-weights", "1.0,0.1"], tmp_path)
    assert dpo["steps"] >= 1 and 0 <= dpo["eval_reward_accuracy"] <= 1
