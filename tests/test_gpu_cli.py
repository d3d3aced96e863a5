"""The command line as a user runs it: `bin/rustinfer --config run.toml` in a process of its
own, started from another folder, with the model made by the run file's [random_weights]
table; its tokens against the plain implementation."""
import json
import os
import subprocess
import sys

import pytest

import plain_llama
from helpers import TINY

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_rustinfer_config_generates_the_plain_models_tokens(tmp_path):
    run_dir = tmp_path / "runs"
    run_dir.mkdir()
    with open(run_dir / "tiny_a.json", "w") as f:
        json.dump(TINY["A"], f)
    prompt = [5, 17, 3, 99, 42, 7, 250]
    (run_dir / "run.toml").write_text(f"""
model = "model_out"                      # relative to this file; made by [random_weights]
model_name = "ignored-by-this-engine"
dtype = "float32"
max_batch_tokens = 64
max_batch_seqs = 4
max_model_len = 96
paged_block_size = 8
chunked_prefill_size = 5
num_blocks = 24
ignore_eos = true
capture_sizes = [1, 2]

[random_weights]
config = "tiny_a.json"                   # relative to this file too
seed = 4
std = 0.2
norm_std = 0.1

[sampling]
temperature = 0.0
max_tokens = 9

[[request]]
prompt_ids = {prompt}

[[request]]
random_len = 13
seed = 3
""")
    other = tmp_path / "elsewhere"
    other.mkdir()
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "rustinfer"), "--config",
                        str(run_dir / "run.toml")], cwd=str(other), capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-3000:]
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.strip()]
    assert [l["request"] for l in lines] == [0, 1]
    assert os.path.isfile(run_dir / "model_out" / "model.safetensors")
    assert not os.path.exists(other / "model_out")
    cfg, w = plain_llama.read_model_folder(str(run_dir / "model_out"))
    import random
    rng = random.Random(3)
    second = [rng.randrange(TINY["A"]["vocab_size"]) for _ in range(13)]
    for line, ids in zip(lines, [prompt, second]):
        assert line["prompt_tokens"] == len(ids) and line["finish_reason"] == "length"
        assert line["tokens"] == plain_llama.greedy_generate(cfg, w, ids, 9)
    stats = json.loads(p.stderr.strip().splitlines()[-1])
    assert stats["generated_tokens"] == 18 and stats["prompt_tokens"] == 20


def test_random_weights_subcommand_writes_a_model_folder(tmp_path):
    with open(tmp_path / "c.json", "w") as f:
        json.dump(TINY["B"], f)
    out = tmp_path / "made"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "rustinfer"), "random-weights", "--config",
                        str(tmp_path / "c.json"), "--seed", "7", "--out", str(out)],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    cfg, w = plain_llama.read_model_folder(str(out))
    assert cfg["hidden_size"] == TINY["B"]["hidden_size"] and "lm_head.weight" in w
    assert w["model.layers.2.mlp.down_proj.weight"].shape == (96, 272)
