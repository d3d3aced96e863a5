"""What `bench.py` answers without a GPU: more than one GPU is refused in one line with exit
code 2, the reference arm says in one JSON line why it cannot run, and the shapes it offers are
configurations the architecture registry takes."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=120)


def test_more_than_one_gpu_is_refused_in_one_line():
    r = _run("--gpus", "2")
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert r.returncode == 0
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and isinstance(out["unavailable"], str) and "\n" not in out["unavailable"]


def test_shapes_are_valid_configurations():
    sys.path.insert(0, ROOT)
    import bench
    from rustinfer_b200.config.registry import resolve_architecture
    assert set(bench.SHAPES) == {"1b", "3b", "8b"}
    for name, (label, cfg) in bench.SHAPES.items():
        fam = resolve_architecture(cfg)
        typed = fam.parse_config(cfg, None)
        assert typed.num_hidden_layers == cfg["num_hidden_layers"] and label
        per_layer, weight_bytes, kv_per_token, q_dim = bench.model_numbers(cfg, cfg["num_hidden_layers"])
        assert q_dim == cfg["num_attention_heads"] * cfg["head_dim"] and weight_bytes > 0 and kv_per_token > 0
