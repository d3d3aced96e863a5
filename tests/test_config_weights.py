"""Configuration, registry, safetensors container and weight errors (no GPU)."""
import json
import os

import pytest
import torch

import rustinfer_b200  # noqa: F401
from helpers import TINY_A, TINY_B, TINY_C, sharp_weights, tensor_shapes, write_model
from rustinfer_b200.config.model_config import ConfigError, LlamaConfig
from rustinfer_b200.config.registry import (load_model_description, resolve_architecture,
                                            supported_architectures)
from rustinfer_b200.config.run_config import RunConfig, RunConfigError
from rustinfer_b200.models.decoder import Decoder
from rustinfer_b200.weights.loader import WeightError, check_against, load_weights, target_dtype
from rustinfer_b200.weights.random_init import write_random_model
from rustinfer_b200.weights.safetensors_io import SafetensorsReader, write_safetensors


def test_config_reads_its_own_keys():
    c = LlamaConfig.from_dict(TINY_B)
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers) == (96, 272, 3)
    assert (c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 1, 32)
    assert c.vocab_size == 391 and c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0
    assert c.rope_scaling.factor == 8.0 and c.rope_scaling.original_max_position_embeddings == 64
    assert not c.tie_word_embeddings
    assert c.q_dim == 96 and c.kv_dim == 32


def test_config_defaults_and_head_dim():
    d = {k: v for k, v in TINY_A.items() if k not in ("head_dim", "rms_norm_eps", "rope_theta")}
    c = LlamaConfig.from_dict(d)
    assert c.head_dim == 64 // 4 and c.rms_norm_eps == 1e-5 and c.rope_theta == 10000.0


def test_config_scaling_ignored_unless_llama3_and_complete():
    d = dict(TINY_B, rope_scaling={"rope_type": "linear", "factor": 2.0})
    assert LlamaConfig.from_dict(d).rope_scaling is None
    d = dict(TINY_B, rope_scaling={"rope_type": "llama3", "factor": 2.0})
    assert LlamaConfig.from_dict(d).rope_scaling is None


@pytest.mark.parametrize("key", ["hidden_size", "num_key_value_heads", "vocab_size", "intermediate_size"])
def test_config_missing_key(key):
    d = {k: v for k, v in TINY_A.items() if k != key}
    with pytest.raises(ConfigError, match=key):
        LlamaConfig.from_dict(d)


def test_config_bad_values():
    with pytest.raises(ConfigError, match="multiple"):
        LlamaConfig.from_dict(dict(TINY_A, num_key_value_heads=3))
    with pytest.raises(ConfigError, match="even"):
        LlamaConfig.from_dict(dict(TINY_A, head_dim=15))


def test_eos_ids_from_generation_config_first():
    c = LlamaConfig.from_dict(dict(TINY_A, eos_token_id=7), {"eos_token_id": [3, 4]})
    assert c.eos_token_ids == (3, 4)
    assert LlamaConfig.from_dict(dict(TINY_A, eos_token_id=7)).eos_token_ids == (7,)
    assert LlamaConfig.from_dict(TINY_A).eos_token_ids == ()


def test_registry_resolves_and_refuses():
    assert resolve_architecture({"architectures": ["LlamaForCausalLM"]}).name == "llama"
    assert resolve_architecture({"model_type": "llama"}).name == "llama"
    with pytest.raises(ConfigError, match="supported"):
        resolve_architecture({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3"})
    with pytest.raises(ConfigError, match="missing"):
        resolve_architecture({})
    assert "llama" in supported_architectures()


def test_model_spec_is_data(tmp_path):
    write_random_model(str(tmp_path), TINY_B, seed=1)
    fam, cfg, spec = load_model_description(str(tmp_path))
    assert len(spec.layers) == 3 and [e.layer for e in spec.run_order] == [0, 1, 2]
    m = spec.layers[0].mixer
    assert m.kind == "gqa_attention" and m.params["head_dim"] == 32 and m.params["num_kv_heads"] == 1
    assert spec.layers[0].ffn.params["intermediate_size"] == 272
    assert spec.layers[0].mixer_norm.params["eps"] == 1e-6
    assert spec.layers[1].names["ffn"] == "model.layers.1.mlp."


def test_declared_tensors_match_a_llama_checkpoint():
    for cfg in (TINY_A, TINY_B, TINY_C):
        fam = resolve_architecture(cfg)
        decls = Decoder(fam.model_spec(fam.parse_config(cfg, None))).param_decls()
        want = tensor_shapes(cfg)
        got = {n: tuple(d.shape) for n, d in decls.items() if not d.optional}
        assert got == want


def test_safetensors_roundtrip_and_foreign_reader(tmp_path):
    ts = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int64),
          "c": torch.randn(2, 2), "d": torch.randn(4).half()}
    path = str(tmp_path / "model.safetensors")
    write_safetensors(path, ts)
    r = SafetensorsReader(str(tmp_path))
    assert r.names() == ["a", "b", "c", "d"]
    for n in ts:
        assert torch.equal(r.tensor(n), ts[n]) and r.dtype(n) == ts[n].dtype
    from safetensors.torch import load_file
    other = load_file(path)
    for n in ts:
        assert torch.equal(other[n], ts[n])


def test_sharded_index(tmp_path):
    w = sharp_weights(TINY_A, 0)
    names = sorted(w)
    half = len(names) // 2
    write_safetensors(str(tmp_path / "s1.safetensors"), {n: w[n] for n in names[:half]})
    write_safetensors(str(tmp_path / "s2.safetensors"), {n: w[n] for n in names[half:]})
    wm = {n: "s1.safetensors" for n in names[:half]}
    wm.update({n: "s2.safetensors" for n in names[half:]})
    with open(tmp_path / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": wm}, f)
    r = SafetensorsReader(str(tmp_path))
    assert r.names() == names and torch.equal(r.tensor(names[-1]), w[names[-1]])


def _decls(cfg):
    fam = resolve_architecture(cfg)
    return Decoder(fam.model_spec(fam.parse_config(cfg, None))).param_decls()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    w = sharp_weights(TINY_B, 0)
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["lm_head.weight"]                                  # untied model: the head is required
    w["model.layers.0.self_attn.q_norm.weight"] = torch.ones(32)
    w["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(16, 96)
    # a buffer some exporters write beside the weights: derived from the configuration, not a fault
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.ones(16)
    write_model(str(tmp_path), TINY_B, w)
    with pytest.raises(WeightError) as ei:
        check_against(SafetensorsReader(str(tmp_path)), _decls(TINY_B), str(tmp_path))
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert e.unexpected == ["model.layers.0.self_attn.q_norm.weight"]
    assert len(e.wrong_shape) == 1 and "k_proj" in e.wrong_shape[0] and "[32, 96]" in e.wrong_shape[0]
    msg = str(e)
    assert "missing" in msg and "unexpected" in msg and "wrong shape" in msg


def test_tied_head_may_be_absent_or_present(tmp_path):
    w = sharp_weights(TINY_A, 0)
    write_model(str(tmp_path / "a"), TINY_A, w)
    check_against(SafetensorsReader(str(tmp_path / "a")), _decls(TINY_A), "a")
    w["lm_head.weight"] = torch.zeros(256, 64)
    write_model(str(tmp_path / "b"), TINY_A, w)
    check_against(SafetensorsReader(str(tmp_path / "b")), _decls(TINY_A), "b")


def test_precision_policy(tmp_path):
    bf, f32 = torch.bfloat16, torch.float32
    assert target_dtype(bf, bf) == bf and target_dtype(torch.float16, bf) == bf
    assert target_dtype(f32, bf) == f32                      # stored in 32-bit: stays so
    assert target_dtype(bf, f32) == f32 and target_dtype(f32, f32) == f32
    assert target_dtype(torch.int64, bf) == torch.int32
    w = sharp_weights(TINY_A, 0)
    w["model.norm.weight"] = w["model.norm.weight"].float()
    write_model(str(tmp_path), TINY_A, w)
    got = load_weights(str(tmp_path), _decls(TINY_A), bf, torch.device("cpu"))
    assert got["model.norm.weight"].dtype == f32
    assert got["model.embed_tokens.weight"].dtype == bf
    assert "lm_head.weight" not in got


def test_random_weights_mode(tmp_path):
    a = write_random_model(str(tmp_path / "a"), TINY_B, seed=1)
    b = write_random_model(str(tmp_path / "b"), TINY_B, seed=1)
    c = write_random_model(str(tmp_path / "c"), TINY_B, seed=2)
    ra, rb, rc = (SafetensorsReader(x) for x in (a, b, c))
    assert sorted(ra.names()) == sorted(tensor_shapes(TINY_B))
    n = "model.layers.2.mlp.down_proj.weight"
    assert torch.equal(ra.tensor(n), rb.tensor(n)) and not torch.equal(ra.tensor(n), rc.tensor(n))
    assert ra.dtype(n) == torch.bfloat16
    assert abs(float(ra.tensor(n).float().std()) - 0.02) < 0.002
    assert torch.all(ra.tensor("model.norm.weight") == 1)
    with open(os.path.join(a, "config.json")) as f:
        cfg = json.load(f)
    assert cfg["hidden_size"] == 96 and cfg["rope_scaling"]["factor"] == 8.0
    tied = write_random_model(str(tmp_path / "t"), TINY_A, seed=0, norm_std=0.1)
    rt = SafetensorsReader(tied)
    assert "lm_head.weight" not in rt
    assert float(rt.tensor("model.norm.weight").float().std()) > 0.01


def test_run_file(tmp_path):
    p = tmp_path / "run.toml"
    p.write_text('model = "./m"\nmax_batch_seqs = 4\nchunked_prefill_size = 24\nport = 8102\n'
                 'capture_sizes = [1, 2]\n[cuda_memory]\nkernel_workspace_mib = 256\n'
                 '[sampling]\ntemperature = 0.8\nseed = 3\n[[request]]\nprompt_ids = [1, 2]\n')
    cfg = RunConfig.load(str(p))
    assert cfg.model == str(tmp_path / "m") and cfg.max_batch_seqs == 4 and cfg.chunked_prefill_size == 24
    assert cfg.max_batch_tokens == 8192 and cfg.max_model_len == 4096 and cfg.capture_sizes == [1, 2]
    assert cfg.sampling["temperature"] == 0.8 and cfg.requests[0]["prompt_ids"] == [1, 2]
    p.write_text('model = "m"\nmax_batch_seq = 4\n')
    with pytest.raises(RunConfigError, match="max_batch_seq"):
        RunConfig.load(str(p))
    p.write_text('model = "m"\nmem_fraction_static = 1.5\n')
    with pytest.raises(RunConfigError, match="mem_fraction_static"):
        RunConfig.load(str(p))
    p.write_text('max_batch_seqs = 4\n')
    with pytest.raises(RunConfigError, match="model"):
        RunConfig.load(str(p))
    # paths inside the run file are relative to the run file, wherever the program is started
    p.write_text('[random_weights]\nconfig = "cfgs/tiny.json"\nseed = 1\n')
    cfg = RunConfig.load(str(p))
    assert cfg.random_weights["config"] == str(tmp_path / "cfgs" / "tiny.json") and cfg.model == ""
    p.write_text('[random_weights]\nconfig = "/abs/tiny.json"\n')
    assert RunConfig.load(str(p)).random_weights["config"] == "/abs/tiny.json"
