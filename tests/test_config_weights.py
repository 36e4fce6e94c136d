"""Configuration, registry, weight loading errors and the random-weights mode (CPU)."""

from __future__ import annotations

import json

import pytest
import torch

from tokenmill_b200.config import ConfigError, EngineConfig, Qwen2Config, add_engine_args, engine_config_from_args
from tokenmill_b200.parts.model import DecoderModel
from tokenmill_b200.registry import RegistryError, architecture_names, get_architecture, get_part
from tokenmill_b200.weights import WeightError, named_config, read_spec, write_random_model
from tokenmill_b200.weights.loader import load_tensors

BASE = named_config("tiny-a")


def test_config_reads_keys_and_defaults():
    cfg = Qwen2Config.from_dict(BASE)
    assert (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (64, 4, 2, 16)
    assert cfg.num_kv_groups == 2 and cfg.tie_word_embeddings and cfg.rope_theta == 10000.0
    minimal = {k: BASE[k] for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                    "num_attention_heads")}
    d = Qwen2Config.from_dict(minimal)
    # defaults of the reference: kv heads = heads, 32768 positions, eps 1e-6, untied, theta 10000
    assert d.num_key_value_heads == 4 and d.max_position_embeddings == 32768 and d.rms_norm_eps == 1e-6
    assert d.tie_word_embeddings is False and d.rope_theta == 10000.0 and d.eos_token_ids == []
    assert Qwen2Config.from_dict({**minimal, "rope_parameters": {"rope_theta": 5e5}}).rope_theta == 5e5
    assert Qwen2Config.from_dict({**minimal, "head_dim": 32}).head_dim == 32


def test_config_eos_merge_order():
    cfg = Qwen2Config.from_dict({**BASE, "eos_token_id": [7, 3]}, {"eos_token_id": [3, 9]})
    assert cfg.eos_token_ids == [3, 9, 7]
    assert Qwen2Config.from_dict({**BASE, "eos_token_id": 5}).eos_token_ids == [5]


@pytest.mark.parametrize("bad,match", [
    ({"use_sliding_window": True}, "sliding"), ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"num_key_value_heads": 3}, "multiple"),
    ({"hidden_size": 66}, "head_dim"), ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_config_refuses_what_it_does_not_implement(bad, match):
    with pytest.raises(ConfigError, match=match):
        Qwen2Config.from_dict({**BASE, **bad})


def test_config_missing_key():
    raw = dict(BASE)
    del raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        Qwen2Config.from_dict(raw)


def test_config_round_trip():
    cfg = Qwen2Config.from_dict(named_config("tiny-b"))
    assert Qwen2Config.from_dict(cfg.to_dict()) == cfg


def test_registry():
    assert "Qwen2ForCausalLM" in architecture_names()
    with pytest.raises(RegistryError, match="Qwen2ForCausalLM"):
        get_architecture("NoSuchModel")
    with pytest.raises(RegistryError, match="gqa_attention"):
        get_part("mixer", "nope")
    assert get_part("norm", "rmsnorm").__name__ == "RMSNorm"


def test_engine_flags_follow_the_reference_names():
    import argparse

    ap = add_engine_args(argparse.ArgumentParser())
    args = ap.parse_args(["--model", "m", "--dtype", "float32", "--block-size", "8", "--kv-cache-mb", "4",
                          "--max-model-len", "256", "--max-num-seqs", "7", "--max-num-batched-tokens", "99",
                          "--watermark", "0.0", "--enable-prefix-caching", "--enable-chunked-prefill",
                          "--cuda-graphs", "--seed", "3", "--gpu-memory-utilization", "0.5", "--debug-steps"])
    cfg = engine_config_from_args(args)
    assert cfg == EngineConfig(model="m", dtype="float32", block_size=8, kv_cache_mb=4.0, max_model_len=256,
                               max_num_seqs=7, max_num_batched_tokens=99, watermark=0.0, enable_prefix_caching=True,
                               enable_chunked_prefill=True, cuda_graphs=True, seed=3, gpu_memory_utilization=0.5,
                               debug_steps=True)
    assert ap.parse_args(["--max-batched-tokens", "5"]).max_num_batched_tokens == 5
    with pytest.raises(ValueError):
        EngineConfig(dtype="float16")


def _specs(folder):
    spec, _ = read_spec(folder)
    return spec, DecoderModel(spec, torch.float32, torch.device("cpu"))


def test_random_weights_are_reproducible_and_load(tmp_path):
    a = write_random_model(tmp_path / "a", named_config("tiny-b"), seed=1)
    b = write_random_model(tmp_path / "b", named_config("tiny-b"), seed=1)
    c = write_random_model(tmp_path / "c", named_config("tiny-b"), seed=2)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    spec, model = _specs(a)
    t = load_tensors(a, model.weight_specs(), torch.bfloat16, torch.device("cpu"))
    assert t["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert t["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32      # small vectors stay 32-bit
    assert t["model.norm.weight"].dtype == torch.float32
    assert abs(float(t["model.norm.weight"].mean()) - 1.0) < 0.02
    assert 0.015 < float(t["model.embed_tokens.weight"].float().std()) < 0.025
    assert "lm_head.weight" in t                                                   # untied
    t32 = load_tensors(a, model.weight_specs(), torch.float32, torch.device("cpu"))
    assert t32["model.embed_tokens.weight"].dtype == torch.float32
    assert torch.equal(t32["model.embed_tokens.weight"], t["model.embed_tokens.weight"].float())
    model.bind(t32)
    assert model.blocks[0].mixer.w_qkv.shape == (3 * 32 + 2 * 32, 96)
    assert model.output_weight is t32["lm_head.weight"]


def test_tied_output_is_the_embedding(tmp_path):
    d = write_random_model(tmp_path / "a", named_config("tiny-a"), seed=0)
    spec, model = _specs(d)
    t = load_tensors(d, model.weight_specs(), torch.float32, torch.device("cpu"), spec.ignored_name_patterns)
    model.bind(t)
    assert model.output_weight is model.embedding and "lm_head.weight" not in t


def test_weight_errors_are_listed_together(tmp_path):
    from safetensors import safe_open
    from safetensors.torch import save_file

    d = write_random_model(tmp_path / "a", named_config("tiny-a"), seed=0)
    with safe_open(d / "model.safetensors", "pt") as f:
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.layers.0.self_attn.k_proj.bias"]
    tensors["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 100, dtype=torch.bfloat16)
    tensors["model.layers.9.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)      # ignorable by name
    tensors["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)        # ignorable when tied
    save_file(tensors, str(d / "model.safetensors"))
    spec, model = _specs(d)
    with pytest.raises(WeightError) as err:
        load_tensors(d, model.weight_specs(), torch.float32, torch.device("cpu"), spec.ignored_name_patterns)
    e = err.value
    assert e.missing == ["model.layers.0.self_attn.k_proj.bias", "model.layers.1.mlp.up_proj.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert [(n, tuple(g), tuple(w)) for n, g, w in e.wrong_shape] == \
        [("model.layers.0.mlp.down_proj.weight", (64, 100), (64, 128))]
    msg = str(e)
    assert "missing" in msg and "unexpected" in msg and "wrong shapes" in msg and "[64, 100]" in msg


def test_no_safetensors_and_unknown_architecture(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(named_config("tiny-a")))
    spec, model = _specs(tmp_path)
    with pytest.raises(FileNotFoundError):
        load_tensors(tmp_path, model.weight_specs(), torch.float32, torch.device("cpu"))
    (tmp_path / "config.json").write_text(json.dumps({**named_config("tiny-a"), "architectures": ["Other"]}))
    with pytest.raises(RegistryError, match="Other"):
        read_spec(tmp_path)


def test_limit_positions_sizes_the_tables(tmp_path):
    """The engine's own limit reaches the position tables through the parts' hooks, and the model reports the
    shortest table as the longest sequence it serves."""
    from tokenmill_b200.parts.model import DecoderModel
    d = write_random_model(tmp_path / "a", named_config("tiny-a"), seed=0)
    spec, _ = read_spec(d)
    model = DecoderModel(spec, torch.float32, torch.device("cpu"))
    assert model.max_positions() == spec.max_positions == 1024
    model.limit_positions(100)
    assert model.max_positions() == 100
    assert all(b.mixer.position.max_positions == 100 for b in model.blocks)
    model.limit_positions(10 ** 9)                     # a larger limit never grows the tables
    assert model.max_positions() == 100
    model.bind({w.name: torch.zeros(w.shape) for w in model.weight_specs()})
    assert model.blocks[0].mixer.cos.shape == (100, spec.layers[0].mixer.params["head_dim"] // 2)
    assert model.activation_bytes(10) > 10 * spec.hidden_size * 8


def test_cache_layout_groups_layers_and_shared_caches():
    from tokenmill_b200.models.qwen2 import qwen2_spec
    from tokenmill_b200.parts.spec import PartSpec, RunEntry
    from dataclasses import replace

    spec = qwen2_spec(Qwen2Config.from_dict(named_config("tiny-b")))
    # layer 1 gets a window: a second group; layer 2 runs twice, its second run reads entry 0's cache
    windowed = PartSpec(spec.layers[1].mixer.kind, {**spec.layers[1].mixer.params, "window": 24})
    layers = [spec.layers[0], replace(spec.layers[1], mixer=windowed), spec.layers[2]]
    spec2 = replace(spec, layers=layers, run_order=[RunEntry(0), RunEntry(1), RunEntry(2), RunEntry(2, cache_of=0)])
    model = DecoderModel(spec2, torch.float32, torch.device("cpu"))
    lay = model.cache_layout()
    assert [g.need.window for g in lay.groups] == [None, 24]
    assert [g.entries for g in lay.groups] == [[0, 2], [1]]
    assert lay.entry_group == {0: (0, 0), 1: (1, 0), 2: (0, 1), 3: (0, 0)}
    with pytest.raises(ValueError, match="earlier"):
        replace(spec, run_order=[RunEntry(0, cache_of=1), RunEntry(1)]).validate()
