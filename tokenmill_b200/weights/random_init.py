"""Random-weights mode: write a model folder (config.json, model.safetensors) from a configuration
and a seed.

The reference has no such mode in its package (its tests build tiny weights through another
library, tests/conftest.py:35-66). Here every tensor the model declares is drawn on the CPU from one
seeded generator, in the model's fixed declaration order: matrices and embeddings ~ N(0, std), norm
weights 1 + N(0, std), biases N(0, std), std = 0.02. The same seed gives the same file on any
machine, and the folder is loaded back through the ordinary loader.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..parts.model import DecoderModel
from ..registry import get_architecture

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(model: DecoderModel, seed: int, store_dtype: torch.dtype) -> dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu").manual_seed(int(seed))
    out: dict[str, torch.Tensor] = {}
    for spec in model.weight_specs():
        kind, std = spec.init
        if spec.dtype == "int32":
            out[spec.name] = torch.zeros(spec.shape, dtype=torch.int32)
            continue
        t = torch.empty(spec.shape, dtype=torch.float32).normal_(0.0, std, generator=gen)
        if kind == "ones_plus_normal":
            t += 1.0
        elif kind != "normal":
            raise ValueError(f"{spec.name}: unknown init rule {kind!r}")
        out[spec.name] = t.to(store_dtype).contiguous()
    return out


def write_random_model(folder: str | Path, config: dict, seed: int = 0, store_dtype: str = "bfloat16") -> Path:
    """``config`` is a config.json dictionary (it must name its architecture). Tensors are stored in
    ``store_dtype``; storing bfloat16 means a float32 run and a bfloat16 run see the same values."""
    from safetensors.torch import save_file

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    names = config.get("architectures") or []
    if not names:
        raise ValueError("the configuration names no architecture (key 'architectures')")
    arch = get_architecture(names[0])
    cfg = arch.config_from_dict(config, None)
    spec = arch.build_spec(cfg)
    model = DecoderModel(spec, torch.float32, torch.device("cpu"))      # declarations only; nothing runs
    tensors = random_tensors(model, seed, _STORE[store_dtype])
    (folder / "config.json").write_text(json.dumps(config, indent=1))
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt"})
    return folder


# Layer sizes of the configurations the benchmarks name (config.json keys).
def qwen2_config(*, vocab_size, hidden_size, intermediate_size, num_hidden_layers, num_attention_heads,
                 num_key_value_heads, rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
                 max_position_embeddings=32768, head_dim=None, eos_token_id=None) -> dict:
    cfg = {
        "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": vocab_size,
        "hidden_size": hidden_size, "intermediate_size": intermediate_size,
        "num_hidden_layers": num_hidden_layers, "num_attention_heads": num_attention_heads,
        "num_key_value_heads": num_key_value_heads, "max_position_embeddings": max_position_embeddings,
        "rope_theta": rope_theta, "rms_norm_eps": rms_norm_eps, "tie_word_embeddings": tie_word_embeddings,
        "hidden_act": "silu", "use_sliding_window": False, "torch_dtype": "bfloat16",
    }
    if head_dim is not None:
        cfg["head_dim"] = head_dim
    if eos_token_id is not None:
        cfg["eos_token_id"] = eos_token_id
    return cfg


NAMED_SIZES = {
    "qwen2.5-0.5b": dict(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
                         num_attention_heads=14, num_key_value_heads=2, tie_word_embeddings=True),
    "qwen2.5-1.5b": dict(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
                         num_attention_heads=12, num_key_value_heads=2, tie_word_embeddings=True),
    "qwen2.5-7b": dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                       num_attention_heads=28, num_key_value_heads=4, tie_word_embeddings=False),
    "tiny-a": dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, rope_theta=10000.0, rms_norm_eps=1e-6,
                   tie_word_embeddings=True, max_position_embeddings=1024),
    "tiny-b": dict(vocab_size=384, hidden_size=96, intermediate_size=160, num_hidden_layers=3,
                   num_attention_heads=3, num_key_value_heads=1, rope_theta=1000000.0, rms_norm_eps=1e-5,
                   tie_word_embeddings=False, max_position_embeddings=2048),
}


def named_config(name: str) -> dict:
    try:
        return qwen2_config(**NAMED_SIZES[name.lower()])
    except KeyError:
        raise ValueError(f"unknown size name {name!r}; known: {sorted(NAMED_SIZES)}") from None
