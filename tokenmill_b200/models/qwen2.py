"""Qwen2 dense decoder as data: config.json -> ``ModelSpec``.

Pre-norm decoder with grouped-query attention (biased q/k/v, rotate-half position encoding), SwiGLU
feed-forward, RMSNorm, and an output matrix tied to the embedding or separate
(src/infer/model/qwen2.py:13-52, src/infer/model/layers.py:127-164). Checkpoint tensor names are the
ones the reference's loader maps (src/infer/model/loader.py:98-119); names containing "rotary_emb"
may be present and are not loaded (loader.py:117-118), and a stray ``lm_head.weight`` next to tied
embeddings is ignored (loader.py:82-83).
"""

from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..registry import register_architecture


def qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    rope = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                             "max_positions": cfg.max_position_embeddings})
    norm = PartSpec("rmsnorm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    mixer = PartSpec("gqa_attention", {
        "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
        "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "qkv_bias": cfg.attention_bias,
        "position": rope, "window": None, "scale": cfg.head_dim ** -0.5})
    ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size})
    layers = [LayerSpec(prefix=f"model.layers.{i}", block="pre_norm", mixer=mixer, feed_forward=ffn,
                        mixer_norm=norm, feed_forward_norm=norm) for i in range(cfg.num_hidden_layers)]
    ignored = ("rotary_emb",) + (("lm_head.weight",) if cfg.tie_word_embeddings else ())
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        embedding_name="model.embed_tokens.weight", layers=layers,
        run_order=[RunEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=norm, final_norm_prefix="model.norm",
        lm_head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        max_positions=cfg.max_position_embeddings, eos_token_ids=list(cfg.eos_token_ids),
        ignored_name_patterns=ignored)


register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict, qwen2_spec)
