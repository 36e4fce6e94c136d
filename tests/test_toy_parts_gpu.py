"""Generality of the parts interface: a toy mixer with per-request state of its own, a toy
feed-forward with routing, and a toy position encoding are defined HERE, registered, built from a
model folder and stepped through the engine's own step function and cache manager, without a
change to any file of the framework. They are not models of anything."""

from __future__ import annotations

import json
from pathlib import Path

import pytest
import torch

from plain_qwen2 import (plain_apply_rope, plain_causal_attention, plain_embedding, plain_qkv,
                         plain_rmsnorm, plain_rope_tables, plain_swiglu)
from replay_util import make_requests, mixed_steps, portion_steps, run_trace, whole_steps

pytestmark = pytest.mark.gpu

H, V, DECAY = 48, 200, 0.75


class ToyStateMixer:
    """state_t = DECAY * state_{t-1} + x_t per request; out_t = state_t @ W^T. The state lives in the
    engine's per-request state slots between steps."""

    def __init__(self, *, hidden_size, dtype, device):
        self.H, self.dtype, self.device = hidden_size, dtype, device

    def weight_specs(self):
        from tokenmill_b200.parts.spec import WeightSpec
        return [WeightSpec("mix.weight", (self.H, self.H), init=("normal", 0.1))]

    def bind(self, tensors):
        self.w = tensors["mix.weight"]

    def cache_need(self):
        return None

    def state_need(self):
        from tokenmill_b200.parts.spec import StateNeed
        return StateNeed((self.H,), "float32")

    def forward(self, x, step, cache):
        out = torch.empty_like(x)
        slots = step.state_slots.tolist()
        pos = 0
        for s, n in enumerate(step.q_lens):
            state = cache.state[slots[s]]
            for t in range(n):
                state = DECAY * state + x[pos + t].float()
                out[pos + t] = (state @ self.w.float().T).to(x.dtype)
            cache.state[slots[s]] = state
            pos += n
        return out


class ToyRoutedFeedForward:
    """Two experts (plain matrices); the router's 32-bit logits pick one per token."""

    def __init__(self, *, hidden_size, dtype, device):
        self.H, self.dtype, self.device = hidden_size, dtype, device

    def weight_specs(self):
        from tokenmill_b200.parts.spec import WeightSpec
        return [WeightSpec("router.weight", (2, self.H), dtype="float32", init=("normal", 0.5)),
                WeightSpec("experts.0.weight", (self.H, self.H), init=("normal", 0.1)),
                WeightSpec("experts.1.weight", (self.H, self.H), init=("normal", 0.1))]

    def bind(self, tensors):
        self.router = tensors["router.weight"]
        self.experts = [tensors["experts.0.weight"], tensors["experts.1.weight"]]

    def forward(self, x, step=None):
        choice = (x.float() @ self.router.T).argmax(-1)
        out = torch.empty_like(x)
        for e, w in enumerate(self.experts):
            rows = choice == e
            out[rows] = (x[rows].float() @ w.float().T).to(x.dtype)
        return out


class ToyHalfSpeedRope:
    """Another position encoding behind the same interface: angles advance at half speed."""

    def __init__(self, *, head_dim, theta, max_positions):
        self.head_dim, self.theta, self.max_positions = head_dim, theta, max_positions

    def tables(self, device):
        inv = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.int64).float() / self.head_dim))
        ang = torch.outer(torch.arange(self.max_positions).float() * 0.5, inv)
        return ang.cos().to(device).contiguous(), ang.sin().to(device).contiguous()


def toy_spec(cfg: dict):
    from tokenmill_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
    norm = PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5})
    attn = PartSpec("gqa_attention", {"hidden_size": H, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16,
                                      "qkv_bias": True, "window": None,
                                      "position": PartSpec("toy_half_rope", {"head_dim": 16, "theta": 100.0,
                                                                             "max_positions": 512})})
    state = PartSpec("toy_state", {"hidden_size": H})
    dense = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 80})
    routed = PartSpec("toy_routed", {"hidden_size": H})
    layers = [LayerSpec("model.layers.0", "pre_norm", state, dense, norm, norm, mixer_name="mixer"),
              LayerSpec("model.layers.1", "pre_norm", attn, routed, norm, norm, feed_forward_name="moe")]
    return ModelSpec("ToyStateLM", H, V, "model.embed_tokens.weight", layers, [RunEntry(0), RunEntry(1), RunEntry(0)],
                     norm, "model.norm", "lm_head.weight", 512)


@pytest.fixture(scope="module")
def toy_dir(tmp_path_factory):
    from tokenmill_b200.registry import (register_architecture, register_feed_forward, register_mixer,
                                         register_position_encoding)
    from tokenmill_b200.weights import write_random_model
    register_mixer("toy_state", ToyStateMixer, replace=True)
    register_feed_forward("toy_routed", ToyRoutedFeedForward, replace=True)
    register_position_encoding("toy_half_rope", ToyHalfSpeedRope, replace=True)
    register_architecture("ToyStateLM", lambda raw, gen: raw, toy_spec, replace=True)
    folder = tmp_path_factory.mktemp("toy")
    write_random_model(folder, {"architectures": ["ToyStateLM"], "vocab_size": V}, seed=3)
    return folder


def plain_toy_logits(folder, ids):
    from safetensors import safe_open
    with safe_open(str(Path(folder) / "model.safetensors"), framework="pt") as f:
        w = {k: f.get_tensor(k).float() for k in f.keys()}
    n = len(ids)
    x = plain_embedding(ids, w["model.embed_tokens.weight"])

    def state_layer(x):
        normed = plain_rmsnorm(x, w["model.layers.0.input_layernorm.weight"], 1e-5)
        state, outs = torch.zeros(H), []
        for t in range(n):
            state = DECAY * state + normed[t]
            outs.append(state @ w["model.layers.0.mixer.mix.weight"].T)
        x = x + torch.stack(outs)
        return x + plain_swiglu(plain_rmsnorm(x, w["model.layers.0.post_attention_layernorm.weight"], 1e-5), w,
                                "model.layers.0.mlp")

    x = state_layer(x)
    p = "model.layers.1"
    cfg = {"heads": 3, "kv_heads": 1, "head_dim": 16}
    inv = 1.0 / (100.0 ** (torch.arange(0, 16, 2, dtype=torch.int64).float() / 16))
    ang = torch.outer(torch.arange(n).float() * 0.5, inv)
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    normed = plain_rmsnorm(x, w[f"{p}.input_layernorm.weight"], 1e-5)
    q, k, v = plain_qkv(normed, w, f"{p}.self_attn", cfg)
    q, k = plain_apply_rope(q, cos, sin, range(n)), plain_apply_rope(k, cos, sin, range(n))
    att = plain_causal_attention(q, k, v, 16 ** -0.5)
    x = x + att.reshape(n, 48) @ w[f"{p}.self_attn.o_proj.weight"].T
    normed = plain_rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], 1e-5)
    choice = (normed @ w[f"{p}.moe.router.weight"].T).argmax(-1)
    routed = torch.stack([normed[t] @ w[f"{p}.moe.experts.{int(choice[t])}.weight"].T for t in range(n)])
    x = state_layer(x + routed)
    return plain_rmsnorm(x, w["model.norm.weight"], 1e-5) @ w["lm_head.weight"].T


@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_toy_parts_register_build_and_step(toy_dir, mode, tmp_path):
    """The third run-order entry runs layer 0 a second time: its state is a slot of its own."""
    reqs = make_requests(V, [40, 75, 23, 90, 31], seed=5)
    steps, max_tokens = {"whole": lambda: whole_steps(reqs), "portions": lambda: portion_steps(reqs, 2),
                         "mixed": lambda: mixed_steps(reqs, 4)}[mode]()
    outputs = run_trace(toy_dir, "float32", steps, max_tokens, tmp_path / "o")
    plain = {rid: plain_toy_logits(toy_dir, t) for rid, t in reqs.items()}
    fed = {rid: 0 for rid in reqs}
    for s in steps:
        row = 0
        for e in s["entries"]:
            for wpos in e["want"]:
                got = torch.from_numpy(outputs[s["step"]][row])
                ref = plain[e["id"]][fed[e["id"]] + wpos]
                assert (got - ref).abs().max() <= 1e-4 * float(ref.abs().max()), (s["step"], e["id"], wpos)
                row += 1
            fed[e["id"]] += len(e["tokens"])
