"""Generality of the parts interface. Defined HERE, registered, built from a model folder and run through
the engine's own step function, cache manager, scheduler and decode graphs, without a change to any file of
the framework:

* a mixer with per-request state of its own that also asks for per-step arrays of its own (the offset of every
  token inside its portion, the last row of every request) through ``step_metadata``;
* a feed-forward with routing;
* a rotary position encoding with other angles (tables), and an encoding that is not a rotation at all and
  brings its own ``apply`` (no tables);
* an architecture that runs one layer twice.

They are not models of anything."""

from __future__ import annotations

import random
from pathlib import Path

import numpy as np
import pytest
import torch

from plain_qwen2 import (plain_apply_rope, plain_causal_attention, plain_embedding, plain_qkv,
                         plain_rmsnorm, plain_swiglu)
from replay_util import make_requests, mixed_steps, portion_steps, run_trace, whole_steps

pytestmark = pytest.mark.gpu

H, V, DECAY = 48, 200, 0.75
metadata_calls = {"step": 0, "graph": 0}


class ToyScanMixer:
    """state_t = DECAY * state_{t-1} + x_t per request; out_t = state_t @ W^T. The state lives in the engine's
    per-request state slots between steps. A portion of n tokens is one matrix product: with the offset j of
    every token inside its portion, state_j = DECAY^(j+1) * state_in + sum_{i<=j} DECAY^(j-i) x_i. The offsets
    and each request's last row come from this part's own ``step_metadata``; nothing is read back to the host,
    so the step can be captured in a graph."""

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

    def metadata_key(self):
        return "toy_scan"

    def step_metadata(self, shape):
        from tokenmill_b200.parts.base import StepMetadata
        metadata_calls["graph" if shape.for_graph else "step"] += 1
        q = shape.q_lens.astype(np.int64)
        first = np.cumsum(q) - q
        offset = np.arange(int(q.sum())) - np.repeat(first, q)
        return StepMetadata({"offset": offset.astype(np.int32), "last_row": (first + q - 1).astype(np.int32)},
                            {"rows": int(q.sum())}, constant_in_graph=False)

    def forward(self, x, step, cache):
        meta = step.meta["toy_scan"]
        off = meta.arrays["offset"].long()
        seq = step.seq_of_token.long()
        slots = step.state_slots.long()
        same = seq[:, None] == seq[None, :]
        gap = off[:, None] - off[None, :]
        mix = torch.pow(DECAY, gap.clamp(min=0).float()) * (same & (gap >= 0))       # (no host values: graph-safe)
        state_in = cache.state.index_select(0, slots).index_select(0, seq)           # [T, H]
        states = mix @ x.float() + torch.pow(DECAY, (off + 1).float())[:, None] * state_in
        cache.state.index_copy_(0, slots, states.index_select(0, meta.arrays["last_row"].long()))
        return (states @ self.w.float().T).to(x.dtype)


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
        first = ((x.float() @ self.router.T).argmax(-1) == 0)[:, None]
        y0, y1 = x.float() @ self.experts[0].float().T, x.float() @ self.experts[1].float().T
        return torch.where(first, y0, y1).to(x.dtype)


class ToyHalfSpeedRope:
    """Another position encoding behind the table interface: angles advance at half speed."""

    def __init__(self, *, head_dim, theta, max_positions):
        self.head_dim, self.theta, self.max_positions = head_dim, theta, max_positions

    def tables(self, device):
        inv = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.int64).float() / self.head_dim))
        ang = torch.outer(torch.arange(self.max_positions).float() * 0.5, inv)
        return ang.cos().to(device).contiguous(), ang.sin().to(device).contiguous()


def toy_gains(positions):
    """(gain of a query, gain of a key) at the given positions: what ToyGainEncoding multiplies by."""
    p = torch.as_tensor(positions).float()
    return 1.0 + 0.05 * (p % 5), 1.0 - 0.04 * (p % 7)


class ToyGainEncoding:
    """An encoding that is not a rotation: q and k are scaled by gains that depend on the position. It has no
    tables; the mixer hands it dense q and k to change in place before k goes to the cache."""

    def __init__(self, *, max_positions):
        self.max_positions = max_positions

    def limit_positions(self, n):
        self.max_positions = min(self.max_positions, n)

    def apply(self, q, k, positions):
        gq, gk = toy_gains(positions)
        q.mul_(gq.to(q.dtype)[:, None, None])
        k.mul_(gk.to(k.dtype)[:, None, None])


def toy_spec(cfg: dict):
    from tokenmill_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
    norm = PartSpec("rmsnorm", {"hidden_size": H, "eps": 1e-5})
    heads = {"hidden_size": H, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "qkv_bias": True, "window": None}
    attn = PartSpec("gqa_attention", {**heads, "position": PartSpec("toy_half_rope", {"head_dim": 16, "theta": 100.0,
                                                                                      "max_positions": 512})})
    gain_attn = PartSpec("gqa_attention", {**heads, "position": PartSpec("toy_gain", {"max_positions": 512})})
    state = PartSpec("toy_scan", {"hidden_size": H})
    dense = PartSpec("swiglu", {"hidden_size": H, "intermediate_size": 80})
    routed = PartSpec("toy_routed", {"hidden_size": H})
    layers = [LayerSpec("model.layers.0", "pre_norm", state, dense, norm, norm, mixer_name="mixer"),
              LayerSpec("model.layers.1", "pre_norm", attn, routed, norm, norm, feed_forward_name="moe"),
              LayerSpec("model.layers.2", "pre_norm", gain_attn, dense, norm, norm)]
    return ModelSpec("ToyStateLM", H, V, "model.embed_tokens.weight", layers,
                     [RunEntry(0), RunEntry(1), RunEntry(2), RunEntry(0)], norm, "model.norm", "lm_head.weight", 512)


@pytest.fixture(scope="module")
def toy_dir(tmp_path_factory):
    from tokenmill_b200.registry import (register_architecture, register_feed_forward, register_mixer,
                                         register_position_encoding)
    from tokenmill_b200.weights import write_random_model
    register_mixer("toy_scan", ToyScanMixer, replace=True)
    register_feed_forward("toy_routed", ToyRoutedFeedForward, replace=True)
    register_position_encoding("toy_half_rope", ToyHalfSpeedRope, replace=True)
    register_position_encoding("toy_gain", ToyGainEncoding, replace=True)
    register_architecture("ToyStateLM", lambda raw, gen: raw, toy_spec, replace=True)
    folder = tmp_path_factory.mktemp("toy")
    write_random_model(folder, {"architectures": ["ToyStateLM"], "vocab_size": V}, seed=3)
    return folder


_weights: dict[str, dict] = {}


def plain_toy_logits(folder, ids):
    """The toy architecture restated plainly: whole sequence, no cache, one loop per recurrence."""
    from safetensors import safe_open
    if str(folder) not in _weights:
        with safe_open(str(Path(folder) / "model.safetensors"), framework="pt") as f:
            _weights[str(folder)] = {k: f.get_tensor(k).float() for k in f.keys()}
    w = _weights[str(folder)]
    n = len(ids)
    x = plain_embedding(ids, w["model.embed_tokens.weight"])
    cfg = {"heads": 3, "kv_heads": 1, "head_dim": 16}

    def state_layer(x):
        normed = plain_rmsnorm(x, w["model.layers.0.input_layernorm.weight"], 1e-5)
        state, outs = torch.zeros(H), []
        for t in range(n):
            state = DECAY * state + normed[t]
            outs.append(state @ w["model.layers.0.mixer.mix.weight"].T)
        x = x + torch.stack(outs)
        return x + plain_swiglu(plain_rmsnorm(x, w["model.layers.0.post_attention_layernorm.weight"], 1e-5), w,
                                "model.layers.0.mlp")

    def attention(x, p, encode):
        normed = plain_rmsnorm(x, w[f"{p}.input_layernorm.weight"], 1e-5)
        q, k, v = plain_qkv(normed, w, f"{p}.self_attn", cfg)
        q, k = encode(q, k)
        att = plain_causal_attention(q, k, v, 16 ** -0.5)
        return x + att.reshape(n, 48) @ w[f"{p}.self_attn.o_proj.weight"].T

    def half_speed(q, k):
        inv = 1.0 / (100.0 ** (torch.arange(0, 16, 2, dtype=torch.int64).float() / 16))
        ang = torch.outer(torch.arange(n).float() * 0.5, inv)
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
        return plain_apply_rope(q, cos, sin, range(n)), plain_apply_rope(k, cos, sin, range(n))

    def gains(q, k):
        gq, gk = toy_gains(range(n))
        return q * gq[:, None, None], k * gk[:, None, None]

    x = state_layer(x)
    p = "model.layers.1"
    x = attention(x, p, half_speed)
    normed = plain_rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], 1e-5)
    choice = (normed @ w[f"{p}.moe.router.weight"].T).argmax(-1)
    x = x + torch.stack([normed[t] @ w[f"{p}.moe.experts.{int(choice[t])}.weight"].T for t in range(n)])
    p = "model.layers.2"
    x = attention(x, p, gains)
    x = x + plain_swiglu(plain_rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], 1e-5), w, f"{p}.mlp")
    x = state_layer(x)
    return plain_rmsnorm(x, w["model.norm.weight"], 1e-5) @ w["lm_head.weight"].T


@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_toy_parts_register_build_and_step(toy_dir, mode, tmp_path):
    """The fourth run-order entry runs layer 0 a second time: its state is a slot of its own."""
    reqs = make_requests(V, [40, 75, 23, 90, 31], seed=5)
    steps, max_tokens = {"whole": lambda: whole_steps(reqs), "portions": lambda: portion_steps(reqs, 2),
                         "mixed": lambda: mixed_steps(reqs, 4)}[mode]()
    before = metadata_calls["step"]
    outputs = run_trace(toy_dir, "float32", steps, max_tokens, tmp_path / "o")
    assert metadata_calls["step"] - before == len(steps)            # the part was asked once per step
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


@pytest.mark.parametrize("graphs,async_decode,chunked", [(True, True, False), (True, False, True), (False, True, False)])
def test_toy_state_through_the_engine(toy_dir, graphs, async_decode, chunked):
    """Fixed-size state through everything above the step function: admission (a state slot per request, zeroed
    when handed out), the scheduler, decode graphs whose padded rows must not touch a live request's slot,
    steps in flight, and a pool so small that requests are evicted and their state is rebuilt from nothing.
    The logits behind every generated token equal the plain restatement's on the request's own history."""
    from tokenmill_b200 import EngineConfig
    from tokenmill_b200.engine import LLMEngine
    from tokenmill_b200.sampling import SamplingParams

    rng = random.Random(7)
    prompts = [[rng.randrange(V) for _ in range(n)] for n in (9, 30, 17, 44, 5, 26, 12)]
    # 20 pages of 8 tokens in each of the two attention layers' pools: seven requests of up to 44 + 20 tokens do not fit
    per_token = 2 * 2 * 16 * 4
    eng = LLMEngine(EngineConfig(model=str(toy_dir), dtype="float32", block_size=8, max_model_len=128, max_num_seqs=5,
                                 kv_cache_mb=(20 * 8 + 1) * per_token / 2 ** 20, watermark=0.0, cuda_graphs=graphs,
                                 cuda_graph_max_batch=8, async_decode=async_decode, enable_chunked_prefill=chunked,
                                 max_num_batched_tokens=24 if chunked else 256))
    assert eng.cache.num_pages == [20] and eng.cache.state_slots.num_slots == 5
    rows: dict[str, list] = {}

    def tap(where, logits):
        cpu = logits.float().cpu()
        for (rid, pos), row in zip(where, cpu):
            rows.setdefault(rid, []).append((pos, row.clone()))

    eng.on_logits = tap
    before = dict(metadata_calls)
    reqs = [eng.add_request(f"t{i}", p, SamplingParams(max_tokens=20, ignore_eos=True)) for i, p in enumerate(prompts)]
    while eng.has_unfinished():
        eng.step()
    eng.drain()
    assert eng.cache.all_free and eng.scheduler.evictions > 0
    if graphs:
        assert eng.runner.stats["graph_steps"] > 0
        assert metadata_calls["graph"] > before["graph"]            # asked again at replays: its arrays are not constant
    compared = 0
    for i, (p, r) in enumerate(zip(prompts, reqs)):
        assert len(r.output_ids) == 20
        plain = plain_toy_logits(toy_dir, p + r.output_ids)
        for pos, row in rows[f"t{i}"]:
            ref = plain[pos]
            assert (row - ref).abs().max() <= 1e-4 * float(ref.abs().max()), (i, pos)
            assert int(row.argmax()) == r.output_ids[pos - len(p) + 1]
            compared += 1
    assert compared >= 7 * 20
