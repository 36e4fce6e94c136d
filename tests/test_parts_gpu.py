"""Each part alone on the GPU against its plain function, at sizes of its own: norm, position tables,
attention mixer (whole prompt, then a later portion, then one token, through a small paged cache),
feed-forward and the pre-norm block; plus a layer order that runs a layer twice and shares a cache."""

from __future__ import annotations

from dataclasses import replace

import pytest
import torch

from plain_qwen2 import (plain_attention_block, plain_decoder_layer, plain_embedding, plain_rmsnorm,
                         plain_rope_tables, plain_swiglu)

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, ref):
    return (3e-5 if dtype == torch.float32 else 2e-2) * float(ref.abs().max())


def rand_weights(part, seed, dtype):
    """{name: tensor} for a part's declared tensors: (device tensors in their held dtype, float32 CPU copies
    of the values the device sees)."""
    g = torch.Generator().manual_seed(seed)
    dev, cpu = {}, {}
    for s in part.weight_specs():
        t = 0.1 * torch.randn(s.shape, generator=g) + (1.0 if s.init[0] == "ones_plus_normal" else 0.0)
        held = t.to(dtype if s.dtype == "compute" else torch.float32)
        dev[s.name], cpu[s.name] = held.to(DEV), held.float()
    return dev, cpu


def step_for(cache, entries, parts=()):
    """The step's inputs with the metadata the given parts ask for, and a workspace for their scratch."""
    from tokenmill_b200.engine.batch import build_step_inputs, metadata_providers
    from tokenmill_b200.engine.workspace import Workspace
    return build_step_inputs(entries, cache, DEV, metadata_providers(parts), workspace=Workspace(DEV))


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    from tokenmill_b200.parts.norm import RMSNorm
    part = RMSNorm(hidden_size=104, eps=3e-5, dtype=dtype, device=DEV)
    dev, cpu = rand_weights(part, 1, dtype)
    part.bind(dev)
    x = torch.randn(6, 104)
    out = part.forward(x.to(DEV).clone())
    ref = plain_rmsnorm(x, cpu["weight"], 3e-5)
    assert out.dtype == dtype and (out.float().cpu() - ref).abs().max() <= tol(dtype, ref)


def test_rotary_tables_equal_the_plain_tables():
    from tokenmill_b200.parts.rope import RotaryEmbedding
    for D, theta in [(16, 1e4), (64, 1e6), (80, 5e5)]:
        cos, sin = RotaryEmbedding(head_dim=D, theta=theta, max_positions=700).tables(DEV)
        pc, ps = plain_rope_tables(700, D, theta)
        assert torch.equal(cos.cpu(), pc[:, :D // 2]) and torch.equal(sin.cpu(), ps[:, :D // 2])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,nh,nkv,D,page", [(40, 6, 2, 16, 4), (72, 7, 1, 32, 16), (128, 4, 4, 48, 8)])
def test_attention_mixer_through_the_cache(dtype, H, nh, nkv, D, page):
    from tokenmill_b200.cache import CacheManager
    from tokenmill_b200.engine.batch import StepEntry
    from tokenmill_b200.parts.attention import GroupedQueryAttention
    from tokenmill_b200.parts.base import LayerCache
    from tokenmill_b200.parts.spec import PartSpec

    rope = PartSpec("rope", {"head_dim": D, "theta": 1e4, "max_positions": 512})
    mixer = GroupedQueryAttention(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=D, qkv_bias=True,
                                  position=rope, dtype=dtype, device=DEV)
    dev, cpu = rand_weights(mixer, 7, dtype)
    mixer.bind(dev)
    n = 45
    x = torch.randn(n, H, generator=torch.Generator().manual_seed(2)).to(dtype)
    cfg = {"heads": nh, "kv_heads": nkv, "head_dim": D}
    cos, sin = plain_rope_tables(n, D, 1e4)
    ref = plain_attention_block(x.float(), {f"p.{k}": v for k, v in cpu.items()}, "p", cfg, cos, sin)

    cache = CacheManager(16, page, watermark=0.0)
    pool_k = torch.randn(16, page, nkv, D, device=DEV).to(dtype)          # stale noise
    pool_v = torch.randn(16, page, nkv, D, device=DEV).to(dtype)
    lc = LayerCache(k=pool_k, v=pool_v, group=0)
    h = cache.new_handle()
    cache.allocate(h, list(range(n)))
    outs = []
    for start, size in [(0, 30), (30, 14), (44, 1)]:                       # whole part, later portion, one token
        step = step_for(cache, [StepEntry(h, list(range(size)), start)], [mixer])
        outs.append(mixer.forward(x[start:start + size].to(DEV), step, lc))
    got = torch.cat(outs).float().cpu()
    assert (got - ref).abs().max() <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    from tokenmill_b200.parts.swiglu import SwiGLUFeedForward
    part = SwiGLUFeedForward(hidden_size=56, intermediate_size=150, dtype=dtype, device=DEV)
    dev, cpu = rand_weights(part, 3, dtype)
    part.bind(dev)
    x = torch.randn(9, 56).to(dtype)
    ref = plain_swiglu(x.float(), {f"p.{k}": v for k, v in cpu.items()}, "p")
    out = part.forward(x.to(DEV))
    assert (out.float().cpu() - ref).abs().max() <= tol(dtype, ref)


def _model_from(spec, dtype, seed):
    from tokenmill_b200.parts.model import DecoderModel
    from tokenmill_b200.weights.random_init import random_tensors
    model = DecoderModel(spec, dtype, DEV)
    stored = random_tensors(model, seed, torch.bfloat16)
    held = {}
    for s in model.weight_specs():
        held[s.name] = stored[s.name].to(DEV, dtype if s.dtype == "compute" else torch.float32)
    model.bind(held)
    return model, {k: v.float() for k, v in stored.items()}


@pytest.mark.parametrize("wide_heads", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
def test_run_order_runs_a_layer_twice_and_shares_a_cache(dtype, wide_heads):
    """Layers 0, 1, 1 again (a cache of its own), then 0 again reading the first run's cache: the plain
    model is the same walk, the shared-cache run attending over the first run's keys and values. With heads of
    64 the bfloat16 prompt portion runs as a step program (an entry that reads another's cache writes none)."""
    from tokenmill_b200.cache import CacheManager
    from tokenmill_b200.cache.pool import CachePools
    from tokenmill_b200.config import Qwen2Config
    from tokenmill_b200.engine.batch import StepEntry
    from tokenmill_b200.engine.runner import ModelRunner
    from tokenmill_b200.models.qwen2 import qwen2_spec
    from tokenmill_b200.parts.spec import RunEntry
    from tokenmill_b200.weights import named_config
    from plain_qwen2 import plain_apply_rope, plain_causal_attention, plain_qkv

    raw = {**named_config("tiny-a"), "num_hidden_layers": 2, "max_position_embeddings": 256}
    nh, nkv, D = 4, 2, 16
    if wide_heads:
        nh, nkv, D = 2, 1, 64
        raw.update(hidden_size=128, num_attention_heads=nh, num_key_value_heads=nkv, head_dim=D)
    spec = qwen2_spec(Qwen2Config.from_dict(raw))
    spec = replace(spec, run_order=[RunEntry(0), RunEntry(1), RunEntry(1), RunEntry(0, cache_of=0)])
    model, w = _model_from(spec, dtype, seed=4)
    layout = model.cache_layout()
    assert [g.entries for g in layout.groups] == [[0, 1, 2]]
    cache = CacheManager(12, 16, watermark=0.0)
    pools = CachePools(layout, [12], 16, dtype, DEV, run_order_cache_of=[e.cache_of for e in spec.run_order])
    runner = ModelRunner(model, cache, pools, max_model_len=256)
    ids = torch.randint(0, 256, (50,), generator=torch.Generator().manual_seed(1)).tolist()
    h = cache.new_handle()
    cache.allocate(h, ids)
    got = torch.cat([runner.step([StepEntry(h, ids[a:b], a, list(range(b - a)))]) for a, b in [(0, 33), (33, 49), (49, 50)]])

    assert runner.stats["program_steps"] == (3 if wide_heads and dtype == torch.bfloat16 else 0)    # every step
    cfg = {"heads": nh, "kv_heads": nkv, "head_dim": D, "eps": raw["rms_norm_eps"], "layers": 2}
    cos, sin = plain_rope_tables(50, D, raw["rope_theta"])
    x = plain_embedding(ids, w["model.embed_tokens.weight"])
    first_kv = None
    for entry in spec.run_order:
        p = f"model.layers.{entry.layer}"
        if entry.cache_of is None:
            if first_kv is None:
                normed = plain_rmsnorm(x, w[f"{p}.input_layernorm.weight"], cfg["eps"])
                _, k, v = plain_qkv(normed, w, f"{p}.self_attn", cfg)
                first_kv = (plain_apply_rope(k, cos, sin, range(50)), v)
            x = plain_decoder_layer(x, w, entry.layer, cfg, cos, sin)
        else:
            normed = plain_rmsnorm(x, w[f"{p}.input_layernorm.weight"], cfg["eps"])
            q, _, _ = plain_qkv(normed, w, f"{p}.self_attn", cfg)
            q = plain_apply_rope(q, cos, sin, range(50))
            att = plain_causal_attention(q, first_kv[0], first_kv[1], D ** -0.5)
            x = x + att.reshape(50, nh * D) @ w[f"{p}.self_attn.o_proj.weight"].T
            x = x + plain_swiglu(plain_rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], cfg["eps"]), w, f"{p}.mlp")
    ref = plain_rmsnorm(x, w["model.norm.weight"], cfg["eps"]) @ w["model.embed_tokens.weight"].T
    assert (got.cpu() - ref).abs().max() <= tol(dtype, ref)
    cache.free(h)
    assert cache.all_free


@pytest.mark.parametrize("case", ["tiny-one-layer", "wide-one-layer", "wide-all-layers"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_windowed_mixers_through_the_runner(dtype, case):
    """Attention with a window of 40 keys in one layer (a cache group of its own beside the full-attention
    layer's) or in every layer (one group; with heads of 64 in bfloat16 the tcgen05 prompt kernel, the step
    program and the whole-step decode kernel all see the window): prompt portions, then tokens one by one, with
    the pages behind the window given back after every step, against the plain walk with the same window."""
    from tokenmill_b200.cache import CacheManager
    from tokenmill_b200.cache.pool import CachePools
    from tokenmill_b200.config import Qwen2Config
    from tokenmill_b200.engine.batch import StepEntry
    from tokenmill_b200.engine.runner import ModelRunner
    from tokenmill_b200.models.qwen2 import qwen2_spec
    from tokenmill_b200.weights import named_config

    W, n = 40, 150
    raw = {**named_config("tiny-a"), "num_hidden_layers": 2, "max_position_embeddings": 256}
    nh, nkv, D = 4, 2, 16
    if case.startswith("wide"):
        nh, nkv, D = 2, 1, 64
        raw.update(hidden_size=128, num_attention_heads=nh, num_key_value_heads=nkv, head_dim=D)
    spec = qwen2_spec(Qwen2Config.from_dict(raw))
    windowed = [0, 1] if case.endswith("all-layers") else [1]
    layers = [replace(l, mixer=replace(l.mixer, params={**l.mixer.params, "window": W})) if i in windowed else l
              for i, l in enumerate(spec.layers)]
    spec = replace(spec, layers=layers)
    model, w = _model_from(spec, dtype, seed=9)
    layout = model.cache_layout()
    assert len(layout.groups) == (1 if case.endswith("all-layers") else 2)
    pages = [14] * len(layout.groups)
    cache = CacheManager(pages, 16, windows=[g.need.window for g in layout.groups], watermark=0.0)
    pools = CachePools(layout, pages, 16, dtype, DEV, run_order_cache_of=[e.cache_of for e in spec.run_order])
    runner = ModelRunner(model, cache, pools, max_model_len=256)
    ids = torch.randint(0, 256, (n,), generator=torch.Generator().manual_seed(2)).tolist()
    h = cache.new_handle()
    cache.allocate(h, ids)
    cuts = [(0, 70), (70, 101)] + [(i, i + 1) for i in range(101, n)]
    got, freed = [], 0
    for a, b in cuts:
        got.append(runner.step([StepEntry(h, ids[a:b], a, list(range(b - a)))]))
        freed += cache.release_behind_window(h, b)
    got = torch.cat(got)
    assert freed >= (n - W) // 16 - 1              # the windowed group gave its old pages back on the way
    if case == "wide-all-layers" and dtype == torch.bfloat16:
        assert runner.fused is not None and runner.stats["fused_steps"] == n - 101 and runner.stats["program_steps"] == 2

    cfg = {"heads": nh, "kv_heads": nkv, "head_dim": D, "eps": raw["rms_norm_eps"], "layers": 2}
    cos, sin = plain_rope_tables(n, D, raw["rope_theta"])
    x = plain_embedding(ids, w["model.embed_tokens.weight"])
    for i in range(2):
        p = f"model.layers.{i}"
        x = x + plain_attention_block(plain_rmsnorm(x, w[f"{p}.input_layernorm.weight"], cfg["eps"]), w,
                                      f"{p}.self_attn", cfg, cos, sin, window=W if i in windowed else None)
        x = x + plain_swiglu(plain_rmsnorm(x, w[f"{p}.post_attention_layernorm.weight"], cfg["eps"]), w, f"{p}.mlp")
    ref = plain_rmsnorm(x, w["model.norm.weight"], cfg["eps"]) @ w["model.embed_tokens.weight"].T
    assert (got.cpu() - ref).abs().max() <= tol(dtype, ref)
    cache.free(h)
    assert cache.all_free


@pytest.mark.parametrize("dtype", DTYPES)
def test_layers_with_different_mixers_and_feed_forwards(dtype):
    """One model, three layers that differ: 2 query heads over 1 kv head, then 2 over 2 (another group size and
    another cache group), then 2 over 1 with a feed-forward twice as wide. Each part takes its sizes from its own
    parameters; in bfloat16 (heads of 64) the step program holds all three."""
    from tokenmill_b200.cache import CacheManager
    from tokenmill_b200.cache.pool import CachePools
    from tokenmill_b200.config import Qwen2Config
    from tokenmill_b200.engine.batch import StepEntry
    from tokenmill_b200.engine.runner import ModelRunner
    from tokenmill_b200.models.qwen2 import qwen2_spec
    from tokenmill_b200.weights import named_config

    raw = {**named_config("tiny-a"), "num_hidden_layers": 3, "max_position_embeddings": 256, "hidden_size": 128,
           "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 64, "intermediate_size": 136}
    spec = qwen2_spec(Qwen2Config.from_dict(raw))
    kv_heads, inter = [1, 2, 1], [136, 136, 272]
    layers = [replace(l, mixer=replace(l.mixer, params={**l.mixer.params, "num_kv_heads": kv_heads[i]}),
                      feed_forward=replace(l.feed_forward, params={**l.feed_forward.params, "intermediate_size": inter[i]}))
              for i, l in enumerate(spec.layers)]
    spec = replace(spec, layers=layers)
    model, w = _model_from(spec, dtype, seed=12)
    layout = model.cache_layout()
    assert [g.entries for g in layout.groups] == [[0, 2], [1]]
    cache = CacheManager([8, 8], 16, windows=[None, None], watermark=0.0)
    pools = CachePools(layout, [8, 8], 16, dtype, DEV, run_order_cache_of=[e.cache_of for e in spec.run_order])
    runner = ModelRunner(model, cache, pools, max_model_len=256)
    assert runner.fused is None                      # the whole-step kernel wants every layer alike
    ids = torch.randint(0, 256, (90,), generator=torch.Generator().manual_seed(4)).tolist()
    h = cache.new_handle()
    cache.allocate(h, ids)
    got = torch.cat([runner.step([StepEntry(h, ids[a:b], a, list(range(b - a)))])
                     for a, b in [(0, 41), (41, 80), (80, 82)] + [(i, i + 1) for i in range(82, 90)]])
    assert runner.stats["program_steps"] == (11 if dtype == torch.bfloat16 else 0)    # every step: no whole-step kernel
    cos, sin = plain_rope_tables(90, 64, raw["rope_theta"])
    x = plain_embedding(ids, w["model.embed_tokens.weight"])
    for i in range(3):
        cfg = {"heads": 2, "kv_heads": kv_heads[i], "head_dim": 64, "eps": raw["rms_norm_eps"], "layers": 3}
        x = plain_decoder_layer(x, w, i, cfg, cos, sin)
    ref = plain_rmsnorm(x, w["model.norm.weight"], raw["rms_norm_eps"]) @ w["model.embed_tokens.weight"].T
    assert (got.cpu() - ref).abs().max() <= tol(dtype, ref)
    cache.free(h)
    assert cache.all_free
