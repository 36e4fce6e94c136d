"""The engine through its Python entry point: greedy generation against the plain implementation,
every scheduling option giving the same tokens, preemption with a tiny pool, decode graphs, long
decoding, the first tokens of a sequence, seeded sampling."""

from __future__ import annotations

import json
import random
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from plain_qwen2 import load_plain, plain_greedy, plain_logits, tolerance
from replay_util import check_against_plain, make_requests, plain_for, run_trace, tail_decode_steps

pytestmark = pytest.mark.gpu

N_NEW = 12


def engine_for(model_dir, dtype="float32", **kw):
    from tokenmill_b200 import EngineConfig
    from tokenmill_b200.engine import LLMEngine
    base = dict(model=str(model_dir), dtype=dtype, kv_cache_mb=8, block_size=16, max_model_len=512,
                max_num_seqs=16, max_num_batched_tokens=512, watermark=0.0)
    base.update(kw)
    return LLMEngine(EngineConfig(**base))


def prompts_for(model_dir, lengths=(1, 2, 3, 5, 8, 17, 31, 40, 64, 3, 11, 90)):
    vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    rng = random.Random(0)
    return [[rng.randrange(vocab) for _ in range(n)] for n in lengths]


def greedy(n=N_NEW):
    from tokenmill_b200.sampling import SamplingParams
    return SamplingParams(max_tokens=n, ignore_eos=True)


class LogitTap:
    """Collects, through ``LLMEngine.on_logits``, the logits row behind every sampled token: by request id, a
    list of (position, row) in the order the steps produced them (a position recomputed after an eviction
    appears again)."""

    def __init__(self, eng):
        self.rows: dict[str, list[tuple[int, torch.Tensor]]] = {}
        eng.on_logits = self

    def __call__(self, where, logits):
        cpu = logits.float().cpu()
        assert cpu.shape[0] == len(where)
        for (rid, pos), row in zip(where, cpu):
            self.rows.setdefault(rid, []).append((pos, row.clone()))


def generate_tapped(eng, prompts, params):
    """``eng.generate`` with a tap on the logits; returns (outputs, tap); request i has the id ``t<i>``."""
    tap = LogitTap(eng)
    reqs = [eng.add_request(f"t{i}", p, params) for i, p in enumerate(prompts)]
    while eng.has_unfinished():
        eng.step()
    eng.drain()
    eng.on_logits = None
    return [r.output_ids for r in reqs], tap


def assert_logits_match_plain(model_dir, prompts, outs, tap, dtype):
    """Every logits row the engine sampled from equals the plain implementation's row at that position of
    the request's own history (prompt + what the engine generated), within the dtype's replay tolerance; and
    every token is the arg-max of the row it was sampled from. Returns the number of rows compared."""
    cfg, w = load_plain(model_dir)
    n = 0
    for i, (p, o) in enumerate(zip(prompts, outs)):
        plain = plain_logits(cfg, w, p + o)
        got = tap.rows.get(f"t{i}", [])
        assert len(got) >= len(o)
        for pos, row in got:
            if pos >= len(plain):          # a surplus step behind an unforeseen end: its token was thrown away
                continue
            ref = plain[pos]
            diff = float((row - ref).abs().max())
            assert diff <= tolerance(ref, dtype), (i, pos, diff, tolerance(ref, dtype))
            k = pos - (len(p) - 1)
            if k < len(o):
                assert int(row.argmax()) == o[k], (i, pos)
            n += 1
    return n


def assert_tokens_are_argmax_of_plain(model_dir, prompts, outs, dtype):
    """Each generated token is the plain implementation's arg-max given the same history, or, in bfloat16,
    within twice the dtype's logit tolerance of it (a near-tie). The engines that can be tapped are checked on
    their logits instead (``assert_logits_match_plain``)."""
    cfg, w = load_plain(model_dir)
    for p, o in zip(prompts, outs):
        logits = plain_logits(cfg, w, p + o)
        for i, tok in enumerate(o):
            row = logits[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= 2 * tolerance(row, dtype), (len(p), i, tok, int(row.argmax()))


@pytest.fixture(scope="module")
def baseline_tokens(tiny_dir):
    eng = engine_for(tiny_dir)
    prompts = prompts_for(tiny_dir)
    outs = eng.generate(prompts, greedy())
    assert eng.cache.all_free and not eng.scheduler.running
    return prompts, outs


def test_greedy_generation_equals_the_plain_implementation(tiny_dir, baseline_tokens):
    prompts, outs = baseline_tokens
    cfg, w = load_plain(tiny_dir)
    assert all(len(o) == N_NEW for o in outs)
    for p, o in list(zip(prompts, outs))[:6]:
        assert o == plain_greedy(cfg, w, p, N_NEW)
    assert_tokens_are_argmax_of_plain(tiny_dir, prompts, outs, "float32")


@pytest.mark.parametrize("kw", [
    dict(block_size=1), dict(block_size=8), dict(max_num_batched_tokens=40), dict(enable_prefix_caching=True),
    dict(enable_chunked_prefill=True, max_num_batched_tokens=16),
    dict(enable_chunked_prefill=True, max_num_batched_tokens=5, block_size=3),
    dict(enable_chunked_prefill=True, max_num_batched_tokens=24, enable_prefix_caching=True),
    dict(policy="decode_first", max_waiting_steps=2), dict(cuda_graphs=True), dict(max_num_seqs=3),
    dict(cuda_graphs=True, enable_chunked_prefill=True, max_num_batched_tokens=32, cuda_graph_max_batch=4),
], ids=["page1", "page8", "small_budget", "prefix", "chunked16", "chunked5_page3", "chunked+prefix", "decode_first",
        "graphs", "three_seats", "graphs+chunked"])
def test_every_scheduling_option_gives_the_same_tokens(tiny_dir, baseline_tokens, kw):
    prompts, outs = baseline_tokens
    eng = engine_for(tiny_dir, **kw)
    assert eng.generate(prompts, greedy()) == outs
    assert eng.cache.all_free and not eng.scheduler.running and not eng.scheduler.queue
    if kw.get("cuda_graphs"):
        assert eng.runner.stats["graph_steps"] > 0


@pytest.mark.parametrize("chunked", [False, True])
def test_preemption_with_a_tiny_pool_keeps_the_tokens(tiny_b_dir, chunked):
    eng = engine_for(tiny_b_dir)
    prompts = prompts_for(tiny_b_dir)
    outs = eng.generate(prompts, greedy(24))
    per_token = eng.model.cache_layout().bytes_per_token(4)
    small = engine_for(tiny_b_dir, block_size=4, kv_cache_mb=(34 * 4 + 1) * per_token / 2 ** 20,
                       enable_chunked_prefill=chunked, max_num_batched_tokens=12 if chunked else 512)
    assert small.cache.num_pages == [34]                    # far fewer than the 12 requests need at once
    assert small.generate(prompts, greedy(24)) == outs
    assert small.scheduler.evictions > 0 and small.cache.all_free


def test_prompt_that_never_fits_and_bad_requests(tiny_a_dir):
    from tokenmill_b200.engine import RequestRejected
    eng = engine_for(tiny_a_dir, block_size=4, kv_cache_mb=(8 * 4 + 1) * 512 / 2 ** 20)   # 8 pages of 4 tokens x 512 B
    assert eng.cache.num_pages == [8]
    with pytest.raises(RequestRejected, match="no tokens"):
        eng.add_request("e", [], greedy())
    with pytest.raises(RequestRejected, match="max_model_len"):
        eng.add_request("l", [1] * 512, greedy())
    with pytest.raises(RequestRejected, match="vocabulary"):
        eng.add_request("v", [10 ** 6], greedy())
    eng.add_request("big", [1] * 40, greedy())              # 10 pages: never fits
    eng.add_request("ok", [1, 2, 3], greedy(4))
    with pytest.raises(RequestRejected, match="already in use"):
        eng.add_request("ok", [1], greedy())
    seen = {}
    while eng.has_unfinished():
        for out in eng.step():
            seen.setdefault(out.request_id, []).append(out)
    assert seen["big"][0].finished and seen["big"][0].error and seen["big"][0].finish_reason == "length"
    assert sum(len(o.new_token_ids) for o in seen["ok"]) == 4 and seen["ok"][-1].finish_reason == "length"
    assert eng.cache.all_free


def test_stop_rules_and_abort(tiny_a_dir):
    from tokenmill_b200.sampling import SamplingParams
    eng = engine_for(tiny_a_dir, max_model_len=40)
    first = eng.generate([[5, 6, 7]], SamplingParams(max_tokens=6, ignore_eos=True))[0]
    eng.eos_ids = {first[2]}
    assert eng.generate([[5, 6, 7]], SamplingParams(max_tokens=6))[0] == first[:first.index(first[2]) + 1]
    assert eng.generate([[5, 6, 7]], SamplingParams(max_tokens=6, ignore_eos=True))[0] == first
    eng.eos_ids = set()
    assert len(eng.generate([[1] * 30], SamplingParams(max_tokens=64, ignore_eos=True))[0]) == 10   # max_model_len
    eng.add_request("x", [1, 2, 3, 4], greedy(50))
    eng.step()
    eng.step()
    out = eng.abort_request("x")
    assert out.finished and out.finish_reason == "abort" and eng.cache.all_free and not eng.has_unfinished()
    assert eng.abort_request("x") is None


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_bfloat16_and_float32_engines_follow_the_plain_argmax(tiny_b_dir, dtype):
    prompts = prompts_for(tiny_b_dir)
    eng = engine_for(tiny_b_dir, dtype=dtype, enable_chunked_prefill=True, max_num_batched_tokens=48, cuda_graphs=True)
    outs, tap = generate_tapped(eng, prompts, greedy())
    assert assert_logits_match_plain(tiny_b_dir, prompts, outs, tap, dtype) >= len(prompts) * N_NEW
    assert eng.model.embedding.dtype == (torch.float32 if dtype == "float32" else torch.bfloat16)
    assert eng.pools.kv[0].dtype == eng.model.embedding.dtype


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_crosses_pages_and_key_cuts(tiny_dir, dtype, tmp_path, plain_cache):
    """10 prompt tokens, then 600 tokens one by one: every page edge and the cuts at 256 and 512 keys."""
    vocab = json.loads((Path(tiny_dir) / "config.json").read_text())["vocab_size"]
    reqs = make_requests(vocab, [610], seed=21)
    steps, max_tokens = tail_decode_steps(reqs, tail=600)
    outputs = run_trace(tiny_dir, dtype, steps, max_tokens, tmp_path / "o")
    check_against_plain(steps, outputs, reqs, plain_for(tiny_dir, reqs, plain_cache), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(tiny_dir, dtype, tmp_path, plain_cache):
    """Positions 0, 1, 2: alone, as a whole, and one by one (no earlier key exists for the first)."""
    vocab = json.loads((Path(tiny_dir) / "config.json").read_text())["vocab_size"]
    reqs = make_requests(vocab, [1, 2, 3, 4], seed=8)
    steps = [{"step": i, "entries": [{"id": rid, "tokens": t, "want": list(range(len(t)))}], "end": [rid]}
             for i, (rid, t) in enumerate(reqs.items())]
    one_by_one = make_requests(vocab, [4], seed=9)
    toks = one_by_one["r0"]
    for p, t in enumerate(toks):
        steps.append({"step": 10 + p, "entries": [{"id": "s", "tokens": [t], "want": [0]}],
                      "end": ["s"] if p == len(toks) - 1 else []})
    all_reqs = {**reqs, "s": toks}
    outputs = run_trace(tiny_dir, dtype, steps, 64, tmp_path / "o")
    check_against_plain(steps, outputs, all_reqs, plain_for(tiny_dir, all_reqs, plain_cache), dtype)


def test_seeded_sampling_does_not_depend_on_batch_company(tiny_b_dir):
    from tokenmill_b200.sampling import SamplingParams
    prompts = prompts_for(tiny_b_dir)
    sp = SamplingParams(max_tokens=10, temperature=0.8, seed=7, ignore_eos=True)
    alone = engine_for(tiny_b_dir).generate([prompts[5]], sp)[0]
    plist = [greedy(10)] * len(prompts)
    plist[5] = sp
    plist[7] = SamplingParams(max_tokens=10, temperature=1.2, top_k=20, top_p=0.9, ignore_eos=True)
    eng = engine_for(tiny_b_dir, enable_chunked_prefill=True, max_num_batched_tokens=32)
    mixed = eng.generate(prompts, plist)
    assert mixed[5] == alone
    assert engine_for(tiny_b_dir).generate([prompts[5]], sp)[0] == alone                  # same seed, same stream
    other = engine_for(tiny_b_dir).generate([prompts[5]], SamplingParams(max_tokens=10, temperature=0.8, seed=8,
                                                                         ignore_eos=True))[0]
    assert other != alone
    greedy_ref = engine_for(tiny_b_dir).generate(prompts, greedy(10))
    assert [m for i, m in enumerate(mixed) if i not in (5, 7)] == [g for i, g in enumerate(greedy_ref) if i not in (5, 7)]
    # sampled tokens lie in the support the plain rules give (temperature 1.2, top-k 20, top-p 0.9)
    from plain_qwen2 import plain_filtered_probs
    cfg, w = load_plain(tiny_b_dir)
    logits = plain_logits(cfg, w, prompts[7] + mixed[7])
    for i, tok in enumerate(mixed[7]):
        probs = plain_filtered_probs(logits[len(prompts[7]) - 1 + i], 1.2, 20, 0.9)
        assert probs[tok] > 0 or float(probs.max()) > 0.999


def test_command_line_generates(tiny_a_dir):
    root = Path(__file__).resolve().parents[1]
    proc = subprocess.run([sys.executable, "-m", "tokenmill_b200.generate", "--model", str(tiny_a_dir), "--dtype",
                           "float32", "--kv-cache-mb", "4", "--max-model-len", "128", "--prompt-ids", "5,6,7",
                           "--prompt-ids", "9", "--max-tokens", "5", "--ignore-eos"],
                          capture_output=True, text=True, cwd=root, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    rows = [json.loads(line) for line in proc.stdout.splitlines() if line.startswith("{")]
    assert [r["prompt_ids"] for r in rows] == [[5, 6, 7], [9]] and all(len(r["output_ids"]) == 5 for r in rows)
    cfg, w = load_plain(tiny_a_dir)
    assert rows[0]["output_ids"] == plain_greedy(cfg, w, [5, 6, 7], 5)


@pytest.mark.parametrize("step_program", ["1", "0"])
@pytest.mark.parametrize("switch", ["1", "0"])
def test_prompt_attention_kernel_choice(tmp_path, monkeypatch, plain_cache, switch, step_program):
    """Heads of 64 in bfloat16 take the tcgen05 prompt-attention kernel (128-row tiles), and the mma.sync one
    when TOKENMILL_TC_ATTENTION=0; both agree with the plain implementation, also on portions cut anywhere and
    beside another request's decoded tokens. The same with the launches walked by a step program (the default)
    and made one by one from Python (TOKENMILL_STEP_PROGRAM=0)."""
    from tokenmill_b200.kernels import lib, program
    from tokenmill_b200.weights import qwen2_config, write_random_model
    cfg = qwen2_config(vocab_size=300, hidden_size=192, intermediate_size=264, num_hidden_layers=2,
                       num_attention_heads=3, num_key_value_heads=1, rope_theta=10000.0, tie_word_embeddings=False,
                       max_position_embeddings=1024)
    folder = write_random_model(tmp_path / "m", cfg, seed=6)
    monkeypatch.setenv("TOKENMILL_TC_ATTENTION", switch)
    monkeypatch.setenv("TOKENMILL_STEP_PROGRAM", step_program)
    calls = []
    real = lib.call
    monkeypatch.setattr(lib, "call", lambda name, *a: (calls.append(name), real(name, *a))[1])
    reqs = make_requests(300, [340, 150], seed=9)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"][:297], "want": list(range(0, 297, 5))}], "end": []},
             {"step": 1, "entries": [{"id": "r1", "tokens": reqs["r1"][:149], "want": [0, 148]},
                                     {"id": "r0", "tokens": reqs["r0"][297:299], "want": [0, 1]}], "end": []},
             {"step": 2, "entries": [{"id": "r0", "tokens": reqs["r0"][299:], "want": list(range(41))},
                                     {"id": "r1", "tokens": reqs["r1"][149:], "want": [0]}], "end": ["r0", "r1"]}]
    before = program.kind_launches()
    outputs = run_trace(folder, "bfloat16", steps, 512, tmp_path / "o")
    check_against_plain(steps, outputs, reqs, plain_for(folder, reqs, plain_cache), "bfloat16")
    used, other = ("prefill_attention_tc", "prefill_attention") if switch == "1" else ("prefill_attention", "prefill_attention_tc")
    if step_program == "1":
        issued = {k: v - before[k] for k, v in program.kind_launches().items()}
        assert issued[used] == 6 and issued[other] == 0 and issued["gemm_bf16"] == 3 * (4 * 2 + 1)
        assert calls.count("tm_program_run") == 3 and not any("attention" in c for c in calls)
    else:
        assert f"tm_{used}_bf16" in calls and f"tm_{other}_bf16" not in calls and "tm_program_run" not in calls


def test_prompt_products_on_tcgen05_when_switched_on(tmp_path, monkeypatch, plain_cache):
    """With TOKENMILL_TC_GEMM on, prompt steps of 128 tokens or more run the fused q/k/v projection, the
    gate/up projection with its SwiGLU epilogue and the down projection on the tcgen05 kernel; logits stay
    within the bfloat16 tolerance of the plain implementation, and decoding afterwards reads what it wrote."""
    from tokenmill_b200.kernels import lib, ops
    from tokenmill_b200.weights import qwen2_config, write_random_model
    cfg = qwen2_config(vocab_size=300, hidden_size=128, intermediate_size=264, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=1, rope_theta=10000.0, tie_word_embeddings=False,
                       max_position_embeddings=1024)
    folder = write_random_model(tmp_path / "m", cfg, seed=5)
    monkeypatch.setattr(ops, "_TC_MODE", "1")
    calls = []
    real = lib.call
    monkeypatch.setattr(lib, "call", lambda name, *a: (calls.append(name), real(name, *a))[1])
    reqs = make_requests(300, [330, 150], seed=4)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"][:300], "want": list(range(0, 300, 7))}], "end": []},
             {"step": 1, "entries": [{"id": "r1", "tokens": reqs["r1"][:140], "want": [139]},
                                     {"id": "r0", "tokens": reqs["r0"][300:310], "want": list(range(10))}], "end": []},
             {"step": 2, "entries": [{"id": "r0", "tokens": reqs["r0"][310:], "want": list(range(20))},
                                     {"id": "r1", "tokens": reqs["r1"][140:], "want": list(range(10))}], "end": ["r0", "r1"]}]
    outputs = run_trace(folder, "bfloat16", steps, 512, tmp_path / "o")
    check_against_plain(steps, outputs, reqs, plain_for(folder, reqs, plain_cache), "bfloat16")
    assert {"tm_tc_qkv_rope_write", "tm_tc_gate_up_swiglu", "tm_tc_linear"} <= set(calls)


def test_fused_qkv_and_narrow_products_on_tcgen05_inside_step_programs(d64_dir, tmp_path, monkeypatch, plain_cache):
    """TOKENMILL_TC_GEMM=qkv: in prompt steps long enough, the q/k/v projection runs as one tcgen05 kernel with bias,
    rotation and cache write in its epilogue (tiles of 128 columns: one wave) and the output projection on the same
    kernel, both as launches of the step program; shorter steps of the same program keep the library products. The
    logits are the plain implementation's, and decoding afterwards reads the keys that epilogue wrote."""
    from tokenmill_b200.kernels import ops, program
    monkeypatch.setattr(ops, "_TC_MODE", "qkv")
    vocab = json.loads((Path(d64_dir) / "config.json").read_text())["vocab_size"]
    reqs = make_requests(vocab, [1130, 420], seed=8)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"][:1100], "want": list(range(0, 1100, 37))}], "end": []},
             {"step": 1, "entries": [{"id": "r1", "tokens": reqs["r1"][:400], "want": [0, 399]},
                                     {"id": "r0", "tokens": reqs["r0"][1100:1110], "want": list(range(10))}], "end": []},
             {"step": 2, "entries": [{"id": "r0", "tokens": reqs["r0"][1110:], "want": list(range(20))},
                                     {"id": "r1", "tokens": reqs["r1"][400:], "want": list(range(20))}], "end": ["r0", "r1"]}]
    before = program.kind_launches()
    outputs = run_trace(d64_dir, "bfloat16", steps, 2048, tmp_path / "o")
    after = program.kind_launches()
    check_against_plain(steps, outputs, reqs, plain_for(d64_dir, reqs, plain_cache), "bfloat16")
    took = {k: after[k] - before[k] for k in after}
    # 3 layers: step 0 (1,100 tokens) takes both tcgen05 launches, step 1 (410 tokens) the fused projection only,
    # step 2 (40 tokens) neither
    assert took["tc_qkv_rope_write"] == 6 and took["tc_linear"] == 3 and took["qkv_rope_write"] == 3


@pytest.mark.parametrize("mode", ["tail", "mixed", "many", "tail-whole", "mixed-whole", "long-whole"])
def test_whole_step_decode_kernel_matches_plain(d64_dir, mode, tmp_path, plain_cache, monkeypatch):
    """Decode steps of at most 16 tokens run as ONE kernel (norms, projections, attention, feed-forward of
    every layer). Logits must match the plain implementation like every other path: one request decoded for
    300 steps across page edges; several requests decoding side by side while others still feed prompt
    portions; twelve requests decoding together (a request's keys are split across blocks, the partials merged by
    the last block to finish); the same with one block attending all keys of a request; and that with a
    context so long that a warp takes its keys in several rounds."""
    from tokenmill_b200.engine import runner as runner_mod
    from replay_util import mixed_steps
    made = []
    real = runner_mod.fused.FusedDecoder
    monkeypatch.setattr(runner_mod.fused, "FusedDecoder", lambda *a, **k: made.append(real(*a, **k)) or made[-1])
    if mode.endswith("whole"):       # one block attends all keys of a (request, kv head): no partials
        monkeypatch.setattr(real, "split_for", lambda self, n, kv: 4096)
    if mode.startswith("tail"):
        reqs = make_requests(500, [310], seed=2)
        steps, max_tokens = tail_decode_steps(reqs, tail=300)
    elif mode.startswith("long"):
        reqs = make_requests(500, [1000], seed=3)
        steps, max_tokens = tail_decode_steps(reqs, tail=40)
    elif mode.startswith("mixed"):
        reqs = make_requests(500, [70, 133, 45, 200, 96, 61], seed=11)
        steps, max_tokens = mixed_steps(reqs, seed=7, decode_tail=20)
    else:
        reqs = make_requests(500, [40 + 7 * i for i in range(12)], seed=5)
        steps = [{"step": 0, "entries": [{"id": r, "tokens": t[:-6], "want": [len(t) - 7]} for r, t in list(reqs.items())[:6]], "end": []},
                 {"step": 1, "entries": [{"id": r, "tokens": t[:-6], "want": [len(t) - 7]} for r, t in list(reqs.items())[6:]], "end": []}]
        for i in range(6):
            steps.append({"step": 2 + i, "entries": [{"id": r, "tokens": [t[len(t) - 6 + i]], "want": [0]} for r, t in reqs.items()],
                          "end": list(reqs) if i == 5 else []})
        max_tokens = sum(-(-len(t) // 64) * 64 for t in reqs.values())
    outputs = run_trace(d64_dir, "bfloat16", steps, max_tokens, tmp_path / "o")
    check_against_plain(steps, outputs, reqs, plain_for(d64_dir, reqs, plain_cache), "bfloat16")
    assert made and made[0].launches >= {"tail": 290, "tail-whole": 290, "long-whole": 36}.get(mode, 6)
    made[0].check()
    assert made[0].bar.item() == 0 and int(made[0].attn_count.abs().sum()) == 0      # left clean for the next launch


def test_whole_step_decode_kernel_through_the_engine(d64_dir):
    """Greedy generation with the whole-step kernel equals generation with it switched off, token for
    token where the plain logits are not a near-tie, and the engine reports which path ran."""
    from tokenmill_b200.kernels import fused
    prompts = prompts_for(d64_dir, lengths=(3, 17, 40, 5, 64, 9, 33, 12))
    eng = engine_for(d64_dir, dtype="bfloat16", max_model_len=512)
    outs, tap = generate_tapped(eng, prompts, greedy(40))
    assert eng.runner.stats["fused_steps"] >= 39 and eng.cache.all_free
    assert_logits_match_plain(d64_dir, prompts, outs, tap, "bfloat16")
    old = fused._ENABLED
    fused._ENABLED = False
    try:
        plain_path = engine_for(d64_dir, dtype="bfloat16", max_model_len=512)
        assert plain_path.runner.fused is None
        outs2, tap2 = generate_tapped(plain_path, prompts, greedy(40))
    finally:
        fused._ENABLED = old
    assert_logits_match_plain(d64_dir, prompts, outs2, tap2, "bfloat16")


def _run_requests(eng, prompts, params, abort_after=None):
    """Drive the step loop by hand; returns per request (token ids, finish reason, tokens seen in outputs)."""
    seqs = [eng.add_request(f"r{i}", p, sp) for i, (p, sp) in enumerate(zip(prompts, params))]
    seen = {s.id: [] for s in seqs}
    reasons = {}
    steps = 0
    while eng.has_unfinished():
        for o in eng.step():
            seen[o.request_id] += o.new_token_ids
            if o.finished:
                reasons[o.request_id] = o.finish_reason
                assert o.num_output_tokens == len(seen[o.request_id])
        steps += 1
        if abort_after and steps == abort_after[1]:
            out = eng.abort_request(abort_after[0])
            assert out is not None and out.finished and out.finish_reason == "abort"
            reasons[abort_after[0]] = "abort"
    eng.drain()
    assert eng.cache.all_free and not eng.scheduler.running
    return [(s.output_ids, reasons.get(s.id), seen[s.id]) for s in seqs]


def test_decode_steps_in_flight_give_the_synchronous_loop_s_results(d64_dir):
    """With one decode step in flight (tokens fed on the device, the host one step behind) every request gets
    the same tokens, stops for the same reason at the same place, and the outputs carry every token once:
    ends by max_tokens at different lengths, by an end-of-sequence token the host cannot foresee, seeded
    sampling, an abort while a step is in flight, and a request joining while others decode."""
    from tokenmill_b200.sampling import SamplingParams
    prompts = prompts_for(d64_dir, lengths=(3, 17, 40, 5, 64, 9))
    # pick an end-of-sequence token that the greedy run of request 2 produces in mid-stream
    probe = engine_for(d64_dir, dtype="bfloat16", async_decode=False)
    eos = probe.generate([prompts[2]], greedy(30))[0][11]
    params = [SamplingParams(max_tokens=7, ignore_eos=True), SamplingParams(max_tokens=1, ignore_eos=True),
              SamplingParams(max_tokens=40), SamplingParams(max_tokens=25, temperature=0.8, top_k=50, seed=11, ignore_eos=True),
              SamplingParams(max_tokens=33, temperature=1.1, top_p=0.9, seed=5, ignore_eos=True),
              SamplingParams(max_tokens=30, ignore_eos=True)]
    results = {}
    for mode in (False, True):
        eng = engine_for(d64_dir, dtype="bfloat16", async_decode=mode)
        eng.eos_ids = {eos}
        assert eng._pipelining() == mode
        results[mode] = _run_requests(eng, prompts, params, abort_after=("r5", 9))
        if mode:
            assert eng.runner.stats["fused_steps"] >= 30
    for (ids_s, why_s, seen_s), (ids_a, why_a, seen_a), sp in zip(results[False], results[True], params):
        if why_s == "abort":          # the abort lands one token apart, by construction; the common part agrees
            n = min(len(ids_s), len(ids_a))
            assert why_a == "abort" and ids_s[:n] == ids_a[:n] and -1 not in ids_a
            continue
        assert ids_s == ids_a and why_s == why_a and seen_s == ids_s and seen_a == ids_a
    assert results[False][2][1] == "stop" and results[False][2][0][-1] == eos and len(results[False][2][0]) <= 12
    assert [r[1] for r in results[False][:2]] == ["length", "length"]

    # a request that arrives while a step is in flight joins after that step; nobody's tokens change
    late = prompts_for(d64_dir, lengths=(21,))[0]
    outs = {}
    for mode in (False, True):
        eng = engine_for(d64_dir, dtype="bfloat16", async_decode=mode)
        seqs = [eng.add_request(f"a{i}", p, greedy(20)) for i, p in enumerate(prompts[:3])]
        for _ in range(6):
            eng.step()
        seqs.append(eng.add_request("late", late, greedy(10)))
        while eng.has_unfinished():
            eng.step()
        eng.drain()
        outs[mode] = [s.output_ids for s in seqs]
        assert eng.cache.all_free
    assert outs[False] == outs[True]


def test_decode_steps_in_flight_survive_preemption(d64_dir):
    """A pool so small that decoding preempts: the request thrown out while a step is in flight keeps the
    token that step chose for it, is recomputed later, and ends with the tokens of the synchronous loop."""
    prompts = prompts_for(d64_dir, lengths=(30, 33, 28, 35))
    outs = {}
    probe = engine_for(d64_dir, dtype="bfloat16")
    per_token = probe.model.cache_layout().bytes_per_token(2)
    for mode in (False, True):
        # 12 pages of 16 tokens: four requests of about 32 + 40 tokens (5 pages each) do not fit together
        eng = engine_for(d64_dir, dtype="bfloat16", async_decode=mode, max_model_len=128, max_num_seqs=4,
                         kv_cache_mb=(12 * 16 + 1) * per_token / 2 ** 20)
        assert eng.cache.num_pages == [12]
        outs[mode], tap = generate_tapped(eng, prompts, greedy(40))
        assert eng.scheduler.evictions > 0 and eng.cache.all_free
        # the logits behind every token, those of recomputed positions included, against the plain implementation
        assert assert_logits_match_plain(d64_dir, prompts, outs[mode], tap, "bfloat16") >= 4 * 40
    assert outs[False] == outs[True]


@pytest.mark.parametrize("batch", [1, 5, 8, 9, 13, 16])
def test_whole_step_kernel_at_model_sizes_equals_the_kernel_per_operation_path(wide_dir, batch, monkeypatch):
    """Same requests, same steps, through the whole-step kernel and through the separate kernels: the logits
    agree within bfloat16 rounding, at batch sizes on both sides of the 8-token staging limit (above it the
    kernel runs with a single ring stage)."""
    from tokenmill_b200.engine.batch import StepEntry
    from tokenmill_b200.kernels import fused
    rng = random.Random(batch)
    prompts = [[rng.randrange(1000) for _ in range(rng.randrange(300, 700))] for _ in range(batch)]
    nxt = [[rng.randrange(1000) for _ in range(batch)] for _ in range(4)]

    def run(use_fused):
        old = fused._ENABLED
        fused._ENABLED = use_fused
        # (the other path: launch by launch from Python, with the weight-streaming kernels for the decode steps)
        monkeypatch.setenv("TOKENMILL_STEP_PROGRAM", "1" if use_fused else "0")
        try:
            eng = engine_for(wide_dir, dtype="bfloat16", max_model_len=1024, max_num_seqs=16, kv_cache_mb=64,
                             max_num_batched_tokens=4096)
        finally:
            fused._ENABLED = old
        assert (eng.runner.fused is not None) == use_fused
        r, cache = eng.runner, eng.cache
        hs = []
        for p in prompts:
            h = cache.new_handle()
            cache.allocate(h, p)
            hs.append(h)
        for lo in range(0, batch, 4):
            r.step([StepEntry(h, p, 0, []) for h, p in zip(hs[lo:lo + 4], prompts[lo:lo + 4])])
        outs = []
        for k, toks in enumerate(nxt):
            for h, p in zip(hs, prompts):
                cache.grow(h, len(p) + k + 1)
            outs.append(r.step([StepEntry(h, [t], len(p) + k, [0]) for h, p, t in zip(hs, prompts, toks)]).float().cpu())
        if use_fused:
            assert r.stats["fused_steps"] == len(nxt)
            r.fused.check()
        return outs

    for a, b in zip(run(True), run(False)):
        assert torch.isfinite(a).all()
        assert float((a - b).abs().max()) <= 3e-2 * float(b.abs().max()), float((a - b).abs().max())


def test_step_program_equals_the_launch_by_launch_path(wide_dir, monkeypatch):
    """The same steps with the launches walked natively from a step program and made one by one from Python:
    prompt portions of growing size (the program's workspace is rebuilt when a step outgrows it), a mixed step,
    a step of 20 single tokens (which takes the decode attention kernel inside the program) and a step that
    wants no logits. Same kernels, same arguments: the logits agree to the last bit wherever the matrix library
    picks the same algorithm, and within bfloat16 rounding otherwise."""
    from tokenmill_b200.engine.batch import StepEntry
    from tokenmill_b200.kernels import program
    rng = random.Random(3)
    prompts = [[rng.randrange(1000) for _ in range(n)] for n in [700] + [40] * 19]

    def run(use_program):
        monkeypatch.setenv("TOKENMILL_STEP_PROGRAM", "1" if use_program else "0")
        eng = engine_for(wide_dir, dtype="bfloat16", max_model_len=1024, max_num_seqs=32, kv_cache_mb=64,
                         max_num_batched_tokens=4096, cuda_graphs=False)
        r, cache = eng.runner, eng.cache
        hs = []
        for p in prompts:
            h = cache.new_handle()
            cache.allocate(h, p + [0])
            hs.append(h)
        before = program.kind_launches()
        outs = [r.step([StepEntry(hs[0], prompts[0][:100], 0, [0, 99])]),                    # capacity 256
                r.step([StepEntry(hs[0], prompts[0][100:130], 100, [])]),                    # no logits wanted
                r.step([StepEntry(hs[0], prompts[0][130:], 130, [569])] +                    # capacity 1024, mixed
                       [StepEntry(h, p, 0, [39]) for h, p in zip(hs[1:], prompts[1:])]),
                r.step([StepEntry(hs[0], [5], 700, [0])] +                                   # 20 decoded tokens
                       [StepEntry(h, [7 + i], 40, [0]) for i, h in enumerate(hs[1:])])]
        issued = {k: v - before[k] for k, v in program.kind_launches().items()}
        if use_program:
            assert r.stats["program_steps"] == 4 and r._program.capacity == 2048
            assert issued["decode_attention_units"] == 2 and issued["decode_attention"] == 0
            assert issued["prefill_attention_tc"] == 6 and issued["prefill_attention"] == 0
        else:
            assert r.stats["program_steps"] == 0 and sum(issued.values()) == 0
        return [o.float().cpu() for o in outs]

    a, b = run(True), run(False)
    assert a[1].shape == (0, 1000) and b[1].shape == (0, 1000)
    for x, y in zip(a, b):
        assert x.shape == y.shape and torch.isfinite(x).all()
        if x.numel():
            assert float((x - y).abs().max()) <= 3e-2 * float(y.abs().max()), float((x - y).abs().max())


def test_output_matrix_kernel_in_the_decode_step(wide_dir, monkeypatch):
    """With TOKENMILL_LM_HEAD=1 the whole-step decode path multiplies by the output matrix with this library's
    streaming kernel instead of the library product: same logits within float32 summation order."""
    from tokenmill_b200.engine.batch import StepEntry
    rng = random.Random(11)
    prompts = [[rng.randrange(1000) for _ in range(rng.randrange(20, 90))] for _ in range(5)]

    def run(switch):
        monkeypatch.setenv("TOKENMILL_LM_HEAD", switch)
        eng = engine_for(wide_dir, dtype="bfloat16", max_model_len=256, max_num_seqs=8, kv_cache_mb=32,
                         max_num_batched_tokens=1024)
        r, cache = eng.runner, eng.cache
        assert (r._packed_output is not None) == (switch == "1")
        hs = []
        for p in prompts:
            h = cache.new_handle()
            cache.allocate(h, p + [0, 0])
            hs.append(h)
        r.step([StepEntry(h, p, 0, []) for h, p in zip(hs, prompts)])
        outs = [r.step([StepEntry(h, [3 + k], len(p) + k, [0]) for h, p in zip(hs, prompts)]).float().cpu() for k in range(2)]
        r.fused.check()
        return outs

    for a, b in zip(run("1"), run("0")):
        assert a.shape == (5, 1000) and float((a - b).abs().max()) <= 1e-4 * float(b.abs().max())


@pytest.mark.parametrize("inter,expect", [(8960, "some"), (13312, "none")])
def test_whole_step_kernel_leaves_wide_models_to_the_other_kernels(tmp_path, inter, expect):
    """A feed-forward so wide that the staged activations of many tokens leave no room for a ring stage: the
    whole-step kernel says how many tokens it takes at these sizes (none at all for the widest), steps beyond
    that run through the separate kernels, and the logits agree either way."""
    from tokenmill_b200.engine.batch import StepEntry
    from tokenmill_b200.kernels import fused
    from tokenmill_b200.weights import qwen2_config, write_random_model
    cfg = qwen2_config(vocab_size=500, hidden_size=256, intermediate_size=inter, num_hidden_layers=2,
                       num_attention_heads=2, num_key_value_heads=1, head_dim=128, rope_theta=10000.0,
                       tie_word_embeddings=True, max_position_embeddings=512)
    folder = write_random_model(tmp_path / "m", cfg, seed=2)
    rng = random.Random(inter)
    prompts = [[rng.randrange(500) for _ in range(rng.randrange(5, 60))] for _ in range(16)]

    def run(use_fused, batches):
        old = fused._ENABLED
        fused._ENABLED = use_fused
        try:
            eng = engine_for(folder, dtype="bfloat16", max_model_len=128, max_num_seqs=16, kv_cache_mb=16,
                             max_num_batched_tokens=1024)
        finally:
            fused._ENABLED = old
        r, cache = eng.runner, eng.cache
        hs = []
        for p in prompts:
            h = cache.new_handle()
            cache.allocate(h, p + [0] * len(batches))
            hs.append(h)
        r.step([StepEntry(h, p, 0, []) for h, p in zip(hs, prompts)])
        outs = [r.step([StepEntry(h, [3 + k], len(p) + k, [0]) for h, p in list(zip(hs, prompts))[:b]]).float().cpu()
                for k, b in enumerate(batches)]
        if r.fused is not None:
            r.fused.check()
        return r, outs

    r0, _ = run(True, [])
    if expect == "none":
        assert r0.fused is None
        batches = [1, 8]
    else:
        limit = r0.fused.max_tokens
        assert 1 <= limit < 16
        batches = [1, limit, limit + 1, 16]
    ra, a = run(True, batches)
    rb, b = run(False, batches)
    if expect == "some":
        assert ra.stats["fused_steps"] == 2 and rb.stats["fused_steps"] == 0
    for x, y in zip(a, b):
        assert torch.isfinite(x).all() and float((x - y).abs().max()) <= 3e-2 * float(y.abs().max())


@pytest.mark.parametrize("max_seqs,graphs,dtype", [(32, True, "bfloat16"), (10, True, "float32"), (32, False, "bfloat16")])
def test_graph_decode_steps_in_flight_give_the_synchronous_loop_s_results(d64_dir, max_seqs, graphs, dtype):
    """(With room for 10 requests the others wait and join as requests end: steps stay in flight while the
    queue is not empty. A request may then join one step later than in the synchronous loop, beside other
    requests, so that case runs in float32, where the company a request keeps does not move its logits enough
    to flip a token. Without decode graphs the steps of 17 and more requests run as step programs, with the
    ids gathered into the step's input buffer.) More requests than the whole-step kernel takes: their decode steps replay captured graphs, and with
    steps in flight the token ids are gathered on the device into the graph's static input. Same tokens, same
    ends as the synchronous loop: greedy and seeded sampling, ends at different lengths (the batch shrinks
    through the graph buckets down into the whole-step kernel's range)."""
    from tokenmill_b200.sampling import SamplingParams
    rng = random.Random(5)
    vocab = json.loads((Path(d64_dir) / "config.json").read_text())["vocab_size"]
    prompts = [[rng.randrange(vocab) for _ in range(rng.randrange(3, 40))] for _ in range(24)]
    params = [SamplingParams(max_tokens=4 + (5 * i) % 23, ignore_eos=True) if i % 3 else
              SamplingParams(max_tokens=6 + i, temperature=0.9, top_k=40, seed=i, ignore_eos=True) for i in range(24)]
    results = {}
    for mode in (False, True):
        eng = engine_for(d64_dir, dtype=dtype, async_decode=mode, max_num_seqs=max_seqs, max_num_batched_tokens=1024,
                         kv_cache_mb=32, cuda_graphs=graphs, cuda_graph_max_batch=32)
        assert eng._pipelining() == mode
        results[mode] = _run_requests(eng, prompts, params)
        st = eng.runner.stats
        if dtype == "bfloat16":
            assert st["fused_steps"] >= 3 and st["graph_steps" if graphs else "program_steps"] >= 3
        else:
            assert st["graph_steps"] >= 10
    for (ids_s, why_s, seen_s), (ids_a, why_a, seen_a), sp in zip(results[False], results[True], params):
        assert ids_s == ids_a and why_s == why_a == "length" and seen_s == ids_s and seen_a == ids_a
        assert len(ids_s) == sp.max_tokens and -1 not in ids_a


@pytest.mark.parametrize("variant", ["default", "units_off", "rope_kernel", "library_down", "own_o_and_gate_up"])
@pytest.mark.parametrize("graphs", [True, False])
def test_decode_steps_of_many_requests_against_plain_under_every_switch(wide_dir, variant, graphs, monkeypatch):
    """Twenty requests decoding together at the Qwen2.5-0.5B layer sizes (more than the whole-step kernel takes):
    captured graph or launch-by-launch, with the default kernels and with each switch turned the other way (the
    decode attention by fixed splits; the rotation kernel between projection and attention; the library's down
    projection; this repository's kernels for the output projection and gate/up too). Every logits row the
    engine sampled from is compared with the plain implementation on the request's own history."""
    from tokenmill_b200.kernels import ops
    from tokenmill_b200.sampling import SamplingParams
    if variant == "units_off":
        monkeypatch.setattr(ops, "_DECODE_UNITS", False)
    elif variant == "rope_kernel":
        monkeypatch.setattr(ops, "_DECODE_ROPE", False)
    elif variant == "library_down":
        monkeypatch.setattr(ops, "_TC_ADD", False)
    elif variant == "own_o_and_gate_up":
        monkeypatch.setattr(ops, "_TC_ADD_ALL", True)
    if not graphs:
        monkeypatch.setenv("TOKENMILL_STEP_PROGRAM", "0")          # (every launch from Python: the parts' forward paths)
    rng = random.Random(23)
    vocab = json.loads((Path(wide_dir) / "config.json").read_text())["vocab_size"]
    prompts = [[rng.randrange(vocab) for _ in range(rng.randrange(5, 150))] for _ in range(20)]
    eng = engine_for(wide_dir, dtype="bfloat16", max_model_len=512, max_num_seqs=32, max_num_batched_tokens=2048,
                     kv_cache_mb=64, cuda_graphs=graphs, cuda_graph_max_batch=32, async_decode=False)
    outs, tap = generate_tapped(eng, prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    st = eng.runner.stats
    assert st["graph_steps" if graphs else "steps"] >= 8
    assert assert_logits_match_plain(wide_dir, prompts, outs, tap, "bfloat16") >= 20 * 12


def test_long_contexts_move_small_decode_steps_from_the_whole_step_kernel_to_the_graph(d64_dir, monkeypatch):
    """Beside decode graphs, four or more requests whose contexts add up to many keys decode in the graph (its
    attention kernel streams long contexts faster), fewer keys or fewer requests in the whole-step kernel. With the
    limit lowered to 150 keys, five short requests cross it while they decode: both paths run, and every logits
    row agrees with the plain implementation."""
    from tokenmill_b200.engine import runner as runner_mod
    from tokenmill_b200.sampling import SamplingParams
    monkeypatch.setattr(runner_mod, "FUSED_DECODE_MAX_KEYS_BESIDE_GRAPHS", 150)
    rng = random.Random(31)
    vocab = json.loads((Path(d64_dir) / "config.json").read_text())["vocab_size"]
    prompts = [[rng.randrange(vocab) for _ in range(20)] for _ in range(5)]
    eng = engine_for(d64_dir, dtype="bfloat16", max_num_seqs=16, cuda_graphs=True, cuda_graph_max_batch=16,
                     async_decode=False, kv_cache_mb=16)
    outs, tap = generate_tapped(eng, prompts, SamplingParams(max_tokens=24, ignore_eos=True))
    st = eng.runner.stats
    assert st["fused_steps"] >= 5 and st["graph_steps"] >= 5, st
    assert assert_logits_match_plain(d64_dir, prompts, outs, tap, "bfloat16") >= 5 * 24
    # three requests stay in the kernel however long they are
    eng2 = engine_for(d64_dir, dtype="bfloat16", max_num_seqs=16, cuda_graphs=True, cuda_graph_max_batch=16,
                      async_decode=False, kv_cache_mb=16)
    generate_tapped(eng2, prompts[:3], SamplingParams(max_tokens=80, ignore_eos=True))
    assert eng2.runner.stats["graph_steps"] == 0 and eng2.runner.stats["fused_steps"] >= 79


@pytest.mark.parametrize("dtype,n_graphs", [("bfloat16", 1), ("float32", 6)])
def test_decode_graphs_captured_at_start_change_nothing_but_when(d64_dir, dtype, n_graphs):
    """``LLMEngine.capture_graphs()`` captures every decode graph before the first request (one graph of the
    largest batch where the whole-step kernel takes the small steps, one per power of two otherwise); the
    requests then get the tokens they get from an engine that captures when it first needs a graph."""
    from tokenmill_b200.sampling import SamplingParams
    rng = random.Random(11)
    vocab = json.loads((Path(d64_dir) / "config.json").read_text())["vocab_size"]
    prompts = [[rng.randrange(vocab) for _ in range(rng.randrange(3, 40))] for _ in range(24)]
    params = [SamplingParams(max_tokens=4 + (7 * i) % 19, ignore_eos=True) for i in range(24)]
    results = []
    for early in (True, False):
        eng = engine_for(d64_dir, dtype=dtype, max_num_seqs=32, max_num_batched_tokens=1024, kv_cache_mb=32,
                         cuda_graphs=True, cuda_graph_max_batch=32, async_decode=False)
        if early:
            assert eng.capture_graphs() == n_graphs and len(eng.runner._graphs) == n_graphs
            assert eng.capture_graphs() == n_graphs                     # (a second call finds them all there)
        results.append(_run_requests(eng, prompts, params))
        assert eng.runner.stats["graph_steps"] >= 3 and len(eng.runner._graphs) <= n_graphs
    assert [r[0] for r in results[0]] == [r[0] for r in results[1]]


@pytest.mark.parametrize("trial", [0, 3, 4])
def test_random_workloads_with_tiny_pools(d64_dir, trial):
    """Sixty requests of random lengths and sampling settings arriving at random times into a pool so small
    that requests are preempted again and again, with decode graphs, chunked prompts in one trial, steps in
    flight or not: every request gets exactly its tokens, no placeholder survives, no page is lost, and in
    float32 the loop with steps in flight produces the synchronous loop's tokens. (Between graph replays a
    mixed step of many short portions needs more attention scratch than the graphs captured.)"""
    from tokenmill_b200.sampling import SamplingParams
    vocab = json.loads((Path(d64_dir) / "config.json").read_text())["vocab_size"]
    rng = random.Random(trial)
    n = 60
    prompts = [[rng.randrange(vocab) for _ in range(rng.choice([1, 2, 5, 17, 40, 90, 150]))] for _ in range(n)]
    params = [SamplingParams(max_tokens=rng.choice([1, 3, 10, 40, 90]), ignore_eos=True) if rng.random() < 0.6 else
              SamplingParams(max_tokens=rng.choice([5, 30, 60]), temperature=0.8, top_k=20, seed=rng.randrange(1000),
                             ignore_eos=True) for _ in range(n)]

    def drive(eng):
        arrivals = random.Random(trial)
        pending = list(range(n))
        seqs, steps = {}, 0
        while pending or eng.has_unfinished():
            for _ in range(min(arrivals.choice([0, 0, 1, 2, 5]) if steps else 6, len(pending))):
                i = pending.pop(0)
                seqs[i] = eng.add_request(f"r{i}", prompts[i], params[i])
            eng.step()
            steps += 1
            assert steps < 20000
        eng.drain()
        assert eng.cache.all_free and not eng.scheduler.running
        return [seqs[i].output_ids for i in range(n)]

    outs = {}
    for dtype, kv_mb in (("float32", 1.2), ("bfloat16", 0.6)):        # room for 400 tokens: any request alone fits
        for mode in (False, True):
            eng = engine_for(d64_dir, dtype=dtype, max_model_len=512, max_num_seqs=24, max_num_batched_tokens=256,
                             kv_cache_mb=kv_mb, async_decode=mode, cuda_graphs=True, cuda_graph_max_batch=32,
                             enable_chunked_prefill=(trial % 3 == 0))
            outs[dtype, mode] = drive(eng)
            for ids, sp in zip(outs[dtype, mode], params):
                assert len(ids) == sp.max_tokens and all(0 <= t < vocab for t in ids)
    assert outs["float32", False] == outs["float32", True]


@pytest.mark.parametrize("trial", [0, 1, 2, 3])
def test_greedy_tokens_survive_preemption_prefix_sharing_and_portions(d64_dir, trial):
    """Sixteen greedy requests (some sharing a 37-token prefix) through a float32 engine with room for 200
    tokens and 8 requests at a time, prompts cut into portions of 32 or 128, prefix caching on in half of the
    trials, decode graphs, steps in flight or not: whatever the scheduler does (preempt and recompute, reuse a
    prefix's pages, cut a prompt), every request's tokens are the plain implementation's greedy continuation."""
    from tokenmill_b200.sampling import SamplingParams
    cfg, w = load_plain(d64_dir)
    vocab = json.loads((Path(d64_dir) / "config.json").read_text())["vocab_size"]
    rng = random.Random(trial)
    shared = [rng.randrange(vocab) for _ in range(rng.choice([0, 37]))]
    prompts = [shared + [rng.randrange(vocab) for _ in range(rng.choice([1, 4, 20, 50]))] for _ in range(16)]
    news = [rng.choice([1, 5, 20]) for _ in range(16)]
    want = [plain_greedy(cfg, w, p, k) for p, k in zip(prompts, news)]
    budget, block = rng.choice([32, 128]), rng.choice([8, 16])
    for mode in (False, True):
        eng = engine_for(d64_dir, dtype="float32", max_model_len=256, max_num_seqs=8, max_num_batched_tokens=budget,
                         kv_cache_mb=3 * 2 * 64 * 2 * 4 * 200 / 2 ** 20, block_size=block, async_decode=mode,
                         cuda_graphs=True, cuda_graph_max_batch=8, enable_chunked_prefill=trial % 2 == 0,
                         enable_prefix_caching=trial >= 2)
        got = eng.generate(prompts, [SamplingParams(max_tokens=k, ignore_eos=True) for k in news])
        assert got == want, (mode, [i for i, (a, b) in enumerate(zip(got, want)) if a != b])
        assert eng.cache.all_free


@pytest.mark.parametrize("block,chunked,async_decode", [(16, False, True), (8, True, True), (32, False, False),
                                                        (8, False, False)])
def test_bfloat16_fast_paths_with_prefix_hits_and_evictions_match_the_plain_logits(d64_dir, block, chunked,
                                                                                   async_decode):
    """The bfloat16 kernels that serving uses (whole-step decode kernel, tensor-core prompt attention, step
    programs) under everything the scheduler can do to a request: pages of a shared prefix found in the cache,
    eviction with recomputation, prompts cut into portions, steps in flight; pages of 8, 16 and 32 tokens. Not
    the tokens are compared but the logits behind every one of them, recomputed positions included, with the
    plain implementation on the request's own history."""
    vocab = json.loads((Path(d64_dir) / "config.json").read_text())["vocab_size"]
    rng = random.Random(block + chunked)
    shared = [rng.randrange(vocab) for _ in range(70)]
    prompts = [shared[:rng.choice([40, 70])] + [rng.randrange(vocab) for _ in range(rng.choice([3, 9, 30]))]
               for _ in range(10)]
    probe = engine_for(d64_dir, dtype="bfloat16")
    per_token = probe.model.cache_layout().bytes_per_token(2)
    # room for 288 tokens: two or three of the ten requests (about 80 + 30 tokens each) at a time, not all
    eng = engine_for(d64_dir, dtype="bfloat16", block_size=block, max_model_len=256, max_num_seqs=6,
                     kv_cache_mb=(288 + 1) * per_token / 2 ** 20, enable_prefix_caching=True,
                     enable_chunked_prefill=chunked, max_num_batched_tokens=48 if chunked else 512,
                     async_decode=async_decode)
    assert eng.runner.fused is not None
    outs, tap = generate_tapped(eng, prompts, greedy(30))
    assert all(len(o) == 30 for o in outs) and eng.cache.all_free
    assert eng.scheduler.evictions > 0 and eng.cache.prefix_hit_tokens > 0 and eng.runner.stats["fused_steps"] > 0
    assert assert_logits_match_plain(d64_dir, prompts, outs, tap, "bfloat16") >= 10 * 30


def test_short_prompts_go_through_the_whole_step_kernel_in_pieces(d64_dir, tmp_path, plain_cache, monkeypatch):
    """Prompts of up to 16 tokens (alone, beside other short prompts, beside decoded tokens) have more rows per
    kv head than one attention unit of the whole-step kernel holds; they enter it as pieces of a few tokens each
    and the logits at every place are the plain implementation's."""
    from tokenmill_b200.kernels import lib
    calls = []
    real = lib.call
    monkeypatch.setattr(lib, "call", lambda name, *a: (calls.append(name), real(name, *a))[1])
    vocab = json.loads((Path(d64_dir) / "config.json").read_text())["vocab_size"]
    reqs = make_requests(vocab, [30, 20, 12, 40], seed=21)
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": reqs["r0"][:11], "want": [0, 5, 10]}], "end": []},
             {"step": 1, "entries": [{"id": "r1", "tokens": reqs["r1"][:7], "want": list(range(7))},
                                     {"id": "r0", "tokens": reqs["r0"][11:12], "want": [0]},
                                     {"id": "r2", "tokens": reqs["r2"][:3], "want": [2]}], "end": []},
             {"step": 2, "entries": [{"id": "r3", "tokens": reqs["r3"][:16], "want": [15]}], "end": []},
             {"step": 3, "entries": [{"id": "r0", "tokens": reqs["r0"][12:18], "want": [0, 5]},
                                     {"id": "r1", "tokens": reqs["r1"][7:13], "want": [5]},
                                     {"id": "r2", "tokens": reqs["r2"][3:4], "want": [0]},
                                     {"id": "r3", "tokens": reqs["r3"][16:17], "want": [0]}], "end": ["r2"]},
             {"step": 4, "entries": [{"id": "r0", "tokens": reqs["r0"][18:], "want": [11]},
                                     {"id": "r3", "tokens": reqs["r3"][17:21], "want": [3]}], "end": ["r0", "r1", "r3"]}]
    outputs = run_trace(d64_dir, "bfloat16", steps, 512, tmp_path / "o")
    check_against_plain(steps, outputs, reqs, plain_for(d64_dir, reqs, plain_cache), "bfloat16")
    assert calls.count("tm_decode_fused") == 5 and "tm_program_run" not in calls


@pytest.mark.parametrize("shape", [(128, 1, 5, 432, 344, 1), (128, 4, 7, 488, 1312, 3), (64, 2, 1, 640, 1632, 2),
                                   (64, 3, 5, 280, 696, 2), (32, 4, 2, 216, 616, 2)],
                         ids=lambda s: "d%d_kv%d_g%d_h%d" % s[:4])
def test_scheduling_options_over_shapes_no_named_model_has(shape, tmp_path):
    """Head sizes, groupings and widths (no multiples of 32 among them) that the named models do not have, through
    ``LLMEngine`` with its options one after the other (plain; decode graphs; chunked prompts under a budget of 64
    tokens; prefix caching with graphs at another page size; a pool so small that requests are evicted): the
    logits behind every generated token against the plain implementation on the request's own history."""
    from tokenmill_b200.weights import qwen2_config, write_random_model
    D, nkv, G, H, I, L = shape
    cfg = qwen2_config(vocab_size=1013, hidden_size=H, intermediate_size=I, num_hidden_layers=L, num_attention_heads=nkv * G,
                       num_key_value_heads=nkv, head_dim=D, rope_theta=50000.0, rms_norm_eps=1e-6,
                       tie_word_embeddings=bool(L % 2), max_position_embeddings=1024)
    folder = write_random_model(tmp_path / "model", cfg, seed=H)
    rng = random.Random(H)
    prompts = prompts_for(folder, [rng.randrange(1, 150) for _ in range(14)])
    small_pool = 700 * L * 2 * nkv * D * 2 / 2 ** 20                   # room for 700 tokens: 14 requests need about 1,400
    for kw in (dict(), dict(cuda_graphs=True, cuda_graph_max_batch=16),
               dict(enable_chunked_prefill=True, max_num_batched_tokens=64),
               dict(enable_prefix_caching=True, cuda_graphs=True, cuda_graph_max_batch=8, block_size=32),
               dict(kv_cache_mb=small_pool, enable_chunked_prefill=True, max_num_batched_tokens=96)):
        eng = engine_for(folder, "bfloat16", **kw)
        outs, tap = generate_tapped(eng, prompts, greedy(24))
        assert assert_logits_match_plain(folder, prompts, outs, tap, "bfloat16") >= 14 * 24
        if "kv_cache_mb" in kw:
            assert eng.scheduler.evictions > 0 and eng.cache.all_free
