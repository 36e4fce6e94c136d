"""Decode and prefill throughput of the engine at the Qwen2.5-0.5B layer sizes, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]
    python bench.py --workload 1.5b-mixed | 7b-prefix [--impl ours|reference] [--layers L]

One JSON line on standard output. A "step" is one decode step of a batch of 8 requests (prompt 512, 512 new
tokens, context limit 4096): after the prompts, decode steps run untimed until the K timed steps lie in the
middle of the 512 new tokens (mean context 768). ``value`` is decoded tokens per second timed on the device
with CUDA events around exactly K steps of the engine's step function (one metadata copy, the whole-step decode
kernel, the output matrix and the arg-max kernel per step); ``e2e`` is the same quantity through the Python
entry point (``LLMEngine.step``: scheduler, pinned host-to-device metadata copy, kernels, sampling, token ids
read back to the host every step), timed on the host between two device synchronisations. ``prefill`` times
one 2,048-token prompt; ``roofline`` relates the decode step to the memory bandwidth it needs (every weight
once plus the live requests' cache); ``points`` holds decode at batch 1 and 64 (device-timed and end to end),
batch 8 end to end with sampled requests (temperature 0.8, top-k 40, top-p 0.95) and batch 8 behind prompts of
3,072 tokens; ``fp32`` the float32 engine's decode step at batch 8 and its 2,048-token prompt.

Profiling aids that print their own lines instead of the contract's: ``--only prefill | decode_b<batch> |
products | sampling | decode_attention[:<case>]``, with ``--prompt-len N`` (decode behind prompts of N tokens),
``--prefill-tokens N``, ``--layers L``, ``--sizes qwen2.5-1.5b | qwen2.5-7b``, ``--no-graphs``.

``--workload`` runs one of the two other workloads the baseline names, through ``LLMEngine`` with every
request submitted at once and stepped to completion (the reference's bench/common.py:58-76 method), and prints
one JSON line with generated tokens per second, preemptions and the prefix-cache hit rate:
``1.5b-mixed``: Qwen2.5-1.5B sizes, 64 requests, prompt lengths uniform in [128, 2048], 256 new tokens,
chunked prefill with a 2,048-token budget; ``7b-prefix``: Qwen2.5-7B sizes, context 8192, 32 requests of
4,096-token prompts that share their first 1,024 tokens, 512 new tokens, prefix caching, a pool too small for
all of them so that requests are preempted.

The engine runs on one GPU: for --gpus N > 1 a line says so and the exit code is 2.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

SIZES = dict(vocab_size=151936, hidden_size=896, intermediate_size=4864, num_hidden_layers=24,
             num_attention_heads=14, num_key_value_heads=2, head_dim=64, rope_theta=1000000.0, rms_norm_eps=1e-6,
             tie_word_embeddings=True, max_position_embeddings=32768)
MODEL_LABEL = "Qwen2.5-0.5B"
PROMPT_LEN, NEW_TOKENS, CONTEXT, BATCH, PREFILL_TOKENS, PAGE = 512, 512, 4096, 8, 2048, 16
LONG_PROMPT = 3072      # the long-context decode point (prompt + new tokens stay within CONTEXT)


def use_sizes(name: str) -> None:
    """Measure another of the named sizes (--sizes qwen2.5-1.5b | qwen2.5-7b) instead of the default one."""
    global MODEL_LABEL
    from tokenmill_b200.weights.random_init import NAMED_SIZES
    if name.lower() not in NAMED_SIZES:
        raise SystemExit(f"bench.py: unknown --sizes {name!r}; known: {sorted(NAMED_SIZES)}")
    named = NAMED_SIZES[name.lower()]
    SIZES.update(named)
    SIZES["head_dim"] = named.get("head_dim", named["hidden_size"] // named["num_attention_heads"])
    MODEL_LABEL = name.replace("qwen", "Qwen").replace("b", "B") if name.lower().startswith("qwen") else name
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            raw = json.loads(f.read_text())
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"])}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples while the timed regions run (read-only queries)."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        rows = [r.split(",") for r in Path(self.file.name).read_text().splitlines() if r.count(",") >= 5]
        os.unlink(self.file.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.strip().lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_flops_bytes(cfg: dict, layers: int) -> dict:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = H * (nh + 2 * nkv) * D + nh * D * H + 3 * H * I
    small = layers * (2 * H + (nh + 2 * nkv) * D) + H
    return {"layer_matrix_params": per_layer, "weight_bytes": 2 * (layers * per_layer + V * H) + 4 * small,
            "kv_bytes_per_token": 2 * layers * nkv * D * 2,
            "prefill_flops": lambda T: layers * (2 * T * per_layer + 4 * nh * D * T * (T + 1) / 2) + 2 * V * H}


def make_model_dir(layers: int) -> tempfile.TemporaryDirectory:
    from tokenmill_b200.weights import qwen2_config, write_random_model
    tmp = tempfile.TemporaryDirectory(prefix="tokenmill_bench_")
    cfg = qwen2_config(**{**SIZES, "num_hidden_layers": layers})
    t0 = time.time()
    write_random_model(tmp.name, cfg, seed=0)
    print(f"[bench] random weights ({layers} layers) written in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
    return tmp


def prompts(batch: int, length: int, seed: int = 0) -> list[list[int]]:
    import random
    rng = random.Random(seed)
    return [[rng.randrange(1000, 150000) for _ in range(length)] for _ in range(batch)]


def decode_device_timed(engine, batch: int, steps: int, warmup: int, skip_ahead: bool = True,
                        prompt_len: int = 0) -> dict:
    """K decode steps of the step function, CUDA events on the launching stream (``prompt_len``: another prompt
    length than the headline's)."""
    import torch
    from tokenmill_b200.engine.batch import StepEntry
    from tokenmill_b200.kernels import lib, ops

    runner, cache = engine.runner, engine.cache
    prompt_len = prompt_len or PROMPT_LEN
    handles = []
    for p in prompts(batch, prompt_len, seed=batch):
        h = cache.new_handle()
        cache.allocate(h, p)
        handles.append((h, p))
    together = 4 if prompt_len <= 2048 else 1                   # prefill, four prompts a step (long ones alone)
    for lo in range(0, batch, together):
        runner.step([StepEntry(h, p, 0, []) for h, p in handles[lo:lo + together]])
    length = prompt_len
    tok = [p[-1] for _, p in handles]
    # The timed steps lie in the middle of the NEW_TOKENS new tokens; the steps before them run untimed.
    forward = max(0, NEW_TOKENS // 2 - steps // 2 - warmup) if skip_ahead else 0

    chosen = torch.zeros(max(batch, 16), dtype=torch.int32, device=runner.device)

    def one():
        nonlocal length
        for h, _ in handles:
            cache.grow(h, length + 1)
        entries = [StepEntry(h, [t], length, [0]) for (h, _), t in zip(handles, tok)]
        if runner.takes_greedy_steps(batch, entries):   # the arg-max comes out of the output matrix's own kernel
            runner.step_greedy(entries, chosen)
        else:
            ops.argmax(runner.step(entries), out=chosen[:batch])
        length += 1

    for _ in range(forward + warmup):
        one()
    torch.cuda.synchronize()
    launches0 = lib.launch_count
    graph_kernels = getattr(runner, "kernels_per_graph", {}).get(batch, 0)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        one()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    launched = (lib.launch_count - launches0) + steps * graph_kernels
    mean_ctx = length - steps / 2
    for h, _ in handles:
        cache.free(h)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "launches": launched, "mean_ctx": mean_ctx}


def decode_end_to_end(engine, batch: int, steps: int, warmup: int, sampled: bool = False) -> dict:
    """K decode steps through LLMEngine.step: host token ids in, host token ids out, every step. ``sampled``:
    temperature 0.8, top-k 40, top-p 0.95 with a seed per request instead of greedy choice."""
    import torch
    from tokenmill_b200.sampling import SamplingParams

    forward = max(0, NEW_TOKENS // 2 - steps // 2 - warmup)
    sp = SamplingParams(max_tokens=forward + steps + warmup + 4, ignore_eos=True,
                        **(dict(temperature=0.8, top_k=40, top_p=0.95, seed=7) if sampled else {}))
    seqs = [engine.add_request(f"e2e-{batch}-{i}", p, sp) for i, p in enumerate(prompts(batch, PROMPT_LEN, seed=99))]
    while any(s.n_output == 0 for s in seqs):
        engine.step()
    for _ in range(forward + warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = 0
    for _ in range(steps):
        n += sum(len(o.new_token_ids) for o in engine.step())
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = engine.runner.stats["h2d_bytes"]          # bytes of the last step's (one) host-to-device copy
    for s in seqs:
        engine.abort_request(s.id)
    return {"tok_s": n / dt, "ms_per_step": 1e3 * dt / steps, "h2d": h2d, "d2h": batch * 4, "tokens": n}


def prefill_timed(engine, tokens: int, reps: int = 5) -> dict:
    import torch
    from tokenmill_b200.engine.batch import StepEntry

    runner, cache = engine.runner, engine.cache
    p = prompts(1, tokens, seed=5)[0]
    times = []
    for i in range(reps + 3):
        h = cache.new_handle()
        cache.allocate(h, p)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry(h, p, 0, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(start.elapsed_time(end))
        cache.free(h)
    return {"ms": statistics.median(times)}


def sampling_timed(vocab: int = 151936, reps: int = 20) -> list[dict]:
    """Profiling aid (--only sampling): the sampling kernel alone over rows of `vocab` random logits (standard
    deviation 3), 1, 8 and 64 rows, by kind of cut; us a launch, CUDA events around `reps` launches."""
    import torch
    from tokenmill_b200.kernels import ops
    dev, out = torch.device("cuda:0"), []
    kinds = {"temperature": (0, 1.0), "top_k 40": (40, 1.0), "top_p 0.9 (below the candidates)": (0, 0.9),
             "top_k 40 + top_p 0.9": (40, 0.9)}
    for n in (1, 8, 64):
        logits = torch.randn(n, vocab, device=dev, generator=torch.Generator(device=dev).manual_seed(n)) * 3
        for name, (k, p) in kinds.items():
            temp, u = torch.full((n,), 0.8, device=dev), torch.rand(n, device=dev)
            tk, tp = torch.full((n,), k, dtype=torch.int32, device=dev), torch.full((n,), p, device=dev)
            res = torch.empty(n, dtype=torch.int32, device=dev)
            for _ in range(3):
                ops.sample(logits, temp, tk, tp, u, out=res)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            for _ in range(reps):
                ops.sample(logits, temp, tk, tp, u, out=res)
            b.record()
            torch.cuda.synchronize()
            out.append({"rows": n, "vocab": vocab, "kind": name, "us": round(a.elapsed_time(b) / reps * 1000, 1)})
    ops.tc_check(dev)
    return out


def products_timed(tokens: int = 8) -> list[dict]:
    """Profiling aid (--only products): a decode step's matrix products at the Qwen2.5 0.5B / 1.5B / 7B layer
    sizes, through this library's weight-streaming kernels ("streaming": plain loads; "ring": packed weights
    through a shared-memory ring of bulk copies, the K range cut into slices) and through the library product
    (plus the SwiGLU kernel for gate/up), each after an L2 flush. It is what the size limits of kernels/ops.py
    (SKINNY_MAX_WEIGHT_BYTES) and kernels/fused.py (MAX_LAYER_WEIGHT_BYTES) were read from."""
    import torch
    from tokenmill_b200.kernels import ops
    from tokenmill_b200.kernels.fused import pack_rows
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, n=12):
        ts = []
        for _ in range(n):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record(); torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1000)
        return sorted(ts)[n // 2]

    rows = []
    for name, (H, QKV, I) in {"0.5B": (896, 1152, 4864), "1.5B": (1536, 2048, 8960), "7B": (3584, 4608, 18944)}.items():
        x = torch.randn(tokens, H, device="cuda").bfloat16()
        xi = torch.randn(tokens, I, device="cuda").bfloat16()
        w_qkv = (torch.randn(QKV, H, device="cuda") * 0.02).bfloat16()
        w_gu = (torch.randn(2 * I, H, device="cuda") * 0.02).bfloat16()
        w_d = (torch.randn(H, I, device="cuda") * 0.02).bfloat16()
        act = torch.empty(tokens, I, device="cuda", dtype=torch.bfloat16)
        gu = torch.empty(tokens, 2 * I, device="cuda", dtype=torch.bfloat16)
        ks = ops.skinny_k_splits(tokens, I)

        def lib_gate_up():
            torch.mm(x, w_gu.t(), out=gu)
            ops.swiglu(gu, act)
        p_qkv, p_gu, p_d = pack_rows(w_qkv), pack_rows(w_gu), pack_rows(w_d)

        def ring_gate_up():
            ops.swiglu_partials(ops.stream_linear(x, p_gu, 2 * I), act)
        for what, ours, ring, theirs, nbytes in (
                ("qkv", lambda: ops.skinny_linear(x, w_qkv), lambda: ops.stream_linear(x, p_qkv, QKV),
                 lambda: torch.mm(x, w_qkv.t()), QKV * H * 2),
                ("gate_up+swiglu", lambda: ops.skinny_gate_up_swiglu(x, w_gu, act), ring_gate_up, lib_gate_up, 2 * I * H * 2),
                ("down", lambda: ops.skinny_linear(xi, w_d, k_splits=ks), lambda: ops.stream_linear(xi, p_d, H),
                 lambda: torch.mm(xi, w_d.t()), H * I * 2)):
            t_ours, t_ring, t_lib = timed(ours), timed(ring), timed(theirs)
            rows.append({"sizes": name, "tokens": tokens, "product": what, "weight_mb": round(nbytes / 2 ** 20, 1),
                         "streaming_us": round(t_ours, 1), "streaming_tb_s": round(nbytes / t_ours / 1e6, 2),
                         "ring_us": round(t_ring, 1), "ring_tb_s": round(nbytes / t_ring / 1e6, 2),
                         "library_us": round(t_lib, 1), "library_tb_s": round(nbytes / t_lib / 1e6, 2)})
    return rows



ATTENTION_CASES = {      # requests, keys a request, heads, kv heads, head size
    "0.5b_b64": (64, 768, 14, 2, 64), "0.5b_b256": (256, 1000, 14, 2, 64), "1.5b_b64": (64, 1200, 12, 2, 128),
    "7b_b27_long": (27, 4400, 28, 4, 128), "7b_b8_long": (8, 4400, 28, 4, 128), "7b_b64_ragged": (64, 4000, 28, 4, 128),
}


def decode_attention_timed(case: str, reps: int = 5, page: int = 16, sequential: bool = False) -> dict:
    """Profiling aid (--only decode_attention:<case>): the decode attention kernel alone over a shuffled paged cache,
    one new token a request, by host-made units (the engine's plan) and by fixed splits of 512 keys; ten launches
    in a captured graph a repetition, so that the time is the device's. "ragged" cases draw the lengths from a
    quarter of the named one up to it. ``decode_attention:<case>:sequential`` lays each request's pages one after
    the other in the pool instead of shuffling them."""
    import numpy as np
    import torch
    from tokenmill_b200.kernels import ops
    from tokenmill_b200.parts.attention_plan import decode_parts_cap, decode_units
    S, ctx, nh, nkv, D = ATTENTION_CASES[case]
    dev = torch.device("cuda:0")
    lens = np.random.default_rng(0).integers(ctx // 4, ctx, S) if "ragged" in case else np.full(S, ctx)
    pages_seq = -(-(ctx + 1) // page)
    n_pages = S * pages_seq + 1
    nbytes = int((lens + 1).sum()) * nkv * D * 2 * 2
    # As many caches as exceed the L2 together, one after the other through the ten launches of a repetition (a
    # model's layers each have their own): every launch reads its keys and values from memory.
    copies = min(10, max(1, -(-(300 << 20) // nbytes)))
    caches = [((torch.randn(n_pages, page, nkv, D, device=dev) * 0.5).bfloat16(),
               (torch.randn(n_pages, page, nkv, D, device=dev) * 0.5).bfloat16()) for _ in range(copies)]
    order = torch.arange(n_pages - 1, device=dev) if sequential else torch.randperm(n_pages - 1, device=dev)
    table = (order.int() + 1)[: S * pages_seq].view(S, pages_seq).contiguous()
    q = torch.randn(S, nh, D, device=dev).bfloat16()
    out = torch.empty_like(q)
    cu = torch.arange(S + 1, device=dev, dtype=torch.int32)
    before = torch.from_numpy(lens.astype(np.int32)).to(dev)
    done = torch.zeros(S * nkv, dtype=torch.int32, device=dev)
    slots = ops.decode_units_slots(D, dev)
    rec, n_units, max_parts = decode_units(np.ones(S, int), lens, 0, kv_heads=nkv, slots=slots,
                                           cap=decode_parts_cap(ctx + 1), head_dim=D)
    units = torch.from_numpy(rec).to(dev)
    n_work = torch.tensor([n_units * nkv], dtype=torch.int32, device=dev)
    split, max_splits = 512, -(-(ctx + 1) // 512)
    parts = max(max_parts, max_splits)
    acc = torch.empty(S * nh * parts * D, device=dev)
    ml = torch.empty(S * nh * parts * 2, device=dev)

    def by_units(kc, vc):
        ops.decode_attention_units_bf16(q, kc, vc, table, cu, before, units, n_work, out, scale=D ** -0.5, window=0,
                                        max_parts=max_parts, grid=min(slots, n_units * nkv), part_acc=acc, part_ml=ml,
                                        done=done)

    def by_splits(kc, vc):
        ops.decode_attention_bf16(q, kc, vc, table, cu, before, S, out, scale=D ** -0.5, window=0, split_keys=split,
                                  max_splits=max_splits, part_acc=acc, part_ml=ml, done=done)

    def timed(fn):
        for kc, vc in caches:
            fn(kc, vc)
        torch.cuda.synchronize()
        ops.tc_check(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(10):
                fn(*caches[i % copies])
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); g.replay(); b.record(); torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 100)
        return sorted(ts)[reps // 2]

    t_units, t_splits = timed(by_units), timed(by_splits)
    return {"only": "decode_attention", "case": case, "requests": S, "keys": ctx, "heads": nh, "kv_heads": nkv,
            "head_dim": D, "page": page, "pages": "sequential" if sequential else "shuffled", "kv_mb": round(nbytes / 1e6, 1),
            "caches": copies, "units": n_units, "parts_a_request": max_parts,
            "stages_a_unit": int((rec[:, 2] - rec[:, 1]).max()), "units_us": round(t_units, 1),
            "units_tb_s": round(nbytes / t_units / 1e6, 2), "splits_of_512_us": round(t_splits, 1),
            "splits_tb_s": round(nbytes / t_splits / 1e6, 2)}


def bench_config(layers: int, mean_ctx: float, extra: dict) -> dict:
    """The ``config`` object of the JSON line (flat, at most 20 keys), the same keys in both arms."""
    cfg = {"model": f"{MODEL_LABEL} sizes", "layers": layers, "layers_in_named_config": SIZES["num_hidden_layers"],
           "hidden": SIZES["hidden_size"], "q_heads": SIZES["num_attention_heads"],
           "kv_heads": SIZES["num_key_value_heads"], "head_dim": SIZES["head_dim"],
           "intermediate": SIZES["intermediate_size"], "vocab": SIZES["vocab_size"],
           "tied_output": bool(SIZES["tie_word_embeddings"]), "global_batch": BATCH, "prompt_len": PROMPT_LEN,
           "new_tokens": NEW_TOKENS, "seq_len": CONTEXT, "kv_page": PAGE, "mean_decode_context": round(mean_ctx, 1),
           "parallelism": "single GPU"}
    cfg.update(extra)
    assert len(cfg) <= 20
    return cfg


def engine_config(model_dir: str, dtype: str, info: dict, graphs: bool):
    from tokenmill_b200 import EngineConfig
    elt = 2 if dtype == "bfloat16" else 4
    return EngineConfig(model=model_dir, dtype=dtype, block_size=PAGE, max_model_len=CONTEXT, max_num_seqs=64,
                        max_num_batched_tokens=4 * PROMPT_LEN,
                        kv_cache_mb=64 * (PROMPT_LEN + NEW_TOKENS + 64) * info["kv_bytes_per_token"] * (elt // 2) / 2 ** 20,
                        watermark=0.0, cuda_graphs=graphs, cuda_graph_max_batch=64)


def run_ours(args) -> dict:
    import torch
    from tokenmill_b200.engine import LLMEngine
    from tokenmill_b200.kernels import lib

    if args.only == "products":
        for row in products_timed():
            print(json.dumps(row))
        return {}
    if args.only == "sampling":
        for row in sampling_timed():
            print(json.dumps(row))
        return {}
    if args.only.startswith("decode_attention"):
        parts = args.only.split(":")
        cases = [parts[1]] if len(parts) > 1 and parts[1] else list(ATTENTION_CASES)
        for case in cases:
            print(json.dumps(decode_attention_timed(case, sequential="sequential" in parts[2:])))
        return {}
    layers = args.layers or SIZES["num_hidden_layers"]
    pk, pk_kind = peaks()
    info = model_flops_bytes(SIZES, layers)
    tmp = make_model_dir(layers)
    fp32 = None
    try:
        engine = LLMEngine(engine_config(tmp.name, "bfloat16", info, not args.no_graphs))
        lib.load()
        if args.only:                                             # a small case for profilers: no JSON contract
            if args.only == "prefill":
                print(json.dumps({"only": "prefill", **prefill_timed(engine, args.prefill_tokens, reps=args.steps)}))
            else:
                batch = int(args.only.split("_b")[1])
                r = decode_device_timed(engine, batch, args.steps, args.warmup, skip_ahead=not args.no_skip)
                print(json.dumps({"only": args.only, "ms_per_step": r["ms_per_step"], "tok_s": r["tok_s"],
                                  "mean_ctx": r["mean_ctx"]}))
            return {}
        sampler = ClockSampler()
        # warm every path once before the clocks are sampled
        decode_device_timed(engine, BATCH, 4, 3, skip_ahead=False)
        sampler.start()
        main = decode_device_timed(engine, BATCH, args.steps, args.warmup)
        e2e = decode_end_to_end(engine, BATCH, args.steps, args.warmup)
        side = max(16, args.steps // 2)
        b1 = decode_device_timed(engine, 1, side, args.warmup)
        b64 = decode_device_timed(engine, 64, side, args.warmup)
        long8 = decode_device_timed(engine, BATCH, side, args.warmup, prompt_len=LONG_PROMPT)
        e1 = decode_end_to_end(engine, 1, side, args.warmup)
        e64 = decode_end_to_end(engine, 64, side, args.warmup)
        es8 = decode_end_to_end(engine, BATCH, side, args.warmup, sampled=True)
        pre = prefill_timed(engine, PREFILL_TOKENS)
        clocks = sampler.stop()
        if not args.no_fp32:
            # The float32 engine (true 32-bit products on CUDA cores): one decode point and the prompt, so that a
            # regression of that path shows. Not part of the clock record above.
            del engine
            torch.cuda.empty_cache()
            engine = LLMEngine(engine_config(tmp.name, "float32", info, False))
            d32 = decode_device_timed(engine, BATCH, min(args.steps, 16), 3)
            p32 = prefill_timed(engine, PREFILL_TOKENS, reps=2)
            fp32 = {"decode_b8": round(d32["tok_s"], 1), "decode_b8_ms": round(d32["ms_per_step"], 4),
                    "prefill_ms": round(p32["ms"], 3), "prefill_tok_s": round(PREFILL_TOKENS / (p32["ms"] / 1e3), 1)}
    finally:
        tmp.cleanup()
    step_bytes = info["weight_bytes"] + BATCH * main["mean_ctx"] * info["kv_bytes_per_token"]
    achieved = step_bytes / (main["ms_per_step"] / 1e3) / 1e9
    pf_flops = info["prefill_flops"](PREFILL_TOKENS)
    pf_frac = pf_flops / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12)

    def hbm_frac(batch, r):
        return round((info["weight_bytes"] + batch * r["mean_ctx"] * info["kv_bytes_per_token"])
                     / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 4)
    out = {
        "metric": f"decode tok/s at batch 8 ({MODEL_LABEL} sizes, prompt 512, bf16)", "value": round(main["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights seed 0", "impl": "ours",
        "config": bench_config(layers, main["mean_ctx"], {
            "l2": "inputs larger than L2 (weights read per step: %.0f MB)" % (info["weight_bytes"] / 1e6),
            "peaks": pk_kind, "cuda_graphs": not args.no_graphs}),
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(e2e["ms_per_step"], 4),
                "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": int(main["launches"]),
        "prefill": {"value": round(PREFILL_TOKENS / (pre["ms"] / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(pre["ms"], 3), "frac": round(pf_frac, 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {"decode_b1": round(b1["tok_s"], 1), "decode_b64": round(b64["tok_s"], 1),
                   "decode_b1_ms": round(b1["ms_per_step"], 4), "decode_b64_ms": round(b64["ms_per_step"], 4),
                   "decode_b1_hbm_frac": hbm_frac(1, b1), "decode_b64_hbm_frac": hbm_frac(64, b64),
                   "e2e_b1": round(e1["tok_s"], 1), "e2e_b64": round(e64["tok_s"], 1),
                   "e2e_b8_sampled": round(es8["tok_s"], 1),      # temperature 0.8, top-k 40, top-p 0.95
                   # batch 8 behind prompts of LONG_PROMPT tokens (mean context LONG_PROMPT + 256)
                   "decode_b8_long": round(long8["tok_s"], 1), "decode_b8_long_ms": round(long8["ms_per_step"], 4),
                   "decode_b8_long_ctx": round(long8["mean_ctx"], 1), "decode_b8_long_hbm_frac": hbm_frac(BATCH, long8)},
        "clocks": clocks,
    }
    if fp32 is not None:
        out["fp32"] = fp32
    return out


# --- the two other workloads the baseline names --------------------------------------------------------------

WORKLOADS = {
    # sizes, context, requests, prompt lengths, shared prefix, new tokens, engine options, share of the need the pool holds
    "1.5b-mixed": dict(sizes="qwen2.5-1.5b", context=4096, n=64, prompt=(128, 2048), shared=0, new=256,
                       engine=dict(enable_chunked_prefill=True, max_num_batched_tokens=2048), pool_share=1.0),
    "7b-prefix": dict(sizes="qwen2.5-7b", context=8192, n=32, prompt=(4096, 4096), shared=1024, new=512,
                      engine=dict(enable_prefix_caching=True, max_num_batched_tokens=8192), pool_share=0.6),
}


def workload_prompts(w: dict, seed: int = 0) -> list[list[int]]:
    import random
    rng = random.Random(seed)
    shared = [rng.randrange(1000, 150000) for _ in range(w["shared"])]
    lo, hi = w["prompt"]
    return [shared + [rng.randrange(1000, 150000) for _ in range(rng.randint(lo, hi) - w["shared"])] for _ in range(w["n"])]


def run_workload(args) -> dict:
    """Everything submitted at once and stepped to completion; generated tokens / wall time."""
    import torch
    w = WORKLOADS[args.workload]
    use_sizes(w["sizes"])
    layers = args.layers or SIZES["num_hidden_layers"]
    info = model_flops_bytes(SIZES, layers)
    prompts_ = workload_prompts(w)
    need_tokens = sum(len(p) for p in prompts_) + w["n"] * w["new"]
    pool_mb = w["pool_share"] * need_tokens * info["kv_bytes_per_token"] / 2 ** 20
    tmp = make_model_dir(layers)
    base = dict(model=tmp.name, dtype="bfloat16", block_size=PAGE, max_model_len=w["context"], max_num_seqs=w["n"],
                kv_cache_mb=pool_mb, **w["engine"])
    try:
        if args.impl == "reference":
            ref = ROOT / "baseline" / "_ref"
            if not (ref / "infer").is_dir():
                return {"impl": "reference", "unavailable": "baseline/_ref/infer is not installed on this machine"}
            sys.path.insert(0, str(ref))
            from infer.config import EngineConfig
            from infer.engine.engine import LLMEngine
            from infer.engine.sequence import SamplingParams
            from infer.model.loader import load_model
            model = load_model(tmp.name, torch.bfloat16, torch.device("cuda:0"), max_positions=w["context"])
            engine = LLMEngine(EngineConfig(device="cuda:0", cuda_graphs=True, request_timeout=None, **base), model=model)
        else:
            from tokenmill_b200 import EngineConfig
            from tokenmill_b200.engine import LLMEngine
            from tokenmill_b200.sampling import SamplingParams
            engine = LLMEngine(EngineConfig(cuda_graphs=True, cuda_graph_max_batch=max(64, w["n"]), **base))   # (graphs on in both arms)
        if hasattr(engine, "capture_graphs"):
            engine.capture_graphs()             # (the reference captures its graphs when the engine is built)
        sp = SamplingParams(max_tokens=w["new"], ignore_eos=True)
        warm = engine.generate([prompts_[0][:64]], SamplingParams(max_tokens=4, ignore_eos=True))    # compile / warm paths
        assert len(warm[0]) == 4
        for i, p in enumerate(prompts_):
            engine.add_request(f"w{i}", p, sp)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        n_out = 0
        while engine.has_unfinished():
            n_out += sum(len(o.new_token_ids) for o in engine.step())
        if hasattr(engine, "drain"):
            n_out += sum(len(o.new_token_ids) for o in engine.drain())
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        sched, cache = engine.scheduler, engine.cache
        preempted = getattr(sched, "evictions", getattr(sched, "num_preemptions", 0))
        hit = getattr(cache, "prefix_hit_tokens", None)
        asked = getattr(cache, "prefix_query_tokens", None)
        if hit is None:                                           # the reference's counters live on its block manager
            hit, asked = getattr(cache, "hit_tokens", 0), getattr(cache, "query_tokens", 0)
        stats = engine.stats
    finally:
        tmp.cleanup()
    return {"workload": args.workload, "impl": args.impl, "metric": "generated tok/s, all requests submitted at once",
            "value": round(n_out / wall, 1), "unit": "tokens/s", "wall_s": round(wall, 3), "generated_tokens": n_out,
            "prompt_tokens": sum(len(p) for p in prompts_), "requests": w["n"], "new_tokens": w["new"],
            "preemptions": int(preempted), "prefix_hit_rate": round(hit / asked, 4) if asked else 0.0,
            "steps": stats.get("steps"), "peak_running": stats.get("peak_running"),
            "config": {"model": f"{MODEL_LABEL} sizes", "layers": layers, "layers_in_named_config": SIZES["num_hidden_layers"],
                       "context": w["context"], "kv_page": PAGE, "kv_pool_mb": round(pool_mb, 1),
                       "pool_share_of_need": w["pool_share"], **{k: v for k, v in w["engine"].items()}},
            "dtype": "bf16", "data": "synthetic token ids, random weights seed 0"}


def run_reference(args) -> dict:
    """The unmodified reference, installed under baseline/_ref, through its own LLMEngine: the same
    random model folder, bfloat16, its paged engine with its CUDA graphs enabled."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "infer").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref/infer is not installed on this machine"}
    sys.path.insert(0, str(ref))
    try:
        import torch
        from infer.config import EngineConfig
        from infer.engine.engine import LLMEngine
        from infer.engine.sequence import SamplingParams
        from infer.model.loader import load_model
    except Exception as e:  # a dependency of the reference is missing
        return {"impl": "reference", "unavailable": f"the reference does not import here: {type(e).__name__}: {e}"}
    layers = args.layers or SIZES["num_hidden_layers"]
    info = model_flops_bytes(SIZES, layers)
    tmp = make_model_dir(layers)
    try:
        dev = torch.device("cuda:0")
        model = load_model(tmp.name, torch.bfloat16, dev, max_positions=CONTEXT)
        cfg = EngineConfig(model=tmp.name, dtype="bfloat16", device="cuda:0", block_size=PAGE, max_model_len=CONTEXT,
                           max_num_seqs=64, max_num_batched_tokens=4 * PROMPT_LEN,
                           kv_cache_mb=64 * CONTEXT * info["kv_bytes_per_token"] / 2 ** 20, watermark=0.0,
                           cuda_graphs=True, cuda_graph_max_batch=64, request_timeout=None)
        engine = LLMEngine(cfg, model=model)
        sampler = ClockSampler()

        def timed(batch, steps, warmup):
            forward = max(0, NEW_TOKENS // 2 - steps // 2 - warmup)      # the timed steps: the middle of the new tokens
            sp = SamplingParams(max_tokens=forward + steps + warmup + 4, ignore_eos=True)
            seqs = [engine.add_request(f"r-{batch}-{i}-{time.time_ns()}", p, sp)
                    for i, p in enumerate(prompts(batch, PROMPT_LEN, seed=99))]
            while any(s.num_output_tokens == 0 for s in seqs):
                engine.step()
            for _ in range(forward + warmup):
                engine.step()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            start.record()
            n = 0
            for _ in range(steps):
                n += sum(len(o.new_token_ids) for o in engine.step())
            end.record()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            ctx = statistics.mean(s.length for s in seqs) - steps / 2
            for s in seqs:
                engine.abort_request(s.id)
            return {"tok_s_dev": n / (start.elapsed_time(end) / 1e3), "tok_s": n / dt, "ms": 1e3 * dt / steps,
                    "mean_ctx": ctx}

        timed(BATCH, 4, 3)
        sampler.start()
        main = timed(BATCH, args.steps, args.warmup)
        b1 = timed(1, max(16, args.steps // 2), args.warmup)
        b64 = timed(64, max(16, args.steps // 2), args.warmup)
        sp = SamplingParams(max_tokens=1, ignore_eos=True)
        pre = []
        for i in range(6):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            engine.generate([prompts(1, PREFILL_TOKENS, seed=5)[0]], sp)
            torch.cuda.synchronize()
            pre.append(1e3 * (time.perf_counter() - t0))
        clocks = sampler.stop()
    finally:
        tmp.cleanup()
    pf_ms = statistics.median(pre[2:])
    return {
        "metric": f"decode tok/s at batch 8 ({MODEL_LABEL} sizes, prompt 512, bf16)", "value": round(main["tok_s_dev"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main["ms"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random weights seed 0", "impl": "reference",
        "config": bench_config(layers, main["mean_ctx"], {
            "l2": "inputs larger than L2 (weights read per step: %.0f MB)" % (info["weight_bytes"] / 1e6),
            "peaks": peaks()[1], "cuda_graphs": True}),
        "e2e": {"value": round(main["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": None,
                "d2h_bytes_per_step": BATCH * 8},
        "prefill": {"value": round(PREFILL_TOKENS / (pf_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pf_ms, 3)},
        "points": {"decode_b1": round(b1["tok_s_dev"], 1), "decode_b64": round(b64["tok_s_dev"], 1),
                   "e2e_b1": round(b1["tok_s"], 1), "e2e_b64": round(b64["tok_s"], 1)},
        "clocks": clocks,
    }


def main() -> int:
    global PROMPT_LEN, CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the named configuration (0 = all)")
    ap.add_argument("--sizes", default="", help="another named size (qwen2.5-1.5b, qwen2.5-7b) instead of Qwen2.5-0.5B")
    ap.add_argument("--only", default="", help="profiling aid: run only 'prefill', 'decode_b<batch>', 'products', 'sampling' or "
                         "'decode_attention[:<case>]' and print its time")
    ap.add_argument("--no-graphs", action="store_true", help="profiling aid: decode without CUDA graphs")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS)
    ap.add_argument("--prompt-len", type=int, default=0,
                    help="profiling aid with --only decode_b<batch>: prompts of this many tokens instead of 512")
    ap.add_argument("--no-skip", action="store_true", help="profiling aid: time the decode steps right behind the prompt")
    ap.add_argument("--no-fp32", action="store_true", help="leave out the float32 engine's points")
    ap.add_argument("--workload", default="", choices=["", *WORKLOADS],
                    help="run one of the other baseline workloads through LLMEngine instead of the headline bench")
    args = ap.parse_args()
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.sizes:
        use_sizes(args.sizes)
    if args.prompt_len:
        if not args.only.startswith("decode_b"):
            print("bench.py: --prompt-len goes with --only decode_b<batch>")
            return 2
        PROMPT_LEN, CONTEXT = args.prompt_len, max(CONTEXT, args.prompt_len + NEW_TOKENS + 64)
    if args.only == "prefill":
        CONTEXT = max(CONTEXT, args.prefill_tokens + 64)
    if args.workload:
        result = run_workload(args)
    else:
        result = run_reference(args) if args.impl == "reference" else run_ours(args)
    if result:
        print(json.dumps(result), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
