"""Helpers for the replay tests: build step lists, run them through the engine's trace replay
in-process, and compare every written row with the plain implementation's whole-sequence logits."""

from __future__ import annotations

import io
import json
import random
from pathlib import Path

import numpy as np
import torch

from plain_qwen2 import load_plain, plain_logits, tolerance


def make_requests(vocab: int, lengths: list[int], seed: int) -> dict[str, list[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(vocab) for _ in range(n)] for i, n in enumerate(lengths)}


def round64(n: int) -> int:
    return -(-n // 64) * 64


def whole_steps(reqs: dict[str, list[int]]):
    """Each request alone and whole, one step each."""
    steps = []
    for i, (rid, toks) in enumerate(reqs.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps, max(round64(len(t)) for t in reqs.values())


def tail_decode_steps(reqs: dict[str, list[int]], tail: int = 32):
    """Most of each request in one step, its last ``tail`` tokens one by one."""
    steps, n = [], 0
    for rid, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for p in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps, max(round64(len(t)) for t in reqs.values())


def portion_steps(reqs: dict[str, list[int]], seed: int):
    """Each request alone, in portions of changing size, down to two tokens."""
    rng = random.Random(seed)
    steps, n = [], 0
    for rid, toks in reqs.items():
        pos = 0
        sizes = [2, 3, 17, 2, 31, 5, 64, 2, 9]
        k = 0
        while pos < len(toks):
            size = sizes[k % len(sizes)] if k < len(sizes) else rng.choice([2, 3, 7, 16, 33, 50])
            size = min(size, len(toks) - pos)
            if len(toks) - pos - size == 1:       # never leave a single token: portions go down to two
                size += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[pos:pos + size],
                                                  "want": list(range(size))}],
                          "end": [rid] if pos + size == len(toks) else []})
            pos += size
            n += 1
            k += 1
    return steps, max(round64(len(t)) for t in reqs.values())


def mixed_steps(reqs: dict[str, list[int]], seed: int, max_live: int = 4, decode_tail: int = 12):
    """Up to ``max_live`` live requests; portions of some beside single decoded tokens of others; a
    request may sit a step out. Returns (steps, max_tokens) with max_tokens the exact peak of the live
    requests' rounded-up lengths, so the pool has no spare page and freed pages are reused."""
    rng = random.Random(seed)
    pending = list(reqs.items())
    live: dict[str, int] = {}            # id -> tokens fed so far
    steps, n, peak = [], 0, 0
    while pending or live:
        while pending and len(live) < max_live and rng.random() < 0.7:
            rid, _ = pending.pop(0)
            live[rid] = 0
        if not live:
            rid, _ = pending.pop(0)
            live[rid] = 0
        peak = max(peak, sum(round64(len(reqs[r])) for r in live))
        entries, ended = [], []
        for rid in list(live):
            toks, fed = reqs[rid], live[rid]
            if fed > 0 and rng.random() < 0.2:
                continue                          # sits this step out
            left = len(toks) - fed
            if left <= decode_tail:
                size = 1                          # decoding, token by token
            else:
                size = min(rng.choice([2, 3, 5, 8, 13, 16, 21, 40]), left - decode_tail)
                if size < 2:
                    size = min(2, left)
            entries.append({"id": rid, "tokens": toks[fed:fed + size], "want": list(range(size))})
            live[rid] = fed + size
            if live[rid] == len(toks):
                ended.append(rid)
        for rid in ended:
            del live[rid]
        if entries:
            steps.append({"step": n, "entries": entries, "end": ended})
            n += 1
    return steps, peak


def run_trace(model_dir: Path, dtype: str, steps: list[dict], max_tokens: int, out_dir: Path,
              page_size: int | None = None) -> dict[int, np.ndarray]:
    from tokenmill_b200.engine.trace import PAGE_SIZE, run

    out_dir.mkdir(parents=True, exist_ok=True)
    stdin = io.StringIO("".join(json.dumps(s) + "\n" for s in steps))
    stdout = io.StringIO()
    assert run(str(model_dir), dtype, str(out_dir), max_tokens, stdin=stdin, stdout=stdout,
               page_size=page_size or PAGE_SIZE) == 0
    done = [line for line in stdout.getvalue().splitlines() if line.startswith("done ")]
    assert [int(d.split()[1]) for d in done] == [s["step"] for s in steps]
    vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    out = {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        f = out_dir / f"{s['step']}.f32"
        if wanted:
            out[s["step"]] = np.fromfile(f, dtype="<f4").reshape(wanted, vocab)
        else:
            assert not f.exists()
    return out


def plain_for(model_dir: Path, reqs: dict[str, list[int]], memo: dict) -> dict[str, torch.Tensor]:
    cfg, w = None, None
    out = {}
    for rid, toks in reqs.items():
        key = (str(model_dir), tuple(toks))
        if key not in memo:
            if cfg is None:
                cfg, w = load_plain(model_dir)
            memo[key] = plain_logits(cfg, w, toks)
        out[rid] = memo[key]
    return out


def check_against_plain(steps, outputs, reqs, plain, dtype: str) -> float:
    """Every written row equals the plain logits at that request's position, within the dtype's
    tolerance. Returns the largest difference seen; on failure names the first wrong row."""
    fed = {rid: 0 for rid in reqs}
    worst = 0.0
    for s in steps:
        row = 0
        for e in s["entries"]:
            start = fed[e["id"]]
            for wpos in e["want"]:
                got = torch.from_numpy(outputs[s["step"]][row])
                ref = plain[e["id"]][start + wpos]
                diff = float((got - ref).abs().max())
                tol = tolerance(ref, dtype)
                assert diff <= tol, (f"step {s['step']} request {e['id']} position {start + wpos} "
                                     f"(portion starts at {start}, {len(e['tokens'])} tokens): "
                                     f"|engine - plain| = {diff:.3e} > {tol:.3e}")
                worst = max(worst, diff)
                row += 1
            fed[e["id"]] = start + len(e["tokens"])
    return worst
