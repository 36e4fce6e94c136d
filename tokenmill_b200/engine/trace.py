"""Trace replay: feed given token ids through the model step by step and write logits.

Nothing is sampled and nothing is scheduled: each input line names the step's entries, and the
step function (``ModelRunner.step``), the cache manager, the page pools and the kernels are the very
ones generation uses. The reference has no such program; its nearest pieces are the teacher-forced
cache-versus-no-cache checks in its tests (tests/test_model_equivalence.py:48-65).

Input, one JSON object per line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at the wanted
places, in the order of the entries and of ``want``, as little-endian float32 [wanted, vocab]. After
every step a line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

PAGE_SIZE = 16           # tokens per cache page unless --page-size says otherwise
LIVE_REQUESTS = 4        # requests that may be live at a time (state slots are kept for twice as many)


def run(model_dir: str, dtype_name: str, out_dir: str, max_tokens: int, stdin=None, stdout=None,
        device: str = "cuda:0", page_size: int = PAGE_SIZE, state_slots: int = 2 * LIVE_REQUESTS) -> int:
    from ..cache.manager import CacheManager
    from ..cache.pool import CachePools
    from ..kernels import ops
    from ..weights.loader import load_model, resolve_dtype
    from .batch import StepEntry
    from .runner import ModelRunner

    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    if not torch.cuda.is_available():
        raise RuntimeError("trace_run drives the engine's CUDA kernels; no CUDA device is visible")
    dtype = resolve_dtype(dtype_name)
    dev = torch.device(device)
    model = load_model(model_dir, dtype, dev)
    layout = model.cache_layout()
    # The pool holds exactly the pages max_tokens needs (live requests each rounded up to 64 tokens,
    # a multiple of the page size), so pages freed by one request are reused by the next.
    if page_size < 1 or 64 % page_size:
        raise ValueError(f"--page-size must divide 64 (requests are counted in units of 64 tokens), got {page_size}")
    num_pages = max(1, -(-max_tokens // page_size))
    n_groups = len(layout.groups)
    n_state = state_slots if layout.entry_state else 0
    cache = CacheManager([num_pages] * n_groups, page_size, layout.windows, watermark=0.0,
                         enable_prefix_caching=False, num_state_slots=n_state)
    pools = CachePools(layout, [num_pages] * n_groups, page_size, dtype, dev, num_state_slots=n_state,
                       run_order_cache_of=[e.cache_of for e in model.spec.run_order])
    runner = ModelRunner(model, cache, pools, max_model_len=model.max_positions())
    vocab = model.spec.vocab_size

    live: dict[str, tuple] = {}         # id -> (handle, tokens held)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        step_no = msg["step"]
        entries = []
        for e in msg.get("entries", []):
            rid, tokens = str(e["id"]), [int(t) for t in e["tokens"]]
            if not tokens:
                continue
            if any(not (0 <= t < vocab) for t in tokens):
                raise ValueError(f"step {step_no}: a token id of request {rid} lies outside the vocabulary")
            handle, held = live.get(rid, (None, 0))
            if handle is None:
                handle = cache.new_handle()
                cache.allocate(handle, tokens)
            else:
                cache.grow(handle, held + len(tokens))
            entries.append(StepEntry(handle, tokens, held, [int(w) for w in e.get("want", [])]))
            live[rid] = (handle, held + len(tokens))
        if entries:
            logits = runner.step(entries)
            if logits.shape[0] > 0:
                arr = logits.detach().to("cpu", torch.float32).contiguous().numpy()
                ops.tc_check(runner.device)          # (the copy above has waited for the step)
                arr.astype("<f4", copy=False).tofile(out / f"{step_no}.f32")
            for e in entries:
                cache.release_behind_window(e.handle, e.start + len(e.tokens))
        for rid in msg.get("end", []):
            handle, _ = live.pop(str(rid), (None, 0))
            if handle is not None:
                cache.free(handle)
        stdout.write(f"done {step_no}\n")
        stdout.flush()
    return 0


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE, help="tokens per cache page (a divisor of 64)")
    ap.add_argument("--state-slots", type=int, default=2 * LIVE_REQUESTS,
                    help="slots for fixed-size per-request state, for models whose mixers keep some")
    args = ap.parse_args(argv)
    return run(args.model, args.dtype, args.out, args.max_tokens, device=args.device, page_size=args.page_size,
               state_slots=args.state_slots)


if __name__ == "__main__":
    sys.exit(main())
