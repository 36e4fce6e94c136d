"""Offline command line: model folder (or seeded random weights) in, generated token ids out.

    python -m tokenmill_b200.generate --model DIR --prompt-ids 1,2,3 --max-tokens 16
    python -m tokenmill_b200.generate --random-weights tiny-a --prompt-file prompts.jsonl --temperature 0.8

The engine flags carry the reference's names and meanings (src/infer/config.py:110-145; its only
command line, ``python -m infer.serve``, starts an HTTP server, which this engine does not have).
Prompts are token ids: ``--prompt-ids`` takes comma-separated ids (repeatable), ``--prompt-file`` a file
with one JSON list of ids per line. One JSON object per prompt is printed.
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile
import time

from .config.engine_config import add_engine_args, engine_config_from_args


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m tokenmill_b200.generate", description=__doc__.split("\n\n")[0])
    add_engine_args(ap)
    ap.set_defaults(max_model_len=None)      # unless given: the engine's default, or the model's own limit if that is less
    ap.add_argument("--prompt-ids", action="append", default=[], help="comma-separated token ids (repeatable)")
    ap.add_argument("--prompt-file", help="file with one JSON list of token ids per line")
    ap.add_argument("--max-tokens", type=int, default=16)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=-1)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--sampling-seed", type=int, default=None, help="seed of each request's random stream")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--random-weights", metavar="SIZE", help="write a random model of a named size "
                    "(tiny-a, tiny-b, qwen2.5-0.5b, qwen2.5-1.5b, qwen2.5-7b) to a temporary folder and use it")
    ap.add_argument("--weights-seed", type=int, default=0)
    args = ap.parse_args(argv)

    prompts = [[int(t) for t in s.split(",") if t.strip()] for s in args.prompt_ids]
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [json.loads(line) for line in f if line.strip()]
    if not prompts:
        ap.error("give --prompt-ids or --prompt-file")

    from .engine.llm_engine import LLMEngine
    from .sampling.params import SamplingParams

    tmp = None
    if args.random_weights:
        from .weights.random_init import named_config, write_random_model

        tmp = tempfile.TemporaryDirectory(prefix="tokenmill_random_")
        write_random_model(tmp.name, named_config(args.random_weights), seed=args.weights_seed)
        args.model = tmp.name
    if not args.model:
        ap.error("give --model or --random-weights")
    if args.max_model_len is None:
        from .config.engine_config import EngineConfig
        from .weights.loader import read_spec

        args.max_model_len = min(EngineConfig().max_model_len, read_spec(args.model)[0].max_positions)
    try:
        engine = LLMEngine(engine_config_from_args(args))
        params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k,
                                top_p=args.top_p, seed=args.sampling_seed, ignore_eos=args.ignore_eos)
        t0 = time.perf_counter()
        outs = engine.generate(prompts, params)
        dt = time.perf_counter() - t0
        for p, o in zip(prompts, outs):
            print(json.dumps({"prompt_ids": p, "output_ids": o}))
        n = sum(len(o) for o in outs)
        print(f"generated {n} tokens in {dt:.3f} s ({n / dt:.1f} tok/s), {engine.stats['steps']} steps",
              file=sys.stderr)
    finally:
        if tmp is not None:
            tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
