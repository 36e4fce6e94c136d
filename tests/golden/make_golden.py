"""Anchor the plain implementation (tests/plain_qwen2.py) on the reference's own model code.

The reference's model package (``infer.model``) imports and runs on the CPU, so this script builds
the two tiny test configurations with this repository's random-weights writer, loads the same
folders with the reference's loader, runs its whole-sequence forward pass (no cache) and its
single-sequence greedy path, and records a few logits and the greedy tokens. The recorded file
(tests/golden/tiny_golden.json) is committed; tests/test_plain.py compares the plain implementation
with it, and re-runs this comparison live (test_plain_matches_the_reference_live) when the reference's
package is present (baseline/_ref of the checkout, or $TOKENMILL_REFERENCE_SRC).

    python tests/golden/make_golden.py --reference-src <reference checkout>/src

Nothing of the reference is copied: it is imported and called.
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

CASES = {
    "tiny-a": {"seed": 0, "prompt_lens": [5, 17, 33], "greedy": 8},
    "tiny-b": {"seed": 1, "prompt_lens": [1, 9, 24, 40], "greedy": 8},
}


def prompts_for(name: str, vocab: int) -> list[list[int]]:
    gen = torch.Generator().manual_seed(1234 + CASES[name]["seed"])
    return [torch.randint(0, vocab, (n,), generator=gen).tolist() for n in CASES[name]["prompt_lens"]]


def reference_outputs(folder: Path, prompts, n_greedy: int):
    from infer.kv.context import NoCacheContext
    from infer.model.loader import load_model
    from infer.model.qwen2 import greedy_generate_reference

    model = load_model(folder, torch.float32, torch.device("cpu"))
    out = []
    with torch.inference_mode():
        for p in prompts:
            ids = torch.tensor(p)
            hidden = model(ids, torch.arange(len(p)), NoCacheContext.single(len(p), model.cfg))
            logits = model.compute_logits(hidden)
            out.append({"logits": logits, "greedy": greedy_generate_reference(model, p, n_greedy)})
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-src", required=True, help="the reference checkout's src folder")
    ap.add_argument("--out", default=str(HERE / "tiny_golden.json"))
    args = ap.parse_args()
    sys.path.insert(0, args.reference_src)

    from plain_qwen2 import load_plain, plain_greedy, plain_logits
    from tokenmill_b200.weights import named_config, write_random_model

    record = {}
    for name, case in CASES.items():
        with tempfile.TemporaryDirectory() as tmp:
            cfg_json = named_config(name)
            folder = write_random_model(Path(tmp) / name, cfg_json, seed=case["seed"], store_dtype="float32")
            prompts = prompts_for(name, cfg_json["vocab_size"])
            ref = reference_outputs(folder, prompts, case["greedy"])
            cfg, w = load_plain(folder)
            rows = []
            for p, r in zip(prompts, ref):
                mine = plain_logits(cfg, w, p)
                diff = float((mine - r["logits"]).abs().max())
                greedy = plain_greedy(cfg, w, p, case["greedy"])
                assert diff < 1e-5, f"{name}: plain implementation differs from the reference by {diff}"
                assert greedy == r["greedy"], f"{name}: greedy tokens differ: {greedy} vs {r['greedy']}"
                last = r["logits"][-1]
                top = last.topk(4)
                rows.append({"prompt": p, "max_abs_diff_vs_reference": diff, "reference_greedy": r["greedy"],
                             "last_logits_first8": [round(float(x), 7) for x in last[:8]],
                             "last_top4_ids": top.indices.tolist(),
                             "last_top4_values": [round(float(x), 7) for x in top.values],
                             "logit_checksum": round(float(r["logits"].double().sum()), 6)})
                print(f"{name} len {len(p)}: max |plain - reference| = {diff:.2e}, greedy equal")
            record[name] = {"config": cfg_json, "seed": case["seed"], "rows": rows}
    Path(args.out).write_text(json.dumps(record, indent=1))
    print("wrote", args.out)


if __name__ == "__main__":
    main()
