"""Trace replay against the plain implementation: whole, tail decoded one by one, portions of
changing size, and mixed batches over a pool with no spare page; float32 and bfloat16; both tiny
configurations."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from replay_util import (check_against_plain, make_requests, mixed_steps, plain_for, portion_steps, run_trace,
                         tail_decode_steps, whole_steps)

pytestmark = pytest.mark.gpu

LENGTHS = [70, 133, 45, 200, 96, 61]


def _vocab(model_dir):
    return json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_matches_plain(tiny_dir, dtype, mode, tmp_path, plain_cache):
    reqs = make_requests(_vocab(tiny_dir), LENGTHS, seed=11)
    if mode == "whole":
        steps, max_tokens = whole_steps(reqs)
    elif mode == "tail":
        steps, max_tokens = tail_decode_steps(reqs)
    elif mode == "portions":
        steps, max_tokens = portion_steps(reqs, seed=5)
    else:
        steps, max_tokens = mixed_steps(reqs, seed=7)
        assert max(len(s["entries"]) for s in steps) >= 3
    outputs = run_trace(tiny_dir, dtype, steps, max_tokens, tmp_path / "out")
    worst = check_against_plain(steps, outputs, reqs, plain_for(tiny_dir, reqs, plain_cache), dtype)
    print(f"{Path(tiny_dir).name} {dtype} {mode}: worst |engine - plain| = {worst:.3e}")


def test_modes_agree_in_float32(tiny_b_dir, tmp_path):
    """The same position's logits under different cuts differ by rounding only."""
    reqs = make_requests(_vocab(tiny_b_dir), [150, 77], seed=3)
    s1, m1 = whole_steps(reqs)
    s2, m2 = portion_steps(reqs, seed=9)
    o1 = run_trace(tiny_b_dir, "float32", s1, m1, tmp_path / "a")
    o2 = run_trace(tiny_b_dir, "float32", s2, m2, tmp_path / "b")
    whole = {rid: o1[i] for i, rid in enumerate(reqs)}
    fed = {rid: 0 for rid in reqs}
    for s in s2:
        e = s["entries"][0]
        got = o2[s["step"]]
        ref = whole[e["id"]][fed[e["id"]]:fed[e["id"]] + len(e["tokens"])]
        assert np.abs(got - ref).max() <= 2e-6 * max(1.0, np.abs(ref).max())
        fed[e["id"]] += len(e["tokens"])


def test_trace_run_program(tiny_a_dir, tmp_path, plain_cache):
    """The executable itself, as a child process: done lines, files, exit code 0."""
    root = Path(__file__).resolve().parents[1]
    reqs = make_requests(_vocab(tiny_a_dir), [40, 23], seed=2)
    steps, max_tokens = mixed_steps(reqs, seed=1, max_live=2, decode_tail=4)
    steps.insert(1, {"step": 1000, "entries": [], "end": []})
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tiny_a_dir), "--dtype",
                           "float32", "--out", str(tmp_path / "o"), "--max-tokens", str(max_tokens)],
                          input=text, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    real = [s for s in steps if s["entries"]]
    outputs = {s["step"]: np.fromfile(tmp_path / "o" / f"{s['step']}.f32", dtype="<f4").reshape(
        sum(len(e["want"]) for e in s["entries"]), _vocab(tiny_a_dir)) for s in real}
    check_against_plain(real, outputs, reqs, plain_for(tiny_a_dir, reqs, plain_cache), "float32")
    assert not (tmp_path / "o" / "1000.f32").exists()
