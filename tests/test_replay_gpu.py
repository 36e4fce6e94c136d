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


def _steps_for(mode, reqs):
    if mode == "whole":
        return whole_steps(reqs)
    if mode == "tail":
        return tail_decode_steps(reqs)
    if mode == "portions":
        return portion_steps(reqs, seed=5)
    return mixed_steps(reqs, seed=7)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["tail", "mixed"])
def test_replay_with_pages_of_8_tokens(tiny_b_dir, dtype, mode, tmp_path, plain_cache):
    """The second tiny configuration with the page size its benchmark configuration names (8): twice as many
    page edges, block tables twice as wide, the same logits."""
    reqs = make_requests(_vocab(tiny_b_dir), LENGTHS, seed=13)
    steps, max_tokens = _steps_for(mode, reqs)
    outputs = run_trace(tiny_b_dir, dtype, steps, max_tokens, tmp_path / "out", page_size=8)
    check_against_plain(steps, outputs, reqs, plain_for(tiny_b_dir, reqs, plain_cache), dtype)


@pytest.mark.parametrize("page", [8, 32])
@pytest.mark.parametrize("mode", ["tail", "mixed", "portions"])
def test_heads_of_64_replay_at_other_page_sizes(d64_dir, page, mode, tmp_path, plain_cache):
    """The kernels serving uses for heads of 64 (whole-step decode kernel, tensor-core decode and prompt
    attention) over pages of 8 and of 32 tokens, against the plain implementation."""
    from tokenmill_b200.kernels import lib
    reqs = make_requests(_vocab(d64_dir), [70, 133, 45, 200, 96, 61], seed=17)
    steps, max_tokens = _steps_for(mode, reqs)
    before = lib.launch_count
    outputs = run_trace(d64_dir, "bfloat16", steps, max_tokens, tmp_path / "out", page_size=page)
    assert lib.launch_count > before
    check_against_plain(steps, outputs, reqs, plain_for(d64_dir, reqs, plain_cache), "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("size", ["0.5b", "1.5b", "7b"])
def test_replay_at_the_real_layer_sizes(real_size_dir, size, dtype, tmp_path, plain_cache):
    """Two layers of the Qwen2.5-0.5B, 1.5B and 7B layer sizes (small vocabulary), each request whole, in
    portions and mixed with others over a pool with no spare page, in float32 and in bfloat16, against the
    plain implementation: the widths, head counts and groupings that serving meets, through the kernels that
    serving picks for them."""
    folder = real_size_dir(size)
    reqs = make_requests(_vocab(folder), [70, 133, 45, 96], seed=19)
    plain = plain_for(folder, reqs, plain_cache)
    for mode in ("whole", "portions", "mixed"):
        steps, max_tokens = _steps_for(mode, reqs)
        outputs = run_trace(folder, dtype, steps, max_tokens, tmp_path / mode)
        worst = check_against_plain(steps, outputs, reqs, plain, dtype)
        print(f"{size} {dtype} {mode}: worst |engine - plain| = {worst:.3e}")


# Shapes no named model has, each a corner of what the kernels say they take: head size, kv heads, heads per kv
# head, width (no multiple of 32: the last 32-wide chunk of a staged row is part padding), feed-forward width,
# vocabulary, layers, page size.
OTHER_SHAPES = [(128, 4, 3, 112, 296, 301, 3, 8), (128, 4, 2, 144, 352, 777, 2, 8), (128, 3, 2, 440, 1032, 2050, 3, 16),
                (64, 4, 3, 112, 296, 301, 3, 32), (128, 4, 5, 280, 696, 777, 2, 16), (64, 1, 7, 72, 200, 515, 2, 16),
                (96, 1, 7, 384, 1192, 515, 2, 8), (16, 2, 8, 552, 272, 515, 2, 32)]


@pytest.mark.parametrize("shape", OTHER_SHAPES, ids=lambda s: "d%d_kv%d_g%d_h%d" % s[:4])
def test_replay_of_shapes_no_named_model_has(shape, tmp_path, plain_cache):
    """Whole, last tokens one by one, portions and mixed, in bfloat16 (the whole-step kernel, the tensor-core
    attention kernels and the generic ones, whichever take the shape) and whole + mixed in float32, against the
    plain implementation. (A width of 112 through the whole-step kernel gave NaN logits in most runs while the
    padding columns of its staged rows were left as an earlier phase had written them.)"""
    from tokenmill_b200.weights import qwen2_config, write_random_model
    D, nkv, G, H, I, V, L, page = shape
    cfg = qwen2_config(vocab_size=V, hidden_size=H, intermediate_size=I, num_hidden_layers=L, num_attention_heads=nkv * G,
                       num_key_value_heads=nkv, head_dim=D, rope_theta=50000.0, rms_norm_eps=3e-6,
                       tie_word_embeddings=bool(H % 16), max_position_embeddings=1024)
    folder = write_random_model(tmp_path / "model", cfg, seed=D + H)
    reqs = make_requests(V, [216, 45, 207, 172, 153], seed=H)
    plain = plain_for(folder, reqs, plain_cache)
    for dtype, modes in (("bfloat16", ("whole", "tail", "portions", "mixed")), ("float32", ("whole", "mixed"))):
        for mode in modes:
            steps, max_tokens = _steps_for(mode, reqs)
            outputs = run_trace(folder, dtype, steps, max_tokens, tmp_path / f"{dtype}_{mode}", page_size=page)
            check_against_plain(steps, outputs, reqs, plain, dtype)


def test_modes_agree_in_float32(tiny_b_dir, tmp_path):
    """The same position's logits under different cuts. Every reduction has a fixed order, so in float32 they
    are EQUAL to the last bit for every position with at most 128 keys, however the tokens were cut and batched.
    Beyond 128 keys one thing moves: a step in which every request brings few rows has each request's keys cut
    at absolute multiples of 128 across blocks and the partial results merged in index order, while a step with
    long portions walks a row's keys in one pass; the two orders differ in the last bits (measured: 4.8e-7 on
    logits of about 0.5)."""
    reqs = make_requests(_vocab(tiny_b_dir), [150, 77, 300], seed=3)
    s1, m1 = whole_steps(reqs)
    o1 = run_trace(tiny_b_dir, "float32", s1, m1, tmp_path / "a")
    whole = {rid: o1[i] for i, rid in enumerate(reqs)}
    cuts = {"portions": portion_steps(reqs, seed=9), "tail": tail_decode_steps(reqs), "mixed": mixed_steps(reqs, seed=7)}
    for label, (s2, m2) in cuts.items():
        o2 = run_trace(tiny_b_dir, "float32", s2, m2, tmp_path / label)
        fed = {rid: 0 for rid in reqs}
        for s in s2:
            row = 0
            for e in s["entries"]:
                start = fed[e["id"]]
                for w in e["want"]:
                    got, ref = o2[s["step"]][row], whole[e["id"]][start + w]
                    if start + w < 128:
                        assert np.array_equal(got, ref), (label, s["step"], e["id"], start + w)
                    else:
                        assert np.abs(got - ref).max() <= 2e-6 * max(1.0, np.abs(ref).max())
                    row += 1
                fed[e["id"]] = start + len(e["tokens"])


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
