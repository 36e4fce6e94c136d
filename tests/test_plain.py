"""The plain implementation against the recorded outputs of the reference's own model code
(tests/golden/tiny_golden.json, made by tests/golden/make_golden.py), and its own consistency (CPU)."""

from __future__ import annotations

import json
from pathlib import Path

import pytest
import torch

from plain_qwen2 import (load_plain, plain_apply_rope, plain_causal_attention, plain_filtered_probs, plain_greedy,
                         plain_inverse_cdf, plain_logits, plain_rmsnorm, plain_rope_tables)
from tokenmill_b200.weights import write_random_model

GOLDEN = json.loads((Path(__file__).parent / "golden" / "tiny_golden.json").read_text())


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_plain_matches_the_reference_recording(name, tmp_path):
    rec = GOLDEN[name]
    folder = write_random_model(tmp_path / name, rec["config"], seed=rec["seed"], store_dtype="float32")
    cfg, w = load_plain(folder)
    for row in rec["rows"]:
        logits = plain_logits(cfg, w, row["prompt"])
        last = logits[-1]
        assert torch.allclose(last[:8], torch.tensor(row["last_logits_first8"]), atol=2e-6, rtol=0)
        top = last.topk(4)
        assert top.indices.tolist() == row["last_top4_ids"]
        assert torch.allclose(top.values, torch.tensor(row["last_top4_values"]), atol=2e-6, rtol=0)
        assert abs(float(logits.double().sum()) - row["logit_checksum"]) < 1e-3
        assert plain_greedy(cfg, w, row["prompt"], len(row["reference_greedy"])) == row["reference_greedy"]
        assert row["max_abs_diff_vs_reference"] < 1e-5


def _reference_src() -> Path | None:
    """Where the reference's ``infer`` package can be imported from: $TOKENMILL_REFERENCE_SRC, or the offline
    install under baseline/_ref of this checkout."""
    import os
    for cand in (os.environ.get("TOKENMILL_REFERENCE_SRC"), Path(__file__).resolve().parents[1] / "baseline" / "_ref"):
        if cand and (Path(cand) / "infer" / "model" / "qwen2.py").is_file():
            return Path(cand)
    return None


@pytest.mark.skipif(_reference_src() is None, reason="the reference's model code is not present in this checkout")
def test_plain_matches_the_reference_live(tmp_path):
    """The anchor again, not from the recording: the reference's own loader and whole-sequence forward pass on
    the CPU against the plain implementation, on a tiny random model (logits and greedy tokens)."""
    import sys
    sys.path.insert(0, str(Path(__file__).parent / "golden"))
    sys.path.insert(0, str(_reference_src()))
    try:
        import make_golden
        from tokenmill_b200.weights import named_config
        cfg_json = named_config("tiny-b")
        folder = write_random_model(tmp_path / "tiny-b", cfg_json, seed=5, store_dtype="float32")
        prompts = make_golden.prompts_for("tiny-b", cfg_json["vocab_size"])[:3]
        ref = make_golden.reference_outputs(folder, prompts, 6)
    finally:
        sys.path.remove(str(_reference_src()))
        for name in [m for m in sys.modules if m == "infer" or m.startswith("infer.")]:
            del sys.modules[name]
    cfg, w = load_plain(folder)
    for p, r in zip(prompts, ref):
        assert float((plain_logits(cfg, w, p) - r["logits"]).abs().max()) < 1e-5
        assert plain_greedy(cfg, w, p, 6) == r["greedy"]


def test_rmsnorm_formula():
    x = torch.randn(5, 12)
    w = torch.rand(12) + 0.5
    y = plain_rmsnorm(x, w, 1e-5)
    assert torch.allclose(y, w * x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5), atol=1e-6)


def test_rope_is_a_rotation_and_relative():
    cos, sin = plain_rope_tables(64, 16, 10000.0)
    assert cos.shape == (64, 16) and torch.equal(cos[:, :8], cos[:, 8:])
    q, k = torch.randn(1, 2, 16), torch.randn(1, 2, 16)
    a = (plain_apply_rope(q, cos, sin, [5]) * plain_apply_rope(k, cos, sin, [3])).sum(-1)
    b = (plain_apply_rope(q, cos, sin, [40]) * plain_apply_rope(k, cos, sin, [38])).sum(-1)
    assert torch.allclose(a, b, atol=1e-4)                       # scores depend on the distance only
    assert torch.allclose(plain_apply_rope(q, cos, sin, [9]).norm(), q.norm(), atol=1e-5)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    full = plain_causal_attention(q, k, v, 8 ** -0.5)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, 9.0                                     # the future does not matter
    assert torch.allclose(plain_causal_attention(q, k2, v2, 8 ** -0.5)[:4], full[:4], atol=1e-6)
    assert torch.allclose(full[0], v[0].repeat_interleave(2, dim=0), atol=1e-6)     # first token sees itself
    win = plain_causal_attention(q, k, v, 8 ** -0.5, window=2)
    k3 = k.clone()
    k3[:3] = 50.0                                                 # keys 0..2 lie outside query 4's window of 2
    assert torch.allclose(plain_causal_attention(q, k3, v, 8 ** -0.5, window=2)[4], win[4], atol=1e-6)
    tail = plain_causal_attention(q[4:], k, v, 8 ** -0.5)         # the last 2 queries over all 6 keys
    assert torch.allclose(tail, full[4:], atol=1e-6)


def test_sampling_reference_rules():
    logits = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0])
    p = plain_filtered_probs(logits, 1.0, top_k=2)
    assert (p > 0).tolist() == [True, True, False, False, False] and abs(float(p.sum()) - 1) < 1e-9
    p = plain_filtered_probs(logits, 1.0, top_p=0.6)              # p0 = .57: token 1 stays (mass before .57 <= .6)
    assert (p > 0).tolist() == [True, True, False, False, False]
    p = plain_filtered_probs(logits, 1.0, top_p=0.5)
    assert (p > 0).tolist() == [True, False, False, False, False]  # the first always stays
    sharp = plain_filtered_probs(logits, 0.25)
    assert sharp[0] > plain_filtered_probs(logits, 1.0)[0]
    probs = torch.tensor([0.1, 0.2, 0.3, 0.4])
    assert [plain_inverse_cdf(probs, u) for u in (0.0, 0.09, 0.1, 0.29, 0.31, 0.999)] == [0, 0, 1, 1, 2, 3]
