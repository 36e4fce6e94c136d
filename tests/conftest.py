"""Shared fixtures: two tiny random Qwen2 model folders that differ in every size and option.

Tiny A: 2 layers, hidden 64, 4 query heads over 2 kv heads, head size 16, feed-forward 128, vocabulary
256, theta 1e4, eps 1e-6, tied output. Tiny B: 3 layers, hidden 96, 3 query heads over 1 kv head, head
size 32, feed-forward 160, vocabulary 384, theta 1e6, eps 1e-5, separate output matrix. Both are
written by the package's random-weights mode into a temporary folder (never into the repository).
"""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (sm_100a) and the compiled kernels")


def _make(tmp_path_factory, name: str, seed: int) -> Path:
    from tokenmill_b200.weights import named_config, write_random_model

    folder = tmp_path_factory.mktemp(name)
    write_random_model(folder, named_config(name), seed=seed)       # stored in bfloat16
    return folder


@pytest.fixture(scope="session")
def tiny_a_dir(tmp_path_factory) -> Path:
    return _make(tmp_path_factory, "tiny-a", 0)


@pytest.fixture(scope="session")
def tiny_b_dir(tmp_path_factory) -> Path:
    return _make(tmp_path_factory, "tiny-b", 1)


@pytest.fixture(scope="session", params=["tiny-a", "tiny-b"])
def tiny_dir(request, tiny_a_dir, tiny_b_dir) -> Path:
    return tiny_a_dir if request.param == "tiny-a" else tiny_b_dir


@pytest.fixture(scope="session")
def d64_dir(tmp_path_factory) -> Path:
    """A small model whose head size (64) the tensor-core kernels and the whole-step decode kernel take:
    3 layers, hidden 192, 6 query heads over 2 kv heads, feed-forward 328, vocabulary 500, untied."""
    from tokenmill_b200.weights import qwen2_config, write_random_model
    cfg = qwen2_config(vocab_size=500, hidden_size=192, intermediate_size=328, num_hidden_layers=3,
                       num_attention_heads=6, num_key_value_heads=2, head_dim=64, rope_theta=50000.0,
                       rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=2048)
    assert cfg["hidden_size"] != cfg["num_attention_heads"] * cfg["head_dim"]      # o_proj is not square
    return write_random_model(tmp_path_factory.mktemp("d64"), cfg, seed=9)


# Two layers of each layer size the benchmarks name, with a small vocabulary (the output matrix is not what
# differs between them): hidden, query heads, kv heads, head size, feed-forward, tied output.
REAL_LAYER_SIZES = {
    "0.5b": dict(hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
                 intermediate_size=4864, tie_word_embeddings=True),
    "1.5b": dict(hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, head_dim=128,
                 intermediate_size=8960, tie_word_embeddings=True),
    "7b": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
               intermediate_size=18944, tie_word_embeddings=False),
}
_real_dirs: dict[str, Path] = {}


@pytest.fixture(scope="session")
def real_size_dir(tmp_path_factory):
    """``real_size_dir(name)`` -> folder of a 2-layer random model with the named layer sizes (made once)."""
    from tokenmill_b200.weights import qwen2_config, write_random_model

    def get(name: str) -> Path:
        if name not in _real_dirs:
            cfg = qwen2_config(vocab_size=1000, num_hidden_layers=2, rope_theta=1000000.0, rms_norm_eps=1e-6,
                               max_position_embeddings=4096, **REAL_LAYER_SIZES[name])
            _real_dirs[name] = write_random_model(tmp_path_factory.mktemp("real_" + name.replace(".", "_")), cfg,
                                                  seed=4)
        return _real_dirs[name]
    return get


@pytest.fixture(scope="session")
def wide_dir(real_size_dir) -> Path:
    """Two layers of the Qwen2.5-0.5B layer sizes (hidden 896, 14 query heads over 2 kv heads of 64,
    feed-forward 4864) with a small vocabulary: the shapes for which the whole-step kernel's work split is
    made (5 gate/up units on some blocks, a down-projection input of 78 KB per 8 tokens, few ring stages)."""
    return real_size_dir("0.5b")


@pytest.fixture(scope="session")
def plain_cache():
    """Memo of plain-implementation logits per (folder, token tuple)."""
    return {}
