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
def plain_cache():
    """Memo of plain-implementation logits per (folder, token tuple)."""
    return {}
