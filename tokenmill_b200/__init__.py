"""tokenmill_b200: a single-GPU inference engine for the Qwen2 dense decoder, written for sm_100a."""

__version__ = "0.1.0"

from .config import EngineConfig  # noqa: E402,F401


def __getattr__(name: str):
    """``LLMEngine`` and ``SamplingParams`` are importable from the package itself; they load on first use
    (the engine pulls in the kernels, which a configuration-only caller does not need)."""
    if name == "LLMEngine":
        from .engine import LLMEngine
        return LLMEngine
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
