"""tokenmill_b200: a single-GPU inference engine for the Qwen2 dense decoder, written for sm_100a."""

__version__ = "0.1.0"

from .config import EngineConfig  # noqa: E402,F401
