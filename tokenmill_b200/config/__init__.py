from .engine_config import EngineConfig, add_engine_args, engine_config_from_args
from .model_config import ConfigError, Qwen2Config, read_config_json

__all__ = ["EngineConfig", "add_engine_args", "engine_config_from_args", "ConfigError", "Qwen2Config",
           "read_config_json"]
