from .loader import WeightError, load_model, load_tensors, read_spec, resolve_dtype
from .random_init import named_config, qwen2_config, write_random_model

__all__ = ["WeightError", "load_model", "load_tensors", "read_spec", "resolve_dtype",
           "named_config", "qwen2_config", "write_random_model"]
