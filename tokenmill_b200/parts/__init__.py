"""Parts a layer is made of. Importing this package registers the built-in kinds."""

from . import attention, block, norm, rope, swiglu  # noqa: F401
from .base import LayerCache, StepInputs
from .model import CacheGroup, CacheLayout, DecoderModel
from .spec import LayerSpec, ModelSpec, PagedKVNeed, PartSpec, RunEntry, StateNeed, WeightSpec

__all__ = ["LayerCache", "StepInputs", "CacheGroup", "CacheLayout", "DecoderModel", "LayerSpec", "ModelSpec",
           "PagedKVNeed", "PartSpec", "RunEntry", "StateNeed", "WeightSpec"]
