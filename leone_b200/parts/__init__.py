"""Parts a layer is built from.  Importing this package registers the built-in kinds."""
from . import attention, block, rms_norm, rotary, swiglu  # noqa: F401
from .base import (Block, FeedForward, FixedState, Mixer, Norm, PagedCacheView, PagedKV, Part,
                   PositionEncoding, Runtime, StateView, WeightSpec)
from .spec import LayerSpec, ModelSpec, PartSpec

__all__ = ["Block", "FeedForward", "FixedState", "Mixer", "Norm", "PagedCacheView", "PagedKV",
           "Part", "PositionEncoding", "Runtime", "StateView", "WeightSpec", "LayerSpec",
           "ModelSpec", "PartSpec"]
