"""Parts a layer is built from.  Importing this package registers the built-in kinds."""
from . import attention, block, embedding, head, rms_norm, rotary, swiglu  # noqa: F401
from .base import (Block, Embedding, FeedForward, FixedState, Head, Mixer, Norm, PagedCacheView, PagedKV, Part,
                   PositionEncoding, Runtime, StateView, WeightSpec)
from .spec import LayerSpec, ModelSpec, PartSpec

__all__ = ["Block", "Embedding", "FeedForward", "FixedState", "Head", "Mixer", "Norm", "PagedCacheView", "PagedKV",
           "Part", "PositionEncoding", "Runtime", "StateView", "WeightSpec", "LayerSpec",
           "ModelSpec", "PartSpec"]
