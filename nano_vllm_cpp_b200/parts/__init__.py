"""Parts that layers are put together from.  Importing this package registers the built-in kinds."""
from .base import (TensorSpec, KVCacheSpec, StateCacheSpec, RunContext, Part, Norm, PositionEncoding,
                   Mixer, FeedForward, PartSpec)
from .registry import register_part, build_part
from . import norm, rotary, attention, feedforward  # noqa: F401  (register themselves)
from .block import Arrangement, LayerSpec, PreNormBlock, build_layer
from .model import LayerCall, ModelSpec, Model

__all__ = ["TensorSpec", "KVCacheSpec", "StateCacheSpec", "RunContext", "Part", "Norm", "PositionEncoding",
           "Mixer", "FeedForward", "PartSpec", "register_part", "build_part", "LayerSpec", "Arrangement", "PreNormBlock",
           "build_layer", "LayerCall", "ModelSpec", "Model"]
