"""Parts a layer is put together from.  Importing this package registers the built-in ones."""

from .base import (Block, CacheSpec, CacheView, FeedForward, Mixer, Norm, Part,
                   PositionEncoding, StateSpec, StepContext, TensorSpec)
from . import norm, position, attention, feedforward, block  # noqa: F401  (registration)
from .model import DecoderModel

__all__ = ["Block", "CacheSpec", "CacheView", "FeedForward", "Mixer", "Norm", "Part",
           "PositionEncoding", "StateSpec", "StepContext", "TensorSpec", "DecoderModel"]
