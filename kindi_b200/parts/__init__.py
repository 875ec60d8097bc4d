"""The parts a layer is put together from: norms, position encodings, mixers, feed-forwards and the block that
arranges them. Importing this package registers the built-in kinds."""
from .base import (Block, Branch, FeedForward, KVNeed, Mixer, Norm, Part, PositionEncoding, StateNeed, StepContext,
                   WeightView)
from . import norm, rope, attention, mlp, block      # noqa: F401  (they register themselves)
