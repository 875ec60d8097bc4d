"""The parts a model is put together from: embeddings, norms, position encodings, mixers, feed-forwards, the block
that arranges them in a layer, and heads. Importing this package registers the built-in kinds."""
from .base import (Block, Branch, Embedding, FeedForward, Head, KVNeed, Mixer, Norm, Part, PositionEncoding, StateNeed,
                   StepContext, WeightView)
from . import embedding, norm, rope, attention, mlp, block, head      # noqa: F401  (they register themselves)
from .rope import RotationEncoding                                     # noqa: F401
