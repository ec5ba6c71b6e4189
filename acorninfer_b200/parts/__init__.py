"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""

from . import attention, block, feed_forward, norms, rope  # noqa: F401
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, BuildContext,  # noqa: F401
                   CacheNeeds, FeedForward, KVNeeds, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec,
                   PositionEncoding, ScheduleEntry, StateNeeds, TensorSpec)
