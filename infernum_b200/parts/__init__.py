"""Parts a decoder is composed of; importing this package registers the
built-in kinds."""

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS,
                   Block, FeedForward, LayerSpec, Mixer, ModelSpec, Norm, PagedCacheSpec, Part,
                   PartSpec, PositionEncoding, ResidualStream, Runtime, ScheduleItem, StateSpec,
                   WeightSpec, build_layer, register_block, register_feed_forward, register_mixer,
                   register_norm, register_position_encoding)
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registration)
