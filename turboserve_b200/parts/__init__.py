"""Parts a model is put together from; importing the package registers the built-in kinds."""

from .base import (
    BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, FeedForward, LogitHead, Mixer, Norm, PagedKVNeed,
    ParamSpec, Part, PositionEncoding, ScaledUpdates, StateNeed, StreamShifts, TokenEmbedding, STREAM_SHIFTS, register_stream_shifts, register_block, register_embedding, register_feed_forward,
    register_head, register_mixer, register_norm, register_position,
)
from . import (attention, block, diff_attention, latent_attention, mamba1, mamba2, mlp, moe, norm, retention, rope, side_by_side,
               sink_attention, vocabulary, wkv)  # noqa: F401,E402  (registration)

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "FeedForward", "LogitHead", "Mixer",
    "Norm", "PagedKVNeed", "ParamSpec", "Part", "PositionEncoding", "ScaledUpdates", "StateNeed", "StreamShifts", "STREAM_SHIFTS",
    "register_stream_shifts", "TokenEmbedding", "register_block",
    "register_embedding", "register_feed_forward", "register_head", "register_mixer", "register_norm", "register_position",
]
