"""Parts a model is put together from, their specs and registries."""
from . import attention, block, mlp, norm, position  # noqa: F401  (register the built-in parts)
from .base import Block, CacheBinding, FeedForward, Mixer, Norm, Part, PositionEncoding
from .registry import (
    build_block, build_feed_forward, build_mixer, build_norm, build_position_encoding,
    register_block, register_feed_forward, register_mixer, register_norm, register_position_encoding,
)
from .spec import (
    AttentionSpec, BlockSpec, GatedMlpSpec, LayerCall, ModelSpec, NormSpec, ParamInfo, PositionSpec,
)

__all__ = [
    "Block", "CacheBinding", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
    "build_block", "build_feed_forward", "build_mixer", "build_norm", "build_position_encoding",
    "register_block", "register_feed_forward", "register_mixer", "register_norm",
    "register_position_encoding", "AttentionSpec", "BlockSpec", "GatedMlpSpec", "LayerCall",
    "ModelSpec", "NormSpec", "ParamInfo", "PositionSpec",
]
