"""Parts a layer is put together from; importing this package registers the built-in kinds."""
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, CacheSpec, TensorDecl, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "CacheSpec", "TensorDecl", "register_block",
           "register_feed_forward", "register_mixer", "register_norm", "register_position"]
