"""The parts that layers are put together from, and their registries."""
from .base import (BLOCKS, EMBEDDINGS, ENTRIES, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS,
                   CacheNeed, Part, StateNeed, TensorNeed, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position)
from . import (attention, block, embedding, feedforward, latent_attention, moe, norm,  # noqa: F401
               position, recurrent, linear_state, side_by_side)
from .linear import Linear

__all__ = ["BLOCKS", "EMBEDDINGS", "ENTRIES", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS",
           "CacheNeed", "Part", "StateNeed", "TensorNeed", "Linear", "register_block",
           "register_feed_forward", "register_mixer", "register_norm", "register_position"]
