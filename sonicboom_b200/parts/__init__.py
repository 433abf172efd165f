"""Parts a layer is put together from: norms, position encodings, mixers, feed-forwards and
their arrangement in a block; each kind is looked up by name in a registry."""
from .base import (BLOCKS, DEPTH_MIXES, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward,
                   Mixer, Norm, Part, PositionEncoding, StepContext, make, register_block,
                   register_depth_mix, register_feed_forward, register_mixer, register_norm,
                   register_position_encoding)
from . import (norm, rotary, attention, latent_attention, mlstm, window_attention, linear_recurrence,
               side_by_side, state_space, delta_rule, sigmoid_attention, feedforward, depth, block)  # noqa: F401  (fill the registries)

__all__ = ["BLOCKS", "DEPTH_MIXES", "register_depth_mix", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block",
           "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "StepContext", "make",
           "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position_encoding"]
