from .base import (KVRequest, ParamSpec, StateRequest, block_class, feed_forward_class,
                   mixer_class, norm_class, position_class, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position,
                   register_stream_position, stream_position_class)
from .norm import RMSNorm
from .rope import RotaryEmbedding
from .attention import AttentionMixer
from .feedforward import GatedFeedForward
from .block import Block
from .linear import GatedLinear, Linear

__all__ = ["KVRequest", "ParamSpec", "StateRequest", "feed_forward_class", "mixer_class",
           "norm_class", "position_class", "block_class", "stream_position_class",
           "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "register_stream_position", "RMSNorm", "RotaryEmbedding",
           "AttentionMixer", "GatedFeedForward", "Block", "GatedLinear", "Linear"]
