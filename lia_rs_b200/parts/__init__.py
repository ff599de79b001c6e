from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Arrangement, FeedForward,
                   KVCacheRequest, Mixer, Norm, Part, PartSpec, PositionEncoding, Runtime, StateRequest,
                   lookup, register_arrangement, register_feed_forward, register_mixer, register_norm,
                   register_position_encoding)
from . import norm, rotary, attention, feed_forward, block  # noqa: F401  (register the built-in parts)
from .block import LayerSpec, build_layer, check_layer, layer_tensor_specs

__all__ = ["ARRANGEMENTS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Arrangement",
           "FeedForward", "KVCacheRequest", "Mixer", "Norm", "Part", "PartSpec", "PositionEncoding",
           "Runtime", "StateRequest", "lookup", "register_arrangement", "register_feed_forward",
           "register_mixer", "register_norm", "register_position_encoding", "LayerSpec", "build_layer", "check_layer",
           "layer_tensor_specs"]
