"""Parts a model is put together from: norms, position encodings, mixers, feed-forwards, gates, arrangements."""
from .base import CacheNeed, Connection, FeedForward, Gate, Mixer, Norm, Part, PositionEncoding, Runtime, WeightDecl
from .registry import build_part, part_class, register_part, registered_parts
from .linear import Linear
from . import (norm, position, attention, feedforward, gate, recurrent, sigmoid_attention, sink_attention,  # noqa: F401
               parallel, connection, block)                                               # (registers the built-in parts)

__all__ = ["CacheNeed", "Connection", "FeedForward", "Gate", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "WeightDecl",
           "build_part", "part_class", "register_part", "registered_parts", "Linear"]
