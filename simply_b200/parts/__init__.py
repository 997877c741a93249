"""Parts a decoder is put together from: mixers, feed-forwards, norms, position encodings, blocks."""

from simply_b200.parts.base import Block, FeedForward, Mixer, Norm, Part, PositionEncoding
from simply_b200.parts.block import ResidualStream
from simply_b200.parts.model import DecoderModel, tensor_specs

__all__ = ["Block", "DecoderModel", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding",
           "ResidualStream", "tensor_specs"]
