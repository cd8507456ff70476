"""Parts a model is put together from: norm, position encoding, mixer, feed-forward,
their arrangement in a block, embedding and output head."""
from .base import (BuildContext, FeedForward, KVSpec, LayerBinding, Mixer, Norm, Part, PositionEncoding,
                   StateSpec, WeightSpec)
from .stream import ResidualStream
from .norms import RMSNormL2
from .positions import RotaryHalf, RotaryInterleaved
from .attention import GqaAttention
from .feed_forward import SwiGLU
from .block import Block
from .embedding import Embedding, LMHead

__all__ = ["BuildContext", "FeedForward", "KVSpec", "LayerBinding", "Mixer", "Norm", "Part",
           "PositionEncoding", "StateSpec", "WeightSpec", "ResidualStream", "RMSNormL2", "RotaryHalf",
           "RotaryInterleaved", "GqaAttention", "SwiGLU", "Block", "Embedding", "LMHead"]
