from .attention import GQAAttention
from .base import (FeedForward, Mixer, Norm, PagedKVSpec, Part, PositionEncoding, Run, Runtime,
                   StateSpec, StreamEncoding, WeightSpec)
from .block import PreNormBlock
from .embedding import Embedding, LMHead
from .linear import Linear
from .mlp import SwiGLU
from .model import Model
from .norm import RMSNorm
from .rope import NoPositionEncoding, RotaryEmbedding, inverse_frequencies

__all__ = ["GQAAttention", "FeedForward", "Mixer", "Norm", "PagedKVSpec", "Part", "PositionEncoding",
           "Run", "Runtime", "StateSpec", "StreamEncoding", "WeightSpec", "PreNormBlock", "Embedding", "LMHead", "Linear",
           "SwiGLU", "Model", "RMSNorm", "NoPositionEncoding", "RotaryEmbedding", "inverse_frequencies"]
