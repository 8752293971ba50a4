from .attention import AttentionNames, GroupedQueryAttention
from .base import (CacheNeed, FeedForward, Mixer, Norm, PagedKV, Part, PositionEncoding, RequestState, TensorSpec,
                   matrix_to, scale_to)
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .mlp import GatedMlp, GatedMlpNames
from .norm import RmsNorm
from .rope import NoPositionEncoding, RotaryEncoding

__all__ = [
    "AttentionNames", "GroupedQueryAttention", "CacheNeed", "FeedForward", "Mixer", "Norm", "PagedKV", "Part",
    "PositionEncoding", "RequestState", "TensorSpec", "matrix_to", "scale_to", "PreNormBlock", "OutputHead",
    "TokenEmbedding", "GatedMlp", "GatedMlpNames", "RmsNorm", "NoPositionEncoding", "RotaryEncoding",
]
