from .attention import Attention, paged_attention
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Delta, FeedForward, Mixer,
                   PagedKVSpec, Part, Registry, StateSpec)
from .block import Block, NormAfterBlock, PostNormBlock, PreNormBlock, ResidualStream
from .conv import InputConv
from .diff_attention import DifferentialAttention
from .embedding import Embedding, OutputHead
from .ffn import DenseFFN, GatedFFN
from .hgrn2 import HGRN2
from .norm import LayerNorm, NoNorm, Norm, RMSNorm, ScalarRMSNorm
from .position import LearnedPositions, NoPositions, PositionEncoding, RotaryPairs

__all__ = ["Attention", "BLOCKS", "Block", "Delta", "DenseFFN", "Embedding", "FEED_FORWARDS", "FeedForward",
           "LayerNorm", "LearnedPositions", "MIXERS", "Mixer", "NORMS", "NoNorm", "NoPositions", "Norm",
           "OutputHead", "POSITION_ENCODINGS", "PagedKVSpec", "Part", "PositionEncoding", "PostNormBlock",
           "PreNormBlock", "RMSNorm", "Registry", "ResidualStream", "StateSpec", "paged_attention",
           "DifferentialAttention", "GatedFFN", "HGRN2", "InputConv", "NormAfterBlock", "RotaryPairs", "ScalarRMSNorm"]
