from .attention import Attention, paged_attention
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Delta, FeedForward, Mixer,
                   PagedKVSpec, Part, Registry, StateSpec)
from .block import Block, NormAfterBlock, ParallelBlock, PostNormBlock, PreNormBlock, ReentryBlock, ResidualStream
from .conv import InputConv
from .diff_attention import DifferentialAttention
from .embedding import Embedding, OutputHead
from .ffn import DenseFFN, GatedFFN
from .hgrn2 import HGRN2
from .latent_attention import LatentAttention
from .moe import RoutedExperts
from .norm import LayerNorm, NoNorm, Norm, OffsetRMSNorm, RMSNorm, ScalarRMSNorm
from .position import LearnedPositions, NoPositions, PositionEncoding, RotaryHalves, RotaryPairs

__all__ = ["Attention", "BLOCKS", "Block", "Delta", "DenseFFN", "Embedding", "FEED_FORWARDS", "FeedForward",
           "LayerNorm", "LearnedPositions", "MIXERS", "Mixer", "NORMS", "NoNorm", "NoPositions", "Norm",
           "OutputHead", "POSITION_ENCODINGS", "PagedKVSpec", "Part", "PositionEncoding", "PostNormBlock",
           "PreNormBlock", "RMSNorm", "Registry", "ResidualStream", "StateSpec", "paged_attention",
           "DifferentialAttention", "GatedFFN", "HGRN2", "InputConv", "NormAfterBlock", "RotaryPairs", "ScalarRMSNorm",
           "LatentAttention", "OffsetRMSNorm", "ParallelBlock", "ReentryBlock", "RotaryHalves", "RoutedExperts"]
