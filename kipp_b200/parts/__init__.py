from .attention import AttentionMixer
from .base import (Block, EmbeddingStage, FeedForward, Mixer, Norm, PagedKVSpec, Part, PlanContext,
                   PositionEncoding, StateSpec)
from .block import HyperConnectionBlock, ParallelBlock, PreNormBlock
from .latent import LatentAttentionMixer
from .embedding import OutputHead, TokenEmbedding
from .mlp import DenseFeedForward, GatedFeedForward, SwiGLUFeedForward
from .norm import LayerNorm, RMSNorm
from .recurrent import (DeltaRuleMixer, GatedMemoryMixer, ParallelMixer, PolyNormFeedForward, RetentionMixer,
                        StateSpaceMixer)
from .rope import NoPositionEncoding, RotaryEncoding, StretchedRotaryEncoding, YarnRotaryEncoding

__all__ = ["AttentionMixer", "Block", "EmbeddingStage", "FeedForward", "Mixer", "Norm", "PagedKVSpec", "Part",
           "PlanContext", "PositionEncoding", "StateSpec", "PreNormBlock", "OutputHead", "TokenEmbedding",
           "SwiGLUFeedForward", "RMSNorm", "NoPositionEncoding", "RotaryEncoding", "DeltaRuleMixer", "ParallelMixer",
           "PolyNormFeedForward", "RetentionMixer", "ParallelBlock", "LatentAttentionMixer", "DenseFeedForward",
           "LayerNorm", "GatedMemoryMixer", "StretchedRotaryEncoding", "HyperConnectionBlock", "GatedFeedForward",
           "StateSpaceMixer", "YarnRotaryEncoding"]
