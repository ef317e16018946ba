"""Layer parts: mixers, feed-forwards, norms, position encodings, blocks (see ``base.py``)."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheSpec,
                   FeedForward, GroupView, LayerCall, Mixer, Norm, ParamSpec, Part,
                   PositionEncoding, Registry, SiteCache, StateSpec, StepContext, StreamPart)
from .linear import Linear, matmul_nt
from .norm import DynamicTanh, OffsetRMSNorm, OutputRMSNorm, RMSNorm
from .rope import NoPositionEncoding, RotaryEmbedding
from .attention import GeneralAttention, PagedAttention
from .delta import ChannelDecayDeltaMixer, GatedDeltaMixer, SideBySideMixer
from .ssm import Mamba2Mixer
from .latent_attention import LatentAttention, LatentRopeAttention
from .gla import GatedLinearAttention
from .loop import LoopEntry
from .mlp import DenseMLP, GatedMLP
from .moe import RoutedExperts
from .embedding import Embedding, LMHead, ScaledEmbedding, SummedEmbedding
from .block import OutputNormBlock, ParallelBlock, PreNormBlock, SandwichBlock

__all__ = [
    "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheSpec",
    "FeedForward", "GroupView", "LayerCall", "Mixer", "Norm", "ParamSpec", "Part",
    "PositionEncoding", "Registry", "SiteCache", "StateSpec", "StepContext", "Linear", "matmul_nt",
    "RMSNorm", "NoPositionEncoding", "RotaryEmbedding", "PagedAttention", "GatedMLP", "Embedding",
    "LMHead", "PreNormBlock", "OutputRMSNorm", "OutputNormBlock", "SummedEmbedding", "GatedDeltaMixer",
    "LatentAttention", "RoutedExperts", "DynamicTanh", "GeneralAttention", "ChannelDecayDeltaMixer",
    "SideBySideMixer", "Mamba2Mixer", "DenseMLP", "ParallelBlock", "StreamPart", "OffsetRMSNorm", "LatentRopeAttention",
    "GatedLinearAttention", "LoopEntry", "ScaledEmbedding", "SandwichBlock",
]
