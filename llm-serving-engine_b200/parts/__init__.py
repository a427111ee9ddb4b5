"""Parts a model is assembled from. Importing this package registers the built-in kinds."""

from . import (attention, blocks, embed_terms, feed_forward, latent_attention, linear_attention, moe, norms,  # noqa: F401
               parallel, positions, token_shift)
from .attention import AttentionSpec, PagedAttention
from .base import (
    BLOCKS,
    FEED_FORWARDS,
    INPUT_FILTERS,
    MIXERS,
    NORMS,
    POSITION_ENCODINGS,
    Block,
    BuildEnv,
    FeedForward,
    Mixer,
    Norm,
    PagedKVNeed,
    ParamDecl,
    Part,
    PositionEncoding,
    StateNeed,
    role_dtype,
)
from .blocks import BranchNormBlock, BranchNormBlockSpec, PreNormBlock, PreNormBlockSpec, SandwichBlock, SandwichBlockSpec
from .linear_attention import (DecayLinearAttention, DecayLinearAttentionSpec, GatedLinearAttention,
                               GatedLinearAttentionSpec)
from .differential_attention import DifferentialAttention, DifferentialAttentionSpec
from .streams import StreamsBlock, StreamsBlockSpec, StreamsRMSNorm, StreamsRMSNormSpec, StreamsWrite, StreamsWriteSpec
from .parallel import ParallelMixer, ParallelMixerSpec
from .token_shift import TokenShift, TokenShiftSpec
from .feed_forward import MLP, MLPSpec, SwiGLU, SwiGLUSpec
from .norms import RMSNorm, RMSNormSpec
from .embed_terms import HashedPairEmbedding, HashedPairSpec
from .latent_attention import LatentAttention, LatentAttentionSpec
from .moe import RoutedExperts, RoutedExpertsSpec
from .positions import NoPositionSpec, RotaryPositionEncoding, RotarySpec, SinusoidSpec

__all__ = [
    "AttentionSpec", "PagedAttention", "BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS",
    "POSITION_ENCODINGS", "Block", "BuildEnv", "FeedForward", "Mixer", "Norm", "PagedKVNeed",
    "ParamDecl", "Part", "PositionEncoding", "StateNeed", "role_dtype", "PreNormBlock",
    "PreNormBlockSpec", "SwiGLU", "SwiGLUSpec", "RMSNorm", "RMSNormSpec", "NoPositionSpec",
    "RotaryPositionEncoding", "RotarySpec", "INPUT_FILTERS", "BranchNormBlock", "BranchNormBlockSpec",
    "DecayLinearAttention", "DecayLinearAttentionSpec", "ParallelMixer", "ParallelMixerSpec", "TokenShift",
    "TokenShiftSpec", "HashedPairEmbedding", "HashedPairSpec", "LatentAttention", "LatentAttentionSpec",
    "RoutedExperts", "RoutedExpertsSpec", "SinusoidSpec", "SandwichBlock", "SandwichBlockSpec", "MLP", "MLPSpec",
    "GatedLinearAttention", "GatedLinearAttentionSpec", "DifferentialAttention", "DifferentialAttentionSpec",
    "StreamsBlock", "StreamsBlockSpec", "StreamsRMSNorm", "StreamsRMSNormSpec", "StreamsWrite", "StreamsWriteSpec",
]
