"""Parts a layer is put together from: norm, position encoding, mixer, feed-forward, block."""

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Block, CastStream, FeedForward, Mixer,
                   Norm, NormedDelta, Part, PositionEncoding, Runtime)
from .norm import DyT, LayerNorm, RMSNorm
from .rotary import Rotary
from .attention import GQAAttention
from .mlp import DenseMLP, GatedMLP
from .block import PreNormBlock
from .sink_attention import SinkAttention
from .ssd import SSDMixer
from .parallel import ParallelMixer
from .sandwich import SandwichBlock, TokenSide
from .latent_attention import LatentAttention
from .experts import RoutedExperts, TableExperts
from .embedding import BigramHashEmbedding
from .postnorm_block import PostNormBlock
from .head_attention import HeadAttention
from .delta_rule import GatedDeltaRule
from .parallel_block import ParallelResidualBlock

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Block", "FeedForward", "Mixer",
           "Norm", "NormedDelta", "Part", "PositionEncoding", "Runtime", "RMSNorm", "Rotary", "GQAAttention",
           "GatedMLP", "PreNormBlock", "SinkAttention", "SSDMixer", "ParallelMixer", "SandwichBlock", "TokenSide",
           "DyT", "DenseMLP", "LatentAttention", "TableExperts", "HeadAttention", "GatedDeltaRule",
           "ParallelResidualBlock", "EMBEDDINGS", "CastStream", "LayerNorm", "RoutedExperts", "BigramHashEmbedding",
           "PostNormBlock"]
