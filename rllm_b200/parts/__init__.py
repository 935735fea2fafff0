from .base import (CacheKind, KVCacheSpec, LayerCache, NormedSum, Param, Part, ScaledSum, Source, StateSpec, Summands, cache_kind_of,
                   make_part, register_cache_kind, register_part, registered_parts)
from .rope_rules import register_rope_rule, registered_rope_rules
from .norm import RMSNorm
from .rope import InterleavedRotary, RotaryEmbedding, inverse_frequencies
from .attention import GQAttention, SinkGQAttention, TalkingHeadsAttention
from .ffn import ActFFN, GluFFN, SwiGLU
from .block import GatedPreNormBlock, LoopStep, ParallelBlock, PostNormBlock, PreNormBlock, SandwichBlock
from .latent_attention import LatentAttention, LatentCacheSpec
from .gla import GatedLinearAttention
from .moe import GatedRoutedExperts, GluRoutedExperts, RoutedExperts
from .recurrent import DeltaRuleMixer, MinGRUMixer, SideBySideMixer, StateSpaceMixer
from .embedding import Embedding, OutputHead, PairEmbedding

__all__ = ["CacheKind", "cache_kind_of", "register_cache_kind", "register_rope_rule", "registered_rope_rules",
           "KVCacheSpec", "LayerCache", "Param", "Part", "Source", "StateSpec", "make_part",
           "register_part", "registered_parts", "RMSNorm", "RotaryEmbedding",
           "inverse_frequencies", "GQAttention", "SwiGLU", "PreNormBlock", "Embedding",
           "OutputHead", "InterleavedRotary", "SandwichBlock", "LoopStep", "LatentAttention",
           "LatentCacheSpec", "GatedLinearAttention", "RoutedExperts", "Summands", "SinkGQAttention", "ActFFN",
           "PostNormBlock", "GatedRoutedExperts", "NormedSum", "TalkingHeadsAttention", "GluFFN", "ParallelBlock",
           "GluRoutedExperts", "DeltaRuleMixer", "SideBySideMixer", "StateSpaceMixer", "PairEmbedding", "ScaledSum",
           "GatedPreNormBlock", "MinGRUMixer"]
