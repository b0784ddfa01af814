"""Typed configurations and the architecture-neutral specs they translate to."""

from .specs import (AttentionSpec, ConfigError, GatedMLPSpec, LayerSpec, MixerBranch, ModelSpec, NormSpec,
                    ParallelMixerSpec, RotarySpec, RunEntry, SandwichLayerSpec, SinkAttentionSpec, SSDSpec,
                    TokenSideSpec, WavelengthScaling, default_schedule, DenseMLPSpec, DyTNormSpec,
                    LatentAttentionSpec, RampScaling, TableExpertsSpec, HeadAttentionSpec, DeltaRuleSpec,
                    BigramHashSpec, LayerNormSpec, PostNormLayerSpec, RoutedExpertsSpec)
from .qwen3 import Qwen3Config
from .lunulix import LunulixConfig
from .panodra import PanodraConfig
from .fuginex import FuginexConfig
from .pununex import PununexConfig

__all__ = ["AttentionSpec", "ConfigError", "GatedMLPSpec", "LayerSpec", "ModelSpec", "NormSpec",
           "RotarySpec", "RunEntry", "default_schedule", "Qwen3Config", "LunulixConfig", "MixerBranch",
           "ParallelMixerSpec", "SandwichLayerSpec", "SinkAttentionSpec", "SSDSpec", "TokenSideSpec",
           "WavelengthScaling", "DenseMLPSpec", "DyTNormSpec", "LatentAttentionSpec", "RampScaling", "TableExpertsSpec",
           "PanodraConfig", "HeadAttentionSpec", "DeltaRuleSpec", "FuginexConfig", "PununexConfig", "BigramHashSpec",
           "LayerNormSpec", "PostNormLayerSpec", "RoutedExpertsSpec"]
