from .qwen3 import Qwen3Config
from .lemesun import LemesunConfig
from .specs import (AttentionSpec, ChannelDeltaSpec, LatentAttentionSpec, RoutedExpertsSpec, EmbeddingSpec, GatedMLPSpec, HeadSpec, ModelPlan, NoPositionSpec,
                    OrderEntry, PreNormBlockSpec, RMSNormSpec, RotarySpec, names)

__all__ = ["Qwen3Config", "LemesunConfig", "ChannelDeltaSpec", "LatentAttentionSpec", "RoutedExpertsSpec", "AttentionSpec", "EmbeddingSpec", "GatedMLPSpec", "HeadSpec", "ModelPlan",
           "NoPositionSpec", "OrderEntry", "PreNormBlockSpec", "RMSNormSpec", "RotarySpec", "names"]
