"""Typed configurations, the model-as-parts records and the architecture registry."""
from .specs import (ConfigError, ConvSpec, PairEmbeddingSpec, DepthMixSpec, FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec,
                    NormSpec, PositionSpec, ScheduleEntry, StreamInjection)
from .registry import (ARCHITECTURES, Architecture, architecture_name, lookup, read_config_json,
                       register_architecture, spec_from_config_dict)
from .qwen2 import Qwen2Config
from .zolulix import ZolulixConfig
from .mefupel import MefupelConfig
from .leguvik import LeguvikConfig
from .bulodra import BulodraConfig

register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict, Qwen2Config.to_spec)
register_architecture("Zolulix", ZolulixConfig.from_dict, ZolulixConfig.to_spec)
register_architecture("Mefupel", MefupelConfig.from_dict, MefupelConfig.to_spec)
register_architecture("Leguvik", LeguvikConfig.from_dict, LeguvikConfig.to_spec)
register_architecture("Bulodra", BulodraConfig.from_dict, BulodraConfig.to_spec)

__all__ = ["ConfigError", "ConvSpec", "PairEmbeddingSpec", "DepthMixSpec", "ZolulixConfig", "MefupelConfig", "LeguvikConfig", "BulodraConfig", "StreamInjection", "FeedForwardSpec", "LayerSpec", "MixerSpec", "ModelSpec", "NormSpec",
           "PositionSpec", "ScheduleEntry", "ARCHITECTURES", "Architecture", "architecture_name",
           "lookup", "read_config_json", "register_architecture", "spec_from_config_dict",
           "Qwen2Config"]
