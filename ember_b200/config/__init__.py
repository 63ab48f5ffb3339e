"""Typed configurations and the architecture registry."""
from .spec import (AttentionSpec, ConfigError, DynamicTanhSpec, HyperConnectionSpec, TimeMixSpec, GatedDeltaSpec, GatedLinearAttentionSpec, GatedMLPSpec, LatentAttentionSpec,
                   LayerNormSpec, LayerSpec, MatrixMemorySpec, ModelSpec, NoPositionSpec, ParallelMixerSpec, PartSpec,
                   RMSNormSpec, RotarySpec, RoutedMLPSpec, ScheduleEntry, SigmoidAttentionSpec, SigmoidGateSpec,
                   SinkAttentionSpec, StateSpaceSpec, default_schedule)
from .registry import (config_from_dict, load_config, load_model_spec, register_architecture,
                       registered_architectures, resolve_architecture)
from .qwen3 import Qwen3Config
from .fadosun import FadosunConfig
from .zufusun import ZufusunConfig
from .fomanex import FomanexConfig
from .pepapel import PepapelConfig

__all__ = [
    "AttentionSpec", "ConfigError", "GatedMLPSpec", "LayerSpec", "ModelSpec", "NoPositionSpec", "PartSpec",
    "RMSNormSpec", "RotarySpec", "ScheduleEntry", "default_schedule", "config_from_dict", "load_config",
    "load_model_spec", "register_architecture", "registered_architectures", "resolve_architecture",
    "Qwen3Config", "FadosunConfig", "GatedDeltaSpec", "LayerNormSpec", "MatrixMemorySpec", "ParallelMixerSpec",
    "SigmoidAttentionSpec", "SigmoidGateSpec", "StateSpaceSpec", "ZufusunConfig", "GatedLinearAttentionSpec",
    "LatentAttentionSpec", "RoutedMLPSpec", "SinkAttentionSpec", "FomanexConfig", "DynamicTanhSpec", "HyperConnectionSpec",
    "TimeMixSpec", "PepapelConfig",
]
