"""Configuration: typed reading of config.json and the architecture registry."""
from .base import ConfigError, KeyReader, read_config_json
from .spec import (AdapterSpec, AttentionSpec, DeltaRuleSpec, DenseMLPSpec, FeedForwardSpec, GatedMLPSpec,
                   GatedRecurrenceSpec, LatentAttentionSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                   ParallelMixersSpec, RoutedExpertsSpec, RunStep, ShortConvSpec, StateSpaceSpec, TableExpertsSpec,
                   TokenInputSpec)
from .registry import (Architecture, find_architecture, load_config, register_architecture,
                       registered_architectures, unregister_architecture)
from .qwen3 import ARCHITECTURE as QWEN3_ARCHITECTURE, MODEL_TYPE as QWEN3_MODEL_TYPE, Qwen3Config

register_architecture(QWEN3_ARCHITECTURE, Qwen3Config.from_dict, Qwen3Config.model_spec,
                      model_type=QWEN3_MODEL_TYPE, replace=True)
from .gitipel import ARCHITECTURE as GITIPEL_ARCHITECTURE, SHAPES_KEY as _GITIPEL_SHAPES, GitipelConfig

register_architecture(GITIPEL_ARCHITECTURE, GitipelConfig.from_dict, GitipelConfig.model_spec, replace=True,
                      shapes_key=_GITIPEL_SHAPES)
from .fokurax import ARCHITECTURE as FOKURAX_ARCHITECTURE, FokuraxConfig

register_architecture(FOKURAX_ARCHITECTURE, FokuraxConfig.from_dict, FokuraxConfig.model_spec, replace=True)
from .pitudra import ARCHITECTURE as PITUDRA_ARCHITECTURE, PitudraConfig

register_architecture(PITUDRA_ARCHITECTURE, PitudraConfig.from_dict, PitudraConfig.model_spec, replace=True)
from .dogetar import ARCHITECTURE as DOGETAR_ARCHITECTURE, DogetarConfig

register_architecture(DOGETAR_ARCHITECTURE, DogetarConfig.from_dict, DogetarConfig.model_spec, replace=True)

__all__ = [
    "ConfigError", "KeyReader", "read_config_json",
    "AdapterSpec", "AttentionSpec", "FeedForwardSpec", "GatedMLPSpec", "LayerSpec", "MixerSpec", "ModelSpec",
    "NormSpec", "PositionSpec", "RunStep", "DeltaRuleSpec", "DenseMLPSpec", "ShortConvSpec", "GitipelConfig",
    "TableExpertsSpec", "TokenInputSpec", "FokuraxConfig", "GatedRecurrenceSpec", "LatentAttentionSpec",
    "RoutedExpertsSpec", "PitudraConfig", "StateSpaceSpec", "ParallelMixersSpec", "DogetarConfig",
    "Architecture", "find_architecture", "load_config", "register_architecture",
    "registered_architectures", "unregister_architecture", "Qwen3Config",
]
