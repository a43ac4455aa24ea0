from .engine_config import EngineConfig
from .qwen3 import ConfigError, Qwen3Config, qwen3_model_spec
from .registry import (
    ARCHITECTURES,
    Architecture,
    load_model_spec,
    read_config_json,
    register_architecture,
    resolve_architecture,
)
from .specs import (
    FeedForwardSpec,
    LayerSpec,
    MixerSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    ScheduleEntry,
)

register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict, qwen3_model_spec)

__all__ = [
    "ARCHITECTURES", "Architecture", "ConfigError", "EngineConfig", "FeedForwardSpec", "LayerSpec",
    "MixerSpec", "ModelSpec", "NormSpec", "PositionSpec", "Qwen3Config", "ScheduleEntry",
    "load_model_spec", "qwen3_model_spec", "read_config_json", "register_architecture",
    "resolve_architecture",
]
