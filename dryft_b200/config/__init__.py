"""Typed configurations, the architecture registry and the architecture-neutral model spec."""

from .spec import ExtraPart, LayerSpec, ModelSpec, PartSpec, RunStep
from .qwen3 import ConfigError, Qwen3Config
from .tevovik import TevovikConfig
from .vobusun import VobusunConfig
from .mogelix import MogelixConfig
from .kerirax import KeriraxConfig
from .registry import (
    Architecture,
    architecture_of,
    config_from_dict,
    known_architectures,
    load_config,
    load_model_spec,
    register_architecture,
    unregister_architecture,
)
from .presets import PRESETS, preset

register_architecture("Qwen3ForCausalLM", Qwen3Config.from_dict)
register_architecture("Tevovik", TevovikConfig.from_dict)
register_architecture("Vobusun", VobusunConfig.from_dict)
register_architecture("Mogelix", MogelixConfig.from_dict)
register_architecture("Kerirax", KeriraxConfig.from_dict)

__all__ = [
    "ExtraPart",
    "Architecture", "ConfigError", "KeriraxConfig", "LayerSpec", "ModelSpec", "MogelixConfig", "PartSpec", "PRESETS", "Qwen3Config", "RunStep", "TevovikConfig", "VobusunConfig",
    "architecture_of", "config_from_dict", "known_architectures", "load_config", "load_model_spec",
    "preset", "register_architecture", "unregister_architecture",
]
