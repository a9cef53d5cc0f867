from .base import ConfigError, ModelConfig, read_config_json, architecture_name
from .options import EngineOptions, canonical_dtype
from .qwen2 import Qwen2Config, QWEN2_ARCHITECTURE
from .kakipel import KakipelConfig, KAKIPEL_ARCHITECTURE
from .libulorn import LibulornConfig, LIBULORN_ARCHITECTURE
from .lipelix import LipelixConfig, LIPELIX_ARCHITECTURE
from .karorax import KaroraxConfig, KARORAX_ARCHITECTURE
from .registry import (Architecture, config_from_dict, load_config, lookup_architecture,
                       register_architecture, registered_architectures, unregister_architecture)

__all__ = [
    "ConfigError", "ModelConfig", "read_config_json", "architecture_name", "EngineOptions",
    "canonical_dtype", "Qwen2Config", "QWEN2_ARCHITECTURE", "KakipelConfig", "KAKIPEL_ARCHITECTURE", "LibulornConfig", "LIBULORN_ARCHITECTURE", "LipelixConfig", "LIPELIX_ARCHITECTURE", "KaroraxConfig", "KARORAX_ARCHITECTURE", "Architecture", "config_from_dict",
    "load_config", "lookup_architecture", "register_architecture", "registered_architectures",
    "unregister_architecture",
]
