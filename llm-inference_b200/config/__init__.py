from .gunedra_config import GunedraConfig
from .lerorax_config import LeroraxConfig
from .zetizen_config import ZetizenConfig
from .model_config import ConfigError, ModelConfig, Qwen2Config, read_config_json
from .registry import (
    Architecture,
    parse_config,
    register_architecture,
    registered_architectures,
    resolve_architecture,
)

__all__ = [
    "Architecture",
    "ConfigError",
    "GunedraConfig",
    "LeroraxConfig",
    "ModelConfig",
    "Qwen2Config",
    "ZetizenConfig",
    "parse_config",
    "read_config_json",
    "register_architecture",
    "registered_architectures",
    "resolve_architecture",
]
