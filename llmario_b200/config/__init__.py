from .spec import ConfigError, LayerCall, LayerSpec, ModelSpec, PartSpec
from .registry import (config_class, load_config, load_spec, read_config_json,
                       register_architecture, registered_architectures, resolve_architecture)
from .qwen3 import Qwen3Config
from .vunasun import VunasunConfig
from .runidra import RunidraConfig
from .pemolorn import PemolornConfig
from .pavatar import PavatarConfig

register_architecture(Qwen3Config.architecture, Qwen3Config, Qwen3Config.model_type, replace=True)
register_architecture(VunasunConfig.architecture, VunasunConfig, VunasunConfig.model_type,
                      replace=True)
register_architecture(RunidraConfig.architecture, RunidraConfig, RunidraConfig.model_type,
                      replace=True)

register_architecture(PemolornConfig.architecture, PemolornConfig, PemolornConfig.model_type,
                      replace=True)
register_architecture(PavatarConfig.architecture, PavatarConfig, PavatarConfig.model_type,
                      replace=True)

__all__ = ["ConfigError", "LayerCall", "LayerSpec", "ModelSpec", "PartSpec", "Qwen3Config",
           "VunasunConfig", "RunidraConfig", "PemolornConfig", "PavatarConfig",
           "config_class", "load_config", "load_spec", "read_config_json",
           "register_architecture", "registered_architectures", "resolve_architecture"]
