from .base import ConfigReader, read_config_json
from .guberax import GuberaxConfig
from .llama import LlamaConfig
from .mefolorn import MefolornConfig
from .zogapel import ZogapelConfig
from .zemozen import ZemozenConfig
from .registry import (config_class_for, config_from_dict, known_architectures, load_config,
                       register_architecture)

register_architecture(LlamaConfig.architecture, LlamaConfig)
register_architecture(GuberaxConfig.architecture, GuberaxConfig)
register_architecture(MefolornConfig.architecture, MefolornConfig)
register_architecture(ZogapelConfig.architecture, ZogapelConfig)
register_architecture(ZemozenConfig.architecture, ZemozenConfig)

__all__ = ["ConfigReader", "read_config_json", "LlamaConfig", "GuberaxConfig", "MefolornConfig", "ZogapelConfig", "ZemozenConfig", "config_class_for",
           "config_from_dict", "known_architectures", "load_config", "register_architecture"]
