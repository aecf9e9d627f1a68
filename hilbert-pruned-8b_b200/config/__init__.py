from .base import ConfigError, read_config_json
from .llama import Llama3RopeScaling, LlamaConfig
from .pogezen import PogezenConfig
from .vuladra import VuladraConfig
from .tonovik import TonovikConfig
from .moponex import MoponexConfig
from .registry import (config_class_for, load_config, register_architecture, registered_architectures,
                       unregister_architecture)
from .spec import LayerSpec, ModelSpec, PartSpec, PlanEntry

__all__ = ["ConfigError", "Llama3RopeScaling", "LlamaConfig", "PogezenConfig", "VuladraConfig", "TonovikConfig", "MoponexConfig", "read_config_json", "config_class_for",
           "load_config", "register_architecture", "registered_architectures", "unregister_architecture",
           "LayerSpec", "ModelSpec", "PartSpec", "PlanEntry"]

register_architecture(LlamaConfig)
register_architecture(PogezenConfig)
register_architecture(VuladraConfig)
register_architecture(TonovikConfig)
register_architecture(MoponexConfig)
