from .base import (ConfigError, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry)
from .divuzen import DivuzenConfig
from .falalix import FalalixConfig
from .govopel import GovopelConfig
from .navulorn import NavulornConfig
from .qwen3 import Qwen3Config
from .registry import (config_class, config_from_dict, load_config, register_architecture,
                       supported_architectures)

register_architecture("Qwen3ForCausalLM", Qwen3Config)
register_architecture("Falalix", FalalixConfig)
register_architecture("Govopel", GovopelConfig)
register_architecture("Divuzen", DivuzenConfig)
register_architecture("Navulorn", NavulornConfig)

__all__ = ["ConfigError", "LayerSpec", "ModelConfig", "ModelSpec", "PartSpec", "RunEntry", "Qwen3Config", "FalalixConfig", "GovopelConfig", "DivuzenConfig", "NavulornConfig",
           "config_class", "config_from_dict", "load_config", "register_architecture",
           "supported_architectures"]
