"""Typed configurations and the registry from architecture name to model."""
from .base import (ConfigError, LayerCall, LayerSpec, ModelConfig, architecture_name, load_config,
                   lookup_architecture, read_config_json, register_architecture, registered_architectures)
from .qwen3 import Qwen3Config
from .vedizen import VedizenConfig
from .pogarax import PogaraxConfig
from .gamanex import GamanexConfig
from .tagulix import TagulixConfig


def _register_builtin() -> None:
    from ..engine.model import build_decoder
    register_architecture("Qwen3ForCausalLM", Qwen3Config, build_decoder)
    register_architecture("Vedizen", VedizenConfig, build_decoder)
    register_architecture("Pogarax", PogaraxConfig, build_decoder)
    register_architecture("Gamanex", GamanexConfig, build_decoder)
    register_architecture("Tagulix", TagulixConfig, build_decoder)


_register_builtin()
