"""Typed configurations, the model as data (``ModelSpec``) and the architecture registry."""
from .spec import LayerSpec, ModelSpec, PartSpec, Run
from .qwen3 import Qwen3Config
from .busavik import BusavikConfig
from .fimudra import FimudraConfig
from .sezopel import SezopelConfig
from .laralix import LaralixConfig
from .registry import (architectures, config_of_folder, family_of, read_config_json,
                       register_architecture)

register_architecture(Qwen3Config, Qwen3Config.ARCHITECTURE, Qwen3Config.MODEL_TYPE)
register_architecture(BusavikConfig, BusavikConfig.ARCHITECTURE, BusavikConfig.MODEL_TYPE)
register_architecture(FimudraConfig, FimudraConfig.ARCHITECTURE, FimudraConfig.MODEL_TYPE)
register_architecture(SezopelConfig, SezopelConfig.ARCHITECTURE, SezopelConfig.MODEL_TYPE)
register_architecture(LaralixConfig, LaralixConfig.ARCHITECTURE, LaralixConfig.MODEL_TYPE)

__all__ = ["LayerSpec", "ModelSpec", "PartSpec", "Run", "Qwen3Config", "BusavikConfig", "FimudraConfig", "SezopelConfig", "LaralixConfig",
           "architectures",
           "config_of_folder", "family_of", "read_config_json", "register_architecture"]
