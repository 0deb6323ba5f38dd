"""Typed configurations and the architecture registry."""

from .base import ConfigError, read_config_json, read_fields
from .fekitar import FekitarConfig, fekitar_model_spec
from .lezepel import LezepelConfig, lezepel_model_spec
from .movalorn import MovalornConfig, movalorn_model_spec
from .qwen3 import Qwen3Config, qwen3_model_spec
from .rabadra import RabadraConfig, rabadra_model_spec
from .registry import (Architecture, find_architecture, parse_config, register_architecture,
                       registered_architectures, unregister_architecture)

register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_model_spec, model_types=("qwen3",))
register_architecture("Lezepel", LezepelConfig, lezepel_model_spec, model_types=("lezepel",))
register_architecture("Rabadra", RabadraConfig, rabadra_model_spec, model_types=("rabadra",))
register_architecture("Movalorn", MovalornConfig, movalorn_model_spec, model_types=("movalorn",))
register_architecture("Fekitar", FekitarConfig, fekitar_model_spec, model_types=("fekitar",))

__all__ = ["ConfigError", "read_config_json", "read_fields", "Qwen3Config", "qwen3_model_spec", "LezepelConfig", "lezepel_model_spec", "RabadraConfig", "rabadra_model_spec", "MovalornConfig", "movalorn_model_spec", "FekitarConfig", "fekitar_model_spec", "Architecture",
           "find_architecture", "parse_config", "register_architecture", "registered_architectures",
           "unregister_architecture"]
