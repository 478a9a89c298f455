from .registry import ARCHITECTURES, ConfigError, architecture_of, load_config, read_config_json, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, Run
from . import qwen3 as _qwen3  # registers "Qwen3ForCausalLM"
from . import vekurax as _vekurax  # registers "Vekurax"
from . import nametar as _nametar  # registers "Nametar"
from . import pepevik as _pepevik  # registers "Pepevik"
from . import lifulorn as _lifulorn  # registers "Lifulorn"
from .qwen3 import Qwen3Config
from .vekurax import VekuraxConfig
from .nametar import NametarConfig
from .pepevik import PepevikConfig
from .lifulorn import LifulornConfig

__all__ = ["ARCHITECTURES", "ConfigError", "architecture_of", "load_config", "read_config_json",
           "register_architecture", "LayerSpec", "ModelSpec", "PartSpec", "Run", "Qwen3Config", "VekuraxConfig", "NametarConfig", "PepevikConfig", "LifulornConfig"]
