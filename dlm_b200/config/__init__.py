from .base import ConfigError, read_config_json
from .faguzen import FaguzenConfig
from .qwen2_moe import Qwen2MoeConfig
from .salolorn import SalolornConfig
from .zasazen import ZasazenConfig
from .zesapel import ZesapelConfig

__all__ = ["ConfigError", "read_config_json", "FaguzenConfig", "Qwen2MoeConfig", "SalolornConfig", "ZasazenConfig", "ZesapelConfig"]
