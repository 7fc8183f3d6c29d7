from .base import ConfigError, FieldReader, architecture_name, read_config_json
from .minicpm import MiniCPMConfig, RopeScaling, SparseConfig
from .reravik import ReravikConfig
from .mufevik import MufevikConfig
from .kipizen import KipizenConfig
from .lukelorn import LukelornConfig

__all__ = ["ConfigError", "FieldReader", "architecture_name", "read_config_json", "MiniCPMConfig", "RopeScaling",
           "SparseConfig", "ReravikConfig", "MufevikConfig", "KipizenConfig", "LukelornConfig"]
