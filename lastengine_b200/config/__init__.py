from .base import ConfigError, architecture_name, read_config_json  # noqa: F401
from .lfm3 import Lfm3Config  # noqa: F401
