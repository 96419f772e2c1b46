from .base import ConfigError, KeyReader, architecture_name, read_config_json
from .gemma2 import FULL, SLIDING, Gemma2Config
