from .base import ConfigError, Key, read_keys  # noqa: F401
from .qwen2 import Qwen2Config  # noqa: F401
