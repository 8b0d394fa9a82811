from .base import ConfigError, architecture_name, read_config_json  # noqa: F401
from .kisilix import KisilixConfig  # noqa: F401
from .lenesun import LenesunConfig  # noqa: F401
from .lfm3 import Lfm3Config  # noqa: F401
from .tevilix import TevilixConfig  # noqa: F401
from .zekivik import ZekivikConfig  # noqa: F401
