from nanotitan_b200.config import *  # noqa: F401,F403
from nanotitan_b200.config import AppConfig, ModelConfig, RuntimeConfig, load_config, resolve_config_path  # noqa: F401
