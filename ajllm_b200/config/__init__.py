"""YAML run configuration: inheritance, named components, dotted overrides, validation."""

from ajllm_b200.config.loader import ConfigError, LoadedConfig, load_run_config, set_dotted_value
from ajllm_b200.config.schema import (
    check_dataset,
    check_model,
    check_parallel,
    check_tokenizer,
    require,
)

__all__ = [
    "ConfigError", "LoadedConfig", "load_run_config", "set_dotted_value",
    "check_dataset", "check_model", "check_parallel", "check_tokenizer", "require",
]
