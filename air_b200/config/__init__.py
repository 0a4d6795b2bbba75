from .model_config import ConfigError, Qwen2Config
from . import architectures  # registers the known architectures
import json
import os


def load_config(path_or_dict):
    """The typed configuration of a model folder (or of a config.json's contents): the class
    is chosen by the first entry of ``architectures`` through the registry."""
    from ..parts.registry import architecture
    if isinstance(path_or_dict, dict):
        d = path_or_dict
    else:
        path = path_or_dict
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        try:
            with open(path) as f:
                d = json.load(f)
        except FileNotFoundError:
            raise ConfigError("data_error", f"no config.json at {path}") from None
        except json.JSONDecodeError as e:
            raise ConfigError("data_error", f"config.json is not valid JSON: {e}") from None
        if not isinstance(d, dict):
            raise ConfigError("data_error", "config.json must hold an object")
    archs = d.get("architectures") or []
    if not archs:
        raise ConfigError("data_error", "config.json lacks 'architectures'")
    return architecture(archs[0]).config_class.from_dict(d)
