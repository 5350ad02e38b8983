"""Configuration and registry, as the library sees them (config/*.cpp, include/friday/config.h).

read_config turns config.json's content into the typed, complete and checked
configuration of its architecture, or raises ConfigError naming the key; describe_model
gives the model as data: parts' tensors, the run order, what each cache entry asks for.
"""
import json

from .. import native
from ..native import ConfigError  # noqa: F401


def read_config(config):
    """config: config.json's content (dict) or a model folder.  Returns the typed configuration as a dict."""
    if not isinstance(config, dict):
        import os
        path = os.path.join(config, "config.json")
        try:
            with open(path) as f:
                config = json.load(f)
        except FileNotFoundError:
            raise ConfigError("%s: no config.json in the model folder" % config) from None
        except json.JSONDecodeError as e:
            raise ConfigError("%s: not JSON: %s" % (path, e)) from None
    return native.call_json("friday_read_config", native.text(json.dumps(config)))


def describe_model(config):
    """architecture, typed config, program (layer, cache, write), cache_requests by entry, params (name, shape, ...)."""
    return native.call_json("friday_describe_model", native.text(json.dumps(config)))


def registered_architectures():
    return native.call_json("friday_registered", b"architectures")
