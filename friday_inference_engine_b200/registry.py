"""One registry from an architecture's name to its configuration and its model.

config.json names the architecture (`architectures[0]`); the registry gives the class
that types its keys and the function that turns the typed configuration into a
ModelSpec (parts, constants and run order as data).  An unknown name is refused with
the list of known names, as the reference refuses an unknown GGUF architecture
(model_config.cpp:56-58).
"""
import json
import os
from dataclasses import dataclass
from typing import Callable

from .config.base import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type             # has from_dict(dict) and to_dict()
    build_spec: Callable           # typed config -> parts.spec.ModelSpec


_architectures = {}


def register_architecture(name, config_class, build_spec):
    _architectures[name] = Architecture(name, config_class, build_spec)
    return _architectures[name]


def architecture(name) -> Architecture:
    try:
        return _architectures[name]
    except KeyError:
        raise ConfigError("unsupported architecture '%s' (supported: %s)"
                          % (name, ", ".join(sorted(_architectures)) or "none")) from None


def registered():
    return sorted(_architectures)


def architecture_name_of(d: dict) -> str:
    archs = d.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    raise ConfigError("config.json: 'architectures' must be a list whose first item names the model class")


def read_config(model_dir_or_dict):
    """(Architecture, typed config) from a model folder or from config.json's dictionary."""
    if isinstance(model_dir_or_dict, dict):
        d = model_dir_or_dict
    else:
        path = os.path.join(model_dir_or_dict, "config.json")
        try:
            with open(path) as f:
                d = json.load(f)
        except FileNotFoundError:
            raise ConfigError("%s: no config.json in the model folder" % model_dir_or_dict) from None
        except json.JSONDecodeError as e:
            raise ConfigError("%s: not JSON: %s" % (path, e)) from None
    arch = architecture(architecture_name_of(d))
    return arch, arch.config_class.from_dict(d)
