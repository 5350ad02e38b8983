"""Typed reading of config.json.

A configuration class declares its keys once, as `Key` entries; `read_keys` turns the
dictionary of config.json into typed values and reports every problem with the name of
the key.  Nothing here knows a particular architecture.
"""
from dataclasses import dataclass
from typing import Any, Callable, Optional


class ConfigError(ValueError):
    """A config.json that cannot be used; the message names the key."""


_REQUIRED = object()


@dataclass(frozen=True)
class Key:
    name: str                       # the key in config.json
    kind: type                      # int, float, bool or str
    default: Any = _REQUIRED        # _REQUIRED, a value, or a callable(values) -> value
    check: Optional[Callable[[Any], bool]] = None
    rule: str = ""                  # said in the error when `check` fails


def _coerce(key: Key, value):
    if key.kind is bool:
        if isinstance(value, bool):
            return value
    elif key.kind is int:
        if isinstance(value, int) and not isinstance(value, bool):
            return value
        if isinstance(value, float) and value == int(value):
            return int(value)
    elif key.kind is float:
        if isinstance(value, (int, float)) and not isinstance(value, bool):
            return float(value)
    elif key.kind is str:
        if isinstance(value, str):
            return value
    raise ConfigError("config.json: '%s' must be %s, got %r" % (key.name, key.kind.__name__, value))


def read_keys(d: dict, keys) -> dict:
    """Values for `keys` from `d`, defaults filled in the order of `keys`."""
    out = {}
    for key in keys:
        if key.name in d and d[key.name] is not None:
            value = _coerce(key, d[key.name])
        elif key.default is _REQUIRED:
            raise ConfigError("config.json: required key '%s' is missing" % key.name)
        elif callable(key.default):
            value = key.default(out)
        else:
            value = key.default
        if key.check is not None and value is not None and not key.check(value):
            raise ConfigError("config.json: '%s' = %r: %s" % (key.name, value, key.rule))
        out[key.name] = value
    return out


def positive(v):
    return v > 0
