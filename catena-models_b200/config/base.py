"""Typed reading of a model folder's config.json.

A configuration class declares its keys once (`fields`), reads them with type and range
checks, and reports every problem of a file in one `ConfigError`.  Sizes and constants live
only in configuration objects; no other module holds a default for them.
"""
from __future__ import annotations

import json
import math
import os

REQUIRED = object()


class ConfigError(ValueError):
    """config.json is missing a key, has a wrong type, or its values contradict each other."""


class Reader:
    """Typed access to a dict read from JSON, collecting problems instead of stopping at one."""

    def __init__(self, data, where="config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: expected a JSON object")
        self.data = data
        self.where = where
        self.problems = []
        self.seen = set()

    def _get(self, key, default):
        self.seen.add(key)
        if key not in self.data or self.data[key] is None:
            if default is REQUIRED:
                self.problems.append(f"missing key '{key}'")
                return None
            return default
        return self.data[key]

    def integer(self, key, default=REQUIRED, minimum=None):
        v = self._get(key, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, int):
            self.problems.append(f"'{key}' must be an integer, got {v!r}")
            return None
        if minimum is not None and v < minimum:
            self.problems.append(f"'{key}' must be at least {minimum}, got {v}")
        return v

    def number(self, key, default=REQUIRED, positive=False):
        v = self._get(key, default)
        if v is None:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            self.problems.append(f"'{key}' must be a number, got {v!r}")
            return None
        v = float(v)
        if not math.isfinite(v) or (positive and v <= 0.0):
            self.problems.append(f"'{key}' must be finite{' and positive' if positive else ''}, got {v}")
        return v

    def boolean(self, key, default=REQUIRED):
        v = self._get(key, default)
        if v is None:
            return v
        if not isinstance(v, bool):
            self.problems.append(f"'{key}' must be true or false, got {v!r}")
            return None
        return v

    def string(self, key, default=REQUIRED):
        v = self._get(key, default)
        if v is None:
            return v
        if not isinstance(v, str):
            self.problems.append(f"'{key}' must be a string, got {v!r}")
            return None
        return v

    def string_list(self, key, default=REQUIRED, allowed=None):
        v = self._get(key, default)
        if v is None:
            return v
        if not isinstance(v, (list, tuple)) or not all(isinstance(x, str) for x in v):
            self.problems.append(f"'{key}' must be a list of strings")
            return None
        if allowed is not None:
            bad = sorted({x for x in v if x not in allowed})
            if bad:
                self.problems.append(f"'{key}' has unknown entries {bad}; allowed: {sorted(allowed)}")
        return tuple(v)

    def integer_list(self, key, default=REQUIRED):
        v = self._get(key, default)
        if v is None:
            return v
        if isinstance(v, int) and not isinstance(v, bool):
            return (v,)
        if not isinstance(v, (list, tuple)) or not all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            self.problems.append(f"'{key}' must be an integer or a list of integers")
            return None
        return tuple(v)

    def problem(self, text):
        self.problems.append(text)

    def finish(self):
        if self.problems:
            raise ConfigError(f"{self.where}: " + "; ".join(self.problems))


def read_config_json(folder):
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as fh:
            return json.load(fh)
    except FileNotFoundError as exc:
        raise ConfigError(f"{path}: no such file") from exc
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from exc


def architecture_name(data):
    """The architecture a config.json declares: `architecture`, else `model_type`."""
    for key in ("architecture", "model_type"):
        v = data.get(key)
        if isinstance(v, str):
            return v
    raise ConfigError("config.json: missing key 'architecture'")
