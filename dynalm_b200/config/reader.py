"""Typed access to the keys of a config.json object.

Mirrors the reference's `get_int / get_int_or / get_float_or` helpers
(dynalm/src/loader/hf/hf_model.cpp:23-46): a missing required key is NotFound,
a key of the wrong JSON type is Corrupt.
"""

from __future__ import annotations

import json
import os
from typing import Any, Mapping, Optional

from ..errors import Corrupt, NotFound


class KeyReader:
    """Reads typed values out of one JSON object and names the key in every error."""

    def __init__(self, obj: Mapping[str, Any], where: str = "config.json"):
        if not isinstance(obj, Mapping):
            raise Corrupt(f"{where} is not an object")
        self.obj = obj
        self.where = where

    def has(self, key: str) -> bool:
        return key in self.obj and self.obj[key] is not None

    def _int(self, key: str, value: Any) -> int:
        # JSON has one number type; 8192.0 is accepted as the integer it is, 0.5 is not.
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise Corrupt(f"{self.where}: '{key}' is not an integer")
        if isinstance(value, float):
            if value != int(value):
                raise Corrupt(f"{self.where}: '{key}' is not an integer")
            value = int(value)
        return value

    def int(self, key: str) -> int:
        if not self.has(key):
            raise NotFound(f"{self.where}: missing '{key}'")
        return self._int(key, self.obj[key])

    def int_or(self, key: str, default: int) -> int:
        return self._int(key, self.obj[key]) if self.has(key) else default

    def float_or(self, key: str, default: float) -> float:
        if not self.has(key):
            return default
        value = self.obj[key]
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise Corrupt(f"{self.where}: '{key}' is not a number")
        return float(value)

    def bool_or(self, key: str, default: bool) -> bool:
        if not self.has(key):
            return default
        value = self.obj[key]
        if not isinstance(value, bool):
            raise Corrupt(f"{self.where}: '{key}' is not a boolean")
        return value

    def str_or(self, key: str, default: Optional[str]) -> Optional[str]:
        if not self.has(key):
            return default
        value = self.obj[key]
        if not isinstance(value, str):
            raise Corrupt(f"{self.where}: '{key}' is not a string")
        return value

    def object_or_none(self, key: str) -> Optional["KeyReader"]:
        if not self.has(key):
            return None
        value = self.obj[key]
        if not isinstance(value, Mapping):
            raise Corrupt(f"{self.where}: '{key}' is not an object")
        return KeyReader(value, f"{self.where}: {key}")


# The reference refuses config files above 16 MiB before parsing them
# (dynalm/src/loader/hf/hf_model.cpp:144-156); the same bound is kept here.
MAX_CONFIG_BYTES = 16 << 20


def read_json_file(path: str) -> dict:
    """Parse a JSON file into a dict with the errors the loader promises."""
    if not os.path.isfile(path):
        raise NotFound(f"{path}: no such file")
    if os.path.getsize(path) > MAX_CONFIG_BYTES:
        raise Corrupt(f"{path}: larger than {MAX_CONFIG_BYTES} bytes")
    with open(path, "rb") as f:
        text = f.read()
    try:
        value = json.loads(text)
    except (ValueError, RecursionError) as e:
        raise Corrupt(f"{path}: {e}") from None
    if not isinstance(value, dict):
        raise Corrupt(f"{path} is not an object")
    return value
