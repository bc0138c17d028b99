"""A leveled log for the package's own lines (kernel builds, engine notes, the command line's statistics).

Levels and their names are the reference's (dynalm/src/logging/log.h:16-54, log.cpp:24-37): trace, debug, info,
warn, error, off, and the user-facing names of `dynalm -q / -v`: quiet = errors only, normal = info, verbose =
debug. Lines go to standard error as `[tag] text`. The level comes from DYNALM_LOG_LEVEL when the package is
imported and from `-q`, `-v` and `--log-level` of the command line.
"""

from __future__ import annotations

import os
import sys
from typing import Optional

TRACE, DEBUG, INFO, WARN, ERROR, OFF = range(6)
_NAMES = {"trace": TRACE, "debug": DEBUG, "info": INFO, "warn": WARN, "error": ERROR, "off": OFF,
          "quiet": ERROR, "normal": INFO, "verbose": DEBUG}
_level = INFO


def parse_level(name: str) -> Optional[int]:
    return _NAMES.get(name)


def set_level(level) -> bool:
    """By number or by name; False (and no change) for an unknown name."""
    global _level
    if isinstance(level, str):
        got = parse_level(level)
        if got is None:
            return False
        level = got
    _level = int(level)
    return True


def level() -> int:
    return _level


def enabled(lvl: int) -> bool:
    return lvl >= _level


def write(lvl: int, tag: str, text: str) -> None:
    if lvl >= _level:
        print(f"[{tag}] {text}", file=sys.stderr, flush=True)


def debug(tag: str, text: str) -> None:
    write(DEBUG, tag, text)


def info(tag: str, text: str) -> None:
    write(INFO, tag, text)


def warn(tag: str, text: str) -> None:
    write(WARN, tag, text)


def error(tag: str, text: str) -> None:
    write(ERROR, tag, text)


_env = os.environ.get("DYNALM_LOG_LEVEL", "")
if _env:
    set_level(_env)
