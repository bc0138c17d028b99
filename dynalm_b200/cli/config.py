"""Where a command's options come from: a config file, DYNALM_* environment variables and the command line,
merged into one argument list that the command's own parser reads; later sources win:

    config file  <  DYNALM_<OPTION>  <  command line

as the reference's commands do (dynalm/src/config/config.h:3-20,56; config.cpp:188-318). The file is `--config PATH`,
else $DYNALM_CONFIG, else ~/.dynalm/config.yaml when it exists. Two formats: the reference's YAML subset (sections
of `key: value`, `#` comments, optional quotes; the documented keys below, of which a command takes those it has an
option for, an unknown key being an error with its line number), and flat lines `option = value` (a bare `option`
for a flag). Environment: DYNALM_ + the option's long name in capitals with '-' as '_'.
"""

from __future__ import annotations

import os
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from ..errors import InvalidArgument, NotFound

# the reference's documented YAML keys -> the long option they set (config.cpp:15-37); the server's keys are known,
# so that one file serves every command, and skipped by commands without the option
YAML_KEYS: Dict[str, str] = {
    "model.path": "model", "model.id": "model-id", "runtime.device": "backend", "runtime.mode": "mode",
    "runtime.execution": "execution", "runtime.threads": "threads", "runtime.context_length": "ctx",
    "runtime.batch_tokens": "batch", "runtime.int8_decode": "int8-decode",
    "scheduler.max_concurrent_requests": "max-active", "scheduler.policy": "policy", "kv_cache.dtype": "kv",
    "sampling.temperature": "temperature", "sampling.max_tokens": "max-tokens", "server.host": "host",
    "server.port": "port", "server.http_threads": "http-threads", "server.request_timeout": "request-timeout",
    "server.shutdown_timeout": "shutdown-timeout", "server.admin": "disable-admin", "server.metrics": "disable-metrics",
}
_TRUE, _FALSE = ("1", "true", "yes", "on"), ("0", "false", "no", "off")

Options = Dict[str, bool]          # long option name without "--" -> whether it takes a value


def env_name(option: str) -> str:
    return "DYNALM_" + option.replace("-", "_").upper()


def _strip_comment(line: str) -> str:
    quote = ""
    for i, c in enumerate(line):
        if quote:
            if c == quote:
                quote = ""
        elif c in "\"'":
            quote = c
        elif c == "#":
            return line[:i]
    return line


def _unquote(v: str) -> str:
    return v[1:-1] if len(v) >= 2 and v[0] in "\"'" and v[-1] == v[0] else v


def _entries(text: str, origin: str) -> Tuple[bool, List[Tuple[str, Optional[str], int]]]:
    """(is YAML, [(key, value or None for a bare flag, line number)])."""
    lines = [(n + 1, _strip_comment(raw)) for n, raw in enumerate(text.splitlines())]
    first = next((l.strip() for _, l in lines if l.strip()), "")
    yaml = "=" not in first and ":" in first
    out: List[Tuple[str, Optional[str], int]] = []
    if not yaml:
        for n, line in lines:
            line = line.strip()
            if not line:
                continue
            key, eq, value = line.partition("=")
            out.append((key.strip(), _unquote(value.strip()) if eq else None, n))
        return False, out
    section = ""
    for n, raw in lines:
        if not raw.strip():
            continue
        indent = len(raw) - len(raw.lstrip(" "))
        if "\t" in raw[:len(raw) - len(raw.lstrip())]:
            raise InvalidArgument(f"{origin}:{n}: tabs are not allowed for indentation")
        key, colon, value = raw.strip().partition(":")
        if not colon or not key.strip():
            raise InvalidArgument(f"{origin}:{n}: expected 'key: value'")
        key, value = key.strip(), value.strip()
        if value.startswith(("[", "{", "&", "*", "|", ">")) or key.startswith("- "):
            raise InvalidArgument(f"{origin}:{n}: lists, anchors and multi-line values are not supported")
        if indent == 0:
            if value == "":
                section = key
            else:
                section = ""
                out.append((key, _unquote(value), n))
        else:
            if not section:
                raise InvalidArgument(f"{origin}:{n}: an indented key outside a section")
            if value == "":
                raise InvalidArgument(f"{origin}:{n}: deeper nesting is not supported")
            out.append((f"{section}.{key}", _unquote(value), n))
    return True, out


def parse_config_text(text: str, options: Options, origin: str) -> List[str]:
    """The file's contents as "--option [value]" arguments for a command that takes `options`."""
    yaml, entries = _entries(text, origin)
    args: List[str] = []
    for key, value, n in entries:
        where = f"{origin}:{n}"
        option = key
        if yaml:
            option = YAML_KEYS.get(key, key)
            if key not in YAML_KEYS and option not in options:
                raise InvalidArgument(f"{where}: unknown key '{key}'")
            if option not in options:
                continue                   # a documented key that this command does not use
        elif option not in options:
            raise InvalidArgument(f"{where}: unknown key '{key}'")
        if options[option]:
            if value is None or value == "":
                raise InvalidArgument(f"{where}: '{key}' needs a value")
            args += [f"--{option}", value]
        elif value is None or value.lower() in _TRUE:
            args.append(f"--{option}")
        elif value.lower() not in _FALSE:
            raise InvalidArgument(f"{where}: '{key}' is a flag (true/false)")
    return args


def default_config_path(env: Callable[[str], Optional[str]] = os.environ.get) -> str:
    return env("DYNALM_CONFIG") or os.path.join(env("HOME") or os.getcwd(), ".dynalm", "config.yaml")


def merge_config(cli_args: Sequence[str], options: Options,
                 env: Optional[Callable[[str], Optional[str]]] = None) -> List[str]:
    """File arguments, then environment arguments, then the command line without its --config. `env` can be given
    for tests; the user's own ~/.dynalm/config.yaml is then not looked at."""
    real_env = env is None
    env = env or os.environ.get
    cli: List[str] = []
    path, explicit = env("DYNALM_CONFIG") or "", bool(env("DYNALM_CONFIG"))
    it = iter(range(len(cli_args)))
    for i in it:
        if cli_args[i] == "--config":
            if i + 1 >= len(cli_args):
                raise InvalidArgument("--config needs a file path")
            path, explicit = cli_args[i + 1], True
            next(it)
        else:
            cli.append(cli_args[i])
    if not explicit and real_env:
        default = default_config_path()
        path = default if os.path.isfile(default) else ""
    merged: List[str] = []
    if path:
        try:
            with open(path, "r") as f:
                text = f.read()
        except OSError:
            raise NotFound(f"cannot open config file {path}") from None
        merged = parse_config_text(text, options, path)
    for option, takes_value in options.items():
        v = env(env_name(option))
        if v is None:
            continue
        if takes_value:
            merged += [f"--{option}", v]
        elif v.lower() in _TRUE:
            merged.append(f"--{option}")
    return merged + cli
