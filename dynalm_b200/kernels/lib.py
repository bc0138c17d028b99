"""Builds and loads the CUDA kernel libraries.

Each `csrc/<name>.cu` becomes one shared library with plain C entry points, compiled by nvcc for
sm_100a and loaded through ctypes. A library is built the first time one of its kernels is called
(or all at once by `build_all`), so a model compiles what it needs. Built files live under
`dynalm_b200/_build/` when that is writable, else under the temporary directory; the file name
carries a hash of the sources and flags, so an edited kernel is rebuilt and a stale library is
never loaded. There is no other path: if nvcc or the build fails, the call raises
ExtensionMissing.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List, Optional

from ..errors import ExtensionMissing
from ..utils import log as _log

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared"]

_lock = threading.Lock()
_load_lock = threading.Lock()
_libs: Dict[str, ctypes.CDLL] = {}


def _say(msg: str) -> None:
    _log.info("dynalm_b200", msg)


def find_nvcc() -> str:
    for cand in (os.environ.get("DYNALM_NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
                 shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise ExtensionMissing("nvcc was not found (looked at $DYNALM_NVCC, $CUDA_HOME/bin, PATH, /usr/local/cuda/bin); "
                           "the engine has no path without its CUDA kernels")


_build_dir: Optional[str] = None


def build_dir() -> str:
    global _build_dir
    with _lock:
        if _build_dir is None:
            _build_dir = _pick_build_dir()
        return _build_dir


def _pick_build_dir() -> str:
    override = os.environ.get("DYNALM_BUILD_DIR")
    cands = [override] if override else []
    cands.append(os.path.join(os.path.dirname(CSRC), "_build"))
    cands.append(os.path.join(tempfile.gettempdir(), f"dynalm_b200_build_{os.getuid()}"))
    for d in cands:
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise ExtensionMissing(f"no writable folder for built kernels (tried {', '.join(cands)})")


def sources() -> List[str]:
    return sorted(f[:-3] for f in os.listdir(CSRC) if f.endswith(".cu"))


_INCLUDE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _with_includes(name: str) -> List[str]:
    """csrc/<name>.cu and every file of csrc/ that it includes, directly or through another."""
    todo, found = [name + ".cu"], []
    while todo:
        f = todo.pop()
        if f in found or not os.path.isfile(os.path.join(CSRC, f)):
            continue
        found.append(f)
        with open(os.path.join(CSRC, f), "r", errors="replace") as fh:
            todo.extend(_INCLUDE.findall(fh.read()))
    return [found[0]] + sorted(found[1:])


def _source_hash(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + extra_flags()).encode())
    for f in _with_includes(name):
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    return h.hexdigest()[:16]


def extra_flags() -> List[str]:
    """Flags that a switch of the environment adds to every kernel build (they are part of a library's hash, so the
    builds with and without them lie side by side). DYNALM_CHECK=1: -DDL_CHECK, the kernels check every index that
    they take from device data before they use it (see csrc/check.cuh)."""
    return ["-DDL_CHECK=1"] if os.environ.get("DYNALM_CHECK", "0") not in ("", "0") else []


def _file_name(name: str) -> str:
    return f"libdl_{name}.{'check.' if extra_flags() else ''}{_source_hash(name)}.so"


def library_path(name: str, directory: Optional[str] = None) -> str:
    return os.path.join(directory or build_dir(), _file_name(name))


def _find_built(name: str) -> Optional[str]:
    """A built library of the current sources, in any of the candidate folders (a read-only
    checkout may carry one that was built elsewhere)."""
    fname = _file_name(name)
    for d in (os.environ.get("DYNALM_BUILD_DIR"), os.path.join(os.path.dirname(CSRC), "_build"),
              os.path.join(tempfile.gettempdir(), f"dynalm_b200_build_{os.getuid()}")):
        if d and os.path.isfile(os.path.join(d, fname)):
            return os.path.join(d, fname)
    return None


def compile_library(name: str, verbose: bool = True) -> str:
    """Compile csrc/<name>.cu if no library of its current sources exists; return the path."""
    src = os.path.join(CSRC, name + ".cu")
    if not os.path.isfile(src):
        raise ExtensionMissing(f"no kernel source {src}")
    have = _find_built(name)
    if have:
        return have
    out = library_path(name)
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + ARCH_FLAGS + NVCC_FLAGS + extra_flags() + ["-I", CSRC, "-o", tmp, src]
    if verbose:
        _say(f"compiling {name}.cu for sm_100a ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    done = threading.Event()

    def beat():
        while not done.wait(10.0):
            if verbose:
                _say(f"  still compiling {name}.cu ({time.time() - t0:.0f} s)")
    th = threading.Thread(target=beat, daemon=True)
    th.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise ExtensionMissing(f"nvcc failed on {name}.cu (exit {proc.returncode}):\n{log}")
    os.replace(tmp, out)
    if verbose:
        _say(f"built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    # older builds of the same source and the same kind (plain or checked) are of no use any more
    checked = bool(extra_flags())
    for f in os.listdir(os.path.dirname(out)):
        if f.startswith(f"libdl_{name}.") and f.endswith(".so") and f != os.path.basename(out) \
                and f.startswith(f"libdl_{name}.check.") == checked:
            try:
                os.unlink(os.path.join(os.path.dirname(out), f))
            except OSError:
                pass
    return out


def build_all(verbose: bool = True, jobs: int = 0) -> List[str]:
    """Compile every kernel source (in parallel); used by the build check and before shipping."""
    from concurrent.futures import ThreadPoolExecutor
    names = sources()
    jobs = jobs or min(len(names), os.cpu_count() or 4)
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        return list(pool.map(lambda n: compile_library(n, verbose), names))


def load(name: str) -> ctypes.CDLL:
    """The loaded library of csrc/<name>.cu, building it first if needed."""
    lib = _libs.get(name)
    if lib is not None:
        return lib
    with _load_lock:
        lib = _libs.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise ExtensionMissing(f"cannot load {path}: {e}") from None
            _libs[name] = lib
    return lib


def loaded_libraries() -> Dict[str, str]:
    return {n: l._name for n, l in _libs.items()}
