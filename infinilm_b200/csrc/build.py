"""Compiles the CUDA sources of this folder for sm_100a and loads them with ctypes.

Each `.cu` file becomes one shared object with `extern "C"` entry points; it is
compiled with plain `nvcc` (no torch headers, so a file takes seconds) the first
time something asks for it (a `.cpp` file is host code and goes through `g++`), and kept under `_build/` beside the sources, keyed by
a hash of the source text, the included headers, the macro definitions and the
compiler flags. Nothing here falls back to another implementation: a missing
compiler or a failed compile raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, Optional, Tuple

_HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]

_lock = threading.Lock()
_loaded: Dict[Tuple[str, Tuple[Tuple[str, str], ...]], ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[infinilm_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cand = [os.environ.get("INFINILM_B200_NVCC"), shutil.which("nvcc"),
            os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
            "/usr/local/cuda/bin/nvcc"]
    for c in cand:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (PATH, CUDA_HOME, /usr/local/cuda): the CUDA kernels of "
                     "infinilm_b200 cannot be built, and there is no other implementation to fall back to")


_build_dir_cached: Optional[str] = None
_dir_lock = threading.Lock()


def build_dir() -> str:
    """`_build/` beside the sources when that is writable, else a per-user temp folder."""
    global _build_dir_cached
    with _dir_lock:
        if _build_dir_cached is None:
            _build_dir_cached = _pick_build_dir()
        return _build_dir_cached


def _pick_build_dir() -> str:
    env = os.environ.get("INFINILM_B200_BUILD_DIR")
    if env:
        os.makedirs(env, exist_ok=True)
        return env
    d = os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}.{threading.get_ident()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"infinilm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _headers_text() -> bytes:
    parts = []
    for fn in sorted(os.listdir(_HERE)):
        if fn.endswith((".cuh", ".h")):
            with open(os.path.join(_HERE, fn), "rb") as f:
                parts.append(fn.encode() + b"\0" + f.read())
    return b"\0".join(parts)


def _key(src_path: str, defines: Tuple[Tuple[str, str], ...], extra: Tuple[str, ...]) -> str:
    h = hashlib.sha256()
    with open(src_path, "rb") as f:
        h.update(f.read())
    h.update(_headers_text())
    h.update(repr(defines).encode())
    h.update(repr(ARCH_FLAGS + BASE_FLAGS + list(extra)).encode())
    return h.hexdigest()[:16]


def _env_flags() -> Tuple[str, ...]:
    """Further nvcc flags from INFINILM_B200_NVCC_FLAGS (space separated); they are part of a library's key."""
    return tuple(os.environ.get("INFINILM_B200_NVCC_FLAGS", "").split())


HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


def source_path(name: str) -> str:
    """`<name>.cu` (device code, nvcc) or `<name>.cpp` (host code, g++)."""
    for ext in (".cu", ".cpp"):
        p = os.path.join(_HERE, name + ext)
        if os.path.isfile(p):
            return p
    raise BuildError(f"no source {os.path.join(_HERE, name)}.cu or .cpp")


def so_path(name: str, defines: Optional[Dict[str, object]] = None,
            extra_flags: Tuple[str, ...] = ()) -> str:
    extra_flags = tuple(extra_flags) + _env_flags()
    dfs = tuple(sorted((k, str(v)) for k, v in (defines or {}).items()))
    src = source_path(name)
    tag = "".join(f"-{k}{v}" for k, v in dfs)
    return os.path.join(build_dir(), f"{name}{tag}-{_key(src, dfs, tuple(extra_flags))}.so")


def compile_source(name: str, defines: Optional[Dict[str, object]] = None,
                   extra_flags: Tuple[str, ...] = (), verbose: bool = False) -> str:
    """Compile `<name>.cu` if its shared object is not there yet; returns the path."""
    src = source_path(name)
    out = so_path(name, defines, extra_flags)
    if os.path.isfile(out):
        return out
    dfs = [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    if src.endswith(".cpp"):
        gxx = shutil.which(os.environ.get("CXX", "g++")) or shutil.which("g++")
        if gxx is None:
            raise BuildError("g++ was not found: the host code of infinilm_b200 cannot be built")
        cmd = [gxx] + HOST_FLAGS + dfs + ["-I", _HERE, "-o", tmp, src]
    else:
        cmd = [find_nvcc()] + ARCH_FLAGS + BASE_FLAGS + list(extra_flags) + list(_env_flags()) + dfs + ["-I", _HERE, "-o", tmp, src]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
    _say(f"compiling {os.path.basename(src)} {' '.join(dfs)}" + ("" if src.endswith(".cpp") else " for sm_100a") + " ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", build_dir())       # nvcc scratch files: HOME may not exist
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, text=True)
    done = threading.Event()

    def beat():
        while not done.wait(10.0):
            _say(f"  still compiling {os.path.basename(src)} ({time.time() - t0:.0f} s)")
    th = threading.Thread(target=beat, daemon=True)
    th.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise BuildError(f"the compiler failed on {os.path.basename(src)} (exit {proc.returncode}):\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    _say(f"  built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    if verbose and log:
        _say(log)
    return out


def load(name: str, defines: Optional[Dict[str, object]] = None,
         extra_flags: Tuple[str, ...] = ()) -> ctypes.CDLL:
    """The loaded library of `<name>.cu` compiled with `defines`; compiles on first use."""
    key = (name, tuple(sorted((k, str(v)) for k, v in (defines or {}).items())) + tuple(extra_flags))
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_source(name, defines, extra_flags)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from e
            _loaded[key] = lib
        return lib


def all_sources():
    return sorted(os.path.splitext(fn)[0] for fn in os.listdir(_HERE) if fn.endswith((".cu", ".cpp")))
