"""Compiles the CUDA sources of this folder for sm_100a and loads them with ctypes.

Each ``<module>.cu`` becomes one shared library ``_build/<module>[-defs]-<hash>.so``,
compiled by ``nvcc`` at the first call that needs it (a few seconds each) and reused
afterwards; the hash covers the source, the shared header, the flags and the
``-D`` definitions a caller specialises the module with (head size and the like), so
a model compiles what it needs and nothing else.  While ``nvcc`` runs, a line is
printed to stderr every few seconds.  There is no fallback: if ``nvcc`` is missing or
fails, the call raises ``PhotonError(NOT_BUILT)``.
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
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, Optional, Tuple

from ..errors import ErrorCode, PhotonError

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
INCLUDE_DIR = os.path.join(os.path.dirname(CSRC_DIR), "include")          # photon/kernels.h
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]
ALL_MODULES = ("elementwise", "rope_kv", "attention", "gemm_f32", "gemm_skinny", "gemm_skinny_fused", "gemm_skinny_static",
               "gemm_tc", "gemm_tc2", "sampling")

_loaded: Dict[Tuple[str, Tuple[Tuple[str, str], ...]], ctypes.CDLL] = {}
_lock = threading.Lock()
_build_dir: Optional[str] = None


def _log(msg: str) -> None:
    print(f"[photon] {msg}", file=sys.stderr, flush=True)


def build_dir() -> str:
    """In-tree ``csrc/_build`` when it can be written, else ``$PHOTON_BUILD_DIR``, else a
    per-user folder under the system's temporary directory."""
    global _build_dir
    if _build_dir is not None:
        return _build_dir
    candidates = []
    if os.environ.get("PHOTON_BUILD_DIR"):
        candidates.append(os.environ["PHOTON_BUILD_DIR"])
    candidates.append(os.path.join(CSRC_DIR, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"photon_build_{os.getuid()}"))
    for c in candidates:
        try:
            os.makedirs(c, exist_ok=True)
            probe = os.path.join(c, f".probe_{os.getpid()}")
            with open(probe, "w") as f:
                f.write("x")
            os.remove(probe)
            _build_dir = c
            return c
        except OSError:
            continue
    raise PhotonError(ErrorCode.NOT_BUILT, "no writable folder for the compiled kernels: tried " + ", ".join(candidates))


def find_nvcc() -> str:
    for cand in (os.environ.get("PHOTON_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise PhotonError(ErrorCode.NOT_BUILT, "nvcc was not found (PATH, $CUDA_HOME, /usr/local/cuda): "
                      "the CUDA kernels cannot be compiled and there is no other path")


def _source_hash(module: str, defines: Tuple[Tuple[str, str], ...], extra_flags: Tuple[str, ...]) -> str:
    h = hashlib.sha256()
    for name in (f"{module}.cu", "common.cuh"):
        with open(os.path.join(CSRC_DIR, name), "rb") as f:
            h.update(f.read())
    for name in sorted(os.listdir(CSRC_DIR)):
        # other headers, and sources that a module may include whole
        if (name.endswith((".cuh", ".h")) and name != "common.cuh") or \
                (name.endswith(".cu") and name != f"{module}.cu" and module.startswith(name[:-3])):
            with open(os.path.join(CSRC_DIR, name), "rb") as f:
                h.update(f.read())
    with open(os.path.join(INCLUDE_DIR, "photon", "kernels.h"), "rb") as f:
        h.update(f.read())
    h.update(repr((ARCH_FLAGS, BASE_FLAGS, defines, extra_flags)).encode())
    return h.hexdigest()[:12]


def library_path(module: str, defines: Optional[Dict[str, object]] = None,
                 extra_flags: Iterable[str] = ()) -> str:
    defs = tuple(sorted((k, str(v)) for k, v in (defines or {}).items()))
    tag = "".join(f"-{k}{v}" for k, v in defs)
    return os.path.join(build_dir(), f"{module}{tag}-{_source_hash(module, defs, tuple(extra_flags))}.so")


def compile_module(module: str, defines: Optional[Dict[str, object]] = None,
                   extra_flags: Iterable[str] = (), verbose: bool = False) -> str:
    """Compile if the library is not there yet; returns its path."""
    src = os.path.join(CSRC_DIR, f"{module}.cu")
    if not os.path.isfile(src):
        raise PhotonError(ErrorCode.NOT_BUILT, f"no CUDA source {src}")
    out = library_path(module, defines, extra_flags)
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [nvcc, *ARCH_FLAGS, *BASE_FLAGS, *extra_flags, "-I", CSRC_DIR, "-I", INCLUDE_DIR]
    for k, v in sorted((defines or {}).items()):
        cmd.append(f"-D{k}={v}")
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", tmp, src]
    _log(f"compiling {os.path.basename(out)} for sm_100a ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    out_text = []
    reader = threading.Thread(target=lambda: out_text.append(proc.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            proc.wait(timeout=5.0)
            break
        except subprocess.TimeoutExpired:
            _log(f"  still compiling {module} ({time.time() - t0:.0f} s)")
    reader.join()
    text = "".join(out_text)
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise PhotonError(ErrorCode.NOT_BUILT, f"nvcc failed on {module}.cu:\n{text}")
    os.replace(tmp, out)
    _log(f"  built {module} in {time.time() - t0:.1f} s")
    if verbose and text:
        print(text, file=sys.stderr)
    return out


def load_module(module: str, defines: Optional[Dict[str, object]] = None,
                extra_flags: Iterable[str] = ()) -> ctypes.CDLL:
    key = (module, tuple(sorted((k, str(v)) for k, v in (defines or {}).items())))
    with _lock:
        lib = _loaded.get(key)
    if lib is not None:
        return lib
    path = compile_module(module, defines, extra_flags)
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        raise PhotonError(ErrorCode.NOT_BUILT, f"cannot load {path}: {e}") from None
    with _lock:
        _loaded.setdefault(key, lib)
        return _loaded[key]


def ensure_built(modules: Iterable[object]) -> None:
    """Compile several modules at once (``nvcc`` processes run side by side).  An item is a module
    name or a pair (name, definitions) for a module specialised with ``-D``."""
    todo = []
    for m in modules:
        name, defines = (m, None) if isinstance(m, str) else (m[0], dict(m[1]) if m[1] else None)
        key = (name, tuple(sorted((defines or {}).items())))
        if key not in [k for k, _, _ in todo] and not os.path.isfile(library_path(name, defines)):
            todo.append((key, name, defines))
    if not todo:
        return
    with ThreadPoolExecutor(max_workers=min(8, len(todo))) as pool:
        list(pool.map(lambda item: compile_module(item[1], item[2]), todo))


# specialisations that the build check compiles besides the plain modules (the Llama 3.2 1B shape)
DEFAULT_SPECIALISATIONS = (("attention_flash", {"HEAD_DIM": 64}), ("attention_tc", {"HEAD_DIM": 64}),
                           ("attention_decode", {"HEAD_DIM": 64}), ("attention_flash", {"HEAD_DIM": 128}),
                           ("attention_tc", {"HEAD_DIM": 128}), ("attention_decode", {"HEAD_DIM": 128}))


def build_all(verbose: bool = False) -> None:
    ensure_built(list(ALL_MODULES) + list(DEFAULT_SPECIALISATIONS))
