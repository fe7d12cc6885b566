"""Compiles the CUDA sources of this folder for sm_100a and loads them through ctypes.

Each `.cu` file becomes one shared library `_build/<name>-<hash>.so`, built by nvcc the first
time something needs it and reused afterwards; the hash covers the source, every file of this
folder that it includes (directly or through another) and the flags, so an edit rebuilds exactly
what depends on it.  Nothing here falls back to another
implementation: a missing compiler or a failed build raises `KernelBuildError`.
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
from pathlib import Path

SRC_DIR = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-O3"]

_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


class KernelBuildError(RuntimeError):
    pass


def sources() -> list[str]:
    """Names (without suffix) of every kernel library of the package."""
    return sorted(p.stem for p in SRC_DIR.glob("*.cu"))


def find_nvcc() -> str:
    cand = [shutil.which("nvcc")]
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root:
            cand.append(str(Path(root) / "bin" / "nvcc"))
    for c in cand:
        if c and Path(c).is_file() and os.access(c, os.X_OK):
            return c
    raise KernelBuildError("nvcc not found (PATH, CUDA_HOME, /usr/local/cuda): the sm_100a kernels cannot be built")


_build_dir_cache: Path | None = None


def _build_dir() -> Path:
    """`_build/` beside the sources; a per-user folder under the temp dir if that is read-only."""
    global _build_dir_cache
    if _build_dir_cache is not None:
        return _build_dir_cache
    d = SRC_DIR / "_build"
    try:
        d.mkdir(exist_ok=True)
        fd, probe = tempfile.mkstemp(dir=d)
        os.close(fd)
        os.unlink(probe)
    except OSError:
        d = Path(tempfile.gettempdir()) / f"zinfer_b200-build-{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
    _build_dir_cache = d
    return d


_INCLUDE = re.compile(rb'^[ \t]*#[ \t]*include[ \t]*"([^"]+)"', re.M)


def _closure(name: str) -> list[Path]:
    """`<name>.cu` and the files of this folder it includes, transitively, in a fixed order."""
    seen: dict[str, Path] = {}
    todo = [SRC_DIR / f"{name}.cu"]
    while todo:
        p = todo.pop()
        if p.name in seen or not p.is_file():
            continue
        seen[p.name] = p
        todo += [SRC_DIR / m.decode() for m in _INCLUDE.findall(p.read_bytes())]
    return [seen[k] for k in sorted(seen)]


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    for p in _closure(name):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def library_path(name: str) -> Path:
    return _build_dir() / f"{name}-{_digest(name)}.so"


def compile_library(name: str, verbose: bool = True) -> Path:
    """Builds `<name>.cu` if its library is absent; returns the library's path."""
    src = SRC_DIR / f"{name}.cu"
    if not src.is_file():
        raise KernelBuildError(f"no kernel source {src}")
    out = library_path(name)
    if out.is_file():
        return out
    nvcc = find_nvcc()
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(SRC_DIR), "-o", str(tmp), str(src)]
    if verbose:
        print(f"[zinfer_b200] compiling {src.name} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", str(out.parent))
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    while True:
        try:
            log, _ = proc.communicate(timeout=20)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[zinfer_b200]   ... still compiling {src.name} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed on {src.name} (exit {proc.returncode}):\n{log}")
    os.replace(tmp, out)
    for old in out.parent.glob(f"{name}-*.so"):          # libraries of earlier versions of the source
        if old != out and ".tmp" not in old.name:
            old.unlink(missing_ok=True)
    if verbose:
        print(f"[zinfer_b200] built {out.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library of `<name>.cu`, compiling it first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> list[Path]:
    """Compiles every kernel library (in parallel); used by the build check."""
    from concurrent.futures import ThreadPoolExecutor

    names = sources()
    with ThreadPoolExecutor(max_workers=min(8, len(names) or 1)) as ex:
        return list(ex.map(lambda n: compile_library(n, verbose), names))
