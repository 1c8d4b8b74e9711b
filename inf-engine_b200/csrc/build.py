"""Build and load the engine's CUDA libraries.

Sources are plain ``.cu`` files with ``extern "C"`` launchers; each library is
compiled with ``nvcc`` for sm_100a into ``_build/`` beside the sources (or into
the temporary folder when that is not writable) and loaded with ``ctypes``.
The folder name carries a hash of the sources and flags, so an edit rebuilds
and two processes that race build the same thing.  A library holds only what
was asked for: the head size of a specialised attention kernel, for example, is
a ``-D`` flag, and only the sizes a model needs get compiled at its first call.

There is no fallback: if a library is absent and cannot be built, loading
raises.
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
from pathlib import Path

SRC_DIR = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

# name -> sources; the headers every library depends on
LIBRARIES = {
    "core": ["elementwise.cu", "attention_general.cu", "gemm_simt.cu", "sampling.cu"],
}
HEADERS = ["common.cuh"]

_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[inf-engine_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found (set NVCC or CUDA_HOME); the engine has no path without its CUDA kernels")


def _digest(sources: list[str], defines: dict, extra_headers: list[str]) -> str:
    h = hashlib.sha256()
    for name in sorted(set(sources) | set(HEADERS) | set(extra_headers)):
        h.update(name.encode())
        h.update((SRC_DIR / name).read_bytes())
    h.update(repr(sorted(defines.items())).encode())
    h.update(repr(ARCH_FLAGS + BASE_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_root() -> Path:
    root = SRC_DIR / "_build"
    try:
        root.mkdir(exist_ok=True)
        probe = root / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return root
    except OSError:
        alt = Path(tempfile.gettempdir()) / f"inf_engine_b200_build_{os.getuid()}"
        alt.mkdir(parents=True, exist_ok=True)
        return alt


def library_path(name: str, sources: list[str], defines: dict | None = None,
                 extra_headers: list[str] | None = None) -> Path:
    defines = defines or {}
    tag = _digest(sources, defines, extra_headers or [])
    return _build_root() / f"{name}-{tag}" / f"lib{name}.so"


def build_library(name: str, sources: list[str], defines: dict | None = None,
                  extra_headers: list[str] | None = None, verbose: bool = True) -> Path:
    """Compile ``sources`` into one shared library unless it is there already."""
    defines = defines or {}
    out = library_path(name, sources, defines, extra_headers)
    if out.is_file():
        return out
    nvcc = find_nvcc()
    work = Path(tempfile.mkdtemp(prefix=f".{name}-", dir=out.parent.parent))
    dflags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
    t0 = time.time()
    if verbose:
        _say(f"compiling {name} ({len(sources)} files) for sm_100a; this happens once")

    def compile_one(src: str) -> Path:
        obj = work / (Path(src).stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *BASE_FLAGS, *dflags, "-I", str(SRC_DIR), "-c", str(SRC_DIR / src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {src}:\n{r.stderr[-4000:]}")
        return obj

    done = []
    stop = threading.Event()

    def ticker():
        while not stop.wait(10.0):
            _say(f"  still compiling {name}: {len(done)}/{len(sources)} files done after {time.time() - t0:.0f} s")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    try:
        with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
            objs = []
            for obj in ex.map(compile_one, sources):
                done.append(obj)
                objs.append(obj)
        tmp_so = work / f"lib{name}.so"
        r = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_so), *map(str, objs), "-lcuda"],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"link of {name} failed:\n{r.stderr[-4000:]}")
        out.parent.mkdir(parents=True, exist_ok=True)
        os.replace(tmp_so, out)
    finally:
        stop.set()
        shutil.rmtree(work, ignore_errors=True)
    if verbose:
        _say(f"built {out.name} in {time.time() - t0:.0f} s")
    return out


def load_library(name: str, sources: list[str] | None = None, defines: dict | None = None,
                 extra_headers: list[str] | None = None) -> ctypes.CDLL:
    key = name + repr(sorted((defines or {}).items()))
    with _lock:
        if key in _loaded:
            return _loaded[key]
        path = build_library(name, sources or LIBRARIES[name], defines, extra_headers)
        try:
            lib = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelBuildError(f"cannot load {path}: {e}") from None
        lib._path = str(path)
        _loaded[key] = lib
        return lib


def build_all(verbose: bool = True) -> list[Path]:
    """Compile every library the package can ask for (used by the build check)."""
    from .catalog import all_build_requests

    return [build_library(n, s, d, h, verbose) for (n, s, d, h) in all_build_requests()]
