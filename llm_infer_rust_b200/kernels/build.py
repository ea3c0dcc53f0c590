"""Compiles the native code of the package at first use and loads it.

Two kinds of libraries live under ``csrc/``:

* CUDA kernels (``*.cu``), compiled by ``nvcc`` for sm_100a into one shared
  library per (source file, compile-time sizes) and loaded with ``ctypes``.  A
  model only ever asks for the sizes that it has, so a first call compiles just
  what that model needs;
* the host runtime (``host/*.cpp``: cache manager, scheduler, batch builder),
  compiled by the C++ compiler into a Python extension module.

Built files go to ``llm_infer_rust_b200/_build`` (or, if the package folder is
read-only, to a folder under the temporary directory).  A library's file name
carries a hash of its sources and flags, so a stale build is never loaded.
There is no fallback: if a library is missing and cannot be compiled, loading
raises.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from typing import Dict, Iterable, List, Optional, Sequence

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(_PKG, "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr"]

_lock = threading.Lock()
_loaded: Dict[str, object] = {}        # library path -> loaded library
_by_name: Dict[tuple, object] = {}       # (source, defines) -> loaded library


class BuildError(RuntimeError):
    pass


_build_dir: Optional[str] = None
_build_dir_lock = threading.Lock()


def build_dir() -> str:
    global _build_dir
    with _build_dir_lock:
        if _build_dir is None:
            preferred = os.path.join(_PKG, "_build")
            try:
                os.makedirs(preferred, exist_ok=True)
                fd, probe = tempfile.mkstemp(dir=preferred)
                os.close(fd)
                os.remove(probe)
                _build_dir = preferred
            except OSError:
                # A read-only checkout: a per-user folder under the temporary directory.  Libraries found there are
                # loaded as they are, so the folder must be this user's own and closed to everybody else; a folder
                # of that name that somebody else made (or left open) is not used.
                shared = os.path.join(tempfile.gettempdir(), f"llm_infer_rust_b200_build_{os.getuid()}")
                try:
                    os.makedirs(shared, mode=0o700, exist_ok=True)
                    st = os.lstat(shared)
                    import stat
                    if not stat.S_ISDIR(st.st_mode) or st.st_uid != os.getuid() or (st.st_mode & 0o022):
                        raise OSError("the build folder is not this user's own")
                    _build_dir = shared
                except OSError:
                    _build_dir = tempfile.mkdtemp(prefix="llm_infer_rust_b200_build_")
        return _build_dir


def _say(text: str) -> None:
    print(f"[llm_infer_rust_b200] {text}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 shutil.which("nvcc")):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                     "the CUDA kernels cannot be compiled and there is no other path")


def _hash(paths: Sequence[str], extra: Iterable[str]) -> str:
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as fh:
            h.update(fh.read())
    for e in extra:
        h.update(e.encode())
    return h.hexdigest()[:12]


def _run(cmd: List[str], what: str) -> None:
    """Run a compiler, printing a line now and then while it works."""
    start = time.time()
    _say(f"compiling {what} ...")
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"  still compiling {what} ({time.time() - start:.0f} s)")

    t = threading.Thread(target=ticker, daemon=True)
    t.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        raise BuildError(f"compiling {what} failed:\n{' '.join(cmd)}\n{out}")
    _say(f"compiled {what} in {time.time() - start:.1f} s")


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _included_sources(path: str, seen: Optional[set] = None) -> List[str]:
    """``.cu`` files of this folder that ``path`` pulls in with #include "..." (headers are always hashed)."""
    seen = set() if seen is None else seen
    with open(path) as fh:
        for line in fh:
            line = line.strip()
            if line.startswith("#include \"") and line.endswith(".cu\""):
                dep = os.path.join(CSRC, line[len("#include \""):-1])
                if dep not in seen and os.path.isfile(dep):
                    seen.add(dep)
                    _included_sources(dep, seen)
    return sorted(seen)


def cuda_library_path(source: str, defines: Optional[Dict[str, object]] = None) -> str:
    defines = defines or {}
    src = os.path.join(CSRC, source)
    tag = "_".join(f"{k}{v}" for k, v in sorted(defines.items()))
    digest = _hash([src] + _included_sources(src) + _headers(),
                   [repr(sorted(defines.items())), " ".join(ARCH_FLAGS + NVCC_FLAGS)])
    stem = os.path.splitext(source)[0] + (f"_{tag}" if tag else "")
    return os.path.join(build_dir(), f"lib{stem}.{digest}.so")


def build_cuda_library(source: str, defines: Optional[Dict[str, object]] = None) -> str:
    """Compile ``csrc/<source>`` with ``-D`` defines unless it is built already; return the path."""
    defines = defines or {}
    path = cuda_library_path(source, defines)
    if os.path.isfile(path):
        return path
    lock_path = path + ".lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not os.path.isfile(path):
                tmp = f"{path}.{os.getpid()}.tmp"
                cmd = [find_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + [f"-D{k}={v}" for k, v in sorted(defines.items())]
                cmd += ["-I", CSRC, "-o", tmp, os.path.join(CSRC, source)]
                _run(cmd, os.path.basename(path))
                os.replace(tmp, path)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    try:
        os.remove(lock_path)
    except OSError:
        pass
    return path


def load_cuda_library(source: str, defines: Optional[Dict[str, object]] = None) -> ctypes.CDLL:
    """The loaded library of ``source`` compiled with ``defines``; compiled at the first call.

    Every kernel call comes through here, so a process looks a library up by name; the
    sources are hashed (and compiled, if that hash has no library yet) only the first time."""
    name = (source, tuple(sorted(defines.items())) if defines else ())
    lib = _by_name.get(name)
    if lib is not None:
        return lib
    key = cuda_library_path(source, defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(build_cuda_library(source, defines))
            _loaded[key] = lib
        _by_name[name] = lib
        return lib


def all_cuda_libraries(head_dims: Iterable[int]) -> List[tuple]:
    """(source, defines) of every CUDA library that the package can ask for, attention for ``head_dims``."""
    per_head = ("attention.cu", "attention_mma.cu", "decode_attention_static.cu")
    libs = [(f, None) for f in sorted(os.listdir(CSRC)) if f.endswith(".cu") and f not in per_head]
    return libs + [(f, {"HEAD_DIM": int(d)}) for f in per_head for d in head_dims]


def _host_sources() -> List[str]:
    d = os.path.join(CSRC, "host")
    return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith((".cpp", ".h")))


def build_host_runtime() -> str:
    import pybind11
    sources = _host_sources()
    cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
    if not cxx:
        raise BuildError("no C++ compiler was found for the host runtime")
    flags = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]
    digest = _hash(sources, [" ".join(flags), sys.version, pybind11.__version__])
    folder = os.path.join(build_dir(), f"host_{digest}")
    path = os.path.join(folder, "_host_runtime" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
    if os.path.isfile(path):
        return path
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not os.path.isfile(path):
                tmp = f"{path}.{os.getpid()}.tmp"
                cmd = [cxx] + flags + ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
                cmd += [s for s in sources if s.endswith(".cpp")] + ["-o", tmp]
                _run(cmd, "the host runtime (cache manager, scheduler, batch builder)")
                os.replace(tmp, path)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return path


def load_host_runtime():
    with _lock:
        mod = _loaded.get("host")
        if mod is None:
            path = build_host_runtime()
            spec = importlib.util.spec_from_file_location("_host_runtime", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _loaded["host"] = mod
        return mod
