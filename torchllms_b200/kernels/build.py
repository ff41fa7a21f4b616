"""Compiling the CUDA sources for sm_100a and loading them as shared libraries.

Each ``csrc/<name>.cu`` becomes one library, built with ``nvcc`` the first time
something in it is called and loaded through ``ctypes``.  The file name of the
built library carries a hash of the source, the shared headers and the flags,
so an edited source is rebuilt and a stale library is never picked up.
Libraries are written next to the sources (``csrc/_build``) when that folder
can be written, else under the system's temporary folder, so a read-only
checkout and a user without a home directory both work.
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
from typing import Dict, Iterable, List, Optional

CSRC = Path(__file__).resolve().parent.parent / "csrc"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--shared", "-Xcompiler", "-fPIC",
]
# TORCHLLMS_B200_DEBUG=1 builds every kernel with -DTL_DEBUG: indices that come from the step's
# index data (cache slots, pages of a block table, rows to gather) are range-checked on the device
# before they are used; a bad one is skipped and reported through the library's debug word (see
# common.cuh), never trapped on.  TORCHLLMS_B200_NVCC_FLAGS adds flags of the caller's own.  Either
# changes the name of the built library, so builds of different kinds live side by side.
if os.environ.get("TORCHLLMS_B200_DEBUG", "") not in ("", "0"):
    NVCC_FLAGS.append("-DTL_DEBUG")
NVCC_FLAGS += os.environ.get("TORCHLLMS_B200_NVCC_FLAGS", "").split()
# libraries that need more than the CUDA runtime
EXTRA_LINK: Dict[str, List[str]] = {}

ALL_LIBRARIES = ("elementwise", "rope", "attention", "attention_mma", "attention_decode", "attention_prefill", "gemm_simt", "gemm_tcgen05", "sampling")


class KernelBuildError(RuntimeError):
    pass


_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def _say(msg: str) -> None:
    print(f"[torchllms_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(Path(os.environ[var]) / "bin" / "nvcc")
    which = shutil.which("nvcc")
    if which:
        candidates.append(Path(which))
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    for c in candidates:
        if c.is_file() and os.access(c, os.X_OK):
            return str(c)
    raise KernelBuildError(
        "nvcc was not found (looked at $CUDA_HOME/bin, $PATH and /usr/local/cuda/bin); the CUDA "
        "kernels of torchllms_b200 cannot be built and there is no other implementation")


def _headers() -> List[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + EXTRA_LINK.get(name, [])).encode())
    for p in [CSRC / f"{name}.cu"] + _headers():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _build_dirs() -> List[Path]:
    dirs = []
    if os.environ.get("TORCHLLMS_B200_BUILD_DIR"):
        dirs.append(Path(os.environ["TORCHLLMS_B200_BUILD_DIR"]))
    dirs.append(CSRC / "_build")
    uid = os.getuid() if hasattr(os, "getuid") else 0
    dirs.append(Path(tempfile.gettempdir()) / f"torchllms_b200_build_{uid}")
    return dirs


def _writable_dir() -> Path:
    for d in _build_dirs():
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".probe_{os.getpid()}_{threading.get_ident()}"
            probe.write_bytes(b"")
            probe.unlink()
            return d
        except OSError:
            continue
    raise KernelBuildError("no writable folder for built kernels: tried " + ", ".join(map(str, _build_dirs())))


def library_path(name: str) -> Optional[Path]:
    """Path of the up-to-date built library, if one exists already."""
    fname = f"{name}.{_digest(name)}.so"
    for d in _build_dirs():
        p = d / fname
        if p.is_file():
            return p
    return None


def compile_library(name: str) -> Path:
    src = CSRC / f"{name}.cu"
    if not src.is_file():
        raise KernelBuildError(f"no kernel source {src}")
    existing = library_path(name)
    if existing is not None:
        return existing
    out_dir = _writable_dir()
    out = out_dir / f"{name}.{_digest(name)}.so"
    tmp = out_dir / f".{out.name}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [find_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), str(src), "-o", str(tmp), *EXTRA_LINK.get(name, [])]
    _say(f"compiling {src.name} for sm_100a ...")
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    next_note = 15.0
    while True:
        try:
            output, _ = proc.communicate(timeout=5.0)
            break
        except subprocess.TimeoutExpired:
            if time.time() - t0 >= next_note:
                _say(f"still compiling {src.name} ({time.time() - t0:.0f} s)")
                next_note += 15.0
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"nvcc failed on {src.name} (exit {proc.returncode}):\n{output}")
    os.replace(tmp, out)
    for stale in out_dir.glob(f"{name}.*.so"):        # libraries of earlier versions of this source
        if stale != out:
            try:
                stale.unlink()
            except OSError:
                pass
    _say(f"built {out.name} in {time.time() - t0:.1f} s")
    return out


def load_library(name: str) -> ctypes.CDLL:
    """The library of ``csrc/<name>.cu``, compiled first if need be."""
    lib = _loaded.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"could not load {path}: {e}") from None
            _loaded[name] = lib
    return lib


def build_libraries(names: Iterable[str] = ALL_LIBRARIES, jobs: Optional[int] = None) -> List[Path]:
    """Compile several libraries side by side (does not load them)."""
    names = [n for n in names]
    missing = [n for n in names if library_path(n) is None]
    if missing:
        with ThreadPoolExecutor(max_workers=jobs or min(len(missing), os.cpu_count() or 2)) as pool:
            list(pool.map(compile_library, missing))
    return [library_path(n) for n in names]


def loaded_libraries() -> Dict[str, str]:
    return {name: lib._name for name, lib in _loaded.items()}
