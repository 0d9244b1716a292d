"""Build and load the native (CUDA sm_100a / C++) libraries of the engine.

Every ``csrc/*.cu`` file becomes ``_lib/lib<name>.so`` (``nvcc -gencode
arch=compute_100a,code=sm_100a``); every ``csrc/host/*.cpp`` file becomes
``_lib/lib<name>.so`` with ``g++``.  The libraries export plain ``extern "C"``
launchers that take raw device pointers and a CUDA stream, so they do not link
against libtorch and compile in seconds.  Python calls them through ``ctypes``.

The reference has no native code (it is pure Python on top of external
libraries), so there is nothing to cite here.
"""
from __future__ import annotations

import contextlib
import ctypes
import fcntl
import hashlib
import os
import re
import shutil
import subprocess
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Dict, List, Optional

_PKG = Path(__file__).resolve().parent
CSRC = _PKG / "csrc"
# LMMS_B200_DEBUG_BOUNDS=1 selects the debug build of every CUDA library: compiled with -DB200_DEBUG_BOUNDS (the
# per-element index checks behind B200_DBG_INDEX in csrc/common.cuh) into its own directory, so that the release
# objects stay in place.  Failed checks raise the per-device status word that ``ops._cuda.check_status`` turns into
# an exception.
DEBUG_BOUNDS = os.environ.get("LMMS_B200_DEBUG_BOUNDS", "0") == "1"
LIBDIR = _PKG / ("_lib_dbg" if DEBUG_BOUNDS else "_lib")

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]
if DEBUG_BOUNDS:
    NVCC_FLAGS.append("-DB200_DEBUG_BOUNDS=1")
GXX_FLAGS = ["-O3", "-std=c++17", "-shared", "-fPIC", "-march=x86-64-v3", "-pthread"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


def _nvcc() -> Optional[str]:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    return None


def cuda_sources() -> List[Path]:
    return sorted(CSRC.glob("*.cu"))


def host_sources() -> List[Path]:
    return sorted((CSRC / "host").glob("*.cpp"))


_INCLUDE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _local_includes(path: Path, seen: set) -> None:
    """Headers of this tree that ``path`` includes, transitively."""
    for name in _INCLUDE.findall(path.read_text(errors="ignore")):
        for base in (path.parent, CSRC):
            hdr = (base / name).resolve()
            if hdr.exists() and hdr not in seen:
                seen.add(hdr)
                _local_includes(hdr, seen)
                break


def _digest(src: Path) -> str:
    """Hash of a source file and of the in-tree headers it pulls in: a library is rebuilt when one of them changes."""
    h = hashlib.sha1()
    h.update(src.read_bytes())
    seen: set = set()
    _local_includes(src, seen)
    for hdr in sorted(seen):
        h.update(hdr.name.encode())
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _lib_path(name: str) -> Path:
    return LIBDIR / f"lib{name}.so"


def _stale(src: Path) -> bool:
    out = _lib_path(src.stem)
    stamp = out.with_suffix(".sha1")
    if not out.exists() or not stamp.exists():
        return True
    return stamp.read_text().strip() != _digest(src)


@contextlib.contextmanager
def _build_lock(name: str):
    """Inter-process lock for one library: under ``torchrun`` every rank may find the same
    library stale at the same moment; only one of them compiles, the others wait and then
    see the fresh stamp."""
    LIBDIR.mkdir(exist_ok=True)
    with open(LIBDIR / f".{name}.lock", "w") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def _compile(src: Path, verbose: bool = False) -> str:
    """Compile to a temporary file and rename it into place, so that a process that is
    loading the library never sees a half-written file."""
    LIBDIR.mkdir(exist_ok=True)
    final = _lib_path(src.stem)
    out = final.with_name(f".{final.name}.{os.getpid()}.tmp")
    if src.suffix == ".cu":
        nvcc = _nvcc()
        if nvcc is None:
            raise RuntimeError(f"nvcc not found; cannot build {src.name}")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-o", str(out), str(src)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
    else:
        cmd = ["g++", *GXX_FLAGS, "-I", str(CSRC), "-o", str(out), str(src)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        with contextlib.suppress(FileNotFoundError):
            out.unlink()
        raise RuntimeError(f"build of {src.name} failed:\n{res.stdout}\n{res.stderr}")
    os.replace(out, final)
    stamp_tmp = final.with_name(f".{final.stem}.{os.getpid()}.sha1.tmp")
    stamp_tmp.write_text(_digest(src))
    os.replace(stamp_tmp, final.with_suffix(".sha1"))
    return res.stderr


def _compile_if_stale(src: Path, force: bool = False, verbose: bool = False) -> Optional[str]:
    with _build_lock(src.stem):
        if force or _stale(src):
            return _compile(src, verbose)
    return None


def build_all(force: bool = False, verbose: bool = False) -> List[str]:
    """Compile every native source that is missing or out of date.  Returns built names."""
    todo = [s for s in cuda_sources() + host_sources() if force or _stale(s)]
    if not todo:
        return []
    with ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
        logs = list(ex.map(lambda s: _compile_if_stale(s, force, verbose), todo))
    if verbose:
        for s, log in zip(todo, logs):
            print(f"== {s.name}\n{log or ''}")
    return [s.stem for s in todo]


def lib(name: str) -> ctypes.CDLL:
    """Load ``_lib/lib<name>.so``, building it first when a compiler is at hand.

    Raises loudly when the library is missing: a GPU code path never falls back to
    eager PyTorch silently.
    """
    with _lock:
        if name in _loaded:
            return _loaded[name]
        src = CSRC / f"{name}.cu"
        if not src.exists():
            src = CSRC / "host" / f"{name}.cpp"
        if not src.exists():
            raise FileNotFoundError(f"no native source for '{name}'")
        path = _lib_path(name)
        if _stale(src):
            if src.suffix == ".cu" and _nvcc() is None and path.exists():
                pass  # use the shipped binary
            else:
                _compile_if_stale(src)
        handle = ctypes.CDLL(str(path))
        _loaded[name] = handle
        return handle


def have_cuda_libs() -> bool:
    return all(_lib_path(s.stem).exists() for s in cuda_sources())
